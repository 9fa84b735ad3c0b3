// Descriptor compiler (host only): strided windows and shard boxes -> 2-D scatter records.
//
// mxb_plan_pull is the closed form of the reference's plan_pull
// (refit/reshard/slice_plan.py:227-339): the window a loader cut out of a full
// source tensor is resolved to a box in source coordinates (with the view ->
// source dim permutation), intersected with every published shard box, and each
// overlap becomes records whose row-by-row expansion is the reference's run
// list in the reference's order.  mxb_plan_reshard clips strided regions of a
// flat tensor to the contiguous byte range one FSDP rank holds.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/mxb200.h"

namespace mxb {
void set_error(const char *fmt, ...);
}
using mxb::set_error;

namespace {

struct Box {
    int64_t lo[MXB_MAX_DIMS], hi[MXB_MAX_DIMS];
};

void row_major(const int64_t *shape, int nd, int64_t *stride) {
    int64_t acc = 1;
    for (int d = nd - 1; d >= 0; --d) {
        stride[d] = acc;
        acc *= shape[d];
    }
}

// Window -> (box in source coordinates, destination strides in source-dim order).
// slice_plan.py:170-225: every window dim of extent > 1 walks exactly one source dim and
// the offset is a corner of the box.
int32_t window_box(const mxb_window &w, Box &box, int64_t *dst_stride) {
    const int nd = w.ndim_src, nw = w.ndim_win;
    if (nd < 0 || nd > MXB_MAX_DIMS || nw < 0 || nw > MXB_MAX_DIMS) {
        set_error("mxb_plan_pull: at most %d dims", MXB_MAX_DIMS);
        return MXB_ERR_ARG;
    }
    if (w.keep_rank && nw != nd) {
        set_error("unsupported window: rank change");
        return MXB_ERR_UNSUPPORTED;
    }
    int64_t gst[MXB_MAX_DIMS];
    row_major(w.global_shape, nd, gst);
    int perm[MXB_MAX_DIMS];
    bool used[MXB_MAX_DIMS] = {};
    for (int d = 0; d < nw; ++d) {
        perm[d] = -1;
        if (w.win_shape[d] == 1) continue;
        for (int s = 0; s < nd; ++s)
            if (gst[s] == w.win_stride[d]) {  // the first source dim with that stride
                perm[d] = s;
                break;
            }
        if (perm[d] < 0) {
            set_error("unsupported window: stride %lld is not a source dim (merged dims)",
                      (long long)w.win_stride[d]);
            return MXB_ERR_UNSUPPORTED;
        }
        if (used[perm[d]]) {
            set_error("unsupported window: not a permutation of the source dims");
            return MXB_ERR_UNSUPPORTED;
        }
        used[perm[d]] = true;
    }
    int64_t corner = 0;
    for (int s = 0; s < nd; ++s) {
        const int64_t g = w.global_shape[s];
        box.lo[s] = g ? (w.win_offset / gst[s]) % g : 0;
        box.hi[s] = g ? box.lo[s] + 1 : box.lo[s];
        dst_stride[s] = 0;
    }
    for (int d = 0; d < nw; ++d)
        if (perm[d] >= 0) {
            box.hi[perm[d]] = box.lo[perm[d]] + w.win_shape[d];
            dst_stride[perm[d]] = w.dst_stride[d];
        }
    for (int s = 0; s < nd; ++s) {
        if (box.hi[s] > w.global_shape[s]) {
            set_error("unsupported window: box leaves the source");
            return MXB_ERR_UNSUPPORTED;
        }
        corner += box.lo[s] * gst[s];
    }
    if (corner != w.win_offset) {
        set_error("unsupported window: offset is not a box corner");
        return MXB_ERR_UNSUPPORTED;
    }
    return MXB_OK;
}

struct Sink {
    mxb_desc2d *out;
    uint32_t *shard_of;
    uint64_t cap, n = 0;
    void push(const mxb_desc2d &d, uint32_t shard) {
        if (n < cap) {
            out[n] = d;
            if (shard_of) shard_of[n] = shard;
        }
        ++n;
    }
};

// Records covering `overlap`; trailing dims merge while both layouts are unit-packed
// (slice_plan.py:278-284), the next dim out is the row dim, the rest are enumerated in
// row-major order, which is the reference's run order.
void box_records(const Box &ov, int nd, const int64_t *src_origin, const int64_t *src_stride,
                 const int64_t *dst_origin, const int64_t *dst_stride, uint64_t elsize,
                 uint64_t src_base, uint64_t dst_base, uint32_t shard, Sink &sink) {
    int64_t size[MXB_MAX_DIMS];
    for (int d = 0; d < nd; ++d) size[d] = ov.hi[d] - ov.lo[d];
    int64_t run = 1;
    int p = nd;
    while (p > 0 && src_stride[p - 1] == run && dst_stride[p - 1] == run) {
        run *= size[p - 1];
        --p;
    }
    int64_t s0 = 0, d0 = 0;
    for (int d = 0; d < nd; ++d) {
        s0 += (ov.lo[d] - src_origin[d]) * src_stride[d];
        d0 += (ov.lo[d] - dst_origin[d]) * dst_stride[d];
    }
    const uint64_t row_bytes = (uint64_t)run * elsize;
    if (p == 0) {
        sink.push({src_base + (uint64_t)s0 * elsize, dst_base + (uint64_t)d0 * elsize, 1, row_bytes,
                   row_bytes, row_bytes},
                  shard);
        return;
    }
    uint64_t rows = (uint64_t)size[p - 1];
    uint64_t sp = (uint64_t)src_stride[p - 1] * elsize, dp = (uint64_t)dst_stride[p - 1] * elsize;
    int p_outer = p - 1;
    if (rows > 1 && (sp < row_bytes || dp < row_bytes)) {  // overlapping rows: one record per row
        p_outer = p;
        rows = 1;
    }
    if (rows == 1) sp = dp = row_bytes;
    int64_t idx[MXB_MAX_DIMS] = {};
    for (;;) {
        int64_t so = 0, dof = 0;
        for (int d = 0; d < p_outer; ++d) {
            so += idx[d] * src_stride[d];
            dof += idx[d] * dst_stride[d];
        }
        sink.push({src_base + (uint64_t)(s0 + so) * elsize, dst_base + (uint64_t)(d0 + dof) * elsize,
                   rows, row_bytes, sp, dp},
                  shard);
        int d = p_outer - 1;
        while (d >= 0 && ++idx[d] == size[d]) idx[d--] = 0;
        if (d < 0) break;
    }
}

}  // namespace

extern "C" {

int32_t mxb_plan_pull(const mxb_window *w, const mxb_shard *shards, uint64_t n_shards,
                      uint64_t dst_base, mxb_desc2d *out, uint32_t *out_shard, uint64_t cap,
                      uint64_t *n_out) {
    if (!w || (!shards && n_shards) || (!out && cap) || !n_out || w->elsize == 0) {
        set_error("mxb_plan_pull: bad arguments");
        return MXB_ERR_ARG;
    }
    Box need;
    int64_t dst_stride[MXB_MAX_DIMS];
    int32_t rc = window_box(*w, need, dst_stride);
    if (rc != MXB_OK) return rc;
    const int nd = w->ndim_src;
    Sink sink{out, out_shard, cap};
    for (uint64_t i = 0; i < n_shards; ++i) {
        const mxb_shard &sh = shards[i];
        if (sh.ndim != nd) {
            set_error("mxb_plan_pull: shard %llu has rank %d, the source has rank %d",
                      (unsigned long long)i, sh.ndim, nd);
            return MXB_ERR_ARG;
        }
        Box ov;
        bool empty = false;
        for (int d = 0; d < nd; ++d) {
            ov.lo[d] = need.lo[d] > sh.offset[d] ? need.lo[d] : sh.offset[d];
            const int64_t end = sh.offset[d] + sh.shape[d];
            ov.hi[d] = need.hi[d] < end ? need.hi[d] : end;
            if (ov.lo[d] >= ov.hi[d]) empty = true;
        }
        if (empty) continue;
        int64_t sst[MXB_MAX_DIMS];
        row_major(sh.shape, nd, sst);
        box_records(ov, nd, sh.offset, sst, need.lo, dst_stride, w->elsize, sh.addr,
                    dst_base + (uint64_t)w->dst_offset * w->elsize, (uint32_t)i, sink);
    }
    *n_out = sink.n;
    if (sink.n > cap) {
        set_error("mxb_plan_pull: %llu records needed, room for %llu", (unsigned long long)sink.n,
                  (unsigned long long)cap);
        return MXB_ERR_NOMEM;
    }
    return MXB_OK;
}

int32_t mxb_plan_reshard(const mxb_desc2d *regions, uint64_t n, uint64_t shard_lo, uint64_t shard_hi,
                         uint64_t src_base, uint64_t max_record_bytes, mxb_desc2d *out, uint64_t cap,
                         uint64_t *n_out) {
    if ((!regions && n) || (!out && cap) || !n_out || shard_hi < shard_lo) {
        set_error("mxb_plan_reshard: bad arguments");
        return MXB_ERR_ARG;
    }
    std::vector<mxb_desc2d> clipped;
    const uint64_t lo = shard_lo, hi = shard_hi;
    for (uint64_t i = 0; i < n; ++i) {
        const mxb_desc2d &g = regions[i];  // src = byte offset inside the flat full tensor
        if (g.rows == 0 || g.row_bytes == 0) continue;
        const uint64_t so = g.src, rb = g.row_bytes, sp = g.src_pitch, dp = g.dst_pitch;
        if (g.rows == 1) {
            const uint64_t a = so > lo ? so : lo, b = so + rb < hi ? so + rb : hi;
            if (a < b) clipped.push_back({src_base + a - lo, g.dst + (a - so), 1, b - a, b - a, b - a});
            continue;
        }
        if (sp < rb || dp < rb) {
            set_error("mxb_plan_reshard: region %llu has a pitch smaller than its rows",
                      (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        // rows that overlap [lo, hi): row r covers [so + r*sp, so + r*sp + rb)
        uint64_t r_lo = 0;
        if (lo > so + rb - 1) r_lo = (lo - so - rb) / sp + 1;  // first row whose end is past lo
        if (hi <= so) continue;
        uint64_t r_hi = (hi - so - 1) / sp;  // last row that starts before hi
        if (r_hi > g.rows - 1) r_hi = g.rows - 1;
        if (r_lo > r_hi) continue;
        uint64_t first_full = r_lo, last_full = r_hi;
        uint64_t start = so + r_lo * sp;
        if (start < lo) {  // first row clipped at its head
            const uint64_t a = lo, b = start + rb < hi ? start + rb : hi;
            clipped.push_back({src_base, g.dst + r_lo * dp + (a - start), 1, b - a, b - a, b - a});
            first_full = r_lo + 1;
        }
        start = so + r_hi * sp;
        bool has_tail = false;
        mxb_desc2d tail{};
        if (start + rb > hi && r_hi >= first_full) {  // last row clipped at its end
            const uint64_t a = start, b = hi;
            tail = {src_base + a - lo, g.dst + r_hi * dp, 1, b - a, b - a, b - a};
            has_tail = true;
            if (r_hi == 0) {
                clipped.push_back(tail);
                continue;
            }
            last_full = r_hi - 1;
        }
        if (last_full + 1 > first_full) {
            const uint64_t rows = last_full - first_full + 1;
            const uint64_t s0 = so + first_full * sp;
            clipped.push_back({src_base + s0 - lo, g.dst + first_full * dp, rows, rb,
                               rows > 1 ? sp : rb, rows > 1 ? dp : rb});
        }
        if (has_tail) clipped.push_back(tail);
    }
    // cut large records so that an all-to-all schedule can interleave destinations finely
    uint64_t m = 0;
    auto emit = [&](const mxb_desc2d &d) {
        if (m < cap) out[m] = d;
        ++m;
    };
    for (const mxb_desc2d &c : clipped) {
        if (!max_record_bytes || c.rows * c.row_bytes <= max_record_bytes) {
            emit(c);
        } else if (c.rows == 1) {
            uint64_t step = max_record_bytes / 256 * 256;
            if (step < 256) step = 256;
            for (uint64_t off = 0; off < c.row_bytes; off += step) {
                const uint64_t len = step < c.row_bytes - off ? step : c.row_bytes - off;
                emit({c.src + off, c.dst + off, 1, len, len, len});
            }
        } else {
            uint64_t per = max_record_bytes / c.row_bytes;
            if (per < 1) per = 1;
            for (uint64_t r0 = 0; r0 < c.rows; r0 += per) {
                const uint64_t rows = per < c.rows - r0 ? per : c.rows - r0;
                emit({c.src + r0 * c.src_pitch, c.dst + r0 * c.dst_pitch, rows, c.row_bytes,
                      rows > 1 ? c.src_pitch : c.row_bytes, rows > 1 ? c.dst_pitch : c.row_bytes});
            }
        }
    }
    *n_out = m;
    if (m > cap) {
        set_error("mxb_plan_reshard: %llu records needed, room for %llu", (unsigned long long)m,
                  (unsigned long long)cap);
        return MXB_ERR_NOMEM;
    }
    return MXB_OK;
}

}  // extern "C"
