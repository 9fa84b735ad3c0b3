// Kernel 1/3: descriptor-driven scatter (sm_100a).
//
// One persistent launch walks a device-resident table of 2-D byte slices
// (mxb_desc2d) cut into tiles of at most 64 KiB.  Sources and destinations may
// be local HBM, a peer GPU's HBM (NVLink P2P loads / stores) or pinned host
// memory (PCIe reads), so the same kernel serves the staging-ring placement,
// the warm install and the refit reshard.
//
// Two tile engines:
//   * vector engine - 512 threads, 16-byte loads/stores unrolled 4 deep, with
//     head/tail handling and narrower vectors when src and dst disagree mod 16;
//   * bulk engine   - one warp per CTA drives cp.async.bulk (TMA, non-tensor)
//     global->shared->global through a 3-stage 64 KiB ring, for tables whose
//     addresses, pitches and row sizes are all multiples of 16.
#include "bulk.cuh"
#include <mutex>

#include "common.cuh"

namespace mxb {

struct Tile {
    uint32_t desc;   // index into the descriptor table
    uint32_t local;  // tile number inside that descriptor
};

// ---------------------------------------------------------------------------
// vector engine
// ---------------------------------------------------------------------------

template <typename V>
__device__ __forceinline__ V ld_stream(const V *p) {
    return __ldcs(p);
}
template <typename V>
__device__ __forceinline__ void st_stream(V *p, V v) {
    __stcs(p, v);
}

// Copy n elements of vector type V with T cooperating threads, 4 loads in flight.
template <typename V>
__device__ __forceinline__ void copy_vec(V *__restrict__ d, const V *__restrict__ s, uint64_t n,
                                         uint32_t t, uint32_t T) {
    uint64_t i = t;
    for (; i + 3ull * T < n; i += 4ull * T) {
        V a = ld_stream(s + i);
        V b = ld_stream(s + i + T);
        V c = ld_stream(s + i + 2ull * T);
        V e = ld_stream(s + i + 3ull * T);
        st_stream(d + i, a);
        st_stream(d + i + T, b);
        st_stream(d + i + 2ull * T, c);
        st_stream(d + i + 3ull * T, e);
    }
    for (; i < n; i += T) st_stream(d + i, ld_stream(s + i));
}

template <typename V>
__device__ __forceinline__ void copy_span_w(char *d, const char *s, uint64_t n, uint32_t t,
                                            uint32_t T) {
    constexpr uint64_t W = sizeof(V);
    // bytes until the destination reaches a W boundary (src then agrees, since
    // the caller chose W as the largest power of two dividing src^dst)
    uint64_t head = (W - ((uint64_t)(uintptr_t)d & (W - 1))) & (W - 1);
    if (head > n) head = n;
    for (uint64_t i = t; i < head; i += T) d[i] = s[i];
    d += head;
    s += head;
    n -= head;
    uint64_t nv = n / W;
    copy_vec<V>(reinterpret_cast<V *>(d), reinterpret_cast<const V *>(s), nv, t, T);
    uint64_t done = nv * W;
    for (uint64_t i = done + t; i < n; i += T) d[i] = s[i];
}

// Destination 16-byte aligned, source only A-byte aligned (A = 8 or 4): every
// 16-byte store is assembled from 16/A narrower loads, so a checkpoint whose
// data section starts 8 bytes off a 16-byte boundary still moves at full width
// on the store side.
template <typename S>
__device__ __forceinline__ uint4 gather16(const S *p);
template <>
__device__ __forceinline__ uint4 gather16<uint2>(const uint2 *p) {
    uint2 a = __ldcs(p), b = __ldcs(p + 1);
    return make_uint4(a.x, a.y, b.x, b.y);
}
template <>
__device__ __forceinline__ uint4 gather16<uint32_t>(const uint32_t *p) {
    return make_uint4(__ldcs(p), __ldcs(p + 1), __ldcs(p + 2), __ldcs(p + 3));
}

template <typename S>
__device__ __forceinline__ void copy_span_shift(char *d, const char *s, uint64_t n, uint32_t t,
                                                uint32_t T) {
    constexpr uint64_t PER = 16 / sizeof(S);
    uint64_t head = (16 - ((uint64_t)(uintptr_t)d & 15)) & 15;
    if (head > n) head = n;
    for (uint64_t i = t; i < head; i += T) d[i] = s[i];
    d += head;
    s += head;
    n -= head;
    const uint64_t nv = n >> 4;
    uint4 *dv = reinterpret_cast<uint4 *>(d);
    const S *sv = reinterpret_cast<const S *>(s);
    uint64_t i = t;
    for (; i + 3ull * T < nv; i += 4ull * T) {
        uint4 a = gather16<S>(sv + i * PER);
        uint4 b = gather16<S>(sv + (i + T) * PER);
        uint4 c = gather16<S>(sv + (i + 2ull * T) * PER);
        uint4 e = gather16<S>(sv + (i + 3ull * T) * PER);
        __stcs(dv + i, a);
        __stcs(dv + i + T, b);
        __stcs(dv + i + 2ull * T, c);
        __stcs(dv + i + 3ull * T, e);
    }
    for (; i < nv; i += T) __stcs(dv + i, gather16<S>(sv + i * PER));
    for (uint64_t j = (nv << 4) + t; j < n; j += T) d[j] = s[j];
}

// Copy an arbitrary byte span with T threads (t = this thread's index).
__device__ __forceinline__ void copy_span(char *d, const char *s, uint64_t n, uint32_t t,
                                          uint32_t T) {
    uint32_t mis = (uint32_t)(((uint64_t)(uintptr_t)d ^ (uint64_t)(uintptr_t)s) & 15u);
    if (mis == 0)
        copy_span_w<uint4>(d, s, n, t, T);
    else if ((mis & 7u) == 0)
        copy_span_shift<uint2>(d, s, n, t, T);
    else if ((mis & 3u) == 0)
        copy_span_shift<uint32_t>(d, s, n, t, T);
    else if ((mis & 1u) == 0)
        copy_span_w<uint16_t>(d, s, n, t, T);
    else
        for (uint64_t i = t; i < n; i += T) d[i] = s[i];
}

constexpr int kVecThreads = 512;

// rows x nvec 16-byte vectors, both sides 16-byte aligned; at most 64 KiB in total
__device__ __forceinline__ void copy_rows16(char *d, const char *s, uint32_t rows, uint32_t nvec,
                                            uint64_t sp, uint64_t dp, uint32_t t) {
    const uint32_t total = rows * nvec;
    uint32_t i = t;
    for (; i + 3 * kVecThreads < total; i += 4 * kVecThreads) {
        uint32_t r[4], v[4];
        uint4 x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t j = i + k * kVecThreads;
            r[k] = j / nvec;
            v[k] = j - r[k] * nvec;
            x[k] = __ldcs(reinterpret_cast<const uint4 *>(s + (uint64_t)r[k] * sp) + v[k]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            __stcs(reinterpret_cast<uint4 *>(d + (uint64_t)r[k] * dp) + v[k], x[k]);
    }
    for (; i < total; i += kVecThreads) {
        const uint32_t r = i / nvec, v = i - r * nvec;
        __stcs(reinterpret_cast<uint4 *>(d + (uint64_t)r * dp) + v,
               __ldcs(reinterpret_cast<const uint4 *>(s + (uint64_t)r * sp) + v));
    }
}

constexpr uint64_t kWarpRowMax = 8192;  // rows up to this size are copied one warp per row

__global__ void __launch_bounds__(kVecThreads)
scatter_vec_kernel(const mxb_desc2d *__restrict__ descs, const Tile *__restrict__ tiles,
                   uint64_t total_tiles) {
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5, nwarps = kVecThreads / 32;
    for (uint64_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const Tile tile = tiles[t];
        const mxb_desc2d d = descs[tile.desc];
        char *dst = reinterpret_cast<char *>(d.dst);
        const char *src = reinterpret_cast<const char *>(d.src);
        if (d.row_bytes >= kTileBytes) {
            // a piece of one long row
            const uint64_t per_row = (d.row_bytes + kTileBytes - 1) / kTileBytes;
            const uint64_t row = tile.local / per_row, piece = tile.local % per_row;
            const uint64_t off = piece * kTileBytes;
            const uint64_t len = d.row_bytes - off < kTileBytes ? d.row_bytes - off : kTileBytes;
            copy_span(dst + row * d.dst_pitch + off, src + row * d.src_pitch + off, len, tid,
                      kVecThreads);
        } else {
            const uint64_t rows_per_tile = kTileBytes / d.row_bytes;
            const uint64_t r0 = (uint64_t)tile.local * rows_per_tile;
            const uint64_t r1 = d.rows < r0 + rows_per_tile ? d.rows : r0 + rows_per_tile;
            if (d.src_pitch == d.row_bytes && d.dst_pitch == d.row_bytes) {
                // rows are back to back on both sides: one flat span
                copy_span(dst + r0 * d.row_bytes, src + r0 * d.row_bytes, (r1 - r0) * d.row_bytes,
                          tid, kVecThreads);
            } else if (((d.src | d.dst | d.src_pitch | d.dst_pitch | d.row_bytes) & 15u) == 0) {
                // aligned strided rows (a row-parallel slice): the tile is a rows x vectors
                // grid walked by the whole CTA, four independent 16-byte loads per thread
                // in flight whatever the row length
                copy_rows16(dst + r0 * d.dst_pitch, src + r0 * d.src_pitch, (uint32_t)(r1 - r0),
                            (uint32_t)(d.row_bytes >> 4), d.src_pitch, d.dst_pitch, tid);
            } else if (d.row_bytes <= kWarpRowMax) {
                for (uint64_t r = r0 + warp; r < r1; r += nwarps)
                    copy_span(dst + r * d.dst_pitch, src + r * d.src_pitch, d.row_bytes, lane, 32);
            } else {
                for (uint64_t r = r0; r < r1; ++r)
                    copy_span(dst + r * d.dst_pitch, src + r * d.src_pitch, d.row_bytes, tid,
                              kVecThreads);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// bulk engine (cp.async.bulk through shared memory)
// ---------------------------------------------------------------------------

constexpr int kBulkStages = 3;
constexpr uint32_t kBulkSpin = 1u << 24;  // bounded mbarrier wait (iterations)

__device__ __forceinline__ uint64_t umin64(uint64_t a, uint64_t b) { return a < b ? a : b; }

struct TileGeom {
    const char *src;
    char *dst;
    uint64_t rows, row_bytes, src_pitch, dst_pitch;  // rows*row_bytes <= 64 KiB
};

__device__ __forceinline__ TileGeom tile_geom(const mxb_desc2d &d, uint32_t local) {
    TileGeom g;
    if (d.row_bytes >= kTileBytes) {
        const uint64_t per_row = (d.row_bytes + kTileBytes - 1) / kTileBytes;
        const uint64_t row = local / per_row, off = (local % per_row) * kTileBytes;
        g.src = reinterpret_cast<const char *>(d.src) + row * d.src_pitch + off;
        g.dst = reinterpret_cast<char *>(d.dst) + row * d.dst_pitch + off;
        g.rows = 1;
        g.row_bytes = umin64(kTileBytes, d.row_bytes - off);
        g.src_pitch = g.dst_pitch = g.row_bytes;
    } else {
        const uint64_t rows_per_tile = kTileBytes / d.row_bytes;
        const uint64_t r0 = (uint64_t)local * rows_per_tile;
        g.rows = umin64(d.rows, r0 + rows_per_tile) - r0;
        g.row_bytes = d.row_bytes;
        g.src_pitch = d.src_pitch;
        g.dst_pitch = d.dst_pitch;
        g.src = reinterpret_cast<const char *>(d.src) + r0 * d.src_pitch;
        g.dst = reinterpret_cast<char *>(d.dst) + r0 * d.dst_pitch;
        if (g.src_pitch == g.row_bytes && g.dst_pitch == g.row_bytes) {
            g.row_bytes *= g.rows;
            g.rows = 1;
            g.src_pitch = g.dst_pitch = g.row_bytes;
        }
    }
    return g;
}

// One warp per CTA.  Lanes share the per-row copy issue; lane 0 owns the
// barriers.  Every wait is bounded: when one runs out the kernel records
// DEV_TIMEOUT, drains its own copies with a bounded wait and returns.
__global__ void __launch_bounds__(32)
scatter_bulk_kernel(const mxb_desc2d *__restrict__ descs, const Tile *__restrict__ tiles,
                    uint64_t total_tiles, uint32_t *status) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[kBulkStages];
    const uint32_t lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < kBulkStages; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // my tiles: blockIdx.x, +gridDim.x, ...
    const uint64_t first = blockIdx.x;
    if (first >= total_tiles) return;
    const uint64_t mine = (total_tiles - first + gridDim.x - 1) / gridDim.x;

    auto issue_load = [&](uint64_t k) {
        const Tile tile = tiles[first + k * gridDim.x];
        const TileGeom g = tile_geom(descs[tile.desc], tile.local);
        const int s = (int)(k % kBulkStages);
        unsigned char *buf = smem + (size_t)s * kTileBytes;
        if (lane == 0) mbar_expect_tx(&bars[s], (uint32_t)(g.rows * g.row_bytes));
        __syncwarp();
        for (uint64_t r = lane; r < g.rows; r += 32)
            bulk_g2s(buf + r * g.row_bytes, g.src + r * g.src_pitch, (uint32_t)g.row_bytes,
                     &bars[s]);
    };

    // Bounded, warp-uniform wait for the load of tile k to land.
    auto wait_tile = [&](uint64_t k, uint32_t limit) -> bool {
        const int s = (int)(k % kBulkStages);
        const uint32_t parity = (uint32_t)((k / kBulkStages) & 1);
        for (uint32_t spins = 0; spins < limit; ++spins)
            if (__all_sync(0xffffffffu, mbar_try_wait(&bars[s], parity))) return true;
        return false;
    };

    bool failed = false;
    uint64_t k = 0, issued = 1;
    issue_load(0);
    for (; k < mine; ++k) {
        const int s = (int)(k % kBulkStages);
        if (k + 1 < mine) {
            // stage (k+1)%3 last held tile k-2: its stores must have read smem
            bulk_wait_read<1>();
            __syncwarp();
            issue_load(k + 1);
            issued = k + 2;
        }
        if (!wait_tile(k, kBulkSpin)) {
            failed = true;
            break;
        }
        const Tile tile = tiles[first + k * gridDim.x];
        const TileGeom g = tile_geom(descs[tile.desc], tile.local);
        unsigned char *buf = smem + (size_t)s * kTileBytes;
        for (uint64_t r = lane; r < g.rows; r += 32)
            bulk_s2g(g.dst + r * g.dst_pitch, buf + r * g.row_bytes, (uint32_t)g.row_bytes);
        bulk_commit();
    }
    bulk_wait_all<0>();
    if (failed) {
        if (lane == 0) atomicExch(status, DEV_TIMEOUT);
        // give the loads still in flight a bounded time to land before the
        // shared memory they target is released
        for (uint64_t j = k; j < issued; ++j) wait_tile(j, 1u << 16);
    }
}

// A plain copy: 16-byte loads and stores, four in flight per thread, grid-stride.  The
// yardstick the other kernels' achieved rates are compared with on the same memory path
// (HBM to HBM, or stores into a peer over NVLink).
__global__ void __launch_bounds__(512) copy_probe_kernel(const uint4 *__restrict__ src,
                                                         uint4 *__restrict__ dst, uint64_t n16) {
    const uint64_t stride = (uint64_t)gridDim.x * 512;
    uint64_t i = (uint64_t)blockIdx.x * 512 + threadIdx.x;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], e = src[i + 3 * stride];
        dst[i] = a;
        dst[i + stride] = b;
        dst[i + 2 * stride] = c;
        dst[i + 3 * stride] = e;
    }
    for (; i < n16; i += stride) dst[i] = src[i];
}

// The same with 32-byte (256-bit) loads and stores, which sm_100 has for global memory.
__global__ void __launch_bounds__(512) copy_probe_kernel_32(const uint4 *__restrict__ src,
                                                            uint4 *__restrict__ dst, uint64_t n32) {
    const uint64_t stride = (uint64_t)gridDim.x * 512;
    for (uint64_t i = (uint64_t)blockIdx.x * 512 + threadIdx.x; i < n32; i += 2 * stride) {
        uint32_t a[8], b[8];
        const bool two = i + stride < n32;
        asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]),
                       "=r"(a[7])
                     : "l"(src + 2 * i));
        if (two)
            asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]),
                           "=r"(b[6]), "=r"(b[7])
                         : "l"(src + 2 * (i + stride)));
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 2 * i), "r"(a[0]),
                     "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7])
                     : "memory");
        if (two)
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 2 * (i + stride)),
                         "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]),
                         "r"(b[7])
                         : "memory");
    }
}

// ---------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------

// A record goes to the bulk engine when every address, pitch and row size is a
// multiple of 16 bytes (cp.async.bulk's rule) and rows are long enough for one
// bulk copy per row to pay; everything else goes to the vector engine.
static bool bulk_shape_ok(const mxb_desc2d &d) {
    if ((d.src | d.dst | d.row_bytes) & 15u) return false;
    if (d.rows > 1 && ((d.src_pitch | d.dst_pitch) & 15u)) return false;
    return d.row_bytes >= 1024;
}

// Which addresses belong to another GPU.  Stores to a peer over NVLink go faster
// from the vector engine (many warps posting 16-byte stores) than from the bulk
// engine (one warp per SM issuing bulk copies), so records that touch peer memory
// are routed to the vector engine.  Allocations are few (one arena per peer), so
// a small cache of ranges answers per record.  (A peer range mapped through CUDA IPC
// answers the pointer query with the device that opened it and so counts as local:
// its records take the bulk engine, whose bulk stores cross NVLink as well.)
class PeerRanges {
  public:
    explicit PeerRanges(int device) : device_(device) {
        if (device_ >= 0) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) ==
                cudaSuccess)
                range_ = reinterpret_cast<range_fn>(fn);
            cudaGetLastError();
        }
    }
    bool is_peer(uint64_t ptr) {
        if (device_ < 0) return false;
        for (const Entry &e : cache_)
            if (ptr >= e.base && ptr < e.end) return e.peer;
        cudaPointerAttributes attr;
        Entry e{ptr, ptr + 1, false};
        if (cudaPointerGetAttributes(&attr, reinterpret_cast<void *>(ptr)) == cudaSuccess) {
            e.peer = (attr.type == cudaMemoryTypeDevice && attr.device != device_);
            unsigned long long base = 0;
            size_t size = 0;
            if (attr.type == cudaMemoryTypeDevice && range_ && range_(&base, &size, ptr) == 0 && size) {
                e.base = base;
                e.end = base + size;
            }
        }
        cudaGetLastError();
        if (cache_.size() < 256) cache_.push_back(e);
        return e.peer;
    }

  private:
    typedef int (*range_fn)(unsigned long long *, size_t *, unsigned long long);
    struct Entry {
        uint64_t base, end;
        bool peer;
    };
    int device_;
    range_fn range_ = nullptr;
    std::vector<Entry> cache_;
};

size_t scatter_table_bytes(const mxb_desc2d *descs, uint64_t n, uint64_t *live_out,
                           uint64_t *tiles_out) {
    uint64_t live = 0, total = 0;
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t t = tiles_of(descs[i]);
        if (t) {
            ++live;
            total += t;
        }
    }
    if (live_out) *live_out = live;
    if (tiles_out) *tiles_out = total;
    return ((live * sizeof(mxb_desc2d) + 255) & ~size_t(255)) + total * sizeof(Tile);
}

int32_t build_scatter_table(const mxb_desc2d *descs, uint64_t n, void *host_buf, void *dev_buf,
                            ScatterTable *out, uint64_t *bulk_begin, uint64_t *vec_begin,
                            int device) {
    PeerRanges peers(device);
    std::vector<uint8_t> use_bulk(n, 0);
    for (uint64_t i = 0; i < n; ++i)
        if (tiles_of(descs[i]) && bulk_shape_ok(descs[i]) && !peers.is_peer(descs[i].dst) &&
            !peers.is_peer(descs[i].src))
            use_bulk[i] = 1;
    uint64_t live = 0, total = 0;
    scatter_table_bytes(descs, n, &live, &total);
    if (live > 0xffffffffull) {
        set_error("too many descriptors (%llu)", (unsigned long long)live);
        return MXB_ERR_ARG;
    }
    const size_t desc_bytes = (live * sizeof(mxb_desc2d) + 255) & ~size_t(255);
    mxb_desc2d *hd = reinterpret_cast<mxb_desc2d *>(host_buf);
    Tile *ht = reinterpret_cast<Tile *>(reinterpret_cast<char *>(host_buf) + desc_bytes);
    // pass 1: count the bulk tiles so the two lists can be laid out back to back
    uint64_t n_bulk = 0;
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t t = tiles_of(descs[i]);
        if (t > 0xffffffffull) {
            set_error("descriptor %llu has too many tiles", (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        if (t && use_bulk[i]) n_bulk += t;
    }
    uint64_t di = 0, bi = 0, vi = 0;
    Tile *hb = ht, *hv = ht + n_bulk;
    for (uint64_t i = 0; i < n; ++i) {
        if (bulk_begin) bulk_begin[i] = bi;
        if (vec_begin) vec_begin[i] = vi;
        uint64_t t = tiles_of(descs[i]);
        if (!t) continue;
        hd[di] = descs[i];
        if (use_bulk[i])
            for (uint64_t k = 0; k < t; ++k) hb[bi++] = Tile{(uint32_t)di, (uint32_t)k};
        else
            for (uint64_t k = 0; k < t; ++k) hv[vi++] = Tile{(uint32_t)di, (uint32_t)k};
        ++di;
    }
    if (bulk_begin) bulk_begin[n] = bi;
    if (vec_begin) vec_begin[n] = vi;
    out->descs = reinterpret_cast<const mxb_desc2d *>(dev_buf);
    out->tiles = reinterpret_cast<const char *>(dev_buf) + desc_bytes;
    out->n_bulk = n_bulk;
    out->n_vec = total - n_bulk;
    out->bytes = desc_bytes + total * sizeof(Tile);
    return MXB_OK;
}

static int32_t launch_vec(mxb_ctx *ctx, DeviceState *dv, const mxb_desc2d *dd, const Tile *dt,
                          uint64_t count, cudaStream_t stream, int ctas_per_sm = 4) {
    if (!count) return MXB_OK;
    uint64_t grid = (uint64_t)dv->sm_count * ctas_per_sm;
    if (grid > count) grid = count;
    scatter_vec_kernel<<<(unsigned)grid, kVecThreads, 0, stream>>>(dd, dt, count);
    MXB_CUDA(cudaGetLastError());
    ctx->launches.fetch_add(1);
    return MXB_OK;
}

static int32_t launch_bulk(mxb_ctx *ctx, DeviceState *dv, const mxb_desc2d *dd, const Tile *dt,
                           uint64_t count, cudaStream_t stream) {
    if (!count) return MXB_OK;
    static std::once_flag attr_once[64];
    const size_t smem = (size_t)kBulkStages * kTileBytes;
    if (dv->device < 64) {
        cudaError_t attr_rc = cudaSuccess;
        std::call_once(attr_once[dv->device], [&]() {
            attr_rc = cudaFuncSetAttribute(scatter_bulk_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        });
        MXB_CUDA(attr_rc);
    }
    uint64_t grid = (uint64_t)dv->sm_count;
    if (grid > count) grid = count;
    scatter_bulk_kernel<<<(unsigned)grid, 32, smem, stream>>>(dd, dt, count, dv->status);
    MXB_CUDA(cudaGetLastError());
    ctx->launches.fetch_add(1);
    return MXB_OK;
}

int32_t launch_scatter_tiles(mxb_ctx *ctx, DeviceState *dv, const ScatterTable &tb,
                             uint64_t bulk_begin, uint64_t bulk_count, uint64_t vec_begin,
                             uint64_t vec_count, uint32_t flags, cudaStream_t stream) {
    const Tile *bulk_tiles = reinterpret_cast<const Tile *>(tb.tiles) + bulk_begin;
    const Tile *vec_tiles = reinterpret_cast<const Tile *>(tb.tiles) + tb.n_bulk + vec_begin;
    int32_t rc;
    if (flags & MXB_SCATTER_VECTOR) {
        rc = launch_vec(ctx, dv, tb.descs, bulk_tiles, bulk_count, stream);
        if (rc != MXB_OK) return rc;
        return launch_vec(ctx, dv, tb.descs, vec_tiles, vec_count, stream);
    }
    // Two engines, two kernels.  One after the other they add their times; a table with much
    // work for both (a reshard: local copies on the bulk engine, peer stores on the vector
    // engine) runs them side by side instead: the bulk kernel first (one warp and most of the
    // shared memory of every SM), the vector kernel on a second stream with three CTAs per SM,
    // which is what still fits beside it, so that HBM copies hide under the slower link.
    if (flags & (MXB_SCATTER_BULK_PART | MXB_SCATTER_VECTOR_PART)) {  // one half only (measurements)
        if (flags & MXB_SCATTER_BULK_PART)
            return launch_bulk(ctx, dv, tb.descs, bulk_tiles, bulk_count, stream);
        return launch_vec(ctx, dv, tb.descs, vec_tiles, vec_count, stream);
    }
    const bool overlap = (flags & MXB_SCATTER_OVERLAP) && stream == dv->stream &&
                         bulk_count >= (uint64_t)dv->sm_count && vec_count >= (uint64_t)dv->sm_count;
    if (!overlap) {
        rc = launch_bulk(ctx, dv, tb.descs, bulk_tiles, bulk_count, stream);
        if (rc != MXB_OK) return rc;
        return launch_vec(ctx, dv, tb.descs, vec_tiles, vec_count, stream);
    }
    if (!dv->fork_ev) {
        MXB_CUDA(cudaEventCreateWithFlags(&dv->fork_ev, cudaEventDisableTiming));
        MXB_CUDA(cudaEventCreateWithFlags(&dv->join_ev, cudaEventDisableTiming));
    }
    MXB_CUDA(cudaEventRecord(dv->fork_ev, stream));
    MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, dv->fork_ev, 0));
    rc = launch_bulk(ctx, dv, tb.descs, bulk_tiles, bulk_count, stream);
    if (rc != MXB_OK) return rc;
    rc = launch_vec(ctx, dv, tb.descs, vec_tiles, vec_count, dv->copy_stream, 3);
    if (rc != MXB_OK) return rc;
    MXB_CUDA(cudaEventRecord(dv->join_ev, dv->copy_stream));
    MXB_CUDA(cudaStreamWaitEvent(stream, dv->join_ev, 0));
    return MXB_OK;
}

int32_t launch_scatter(mxb_ctx *ctx, DeviceState *dv, const mxb_desc2d *descs, uint64_t n,
                       uint32_t flags, cudaStream_t stream) {
    uint64_t total = 0;
    const size_t bytes = scatter_table_bytes(descs, n, nullptr, &total);
    if (total == 0) return MXB_OK;
    int32_t rc = ensure_table(dv, bytes);
    if (rc != MXB_OK) return rc;
    // the pinned staging copy is reused by every call: wait for the previous upload
    MXB_CUDA(cudaStreamSynchronize(stream));
    ScatterTable tb;
    dv->table_tag = 0;  // the shared table no longer holds a digest tile list
    rc = build_scatter_table(descs, n, dv->table_host, dv->table, &tb, nullptr, nullptr, dv->device);
    if (rc != MXB_OK) return rc;
    MXB_CUDA(cudaMemcpyAsync(dv->table, dv->table_host, tb.bytes, cudaMemcpyHostToDevice, stream));
    return launch_scatter_tiles(ctx, dv, tb, 0, tb.n_bulk, 0, tb.n_vec, flags, stream);
}

}  // namespace mxb

using namespace mxb;

struct mxb_table {
    mxb_ctx *ctx = nullptr;
    DeviceState *dv = nullptr;
    void *dev_buf = nullptr;
    ScatterTable tb;
    uint64_t bytes_moved = 0;
};

extern "C" {

int32_t mxb_table_create(mxb_ctx *ctx, int32_t dev, const mxb_desc2d *descs, uint64_t n,
                         mxb_table **out) {
    if (!ctx || (!descs && n) || !out) {
        set_error("mxb_table_create: bad arguments");
        return MXB_ERR_ARG;
    }
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    int32_t rc = validate_descs(ctx, descs, n);
    if (rc != MXB_OK) return rc;
    DeviceGuard g(dev);
    mxb_table *t = new mxb_table();
    t->ctx = ctx;
    t->dv = d;
    const size_t bytes = scatter_table_bytes(descs, n, nullptr, nullptr);
    for (uint64_t i = 0; i < n; ++i) t->bytes_moved += descs[i].rows * descs[i].row_bytes;
    if (bytes) {
        std::vector<char> host(bytes);
        if (cudaMalloc(&t->dev_buf, bytes) != cudaSuccess) {
            set_error("cudaMalloc(table) failed");
            cudaGetLastError();
            delete t;
            return MXB_ERR_NOMEM;
        }
        rc = build_scatter_table(descs, n, host.data(), t->dev_buf, &t->tb, nullptr, nullptr, d->device);
        if (rc == MXB_OK &&
            cudaMemcpy(t->dev_buf, host.data(), t->tb.bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
            set_error("table upload failed");
            cudaGetLastError();
            rc = MXB_ERR_CUDA;
        }
        if (rc != MXB_OK) {
            cudaFree(t->dev_buf);
            delete t;
            return rc;
        }
    }
    *out = t;
    return MXB_OK;
}

int32_t mxb_table_launch(mxb_table *t, uint32_t flags) {
    if (!t) return MXB_ERR_ARG;
    DeviceGuard g(t->dv->device);
    return launch_scatter_tiles(t->ctx, t->dv, t->tb, 0, t->tb.n_bulk, 0, t->tb.n_vec, flags,
                                t->dv->stream);
}

uint64_t mxb_table_bytes(mxb_table *t) { return t ? t->bytes_moved : 0; }

int32_t mxb_table_engine(mxb_table *t, uint32_t flags) {
    if (!t) return MXB_ERR_ARG;
    if ((flags & MXB_SCATTER_VECTOR) || t->tb.n_bulk == 0) return 0;
    return t->tb.n_vec == 0 ? 1 : 2;
}

int32_t mxb_table_destroy(mxb_table *t) {
    if (!t) return MXB_OK;
    DeviceGuard g(t->dv->device);
    cudaStreamSynchronize(t->dv->stream);
    if (t->dev_buf) cudaFree(t->dev_buf);
    delete t;
    return MXB_OK;
}

int32_t mxb_copy_probe(mxb_ctx *ctx, int32_t dev, uint64_t src, uint64_t dst, uint64_t nbytes,
                       int32_t reps, float *ms_per_rep) {
    if (!ctx || !src || !dst || !ms_per_rep || reps < 1 || nbytes < 16 || ((src | dst | nbytes) & 15u)) {
        set_error("mxb_copy_probe: addresses and size must be multiples of 16 bytes");
        return MXB_ERR_ARG;
    }
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    DeviceGuard g(dev);
    std::lock_guard<std::mutex> lk(*d->mu);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    MXB_CUDA(cudaEventCreate(&e0));
    MXB_CUDA(cudaEventCreate(&e1));
    const uint64_t n16 = nbytes / 16;
    const unsigned grid = (unsigned)d->sm_count * 4;
    // MXB_PROBE_WIDTH=32: 256-bit loads and stores (addresses and size multiples of 32 bytes)
    const char *width = getenv("MXB_PROBE_WIDTH");
    const bool wide = width && !strcmp(width, "32") && !((src | dst | nbytes) & 31u);
    auto launch = [&]() {
        if (wide)
            copy_probe_kernel_32<<<grid, 512, 0, d->stream>>>(reinterpret_cast<const uint4 *>(src),
                                                              reinterpret_cast<uint4 *>(dst), n16 / 2);
        else
            copy_probe_kernel<<<grid, 512, 0, d->stream>>>(reinterpret_cast<const uint4 *>(src),
                                                           reinterpret_cast<uint4 *>(dst), n16);
    };
    launch();  // warm
    cudaEventRecord(e0, d->stream);
    for (int32_t r = 0; r < reps; ++r) launch();
    cudaEventRecord(e1, d->stream);
    cudaError_t e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) {
        set_error("mxb_copy_probe: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return MXB_ERR_CUDA;
    }
    ctx->launches.fetch_add((uint64_t)reps + 1);
    *ms_per_rep = ms / reps;
    return MXB_OK;
}

int32_t mxb_scatter(mxb_ctx *ctx, int32_t dev, const mxb_desc2d *descs, uint64_t n,
                    uint32_t flags) {
    if (!ctx || (!descs && n)) {
        set_error("mxb_scatter: bad arguments");
        return MXB_ERR_ARG;
    }
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    int32_t rc = validate_descs(ctx, descs, n);
    if (rc != MXB_OK) return rc;
    DeviceGuard g(dev);
    std::lock_guard<std::mutex> lk(*d->mu);
    rc = launch_scatter(ctx, d, descs, n, flags, d->stream);
    if (rc != MXB_OK) return rc;
    if (flags & MXB_SCATTER_NO_SYNC) return MXB_OK;
    return check_status(d);
}

int32_t mxb_read_runs(mxb_ctx *ctx, int32_t dev, const mxb_run *runs, uint64_t n) {
    if (!ctx || (!runs && n)) {
        set_error("mxb_read_runs: bad arguments");
        return MXB_ERR_ARG;
    }
    std::vector<mxb_desc2d> descs(n ? n : 1);
    int64_t m = mxb_coalesce_runs(runs, n, descs.data(), descs.size());
    if (m < 0) return MXB_ERR_ARG;
    return mxb_scatter(ctx, dev, descs.data(), (uint64_t)m, MXB_SCATTER_DEFAULT);
}

}  // extern "C"
