// Kernel 4: integrity digests (sm_100a), one pass over the bytes.
//
// A persistent launch walks 64 KiB tiles of a batch of byte ranges.  One warp
// owns one 4 KiB row: lane L loads the 16 bytes at row + step*512 + L*16 for
// step 0..7 (eight independent 16-byte loads in flight per lane) and feeds up
// to three reductions from the same registers:
//   SAFE32  - sum of byte * ((index*2654435761 + 1) mod 2^32), mod 2^32, via
//             two dp4a per word (byte sum and 0,1,2,3-weighted byte sum);
//   ROWS    - signed int32 row sums widened to 64 bit, folded into
//             sum(row) and sum(row * (k+1)) mod 2^64, plus the word tail and
//             ragged-byte terms;
//   BLOCK64 - a 64-bit hash per 4 KiB block: per lane two 32-bit accumulators take
//             xxHash32 rounds over its 32 words, the pair is avalanched (64 bit) with
//             the block index, lanes summed.
// All three are sums in a wrap-around ring, so partial results are merged with
// atomics in any order and the answer is exact.
#include <cstdlib>

#include "bulk.cuh"
#include "common.cuh"

namespace mxb {

struct DigestAcc {  // device accumulator, one per span; same layout as mxb_digest_out
    unsigned long long nbytes, row_sum, row_sum_w, tail_sum, tail_sum_w, ragged_sum, block_hash;
    uint32_t safe_checksum, reserved;
};
static_assert(sizeof(DigestAcc) == sizeof(mxb_digest_out), "accumulator mirrors the ABI record");

struct DTile {
    uint32_t span;
    uint32_t local;  // 64 KiB tile inside the span
};

constexpr uint64_t kP1 = 0x9E3779B185EBCA87ull;
constexpr uint64_t kP2 = 0xC2B2AE3D27D4EB4Full;
constexpr uint64_t kP3 = 0x165667B19E3779F9ull;
constexpr uint64_t kP4 = 0x85EBCA77C2B2AE63ull;
constexpr uint64_t kP5 = 0x27D4EB2F165667C5ull;
constexpr uint32_t kKnuth = 2654435761u;
constexpr uint32_t kQ1 = 0x9E3779B1u, kQ2 = 0x85EBCA77u, kQ3 = 0xC2B2AE3Du, kQ4 = 0x27D4EB2Fu,
                   kQ5 = 0x165667B1u;

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) { return __funnelshift_l(x, x, r); }
__device__ __forceinline__ uint64_t avalanche(uint64_t h) {
    h ^= h >> 33;
    h *= kP2;
    h ^= h >> 29;
    h *= kP3;
    h ^= h >> 32;
    return h;
}

// Streaming 16-byte load: read-only path, no L1 allocation, 256-byte L2 sectors
// fetched together (every byte of the span is read exactly once, in order).
__device__ __forceinline__ uint4 ld_stream16(const uint4 *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// 16 bytes at p + off, zero beyond n; any alignment.
__device__ __forceinline__ uint4 load16(const unsigned char *p, uint64_t off, uint64_t n,
                                        bool aligned16) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (off >= n) return v;
    const unsigned char *q = p + off;
    if (off + 16 <= n) {
        if (aligned16) return ld_stream16(reinterpret_cast<const uint4 *>(q));
        const uint64_t a = (uint64_t)(uintptr_t)q;
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~3ull);
        const uint32_t sh = (uint32_t)(a & 3ull) * 8u;
        uint32_t w0 = __ldcs(w), w1 = __ldcs(w + 1), w2 = __ldcs(w + 2), w3 = __ldcs(w + 3);
        if (sh == 0) return make_uint4(w0, w1, w2, w3);
        // the fifth word shares its aligned 4 bytes with byte off+15, which is valid
        uint32_t w4 = __ldcs(w + 4);
        v.x = __funnelshift_r(w0, w1, sh);
        v.y = __funnelshift_r(w1, w2, sh);
        v.z = __funnelshift_r(w2, w3, sh);
        v.w = __funnelshift_r(w3, w4, sh);
        return v;
    }
    uint32_t w[4] = {0, 0, 0, 0};
    const uint32_t left = (uint32_t)(n - off);
    for (uint32_t i = 0; i < left; ++i) w[i >> 2] |= (uint32_t)q[i] << (8 * (i & 3));
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ uint64_t warp_sum_u64(uint64_t v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, (unsigned long long)v, o);
    return v;
}
__device__ __forceinline__ uint64_t warp_xor_u64(uint64_t v) {
    for (int o = 16; o > 0; o >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int kDigestThreads = 512;
constexpr uint64_t kRowBytes = 4096;
constexpr uint64_t kDigestTile = 64 * 1024;

// Per-LANE partial sums.  Every digest term is a sum that separates over lanes
// (sum_k (k+1) * sum_lanes p = sum_lanes sum_k (k+1) * p), so lanes accumulate on
// their own and the warp reduces once per span, not once per row.
struct WarpAcc {
    uint64_t row_sum = 0, row_sum_w = 0, tail_sum = 0, tail_sum_w = 0, ragged = 0, block = 0;
    uint32_t safe = 0;
    uint32_t span = 0xffffffffu;
};

__device__ __forceinline__ void flush(WarpAcc &a, DigestAcc *acc, uint32_t lane) {
    if (a.span != 0xffffffffu) {
        a.row_sum = warp_sum_u64(a.row_sum);
        a.row_sum_w = warp_sum_u64(a.row_sum_w);
        a.tail_sum = warp_sum_u64(a.tail_sum);
        a.tail_sum_w = warp_sum_u64(a.tail_sum_w);
        a.ragged = warp_sum_u64(a.ragged);
        a.block = warp_sum_u64(a.block);
        a.safe = warp_sum_u32(a.safe);
    }
    if (a.span != 0xffffffffu && lane == 0) {
        DigestAcc *o = acc + a.span;
        if (a.row_sum) atomicAdd(&o->row_sum, (unsigned long long)a.row_sum);
        if (a.row_sum_w) atomicAdd(&o->row_sum_w, (unsigned long long)a.row_sum_w);
        if (a.tail_sum) atomicAdd(&o->tail_sum, (unsigned long long)a.tail_sum);
        if (a.tail_sum_w) atomicAdd(&o->tail_sum_w, (unsigned long long)a.tail_sum_w);
        if (a.ragged) atomicAdd(&o->ragged_sum, (unsigned long long)a.ragged);
        if (a.block) atomicAdd(&o->block_hash, (unsigned long long)a.block);
        if (a.safe) atomicAdd(&o->safe_checksum, a.safe);
    }
    a.row_sum = a.row_sum_w = a.tail_sum = a.tail_sum_w = a.ragged = a.block = 0;
    a.safe = 0;
}

// What one warp needs to know about the row it is digesting.
struct RowMeta {
    uint64_t n = 0;        // span length
    uint64_t row = 0;      // 4 KiB row index inside the span
    uint32_t span = 0xffffffffu;
    bool valid = false;    // the row holds at least one byte
};

// 16 bytes at q, all of them inside the span; any alignment.
__device__ __forceinline__ uint4 load16_inside(const unsigned char *q, bool aligned16) {
    if (aligned16) return ld_stream16(reinterpret_cast<const uint4 *>(q));
    const uint64_t a = (uint64_t)(uintptr_t)q;
    const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~3ull);
    const uint32_t sh = (uint32_t)(a & 3ull) * 8u;
    uint32_t w0 = __ldcs(w), w1 = __ldcs(w + 1), w2 = __ldcs(w + 2), w3 = __ldcs(w + 3);
    if (sh == 0) return make_uint4(w0, w1, w2, w3);
    // the fifth word shares its aligned 4 bytes with byte 15, which is valid
    uint32_t w4 = __ldcs(w + 4);
    return make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh),
                      __funnelshift_r(w2, w3, sh), __funnelshift_r(w3, w4, sh));
}

// Issue this lane's eight 16-byte loads of the row that `tile` assigns to `warp`.
// FULL: the tile is a whole 64 KiB inside its span, so no load needs a bound check.
template <bool FULL>
__device__ __forceinline__ void load_row(const DTile tile, const mxb_span sp, uint32_t warp,
                                         uint32_t lane, RowMeta &m, uint4 (&v)[8]) {
    m.span = tile.span;
    m.n = sp.nbytes;
    m.row = (uint64_t)tile.local * (kDigestTile / kRowBytes) + warp;
    const uint64_t row_off = m.row * kRowBytes;
    const unsigned char *p = reinterpret_cast<const unsigned char *>(sp.ptr);
    const bool aligned16 = ((sp.ptr & 15ull) == 0);
    if (FULL) {
        m.valid = true;
        const unsigned char *q = p + row_off + lane * 16;
#pragma unroll
        for (int s = 0; s < 8; ++s) v[s] = load16_inside(q + s * 512, aligned16);
        return;
    }
    m.valid = row_off < m.n;
    if (!m.valid) return;
#pragma unroll
    for (int s = 0; s < 8; ++s) v[s] = load16(p, row_off + s * 512 + lane * 16, m.n, aligned16);
}

// The partial last row of a span: whole words are the "tail" terms, the bytes
// after the last whole word the "ragged" term.  Only the kernels instantiated
// with TAIL = true carry this code; full tiles never need it.
__device__ __forceinline__ void digest_tail_row(const RowMeta &m, const uint4 (&v)[8], uint32_t lane,
                                             WarpAcc &a) {
    const uint64_t row_off = m.row * kRowBytes;
    const uint64_t body = m.n - (m.n % 4);
    uint64_t ts = 0, tw = 0, rg = 0;
    for (int s = 0; s < 8; ++s) {
        const uint64_t off = row_off + s * 512 + lane * 16;
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
        for (int q = 0; q < 4; ++q) {
            const uint64_t wo = off + 4 * q;
            if (wo + 4 <= body) {
                const uint64_t val = (uint64_t)(int64_t)(int32_t)w[q];
                ts += val;
                tw += val * ((wo - row_off) / 4 + 1);
            } else if (wo < m.n) {
                rg += __dp4a(w[q], 0x01010101u, 0u);  // zero-filled above n
            }
        }
    }
    a.tail_sum += ts;
    a.tail_sum_w += tw;
    a.ragged += rg;
}

template <uint32_t MODES, bool TAIL>
__device__ __forceinline__ void digest_row(const RowMeta &m, const uint4 (&v)[8], uint32_t lane,
                                           WarpAcc &a, unsigned long long *__restrict__ block_out) {
    const uint64_t row_off = m.row * kRowBytes;
    if (MODES & MXB_DIGEST_SAFE32) {
        // weight of byte k of word m of step s of this lane:
        //   ((row_off + lane*16) * K + 1)  +  (512*s) * K  +  (4*m + k) * K      (mod 2^32)
        // so three dp4a chains over the 32 words are enough: A = sum of bytes,
        // B = sum of bytes * s, X = sum of bytes * (4*m + k).  Bytes past the end
        // of the span were loaded as zero and add nothing.
        uint32_t A = 0, B = 0, X = 0;
        // steps are walked from the last to the first so that A, after step s, is the
        // byte sum of steps s..7; adding it once per step s >= 1 gives sum(s * A_s)
        // without a third dp4a per word
#pragma unroll
        for (int s = 7; s >= 0; --s) {
            const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                A = __dp4a(w[q], 0x01010101u, A);
                X = __dp4a(w[q], 0x03020100u + 0x04040404u * (uint32_t)q, X);
            }
            if (s) B += A;
        }
        const uint32_t base = (uint32_t)(row_off + lane * 16) * kKnuth + 1u;
        a.safe += base * A + (512u * kKnuth) * B + kKnuth * X;
    }
    if (MODES & MXB_DIGEST_ROWS) {
        // rows made only of whole words; every row of a full tile is one
        if (!TAIL || m.row < (m.n / 4) / 1024) {
            // (a widening multiply-add per word, 16-bit halves through dp2a and unsigned sums
            // with a count of negatives all measured the same as this plain form)
            int64_t s64 = 0;
#pragma unroll
            for (int s = 0; s < 8; ++s)
                s64 += (int64_t)(int32_t)v[s].x + (int64_t)(int32_t)v[s].y +
                       (int64_t)(int32_t)v[s].z + (int64_t)(int32_t)v[s].w;
            a.row_sum += (uint64_t)s64;
            a.row_sum_w += (uint64_t)s64 * (m.row + 1);
        } else if (TAIL) {
            digest_tail_row(m, v, lane, a);
        }
    }
    if (MODES & MXB_DIGEST_BLOCK64) {
        // two 32-bit accumulators per lane (xxHash32 rounds: one multiply-add, one funnel
        // shift, one multiply per word), even words into the first, odd words into the
        // second; together they are the lane's 64-bit state
        uint32_t a0 = kQ5 + lane * kQ4, a1 = kQ3 ^ (lane * kQ1);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            a0 = rotl32(a0 + v[s].x * kQ2, 13) * kQ1;
            a1 = rotl32(a1 + v[s].y * kQ2, 13) * kQ1;
            a0 = rotl32(a0 + v[s].z * kQ2, 13) * kQ1;
            a1 = rotl32(a1 + v[s].w * kQ2, 13) * kQ1;
        }
        const uint64_t h = ((uint64_t)a0 << 32) | (uint64_t)a1;
        // the lane's share of block `row`; the block hash is the sum of its 32 lane shares
        const uint64_t share = avalanche(h + (m.row + 1) * kP1);
        if (block_out) {
            const uint64_t hb = warp_sum_u64(share);
            if (lane == 0) block_out[m.row] = hb;
        }
        a.block += share;
    }
}

// Vector engine: any alignment; one row per warp per tile.  The tile record and
// span of the NEXT tile are fetched while the current row's loads are in flight,
// so a warp never sits through two dependent table reads before it can issue
// data loads.
//
// Registers: 512 threads x 2 CTAs per SM leave 64 per thread, 32 of which hold the
// row in flight.  The full-tile kernels therefore keep their per-lane partial sums
// in shared memory (each thread owns one slot, no synchronisation), where the
// compiler would otherwise spill them to local memory inside the loop.
struct LaneSums {
    unsigned long long row_sum[kDigestThreads], row_sum_w[kDigestThreads], block[kDigestThreads];
    uint32_t safe[kDigestThreads];
};

template <uint32_t MODES, bool TAIL>
__global__ void __launch_bounds__(kDigestThreads, 2)
digest_kernel(const mxb_span *__restrict__ spans, const DTile *__restrict__ tiles,
              uint64_t total_tiles, DigestAcc *__restrict__ acc,
              unsigned long long *__restrict__ block_out) {
    __shared__ LaneSums sums;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    WarpAcc a;
    RowMeta cur;
    uint4 vc[8];
    const uint32_t ntiles = (uint32_t)total_tiles;  // the host refuses more than 2^32 tiles
    uint32_t t = blockIdx.x;
    if (t >= ntiles) return;
    if (!TAIL) {
        sums.row_sum[tid] = sums.row_sum_w[tid] = sums.block[tid] = 0;
        sums.safe[tid] = 0;
    }
    // the sums of the span this warp is in, out of shared memory and into `a`
    auto collect = [&]() {
        if (!TAIL) {
            a.row_sum = sums.row_sum[tid];
            a.row_sum_w = sums.row_sum_w[tid];
            a.block = sums.block[tid];
            a.safe = sums.safe[tid];
            sums.row_sum[tid] = sums.row_sum_w[tid] = sums.block[tid] = 0;
            sums.safe[tid] = 0;
        }
    };
    DTile tile = tiles[t];
    mxb_span sp;
    sp.ptr = spans[tile.span].ptr;
    sp.nbytes = TAIL ? spans[tile.span].nbytes : 0;  // full tiles never look at the length
    for (;;) {
        load_row<!TAIL>(tile, sp, warp, lane, cur, vc);
        const uint32_t tn = t + gridDim.x;
        const bool more = tn < ntiles;
        DTile ntile = tile;
        mxb_span nsp = sp;
        if (more) {
            ntile = tiles[tn];
            nsp.ptr = spans[ntile.span].ptr;
            if (TAIL) nsp.nbytes = spans[ntile.span].nbytes;
        }
        if (cur.span != a.span) {
            collect();
            flush(a, acc, lane);
            a.span = cur.span;
        }
        if (TAIL) {
            if (cur.valid) digest_row<MODES, TAIL>(cur, vc, lane, a, block_out);
        } else {
            WarpAcc r;  // this row's terms only: short-lived registers
            digest_row<MODES, TAIL>(cur, vc, lane, r, block_out);
            if (MODES & MXB_DIGEST_ROWS) {
                sums.row_sum[tid] += r.row_sum;
                sums.row_sum_w[tid] += r.row_sum_w;
            }
            if (MODES & MXB_DIGEST_BLOCK64) sums.block[tid] += r.block;
            if (MODES & MXB_DIGEST_SAFE32) sums.safe[tid] += r.safe;
        }
        if (!more) break;
        tile = ntile;
        sp = nsp;
        t = tn;
    }
    collect();
    flush(a, acc, lane);
}

// Bulk engine: whole 64 KiB tiles of 16-byte-aligned spans.  One elected thread
// streams tiles into a 3-stage shared-memory ring with cp.async.bulk (192 KiB
// in flight per SM at no register cost); the 16 warps each reduce one 4 KiB row
// of the landed tile out of shared memory.  Waits are bounded.
constexpr int kDigestStages = 3;
constexpr uint32_t kDigestSpin = 1u << 22;

template <uint32_t MODES>
__global__ void __launch_bounds__(kDigestThreads, 1)
digest_bulk_kernel(const mxb_span *__restrict__ spans, const DTile *__restrict__ tiles,
                   uint64_t total_tiles, DigestAcc *__restrict__ acc,
                   unsigned long long *__restrict__ block_out, uint32_t *status) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full[kDigestStages];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kDigestStages; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint64_t first = blockIdx.x;
    if (first >= total_tiles) return;
    const uint64_t mine = (total_tiles - first + gridDim.x - 1) / gridDim.x;
    auto issue = [&](uint64_t k) {  // thread 0 only
        const DTile tile = tiles[first + k * gridDim.x];
        const unsigned char *src = reinterpret_cast<const unsigned char *>(spans[tile.span].ptr) +
                                   (uint64_t)tile.local * kDigestTile;
        const int s = (int)(k % kDigestStages);
        mbar_expect_tx(&full[s], (uint32_t)kDigestTile);
        bulk_g2s(smem + (size_t)s * kDigestTile, src, (uint32_t)kDigestTile, &full[s]);
    };
    if (tid == 0) {
        issue(0);
        if (mine > 1) issue(1);
    }
    WarpAcc a;
    uint64_t issued = mine > 1 ? 2 : 1;
    uint64_t k = 0;
    bool failed = false;
    for (; k < mine; ++k) {
        const int s = (int)(k % kDigestStages);
        // stage (k+2)%3 held tile k-1, which every warp finished before the barrier below
        if (tid == 0 && k + 2 < mine) issue(k + 2);
        if (k + 2 < mine) issued = k + 3;
        const DTile tile = tiles[first + k * gridDim.x];
        RowMeta m;
        m.span = tile.span;
        m.n = spans[tile.span].nbytes;
        m.row = (uint64_t)tile.local * (kDigestTile / kRowBytes) + warp;
        m.valid = true;
        const uint32_t parity = (uint32_t)((k / kDigestStages) & 1);
        bool ok = false;
        for (uint32_t spin = 0; spin < kDigestSpin && !ok; ++spin) ok = mbar_try_wait(&full[s], parity);
        if (__syncthreads_or(!ok)) {
            failed = true;
            break;
        }
        const uint4 *row = reinterpret_cast<const uint4 *>(smem + (size_t)s * kDigestTile +
                                                           (size_t)warp * kRowBytes);
        uint4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = row[q * 32 + lane];
        if (m.span != a.span) {
            flush(a, acc, lane);
            a.span = m.span;
        }
        digest_row<MODES, false>(m, v, lane, a, block_out);
        __syncthreads();  // the stage may be refilled
    }
    flush(a, acc, lane);
    if (failed) {
        if (tid == 0) atomicExch(status, DEV_TIMEOUT);
        // bounded wait for the copies still in flight before shared memory is released
        for (uint64_t j = k; j < issued; ++j) {
            const int s = (int)(j % kDigestStages);
            const uint32_t parity = (uint32_t)((j / kDigestStages) & 1);
            for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                if (mbar_try_wait(&full[s], parity)) break;
        }
    }
}

typedef void (*digest_fn)(const mxb_span *, const DTile *, uint64_t, DigestAcc *,
                          unsigned long long *);
typedef void (*digest_bulk_fn)(const mxb_span *, const DTile *, uint64_t, DigestAcc *,
                               unsigned long long *, uint32_t *);
static digest_bulk_fn digest_bulk_variant(uint32_t modes) {
    switch (modes) {
        case 1: return digest_bulk_kernel<1>;
        case 2: return digest_bulk_kernel<2>;
        case 3: return digest_bulk_kernel<3>;
        case 4: return digest_bulk_kernel<4>;
        case 5: return digest_bulk_kernel<5>;
        case 6: return digest_bulk_kernel<6>;
        default: return digest_bulk_kernel<7>;
    }
}
template <bool TAIL>
static digest_fn digest_variant(uint32_t modes) {
    switch (modes) {
        case 1: return digest_kernel<1, TAIL>;
        case 2: return digest_kernel<2, TAIL>;
        case 3: return digest_kernel<3, TAIL>;
        case 4: return digest_kernel<4, TAIL>;
        case 5: return digest_kernel<5, TAIL>;
        case 6: return digest_kernel<6, TAIL>;
        default: return digest_kernel<7, TAIL>;
    }
}

}  // namespace mxb

using namespace mxb;

extern "C" {

static int32_t run_digest(mxb_ctx *ctx, int32_t dev, const mxb_span *spans, uint64_t n,
                          uint32_t modes, mxb_digest_out *out, uint64_t block_out) {
    if (!ctx || (!spans && n) || (!out && n) || (modes & ~7u) || modes == 0) {
        set_error("mxb_digest: bad arguments");
        return MXB_ERR_ARG;
    }
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    if (n == 0) return MXB_OK;
    if (n > 0xffffffffull) return MXB_ERR_ARG;
    uint64_t total = 0;
    for (uint64_t i = 0; i < n; ++i) {
        if (spans[i].nbytes && !spans[i].ptr) {
            set_error("span %llu has a null address", (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        total += (spans[i].nbytes + kDigestTile - 1) / kDigestTile;
    }
    if (total > 0xffffffffull) {
        set_error("mxb_digest: more than 2^32 tiles (256 TiB) in one call");
        return MXB_ERR_ARG;
    }
    DeviceGuard g(dev);
    std::lock_guard<std::mutex> lk(*d->mu);
    const size_t span_bytes = (n * sizeof(mxb_span) + 255) & ~size_t(255);
    const size_t tile_bytes = (total * sizeof(DTile) + 255) & ~size_t(255);
    int32_t rc = ensure_table(d, span_bytes + tile_bytes);
    if (rc != MXB_OK) return rc;
    rc = ensure_digest(d, n * sizeof(DigestAcc));
    if (rc != MXB_OK) return rc;
    mxb_span *hs = reinterpret_cast<mxb_span *>(d->table_host);
    DTile *ht = reinterpret_cast<DTile *>(reinterpret_cast<char *>(d->table_host) + span_bytes);
    // The same list of ranges is digested over and over (every refit cycle verifies the
    // same shards): the tile list on the device is kept and reused while nothing else
    // has used the table and the ranges are the same, which saves building and
    // uploading a few hundred thousand tile records per call.
    uint64_t tag = 0xcbf29ce484222325ull ^ n;
    for (uint64_t i = 0; i < n; ++i) {
        tag = (tag ^ spans[i].ptr) * 0x100000001b3ull;
        tag = (tag ^ spans[i].nbytes) * 0x100000001b3ull;
    }
    if (tag == 0) tag = 1;
    const bool reuse = d->table_tag == tag && memcmp(hs, spans, n * sizeof(mxb_span)) == 0;
    // Full 64 KiB tiles are listed first, ragged last tiles after them.  Full tiles
    // of 16-byte-aligned spans may use the bulk engine (shared-memory staging); the
    // ragged ones always use the vector engine with tail handling.
    // The vector engine measured faster in every mode on B200 (two resident CTAs
    // hide the arithmetic better than one CTA with a shared-memory ring), so the
    // bulk engine runs only on request: MXB_DIGEST_ENGINE=bulk.
    const char *eng = getenv("MXB_DIGEST_ENGINE");
    bool want_bulk = false;
    if (eng && !strcmp(eng, "bulk")) want_bulk = true;
    if (eng && !strcmp(eng, "vector")) want_bulk = false;
    bool all_aligned = true;
    uint64_t n_full = 0;
    for (uint64_t i = 0; i < n; ++i) {
        n_full += spans[i].nbytes / kDigestTile;
        if (spans[i].nbytes >= kDigestTile && (spans[i].ptr & 15ull)) all_aligned = false;
    }
    const bool use_bulk = want_bulk && all_aligned;
    if (!reuse) {
        MXB_CUDA(cudaStreamSynchronize(d->stream));
        d->table_tag = 0;
        uint64_t fi = 0, gi = n_full;
        for (uint64_t i = 0; i < n; ++i) {
            hs[i] = spans[i];
            uint64_t t = (spans[i].nbytes + kDigestTile - 1) / kDigestTile;
            if (t > 0xffffffffull) return MXB_ERR_ARG;
            const uint64_t fullt = spans[i].nbytes / kDigestTile;
            for (uint64_t k = 0; k < t; ++k) {
                if (k < fullt) ht[fi++] = DTile{(uint32_t)i, (uint32_t)k};
                else ht[gi++] = DTile{(uint32_t)i, (uint32_t)k};
            }
        }
        MXB_CUDA(cudaMemcpyAsync(d->table, d->table_host, span_bytes + tile_bytes,
                                 cudaMemcpyHostToDevice, d->stream));
        d->table_tag = tag;
    }
    MXB_CUDA(cudaMemsetAsync(d->digest, 0, n * sizeof(DigestAcc), d->stream));
    const mxb_span *dspans = reinterpret_cast<const mxb_span *>(d->table);
    const DTile *dtiles = reinterpret_cast<const DTile *>(reinterpret_cast<char *>(d->table) + span_bytes);
    DigestAcc *dacc = reinterpret_cast<DigestAcc *>(d->digest);
    unsigned long long *dblk = reinterpret_cast<unsigned long long *>(block_out);
    if (n_full && use_bulk) {
        const size_t smem = (size_t)kDigestStages * kDigestTile;
        digest_bulk_fn fn = digest_bulk_variant(modes);
        // idempotent and cheap: set on every launch rather than keep a flag several threads share
        MXB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        uint64_t grid = (uint64_t)d->sm_count;
        if (grid > n_full) grid = n_full;
        fn<<<(unsigned)grid, kDigestThreads, smem, d->stream>>>(dspans, dtiles, n_full, dacc, dblk,
                                                                 d->status);
        MXB_CUDA(cudaGetLastError());
        ctx->launches.fetch_add(1);
    } else if (n_full) {
        uint64_t grid = (uint64_t)d->sm_count * 2;
        if (grid > n_full) grid = n_full;
        digest_variant<false>(modes)<<<(unsigned)grid, kDigestThreads, 0, d->stream>>>(
            dspans, dtiles, n_full, dacc, dblk);
        MXB_CUDA(cudaGetLastError());
        ctx->launches.fetch_add(1);
    }
    if (total > n_full) {
        uint64_t grid = (uint64_t)d->sm_count * 2;
        if (grid > total - n_full) grid = total - n_full;
        digest_variant<true>(modes)<<<(unsigned)grid, kDigestThreads, 0, d->stream>>>(
            dspans, dtiles + n_full, total - n_full, dacc, dblk);
        MXB_CUDA(cudaGetLastError());
        ctx->launches.fetch_add(1);
    }
    MXB_CUDA(cudaMemcpyAsync(d->digest_host, d->digest, n * sizeof(DigestAcc),
                             cudaMemcpyDeviceToHost, d->stream));
    rc = check_status(d);
    if (rc != MXB_OK) return rc;
    const DigestAcc *res = reinterpret_cast<const DigestAcc *>(d->digest_host);
    for (uint64_t i = 0; i < n; ++i) {
        memcpy(&out[i], &res[i], sizeof(mxb_digest_out));
        out[i].nbytes = spans[i].nbytes;
        if (modes & MXB_DIGEST_BLOCK64) {
            // the length term keeps zero padding from aliasing shorter inputs
            uint64_t h = spans[i].nbytes * 0x27D4EB2F165667C5ull;
            h ^= h >> 33;
            h *= 0xC2B2AE3D27D4EB4Full;
            h ^= h >> 29;
            h *= 0x165667B19E3779F9ull;
            h ^= h >> 32;
            out[i].block_hash += h;
        }
    }
    return MXB_OK;
}

int32_t mxb_digest(mxb_ctx *ctx, int32_t dev, const mxb_span *spans, uint64_t n, uint32_t modes,
                   mxb_digest_out *out) {
    return run_digest(ctx, dev, spans, n, modes, out, 0);
}

int32_t mxb_block_hashes(mxb_ctx *ctx, int32_t dev, uint64_t ptr, uint64_t nbytes,
                         uint64_t out_blocks) {
    if (!ptr || !out_blocks) return MXB_ERR_ARG;
    mxb_span sp{ptr, nbytes};
    mxb_digest_out o;
    return run_digest(ctx, dev, &sp, 1, MXB_DIGEST_BLOCK64, &o, out_blocks);
}

}  // extern "C"

/* ---- digests for callers that must not allocate device memory ---------------------------- */

namespace {

constexpr uint64_t kNoAllocMaxSpans = 256;
constexpr uint64_t kNoAllocMaxTiles = 16384;  // 1 GiB of 64 KiB tiles

struct NoAllocScratch {
    mxb_span spans[kNoAllocMaxSpans];
    DTile tiles[kNoAllocMaxTiles];
    DigestAcc acc[kNoAllocMaxSpans];
};

// The whole scratch of the allocation-free entry point: 4 KiB of spans, 128 KiB
// of tiles and 16 KiB of accumulators, resident on every GPU that loads the
// library until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel as if it were an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

std::mutex g_noalloc_mu;
NoAllocScratch *g_noalloc_ptr[64] = {};  // device address of the scratch, per device

}  // namespace

extern "C" int32_t mxb_digest_noalloc(int32_t dev, const mxb_span *spans, uint64_t n,
                                      uint32_t modes, mxb_digest_out *out, void *stream) {
    if ((!spans && n) || (!out && n) || (modes & ~7u) || modes == 0 || dev < 0 || dev >= 64) {
        set_error("mxb_digest_noalloc: bad arguments");
        return MXB_ERR_ARG;
    }
    if (n > kNoAllocMaxSpans) {
        set_error("mxb_digest_noalloc: %llu ranges exceed the fixed scratch (at most %llu per call)",
                  (unsigned long long)n, (unsigned long long)kNoAllocMaxSpans);
        return MXB_ERR_ARG;
    }
    uint64_t total = 0;
    for (uint64_t i = 0; i < n; ++i) {
        if (spans[i].nbytes && !spans[i].ptr) {
            set_error("span %llu has a null address", (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        total += (spans[i].nbytes + kDigestTile - 1) / kDigestTile;
    }
    if (total > kNoAllocMaxTiles) {
        set_error("mxb_digest_noalloc: %llu tiles of 64 KiB exceed the fixed scratch (at most %llu "
                  "per call, i.e. 1 GiB); split the ranges over several calls",
                  (unsigned long long)total, (unsigned long long)kNoAllocMaxTiles);
        return MXB_ERR_ARG;
    }
    if (n == 0) return MXB_OK;
    DeviceGuard g(dev);
    if (!g.ok) {
        set_error("cudaSetDevice(%d) failed", dev);
        cudaGetLastError();
        return MXB_ERR_CUDA;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // The scratch is shared by every call on this device; calls are serialised on the
    // host here, and each call finishes (stream synchronised) before it returns.
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocScratch *sc = g_noalloc_ptr[dev];
    if (!sc) {
        // set-up, once per device, with that device current
        void *p = nullptr;
        MXB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        sc = g_noalloc_ptr[dev] = reinterpret_cast<NoAllocScratch *>(p);
    }
    // host image of the table: spans, then tiles (full tiles first, ragged last tiles after)
    static thread_local mxb_span h_spans[kNoAllocMaxSpans];
    static thread_local DTile h_tiles[kNoAllocMaxTiles];
    uint64_t n_full = 0;
    for (uint64_t i = 0; i < n; ++i) n_full += spans[i].nbytes / kDigestTile;
    uint64_t fi = 0, gi = n_full;
    for (uint64_t i = 0; i < n; ++i) {
        h_spans[i] = spans[i];
        const uint64_t t = (spans[i].nbytes + kDigestTile - 1) / kDigestTile;
        const uint64_t fullt = spans[i].nbytes / kDigestTile;
        for (uint64_t k = 0; k < t; ++k) {
            if (k < fullt) h_tiles[fi++] = DTile{(uint32_t)i, (uint32_t)k};
            else h_tiles[gi++] = DTile{(uint32_t)i, (uint32_t)k};
        }
    }
    MXB_CUDA(cudaMemcpyAsync(sc->spans, h_spans, n * sizeof(mxb_span), cudaMemcpyHostToDevice, st));
    if (total)
        MXB_CUDA(cudaMemcpyAsync(sc->tiles, h_tiles, total * sizeof(DTile), cudaMemcpyHostToDevice, st));
    // the accumulators keep the previous call's sums: clear the ones this call uses
    MXB_CUDA(cudaMemsetAsync(sc->acc, 0, n * sizeof(DigestAcc), st));
    int sms = 0;
    MXB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (n_full) {
        uint64_t grid = (uint64_t)sms * 2;
        if (grid > n_full) grid = n_full;
        digest_variant<false>(modes)<<<(unsigned)grid, kDigestThreads, 0, st>>>(
            sc->spans, sc->tiles, n_full, sc->acc, nullptr);
        MXB_CUDA(cudaGetLastError());
    }
    if (total > n_full) {
        uint64_t grid = (uint64_t)sms * 2;
        if (grid > total - n_full) grid = total - n_full;
        digest_variant<true>(modes)<<<(unsigned)grid, kDigestThreads, 0, st>>>(
            sc->spans, sc->tiles + n_full, total - n_full, sc->acc, nullptr);
        MXB_CUDA(cudaGetLastError());
    }
    static thread_local DigestAcc h_acc[kNoAllocMaxSpans];
    MXB_CUDA(cudaMemcpyAsync(h_acc, sc->acc, n * sizeof(DigestAcc), cudaMemcpyDeviceToHost, st));
    MXB_CUDA(cudaStreamSynchronize(st));
    for (uint64_t i = 0; i < n; ++i) {
        memcpy(&out[i], &h_acc[i], sizeof(mxb_digest_out));
        out[i].nbytes = spans[i].nbytes;
        if (modes & MXB_DIGEST_BLOCK64) {
            uint64_t h = spans[i].nbytes * 0x27D4EB2F165667C5ull;
            h ^= h >> 33;
            h *= 0xC2B2AE3D27D4EB4Full;
            h ^= h >> 29;
            h *= 0x165667B19E3779F9ull;
            h ^= h >> 32;
            out[i].block_hash += h;
        }
    }
    return MXB_OK;
}
