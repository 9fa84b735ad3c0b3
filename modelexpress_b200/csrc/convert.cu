// Kernel 5: box convert (sm_100a).  A staged source box (contiguous, in the source's own
// dimension order) lands in a live parameter with the destination's strides, cast on the way
// when the served dtype differs.  It replaces the per-tensor `dst.copy_(src)` the reference
// leaves to torch after a pull (refit/reshard/receiver.py:964-971) and the transposed boxes
// of slice_plan.py:170-224, with one persistent launch for the whole list.
//
// Each box is canonicalised on the host (extent-1 dims dropped, dims merged where the
// destination walks them like the source does) into at most four dims.  Two tile shapes:
//   rows       the destination is unit-stride along the source's inner dim: a tile is up to
//              16384 elements of one row; 16-byte vectors when both sides are aligned.
//   transpose  some other dim is the destination's unit-stride dim: a tile is 64 x 64 elements,
//              read along the source's inner dim, turned in shared memory, written along the
//              destination's inner dim (element pairs when both sides allow 4-byte accesses).
// HBM-bound: one read of the source element and one write of the destination element, nothing
// else.  One launch per conversion present in the list.  Casts use the conversions torch's own device code uses (__float2bfloat16_rn,
// __float2half_rn, widening by bit placement), so results equal torch's bit for bit.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"

namespace mxb {

constexpr int kCvtThreads = 256;
constexpr uint32_t kRowTile = 16384;
constexpr uint32_t kTT = 64;  // transpose tile edge

struct CvtItem {
    uint64_t src, dst;
    uint32_t n[4];     // canonical extents, n[3] = the source's inner dim
    int64_t ds[4];     // destination strides (elements)
    int64_t ss[3];     // source strides of the three outer dims (elements); the inner dim's is 1
    uint64_t tile0;    // first tile of this item
    uint32_t mode;     // 0 rows, 1 transpose (64 x 64), 2 transpose, wide accesses
    uint32_t bdim;     // transpose: the dim the destination walks with stride 1
    uint32_t pair;     // pair (4-byte / 8-byte) accesses allowed on both sides
    uint32_t kind;     // conversion, see CvtKind
    uint32_t tiles_a, tiles_b;  // tiles along n[3] and along n[bdim] (rows: tiles_b = 1)
    uint64_t n_tiles;
};

enum CvtKind : uint32_t {
    kRaw1, kRaw2, kRaw4, kRaw8, kBf16ToF32, kF16ToF32, kF32ToBf16, kF32ToF16, kBf16ToF16, kF16ToBf16,
    kKinds
};

// Element tags: how a value is stored and how it passes through float.
template <typename U>
struct Raw {
    using store = U;
};
struct F32 {
    using store = uint32_t;
    __device__ static __forceinline__ float to_float(store v) { return __uint_as_float(v); }
    __device__ static __forceinline__ store from_float(float f) { return __float_as_uint(f); }
};
struct F16 {
    using store = uint16_t;
    __device__ static __forceinline__ float to_float(store v) { return __half2float(__ushort_as_half(v)); }
    __device__ static __forceinline__ store from_float(float f) { return __half_as_ushort(__float2half_rn(f)); }
};
struct BF16 {
    using store = uint16_t;
    __device__ static __forceinline__ float to_float(store v) { return __uint_as_float((uint32_t)v << 16); }
    __device__ static __forceinline__ store from_float(float f) {
        return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    }
};

template <typename S, typename D>
struct Cast {
    __device__ static __forceinline__ typename D::store run(typename S::store v) {
        return D::from_float(S::to_float(v));
    }
};
template <typename U>
struct Cast<Raw<U>, Raw<U>> {
    __device__ static __forceinline__ U run(U v) { return v; }
};

template <int N>
struct Bytes;
template <>
struct Bytes<2> { using type = uint16_t; };
template <>
struct Bytes<4> { using type = uint32_t; };
template <>
struct Bytes<8> { using type = uint2; };
template <>
struct Bytes<16> { using type = uint4; };

// V elements of S -> V elements of D through registers; addresses aligned to their vectors
template <typename S, typename D, int V>
__device__ __forceinline__ void cast_vec(const typename S::store *__restrict__ s,
                                         typename D::store *__restrict__ d) {
    using SE = typename S::store;
    using DE = typename D::store;
    using SV = typename Bytes<sizeof(SE) * V>::type;
    using DV = typename Bytes<sizeof(DE) * V>::type;
    union { SV v; SE e[V]; } in;
    union { DV v; DE e[V]; } out;
    in.v = *reinterpret_cast<const SV *>(s);
#pragma unroll
    for (int i = 0; i < V; ++i) out.e[i] = Cast<S, D>::run(in.e[i]);
    *reinterpret_cast<DV *>(d) = out.v;
}

template <typename S, typename D>
__device__ void rows_tile(const CvtItem &it, uint32_t t, unsigned char *) {
    using SE = typename S::store;
    using DE = typename D::store;
    const uint32_t ta = t % it.tiles_a;
    uint32_t row = t / it.tiles_a;   // a box's tile count fits 32 bits (checked on the host)
    const uint32_t a0 = ta * kRowTile;
    const uint32_t len = min(kRowTile, it.n[3] - a0);
    int64_t off = 0, soff = 0;
    for (int d = 2; d >= 0; --d) {
        const int64_t idx = (int64_t)(row % it.n[d]);
        off += idx * it.ds[d];
        soff += idx * it.ss[d];
        row /= it.n[d];
    }
    const SE *s = reinterpret_cast<const SE *>(it.src) + soff + a0;
    const int64_t step = it.ds[3];
    DE *dbase = reinterpret_cast<DE *>(it.dst) + off + (int64_t)a0 * step;
    uint32_t done = 0;
    if (step == 1 && (reinterpret_cast<uintptr_t>(s) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(dbase) & 15u) == 0) {
        // W elements per access: 16 bytes on the wider side
        constexpr int kWide = sizeof(SE) > sizeof(DE) ? sizeof(SE) : sizeof(DE);
        constexpr int W = 16 / kWide;
        using SV = typename Bytes<sizeof(SE) * W>::type;
        using DV = typename Bytes<sizeof(DE) * W>::type;
        const uint32_t nv = len / W;
        const SV *sv = reinterpret_cast<const SV *>(s);
        DV *dv = reinterpret_cast<DV *>(dbase);
        uint32_t i = threadIdx.x;
        for (; i + 7 * kCvtThreads < nv; i += 8 * kCvtThreads) {   // eight independent loads in flight
            SV in[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) in[k] = sv[i + k * kCvtThreads];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                union { SV v; SE e[W]; } a;
                union { DV v; DE e[W]; } b;
                a.v = in[k];
#pragma unroll
                for (int e = 0; e < W; ++e) b.e[e] = Cast<S, D>::run(a.e[e]);
                dv[i + k * kCvtThreads] = b.v;
            }
        }
        for (; i < nv; i += kCvtThreads) cast_vec<S, D, W>(s + (size_t)i * W, dbase + (size_t)i * W);
        done = nv * W;
    }
    for (uint32_t i = done + threadIdx.x; i < len; i += kCvtThreads)
        dbase[(int64_t)i * step] = Cast<S, D>::run(s[i]);
}

// Where tile t of a transposed item lies: `edge_a` x `edge_b` elements along the source's
// inner dim (a) and the destination's unit-stride dim (b).
struct TileAt {
    uint64_t src_elem;   // source element of the tile's corner
    int64_t dst_elem;    // destination element of the tile's corner
    uint64_t sstride_b;  // source elements between consecutive b
    uint32_t na, nb;     // valid extent of this tile
};

__device__ __forceinline__ TileAt tile_at(const CvtItem &it, uint32_t t, uint32_t edge_a, uint32_t edge_b) {
    const uint32_t b = it.bdim;
    const uint32_t ta = t % it.tiles_a;
    t /= it.tiles_a;
    const uint32_t tb = t % it.tiles_b;
    uint32_t rest = t / it.tiles_b;
    // the two dims that are neither the source's inner dim nor the destination's
    uint32_t idx[3] = {0, 0, 0};
    for (int d = 2; d >= 0; --d) {
        if ((uint32_t)d == b) continue;
        idx[d] = rest % it.n[d];
        rest /= it.n[d];
    }
    const uint32_t a0 = ta * edge_a, b0 = tb * edge_b;
    TileAt at;
    at.na = min(edge_a, it.n[3] - a0);
    at.nb = min(edge_b, it.n[b] - b0);
    int64_t soff = 0, doff = 0;
    for (int d = 0; d < 3; ++d) {
        const uint32_t v = (uint32_t)d == b ? b0 : idx[d];
        soff += (int64_t)v * it.ss[d];
        doff += (int64_t)v * it.ds[d];
    }
    at.sstride_b = (uint64_t)it.ss[b];
    at.src_elem = (uint64_t)soff + a0;
    at.dst_elem = doff + (int64_t)a0 * it.ds[3];
    return at;
}

// Elements a lane moves per access in the wide transposed path: 8 bytes (4 for one-byte elements)
template <typename E>
struct Group {
    static constexpr int n = sizeof(E) >= 4 ? 8 / sizeof(E) : 4;
};

// Transposed tile, wide: every lane reads Group<source> elements along the source's inner dim
// and writes Group<destination> elements along the destination's, eight rows in flight per
// warp.  The host selects it only when every such group is naturally aligned on both sides.
template <typename S, typename D>
__device__ void wide_tile(const CvtItem &it, uint32_t t, unsigned char *smem_raw) {
    using SE = typename S::store;
    using DE = typename D::store;
    constexpr int GS = Group<SE>::n, GD = Group<DE>::n;
    constexpr uint32_t TA = 32 * GS, TB = 32 * GD;
    using SG = typename Bytes<GS * sizeof(SE)>::type;
    using DG = typename Bytes<GD * sizeof(DE)>::type;
    DE(*tile)[TA + 1] = reinterpret_cast<DE(*)[TA + 1]>(smem_raw);
    const TileAt at = tile_at(it, t, TA, TB);
    const SE *s = reinterpret_cast<const SE *>(it.src) + at.src_elem;
    DE *dp = reinterpret_cast<DE *>(it.dst) + at.dst_elem;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t kWarps = kCvtThreads / 32;
    constexpr int kBatch = 8;
    const bool lane_a = GS * lane < at.na, lane_b = GD * lane < at.nb;
#pragma unroll 1
    for (uint32_t j0 = 0; j0 < at.nb; j0 += kBatch * kWarps) {
        SG in[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const uint32_t j = j0 + warp + k * kWarps;
            if (lane_a && j < at.nb) in[k] = *reinterpret_cast<const SG *>(s + (uint64_t)j * at.sstride_b + GS * lane);
        }
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const uint32_t j = j0 + warp + k * kWarps;
            if (lane_a && j < at.nb) {
                union { SG v; SE e[GS]; } a;
                a.v = in[k];
#pragma unroll
                for (int g = 0; g < GS; ++g) tile[j][GS * lane + g] = Cast<S, D>::run(a.e[g]);
            }
        }
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t i0 = 0; i0 < at.na; i0 += kBatch * kWarps) {
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const uint32_t i = i0 + warp + k * kWarps;
            if (lane_b && i < at.na) {
                union { DG v; DE e[GD]; } o;
#pragma unroll
                for (int g = 0; g < GD; ++g) o.e[g] = tile[GD * lane + g][i];
                *reinterpret_cast<DG *>(dp + (int64_t)i * it.ds[3] + GD * lane) = o.v;
            }
        }
    }
    __syncthreads();  // the tile is reused by this CTA's next tile
}

// Transposed tile for two-byte destinations, packed: shared memory holds 32-bit words of two
// elements that are neighbours along the destination's inner dim (source rows 2p and 2p+1, same
// column), so neither phase touches shared memory in two-byte units.  A warp loads a pair of
// source rows (8 bytes per lane from each), zips them into words and stores word g of every lane
// at column g*32 + lane (conflict-free); on the way out lane l fetches the words of row pairs l
// and l + 32 at one column (conflict-free with the odd pitch) and writes 4 bytes each, 128
// contiguous bytes per warp instruction.  Same tile shape and alignment rules as wide_tile.
template <typename S, typename D>
__device__ void packed_tile(const CvtItem &it, uint32_t t, unsigned char *smem_raw) {
    using SE = typename S::store;
    using DE = typename D::store;
    static_assert(sizeof(DE) == 2, "packed tiles hold two-byte destination elements");
    constexpr int GS = Group<SE>::n;
    constexpr uint32_t TA = 32 * GS, TB = 128;
    using SG = typename Bytes<GS * sizeof(SE)>::type;
    uint32_t(*words)[TA + 1] = reinterpret_cast<uint32_t(*)[TA + 1]>(smem_raw);
    const TileAt at = tile_at(it, t, TA, TB);
    const SE *s = reinterpret_cast<const SE *>(it.src) + at.src_elem;
    DE *dp = reinterpret_cast<DE *>(it.dst) + at.dst_elem;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t kWarps = kCvtThreads / 32;
    constexpr int kBatch = 4;   // row pairs in flight per warp: eight 8-byte loads per lane
    const bool lane_a = GS * lane < at.na;
    const uint32_t pairs = at.nb / 2;  // nb is a multiple of 4 here
#pragma unroll 1
    for (uint32_t p0 = 0; p0 < pairs; p0 += kBatch * kWarps) {
        SG in0[kBatch], in1[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const uint32_t p = p0 + warp + k * kWarps;
            if (lane_a && p < pairs) {
                const SE *row = s + (uint64_t)(2 * p) * at.sstride_b + GS * lane;
                in0[k] = *reinterpret_cast<const SG *>(row);
                in1[k] = *reinterpret_cast<const SG *>(row + at.sstride_b);
            }
        }
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const uint32_t p = p0 + warp + k * kWarps;
            if (lane_a && p < pairs) {
                union { SG v; SE e[GS]; } a, b;
                a.v = in0[k];
                b.v = in1[k];
#pragma unroll
                for (int g = 0; g < GS; ++g)
                    words[p][g * 32 + lane] = (uint32_t)Cast<S, D>::run(a.e[g]) |
                                              ((uint32_t)Cast<S, D>::run(b.e[g]) << 16);
            }
        }
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t i0 = 0; i0 < at.na; i0 += 8 * kWarps) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t i = i0 + warp + k * kWarps;
            if (i < at.na) {
                const uint32_t col = (i % GS) * 32 + i / GS;   // where the load phase put column i
                uint32_t *out = reinterpret_cast<uint32_t *>(dp + (int64_t)i * it.ds[3]);
                if (lane < pairs) out[lane] = words[lane][col];
                if (lane + 32 < pairs) out[lane + 32] = words[lane + 32][col];
            }
        }
    }
    __syncthreads();  // the tile is reused by this CTA's next tile
}

template <typename S, typename D>
__device__ void transpose_tile(const CvtItem &it, uint32_t t, unsigned char *smem_raw) {
    using SE = typename S::store;
    using DE = typename D::store;
    DE(*tile)[kTT + 1] = reinterpret_cast<DE(*)[kTT + 1]>(smem_raw);
    const TileAt at = tile_at(it, t, kTT, kTT);
    const uint32_t na = at.na, nb = at.nb;
    const uint64_t sstride_b = at.sstride_b;
    const SE *s = reinterpret_cast<const SE *>(it.src) + at.src_elem;
    DE *dp = reinterpret_cast<DE *>(it.dst) + at.dst_elem;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t kWarps = kCvtThreads / 32;
    if constexpr (sizeof(SE) <= 4 && sizeof(DE) <= 4) {
      if (it.pair && na == kTT && nb == kTT) {
        // a full tile: the warp's eight rows are loaded before any of them is turned
        using S2 = typename Bytes<2 * sizeof(SE)>::type;
        using D2 = typename Bytes<2 * sizeof(DE)>::type;
        constexpr int kRows = kTT / kWarps;
        S2 in[kRows];
#pragma unroll
        for (int k = 0; k < kRows; ++k)
            in[k] = *reinterpret_cast<const S2 *>(s + (uint64_t)(warp + k * kWarps) * sstride_b + 2 * lane);
#pragma unroll
        for (int k = 0; k < kRows; ++k) {
            union { S2 v; SE e[2]; } a;
            a.v = in[k];
            tile[warp + k * kWarps][2 * lane] = Cast<S, D>::run(a.e[0]);
            tile[warp + k * kWarps][2 * lane + 1] = Cast<S, D>::run(a.e[1]);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kRows; ++k) {
            const uint32_t i = warp + k * kWarps;
            union { D2 v; DE e[2]; } out;
            out.e[0] = tile[2 * lane][i];
            out.e[1] = tile[2 * lane + 1][i];
            *reinterpret_cast<D2 *>(dp + (int64_t)i * it.ds[3] + 2 * lane) = out.v;
        }
        __syncthreads();  // the tile is reused by this CTA's next tile
        return;
      }
      if (it.pair) {
        using S2 = typename Bytes<2 * sizeof(SE)>::type;
        using D2 = typename Bytes<2 * sizeof(DE)>::type;
        for (uint32_t j = warp; j < nb; j += kWarps) {
            const uint32_t i = 2 * lane;
            if (i < na) {  // na is even when pairs are allowed
                union { S2 v; SE e[2]; } in;
                in.v = *reinterpret_cast<const S2 *>(s + (uint64_t)j * sstride_b + i);
                tile[j][i] = Cast<S, D>::run(in.e[0]);
                tile[j][i + 1] = Cast<S, D>::run(in.e[1]);
            }
        }
        __syncthreads();
        for (uint32_t i = warp; i < na; i += kWarps) {
            const uint32_t j = 2 * lane;
            if (j < nb) {
                union { D2 v; DE e[2]; } out;
                out.e[0] = tile[j][i];
                out.e[1] = tile[j + 1][i];
                *reinterpret_cast<D2 *>(dp + (int64_t)i * it.ds[3] + j) = out.v;
            }
        }
        __syncthreads();  // the tile is reused by this CTA's next tile
        return;
      }
    }
    {
        for (uint32_t j = warp; j < nb; j += kWarps)
            for (uint32_t i = lane; i < na; i += 32)
                tile[j][i] = Cast<S, D>::run(s[(uint64_t)j * sstride_b + i]);
        __syncthreads();
        for (uint32_t i = warp; i < na; i += kWarps)
            for (uint32_t j = lane; j < nb; j += 32) dp[(int64_t)i * it.ds[3] + j] = tile[j][i];
    }
    __syncthreads();  // the tile is reused by this CTA's next tile
}

template <typename S, typename D>
__device__ __forceinline__ void one_tile(const CvtItem &it, uint32_t t, unsigned char *smem) {
    if (it.mode == 0) rows_tile<S, D>(it, t, smem);
    else if (it.mode == 2) {
        if constexpr (sizeof(typename D::store) == 2 && sizeof(typename S::store) >= 2 &&
                      sizeof(typename S::store) <= 4) packed_tile<S, D>(it, t, smem);
        else wide_tile<S, D>(it, t, smem);
    }
    else transpose_tile<S, D>(it, t, smem);
}

// One instantiation per conversion: a single kernel switching over all of them needs the
// registers of every case at once (243 per thread against 48-77 for any one of them).
template <typename S, typename D>
__global__ void __launch_bounds__(kCvtThreads, 4) convert_kernel(const CvtItem *__restrict__ items,
                                                             uint32_t n_items, uint64_t n_tiles) {
    constexpr uint32_t kElem = sizeof(typename D::store);
    constexpr uint32_t kEdgeA = 32 * Group<typename S::store>::n, kEdgeB = 32 * Group<typename D::store>::n;
    constexpr uint32_t kWide = kEdgeB * (kEdgeA + 1) * kElem, kPlain = kTT * (kTT + 1) * kElem;
    __shared__ __align__(16) unsigned char smem[kWide > kPlain ? kWide : kPlain];
    __shared__ CvtItem cur;
    __shared__ uint32_t cur_index;
    if (threadIdx.x == 0) cur_index = 0xffffffffu;
    __syncthreads();
    for (uint64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        // the item that owns tile t: usually still the one this CTA holds; else the last item
        // whose first tile is <= t
        uint32_t lo = cur_index;
        if (lo == 0xffffffffu || t < cur.tile0 || t >= cur.tile0 + cur.n_tiles) {
            lo = 0;
            uint32_t hi = n_items - 1;
            while (lo < hi) {
                const uint32_t mid = (lo + hi + 1) >> 1;
                if (items[mid].tile0 <= t) lo = mid;
                else hi = mid - 1;
            }
        }
        if (cur_index != lo) {
            __syncthreads();
            if (threadIdx.x < sizeof(CvtItem) / 8)
                reinterpret_cast<uint64_t *>(&cur)[threadIdx.x] =
                    reinterpret_cast<const uint64_t *>(items + lo)[threadIdx.x];
            if (threadIdx.x == 0) cur_index = lo;
            __syncthreads();
        }
        one_tile<S, D>(cur, (uint32_t)(t - cur.tile0), smem);
        __syncthreads();  // `cur` may be replaced for the next tile
    }
}

template <typename S, typename D>
cudaError_t launch_convert(const CvtItem *items, uint32_t n_items, uint64_t tiles, int sm_count,
                           cudaStream_t stream) {
    // as many resident CTAs per SM as registers and shared memory allow
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, convert_kernel<S, D>, kCvtThreads, 0);
    if (e != cudaSuccess) return e;
    uint64_t grid = (uint64_t)sm_count * (per_sm > 0 ? per_sm : 1);
    if (grid > tiles) grid = tiles;
    convert_kernel<S, D><<<(unsigned)grid, kCvtThreads, 0, stream>>>(items, n_items, tiles);
    return cudaGetLastError();
}

cudaError_t launch_kind(uint32_t kind, const CvtItem *items, uint32_t n_items, uint64_t tiles, int sm_count,
                        cudaStream_t stream) {
    switch (kind) {
        case kRaw1: return launch_convert<Raw<uint8_t>, Raw<uint8_t>>(items, n_items, tiles, sm_count, stream);
        case kRaw2: return launch_convert<Raw<uint16_t>, Raw<uint16_t>>(items, n_items, tiles, sm_count, stream);
        case kRaw4: return launch_convert<Raw<uint32_t>, Raw<uint32_t>>(items, n_items, tiles, sm_count, stream);
        case kRaw8: return launch_convert<Raw<uint64_t>, Raw<uint64_t>>(items, n_items, tiles, sm_count, stream);
        case kBf16ToF32: return launch_convert<BF16, F32>(items, n_items, tiles, sm_count, stream);
        case kF16ToF32: return launch_convert<F16, F32>(items, n_items, tiles, sm_count, stream);
        case kF32ToBf16: return launch_convert<F32, BF16>(items, n_items, tiles, sm_count, stream);
        case kF32ToF16: return launch_convert<F32, F16>(items, n_items, tiles, sm_count, stream);
        case kBf16ToF16: return launch_convert<BF16, F16>(items, n_items, tiles, sm_count, stream);
        case kF16ToBf16: return launch_convert<F16, BF16>(items, n_items, tiles, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mxb

using namespace mxb;

namespace {

uint32_t kind_size(uint32_t kind, uint32_t raw_bytes) {
    switch (kind) {
        case MXB_ELEM_RAW: return raw_bytes;
        case MXB_ELEM_F32: return 4;
        case MXB_ELEM_F16: case MXB_ELEM_BF16: return 2;
        default: return 0;
    }
}

// MXB_OK and a filled item, or MXB_ERR_UNSUPPORTED / MXB_ERR_ARG
int32_t canonical(const mxb_convert &c, CvtItem *out, uint64_t *bytes) {
    const uint32_t ssz = kind_size(c.src_kind, c.elem_bytes), dsz = kind_size(c.dst_kind, c.elem_bytes);
    if (!ssz || !dsz || c.ndim > MXB_MAX_DIMS) return MXB_ERR_ARG;
    uint32_t kind;
    if (c.src_kind == c.dst_kind) {
        kind = ssz == 1 ? kRaw1 : ssz == 2 ? kRaw2 : ssz == 4 ? kRaw4 : ssz == 8 ? kRaw8 : (uint32_t)kKinds;
    } else if (c.src_kind == MXB_ELEM_BF16 && c.dst_kind == MXB_ELEM_F32) kind = kBf16ToF32;
    else if (c.src_kind == MXB_ELEM_F16 && c.dst_kind == MXB_ELEM_F32) kind = kF16ToF32;
    else if (c.src_kind == MXB_ELEM_F32 && c.dst_kind == MXB_ELEM_BF16) kind = kF32ToBf16;
    else if (c.src_kind == MXB_ELEM_F32 && c.dst_kind == MXB_ELEM_F16) kind = kF32ToF16;
    else if (c.src_kind == MXB_ELEM_BF16 && c.dst_kind == MXB_ELEM_F16) kind = kBf16ToF16;
    else if (c.src_kind == MXB_ELEM_F16 && c.dst_kind == MXB_ELEM_BF16) kind = kF16ToBf16;
    else kind = kKinds;
    if (kind == kKinds) return MXB_ERR_UNSUPPORTED;
    if ((c.src % ssz) || (c.dst % dsz)) return MXB_ERR_ALIGN;
    // source strides: as given, or those of a contiguous row-major box when all are zero
    int64_t given[MXB_MAX_DIMS];
    bool strided = false;
    for (uint32_t d = 0; d < c.ndim; ++d) strided = strided || c.src_stride[d] != 0;
    {
        int64_t run = 1;
        for (int d = (int)c.ndim - 1; d >= 0; --d) {
            given[d] = strided ? c.src_stride[d] : run;
            if (given[d] < 0) return MXB_ERR_ARG;
            run *= (int64_t)(c.extent[d] ? c.extent[d] : 1);
        }
    }
    // drop extent-1 dims, merge dims that source and destination both walk as one
    uint64_t n[MXB_MAX_DIMS];
    int64_t ds[MXB_MAX_DIMS], ss[MXB_MAX_DIMS];
    uint32_t nd = 0;
    uint64_t total = 1;
    for (uint32_t d = 0; d < c.ndim; ++d) {
        if (c.extent[d] == 0) { total = 0; break; }
        if (c.dst_stride[d] < 0) return MXB_ERR_ARG;
        total *= c.extent[d];
        if (c.extent[d] == 1) continue;
        if (nd && ds[nd - 1] == c.dst_stride[d] * (int64_t)c.extent[d] &&
            ss[nd - 1] == given[d] * (int64_t)c.extent[d]) {
            n[nd - 1] *= c.extent[d];
            ds[nd - 1] = c.dst_stride[d];
            ss[nd - 1] = given[d];
        } else {
            n[nd] = c.extent[d];
            ds[nd] = c.dst_stride[d];
            ss[nd] = given[d];
            ++nd;
        }
    }
    memset(out, 0, sizeof *out);
    *bytes = total * (ssz + dsz);
    if (total == 0) return MXB_OK;  // nothing to move: zero tiles
    if (nd == 0) { n[0] = 1; ds[0] = 1; ss[0] = 1; nd = 1; }
    if (nd > 4) return MXB_ERR_UNSUPPORTED;
    if (ss[nd - 1] != 1) return MXB_ERR_UNSUPPORTED;  // the source's inner dim must be unit-stride
    for (uint32_t d = 0; d < nd; ++d)
        if (n[d] > 0xffffffffull) return MXB_ERR_UNSUPPORTED;
    out->src = c.src;
    out->dst = c.dst;
    for (uint32_t d = 0; d < 4; ++d) { out->n[d] = 1; out->ds[d] = 0; }
    for (uint32_t d = 0; d < 3; ++d) out->ss[d] = 0;
    for (uint32_t d = 0; d < nd; ++d) {
        out->n[4 - nd + d] = (uint32_t)n[d];
        out->ds[4 - nd + d] = ds[d];
        if (4 - nd + d < 3) out->ss[4 - nd + d] = ss[d];
    }
    out->kind = kind;
    out->bdim = 3;
    if (out->ds[3] != 1)
        for (uint32_t d = 0; d < 3; ++d)
            if (out->n[d] > 1 && out->ds[d] == 1) out->bdim = d;
    uint64_t tiles;
    if (out->bdim == 3) {
        out->mode = 0;
        out->tiles_a = (out->n[3] + kRowTile - 1) / kRowTile;
        out->tiles_b = 1;
        tiles = (uint64_t)out->tiles_a * out->n[0] * out->n[1] * out->n[2];
    } else {
        out->mode = 1;
        const uint32_t b = out->bdim;
        // wide accesses: groups of 8 bytes (4 for one-byte elements) naturally aligned on both sides
        const uint32_t gs = ssz >= 4 ? 8 / ssz : 4, gd = dsz >= 4 ? 8 / dsz : 4;
        bool wide = ssz < 8 && dsz < 8 && out->n[3] % gs == 0 && out->n[b] % gd == 0 &&
                    c.src % (gs * ssz) == 0 && c.dst % (gd * dsz) == 0;
        for (uint32_t d = 0; d < 4 && wide; ++d)
            if (d != b && out->n[d] > 1 && out->ds[d] % gd) wide = false;
        for (uint32_t d = 0; d < 3 && wide; ++d)
            if (out->n[d] > 1 && out->ss[d] % gs) wide = false;
        const uint32_t edge_a = wide ? 32 * gs : kTT, edge_b = wide ? 32 * gd : kTT;
        if (wide) out->mode = 2;
        out->tiles_a = (out->n[3] + edge_a - 1) / edge_a;
        out->tiles_b = (out->n[b] + edge_b - 1) / edge_b;
        tiles = (uint64_t)out->tiles_a * out->tiles_b;
        for (uint32_t d = 0; d < 3; ++d)
            if (d != b) tiles *= out->n[d];
        // pairs: every pair of source elements along the inner dim and every pair of destination
        // elements along its unit-stride dim must be a naturally aligned 2-element word
        bool pair = ssz <= 4 && dsz <= 4 && out->n[3] % 2 == 0 && out->n[b] % 2 == 0 &&
                    c.src % (2 * ssz) == 0 && c.dst % (2 * dsz) == 0;
        for (uint32_t d = 0; d < 4 && pair; ++d)
            if (d != b && out->n[d] > 1 && out->ds[d] % 2) pair = false;
        for (uint32_t d = 0; d < 3 && pair; ++d)
            if (out->n[d] > 1 && out->ss[d] % 2) pair = false;
        out->pair = pair ? 1u : 0u;
    }
    if (tiles > 0xffffffffull) return MXB_ERR_UNSUPPORTED;  // the kernel indexes a box's tiles with 32 bits
    out->tile0 = tiles;  // the caller turns counts into a prefix
    return MXB_OK;
}

}  // namespace

extern "C" int32_t mxb_convert_boxes(mxb_ctx *ctx, int32_t dev, const mxb_convert *items, uint64_t n,
                                     uint32_t flags, uint64_t *bytes_out) {
    if (!ctx || (!items && n)) {
        set_error("mxb_convert_boxes: bad arguments");
        return MXB_ERR_ARG;
    }
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    // boxes grouped by conversion: one launch per conversion present (usually one or two)
    std::vector<CvtItem> groups[kKinds];
    uint64_t group_tiles[kKinds] = {};
    uint64_t bytes = 0;
    size_t live = 0;
    for (uint64_t i = 0; i < n; ++i) {
        CvtItem it;
        uint64_t b = 0;
        const int32_t rc = canonical(items[i], &it, &b);
        if (rc != MXB_OK) {
            set_error("mxb_convert_boxes: box %llu: %s", (unsigned long long)i,
                      rc == MXB_ERR_UNSUPPORTED ? "element kinds or rank not supported"
                      : rc == MXB_ERR_ALIGN     ? "address not aligned to its element"
                                                : "bad geometry");
            return rc;
        }
        bytes += b;
        const uint64_t count = it.tile0;
        if (!count) continue;
        it.tile0 = group_tiles[it.kind];
        it.n_tiles = count;
        group_tiles[it.kind] += count;
        groups[it.kind].push_back(it);
        ++live;
    }
    if (bytes_out) *bytes_out = bytes;
    if (!live) return MXB_OK;
    DeviceGuard g(dev);
    std::lock_guard<std::mutex> lk(*d->mu);
    const size_t table_bytes = live * sizeof(CvtItem);
    int32_t rc = ensure_table(d, table_bytes);
    if (rc != MXB_OK) return rc;
    MXB_CUDA(cudaStreamSynchronize(d->stream));  // the pinned staging copy is shared by every call
    d->table_tag = 0;
    CvtItem *host = reinterpret_cast<CvtItem *>(d->table_host);
    size_t at = 0;
    for (uint32_t k = 0; k < kKinds; ++k) {
        memcpy(host + at, groups[k].data(), groups[k].size() * sizeof(CvtItem));
        at += groups[k].size();
    }
    MXB_CUDA(cudaMemcpyAsync(d->table, d->table_host, table_bytes, cudaMemcpyHostToDevice, d->stream));
    at = 0;
    for (uint32_t k = 0; k < kKinds; ++k) {
        if (groups[k].empty()) continue;
        MXB_CUDA(launch_kind(k, reinterpret_cast<const CvtItem *>(d->table) + at, (uint32_t)groups[k].size(),
                             group_tiles[k], d->sm_count, d->stream));
        at += groups[k].size();
        ctx->launches.fetch_add(1);
    }
    if (flags & MXB_SCATTER_NO_SYNC) return MXB_OK;
    return check_status(d);
}
