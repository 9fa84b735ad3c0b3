// Kernel 2: serving-peer fan-out over NVLink (sm_100a).
//
// Every GPU of the broadcast runs one persistent launch of the same kernel on
// its own device.  The payload (a list of byte ranges, identical in size on
// every GPU) is cut into pieces of at most 64 KiB that never cross a chunk or a
// range boundary.  CTA b owns pieces b, b+grid, ...  For each piece it
//   1. waits (bounded) until this GPU's arrival counter of the piece's chunk
//      shows that the parent delivered the whole chunk (the root skips this),
//   2. stores the piece from local HBM into every child's range with 16-byte
//      P2P stores,
//   3. after a CTA barrier and a system-scope fence, raises the child's counter
//      for that chunk by one (release, system scope).
// A chunk is complete on a GPU when its counter reached run_index * (pieces in
// the chunk); counters only grow, so repeated broadcasts need no reset.  Leaves
// run the same kernel with no children: it returns once every chunk arrived.
// No wait is unbounded: when the time budget runs out the kernel records
// DEV_TIMEOUT in its status word and returns.
// A leaf only watches its counters (one thread per chunk).  A root whose children only
// receive may hand the bytes to the copy engines instead (MXB_FANOUT_ENGINE_DMA: one peer
// copy per run of adjacent ranges, then one launch that raises every counter).
#include <cstdlib>

#include "bulk.cuh"
#include "common.cuh"

namespace mxb {

struct FanPiece {
    uint64_t local;   // address in this GPU's copy
    uint32_t nbytes;  // <= 64 KiB
    uint32_t chunk;
};

constexpr int kFanThreads = 512;
// the copy-engine push is used when its copies average at least this much (about 7 us of setup
// per peer copy were measured: 4 MiB at 750 GB/s take 5.6 us)
constexpr uint64_t kDmaMinMeanCopy = 4ull << 20;
constexpr uint32_t kFanPiece = 64 * 1024;

struct FanArgs {
    const FanPiece *pieces;
    const uint64_t *child_ptr;        // [children][n_pieces] destination of each piece
    const uint32_t *chunk_pieces;     // pieces per chunk
    uint32_t *counters;               // this GPU's arrival counters, one per chunk
    uint64_t child_counters[MXB_FANOUT_MAX_CHILDREN];
    uint64_t n_pieces;
    uint32_t n_chunks;
    uint32_t n_children;
    uint32_t is_root;
    uint32_t run_index;  // 1-based
    uint64_t timeout_ns;
    uint32_t *status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t *p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kFanThreads) fanout_kernel(FanArgs a) {
    __shared__ uint32_t s_abort;
    const uint32_t tid = threadIdx.x;
    if (a.n_children == 0) {
        // a leaf forwards nothing: it only has to see every chunk arrive, one thread per chunk
        if (a.is_root) return;
        const uint64_t t0 = globaltimer_ns();
        for (uint64_t c = (uint64_t)blockIdx.x * kFanThreads + tid; c < a.n_chunks;
             c += (uint64_t)gridDim.x * kFanThreads) {
            const uint32_t want = a.run_index * a.chunk_pieces[c];
            uint32_t spins = 0;
            while ((int32_t)(ld_acquire_sys(a.counters + c) - want) < 0) {
                if ((++spins & 63u) == 0) {
                    if (globaltimer_ns() - t0 > a.timeout_ns) {
                        atomicExch(a.status, DEV_TIMEOUT);
                        return;
                    }
                    __nanosleep(200);
                }
            }
        }
        return;
    }
    if (tid == 0) s_abort = 0;
    __syncthreads();
    for (uint64_t p = blockIdx.x; p < a.n_pieces; p += gridDim.x) {
        const FanPiece pc = a.pieces[p];
        if (!a.is_root) {
            if (tid == 0) {
                const uint32_t want = a.run_index * a.chunk_pieces[pc.chunk];
                const uint32_t *ctr = a.counters + pc.chunk;
                const uint64_t t0 = globaltimer_ns();
                uint32_t spins = 0;
                // counters grow monotonically and may wrap: compare as a signed distance
                while ((int32_t)(ld_acquire_sys(ctr) - want) < 0) {
                    if ((++spins & 63u) == 0) {
                        if (globaltimer_ns() - t0 > a.timeout_ns) {
                            s_abort = 1;
                            atomicExch(a.status, DEV_TIMEOUT);
                            break;
                        }
                        __nanosleep(200);
                    }
                }
            }
            __syncthreads();
            if (s_abort) return;
        }
        const uint4 *src = reinterpret_cast<const uint4 *>(pc.local);
        const uint32_t nvec = pc.nbytes >> 4;
        for (uint32_t c = 0; c < a.n_children; ++c) {
            uint4 *dst = reinterpret_cast<uint4 *>(a.child_ptr[(uint64_t)c * a.n_pieces + p]);
            uint32_t i = tid;
            for (; i + 3 * kFanThreads < nvec; i += 4 * kFanThreads) {
                uint4 v0 = src[i], v1 = src[i + kFanThreads], v2 = src[i + 2 * kFanThreads],
                      v3 = src[i + 3 * kFanThreads];
                dst[i] = v0;
                dst[i + kFanThreads] = v1;
                dst[i + 2 * kFanThreads] = v2;
                dst[i + 3 * kFanThreads] = v3;
            }
            for (; i < nvec; i += kFanThreads) dst[i] = src[i];
            // ranges need not be multiples of 16 bytes
            const unsigned char *sb = reinterpret_cast<const unsigned char *>(pc.local);
            unsigned char *db = reinterpret_cast<unsigned char *>(dst);
            for (uint32_t j = (nvec << 4) + tid; j < pc.nbytes; j += kFanThreads) db[j] = sb[j];
        }
        if (a.n_children) {
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();
                for (uint32_t c = 0; c < a.n_children; ++c)
                    red_release_sys_add(reinterpret_cast<uint32_t *>(a.child_counters[c]) + pc.chunk,
                                        1u);
            }
        }
    }
}

// Bulk engine: one warp per CTA, one CTA per SM, pieces staged through a 3-stage
// 64 KiB shared-memory ring with cp.async.bulk (local HBM -> shared -> every
// child's HBM over NVLink).  The child's counter for piece k is raised only after
// the bulk stores of piece k have completed (wait_group, not wait_group.read).
constexpr int kFanStages = 3;

__device__ __forceinline__ bool fan_wait_chunk(const FanArgs &a, uint32_t chunk) {
    const uint32_t want = a.run_index * a.chunk_pieces[chunk];
    const uint32_t *ctr = a.counters + chunk;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(ctr) - want) < 0) {
        if ((++spins & 63u) == 0) {
            if (globaltimer_ns() - t0 > a.timeout_ns) return false;
            __nanosleep(200);
        }
    }
    // what the parent wrote is read next by the async proxy (bulk load)
    asm volatile("fence.proxy.async;" ::: "memory");
    return true;
}

__device__ __forceinline__ void fan_signal(const FanArgs &a, uint32_t chunk) {
    __threadfence_system();
    for (uint32_t c = 0; c < a.n_children; ++c)
        red_release_sys_add(reinterpret_cast<uint32_t *>(a.child_counters[c]) + chunk, 1u);
}

__global__ void __launch_bounds__(32) fanout_bulk_kernel(FanArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full[kFanStages];
    const uint32_t lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < kFanStages; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const uint64_t first = blockIdx.x;
    if (first >= a.n_pieces) return;
    const uint64_t mine = (a.n_pieces - first + gridDim.x - 1) / gridDim.x;
    bool failed = false;
    // A ragged piece takes its stage without loading into it, so a stage's barrier phase
    // follows the number of loads that went through that stage, not the piece index.
    uint32_t waits_done[kFanStages] = {};

    // wait for the piece's chunk (unless root) and start its load; warp-uniform result
    auto start_piece = [&](uint64_t k) -> bool {
        const FanPiece pc = a.pieces[first + k * gridDim.x];
        bool ok = true;
        if (!a.is_root) {
            if (lane == 0) ok = fan_wait_chunk(a, pc.chunk);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok) return false;
        if ((pc.nbytes & 15u) == 0 && a.n_children) {  // bulk-eligible (addresses are 16-byte aligned)
            const int s = (int)(k % kFanStages);
            if (lane == 0) {
                mbar_expect_tx(&full[s], pc.nbytes);
                bulk_g2s(smem + (size_t)s * kFanPiece, reinterpret_cast<const void *>(pc.local),
                         pc.nbytes, &full[s]);
            }
        }
        return true;
    };

    uint64_t signalled = 0;  // pieces [0, signalled) have raised the children's counters
    if (!start_piece(0)) failed = true;
    uint64_t k = 0;
    for (; k < mine && !failed; ++k) {
        const FanPiece pc = a.pieces[first + k * gridDim.x];
        const int s = (int)(k % kFanStages);
        if (k + 1 < mine) {
            // stage (k+1)%3 held piece k-2, whose stores completed before piece k-2 was signalled
            if (!start_piece(k + 1)) {
                failed = true;
                break;
            }
        }
        if (a.n_children) {
            if ((pc.nbytes & 15u) == 0) {
                const uint32_t parity = waits_done[s] & 1u;
                ++waits_done[s];
                bool ok = false;
                for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
                    ok = __all_sync(0xffffffffu, mbar_try_wait(&full[s], parity));
                    if (ok) break;
                }
                if (!ok) {
                    failed = true;
                    break;
                }
                if (lane == 0) {
                    for (uint32_t c = 0; c < a.n_children; ++c)
                        bulk_s2g(reinterpret_cast<void *>(a.child_ptr[(uint64_t)c * a.n_pieces + first +
                                                                       k * gridDim.x]),
                                 smem + (size_t)s * kFanPiece, pc.nbytes);
                }
            } else {
                // ragged last piece of a range: plain loads and stores by the warp
                const unsigned char *sb = reinterpret_cast<const unsigned char *>(pc.local);
                for (uint32_t c = 0; c < a.n_children; ++c) {
                    unsigned char *db = reinterpret_cast<unsigned char *>(
                        a.child_ptr[(uint64_t)c * a.n_pieces + first + k * gridDim.x]);
                    for (uint32_t j = lane; j < pc.nbytes; j += 32) db[j] = sb[j];
                }
                __syncwarp();
            }
            bulk_commit();  // every piece closes one group (possibly empty), so groups count pieces
            // all groups but the newest are complete: pieces up to k-1 may be announced
            bulk_wait_all<1>();
            __syncwarp();
            if (lane == 0)
                for (; signalled < k; ++signalled)
                    fan_signal(a, a.pieces[first + signalled * gridDim.x].chunk);
            signalled = k;
        }
    }
    bulk_wait_all<0>();
    __syncwarp();
    if (!failed && a.n_children && lane == 0)
        for (; signalled < mine; ++signalled)
            fan_signal(a, a.pieces[first + signalled * gridDim.x].chunk);
    if (failed) {
        if (lane == 0) atomicExch(a.status, DEV_TIMEOUT);
        // bounded wait for a load that may still be in flight before shared memory is released
        for (uint64_t j = k; j < k + 2 && j < mine; ++j) {
            const uint32_t parity = (uint32_t)((j / kFanStages) & 1);
            for (uint32_t spin = 0; spin < (1u << 14); ++spin)
                if (mbar_try_wait(&full[j % kFanStages], parity)) break;
        }
    }
}

// Copy-engine push (root only): after the peer copies of every range have completed in stream
// order, one launch announces every chunk to every child at once.
__global__ void __launch_bounds__(256) fanout_announce_kernel(FanArgs a, uint32_t n_chunks) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_chunks) return;
    __threadfence_system();
    const uint32_t add = a.chunk_pieces[c];
    for (uint32_t k = 0; k < a.n_children; ++k)
        red_release_sys_add(reinterpret_cast<uint32_t *>(a.child_counters[k]) + c, add);
}

}  // namespace mxb

using namespace mxb;

struct mxb_fanout {
    mxb_ctx *ctx = nullptr;
    DeviceState *dv = nullptr;
    std::vector<mxb_span> local;
    uint64_t chunk_bytes = 0;
    std::vector<FanPiece> pieces;
    std::vector<uint64_t> piece_range, piece_off;  // provenance of each piece
    std::vector<uint32_t> chunk_pieces;
    std::vector<uint64_t> child_ptr[MXB_FANOUT_MAX_CHILDREN];
    uint64_t child_counters[MXB_FANOUT_MAX_CHILDREN] = {};
    uint32_t n_children = 0;
    uint32_t *counters = nullptr;  // device
    void *dev_tables = nullptr;
    size_t dev_tables_bytes = 0;
    bool dirty = true;
    uint32_t run_index = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int32_t engine = MXB_FANOUT_ENGINE_VECTOR;
    // copy-engine push: one stream and one completion event per child
    cudaStream_t child_stream[MXB_FANOUT_MAX_CHILDREN] = {};
    cudaEvent_t child_done[MXB_FANOUT_MAX_CHILDREN] = {};
};

namespace {

// Pieces of a payload: walk the concatenated byte space of the ranges; cut at range ends,
// chunk ends and the piece size (64 KiB unless the caller names another).  Every piece start stays 16-byte aligned inside its range: only a
// range's last piece may be ragged.  Depends on the range sizes alone, so every GPU of a
// broadcast (same sizes, own addresses) cuts the same pieces and counts the same chunks.
void plan_pieces(const mxb_span *local, uint64_t n, uint64_t chunk_bytes, uint64_t piece_max,
                 std::vector<mxb_fanout_piece> &pieces, std::vector<uint32_t> &chunk_pieces) {
    uint64_t vpos = 0;
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t off = 0;
        while (off < local[i].nbytes) {
            const uint64_t chunk = vpos / chunk_bytes;
            const uint64_t to_chunk_end = (chunk + 1) * chunk_bytes - vpos;
            uint64_t len = local[i].nbytes - off;
            if (len > to_chunk_end) len = to_chunk_end;
            if (len > piece_max) len = piece_max;
            if (len < local[i].nbytes - off) len &= ~uint64_t(15);
            if (len == 0) len = local[i].nbytes - off < 16 ? local[i].nbytes - off : 16;
            pieces.push_back({i, off, (uint32_t)len, (uint32_t)chunk});
            if (chunk_pieces.size() <= chunk) chunk_pieces.resize(chunk + 1, 0);
            chunk_pieces[chunk] += 1;
            off += len;
            vpos += len;
        }
    }
}

}  // namespace

extern "C" {

static bool piece_ok(uint64_t piece_bytes) {
    return piece_bytes >= 4096 && piece_bytes <= MXB_FANOUT_PIECE_MAX && !(piece_bytes & 15u);
}

int32_t mxb_fanout_plan(const mxb_span *local, uint64_t n, uint64_t chunk_bytes,
                        mxb_fanout_piece *pieces, uint64_t piece_cap, uint64_t *n_pieces,
                        uint32_t *chunk_pieces, uint64_t chunk_cap, uint64_t *n_chunks) {
    return mxb_fanout_plan_pieces(local, n, chunk_bytes, kFanPiece, pieces, piece_cap, n_pieces, chunk_pieces,
                                  chunk_cap, n_chunks);
}

int32_t mxb_fanout_plan_pieces(const mxb_span *local, uint64_t n, uint64_t chunk_bytes, uint64_t piece_bytes,
                               mxb_fanout_piece *pieces, uint64_t piece_cap, uint64_t *n_pieces,
                               uint32_t *chunk_pieces, uint64_t chunk_cap, uint64_t *n_chunks) {
    if ((!local && n) || !n_pieces || !n_chunks || chunk_bytes < 4096 || (chunk_bytes & 15u) ||
        !piece_ok(piece_bytes) || (!pieces && piece_cap) || (!chunk_pieces && chunk_cap)) {
        set_error("mxb_fanout_plan: bad arguments (chunk and piece must be multiples of 16, >= 4096; "
                  "a piece at most 1 MiB)");
        return MXB_ERR_ARG;
    }
    std::vector<mxb_fanout_piece> plan;
    std::vector<uint32_t> per_chunk;
    plan_pieces(local, n, chunk_bytes, piece_bytes, plan, per_chunk);
    *n_pieces = plan.size();
    *n_chunks = per_chunk.size();
    for (uint64_t i = 0; i < plan.size() && i < piece_cap; ++i) pieces[i] = plan[i];
    for (uint64_t i = 0; i < per_chunk.size() && i < chunk_cap; ++i) chunk_pieces[i] = per_chunk[i];
    if (plan.size() > piece_cap || per_chunk.size() > chunk_cap) {
        set_error("mxb_fanout_plan: %llu pieces in %llu chunks, room for %llu and %llu",
                  (unsigned long long)plan.size(), (unsigned long long)per_chunk.size(),
                  (unsigned long long)piece_cap, (unsigned long long)chunk_cap);
        return MXB_ERR_NOMEM;
    }
    return MXB_OK;
}

int32_t mxb_fanout_create(mxb_ctx *ctx, int32_t dev, const mxb_span *local, uint64_t n,
                          uint64_t chunk_bytes, mxb_fanout **out) {
    return mxb_fanout_create_pieces(ctx, dev, local, n, chunk_bytes, kFanPiece, out);
}

int32_t mxb_fanout_create_pieces(mxb_ctx *ctx, int32_t dev, const mxb_span *local, uint64_t n,
                                 uint64_t chunk_bytes, uint64_t piece_bytes, mxb_fanout **out) {
    if (!ctx || !local || !n || !out || chunk_bytes < 4096 || (chunk_bytes & 15u) || !piece_ok(piece_bytes)) {
        set_error("mxb_fanout_create: bad arguments (chunk and piece must be multiples of 16, >= 4096; "
                  "a piece at most 1 MiB)");
        return MXB_ERR_ARG;
    }
    DeviceState *dv = ctx->find(dev);
    if (!dv) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    for (uint64_t i = 0; i < n; ++i)
        if (local[i].nbytes && ((local[i].ptr & 15u) || !local[i].ptr)) {
            set_error("range %llu: address must be non-null and 16-byte aligned",
                      (unsigned long long)i);
            return MXB_ERR_ALIGN;
        }
    mxb_fanout *f = new mxb_fanout();
    f->ctx = ctx;
    f->dv = dv;
    f->local.assign(local, local + n);
    f->chunk_bytes = chunk_bytes;
    std::vector<mxb_fanout_piece> plan;
    plan_pieces(local, n, chunk_bytes, piece_bytes, plan, f->chunk_pieces);
    for (const mxb_fanout_piece &p : plan) {
        f->pieces.push_back({local[p.range].ptr + p.offset, p.nbytes, p.chunk});
        f->piece_range.push_back(p.range);
        f->piece_off.push_back(p.offset);
    }
    if (const char *eng = getenv("MXB_FANOUT_ENGINE")) {
        if (!strcmp(eng, "bulk")) f->engine = MXB_FANOUT_ENGINE_BULK;
        else if (!strcmp(eng, "dma")) f->engine = MXB_FANOUT_ENGINE_DMA;
    }
    DeviceGuard g(dev);
    const size_t nchunks = f->chunk_pieces.size() ? f->chunk_pieces.size() : 1;
    // a whole 2 MiB allocation of its own, so that an IPC handle of the counters
    // exposes nothing else of this process
    size_t ctr_bytes = nchunks * sizeof(uint32_t);
    if (ctr_bytes < (2u << 20)) ctr_bytes = 2u << 20;
    if (cudaMalloc((void **)&f->counters, ctr_bytes) != cudaSuccess ||
        cudaMemset(f->counters, 0, ctr_bytes) != cudaSuccess ||
        cudaEventCreate(&f->ev0) != cudaSuccess || cudaEventCreate(&f->ev1) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        set_error("mxb_fanout_create: CUDA allocation failed: %s",
                  cudaGetErrorString(cudaGetLastError()));
        mxb_fanout_destroy(f);
        return MXB_ERR_CUDA;
    }
    *out = f;
    return MXB_OK;
}

int32_t mxb_fanout_set_engine(mxb_fanout *f, int32_t engine) {
    if (!f || (engine != MXB_FANOUT_ENGINE_VECTOR && engine != MXB_FANOUT_ENGINE_BULK &&
               engine != MXB_FANOUT_ENGINE_DMA)) {
        set_error("mxb_fanout_set_engine: unknown engine");
        return MXB_ERR_ARG;
    }
    f->engine = engine;
    return MXB_OK;
}

uint64_t mxb_fanout_counters(mxb_fanout *f) { return f ? (uint64_t)(uintptr_t)f->counters : 0; }

int32_t mxb_fanout_set_child(mxb_fanout *f, int32_t k, const mxb_span *child, uint64_t n,
                             uint64_t child_counters) {
    if (!f || k < 0 || k >= MXB_FANOUT_MAX_CHILDREN || !child || !child_counters ||
        n != f->local.size()) {
        set_error("mxb_fanout_set_child: bad arguments");
        return MXB_ERR_ARG;
    }
    if ((uint32_t)k > f->n_children) {
        set_error("mxb_fanout_set_child: children must be set in order");
        return MXB_ERR_STATE;
    }
    for (uint64_t i = 0; i < n; ++i) {
        if (child[i].nbytes != f->local[i].nbytes) {
            set_error("child range %llu: size %llu differs from the local size %llu",
                      (unsigned long long)i, (unsigned long long)child[i].nbytes,
                      (unsigned long long)f->local[i].nbytes);
            return MXB_ERR_ARG;
        }
        if (child[i].nbytes && (child[i].ptr & 15u)) return MXB_ERR_ALIGN;
    }
    std::vector<uint64_t> &cp = f->child_ptr[k];
    cp.resize(f->pieces.size());
    for (size_t p = 0; p < f->pieces.size(); ++p)
        cp[p] = child[f->piece_range[p]].ptr + f->piece_off[p];
    f->child_counters[k] = child_counters;
    if ((uint32_t)k == f->n_children) f->n_children = k + 1;
    f->dirty = true;
    return MXB_OK;
}

int32_t mxb_fanout_run(mxb_fanout *f, int32_t is_root, uint32_t timeout_ms) {
    if (!f) return MXB_ERR_ARG;
    DeviceState *dv = f->dv;
    DeviceGuard g(dv->device);
    const size_t np = f->pieces.size();
    const size_t b_pieces = (np * sizeof(FanPiece) + 255) & ~size_t(255);
    const size_t b_child = (np * sizeof(uint64_t) * (f->n_children ? f->n_children : 1) + 255) &
                           ~size_t(255);
    const size_t b_chunk = (f->chunk_pieces.size() * sizeof(uint32_t) + 255) & ~size_t(255);
    if (f->dirty) {
        const size_t total = b_pieces + b_child + b_chunk;
        if (total > f->dev_tables_bytes) {
            if (f->dev_tables) cudaFree(f->dev_tables);
            f->dev_tables = nullptr;
            MXB_CUDA(cudaMalloc(&f->dev_tables, total));
            f->dev_tables_bytes = total;
        }
        char *base = reinterpret_cast<char *>(f->dev_tables);
        MXB_CUDA(cudaMemcpy(base, f->pieces.data(), np * sizeof(FanPiece), cudaMemcpyHostToDevice));
        for (uint32_t c = 0; c < f->n_children; ++c)
            MXB_CUDA(cudaMemcpy(base + b_pieces + (size_t)c * np * sizeof(uint64_t),
                                f->child_ptr[c].data(), np * sizeof(uint64_t),
                                cudaMemcpyHostToDevice));
        MXB_CUDA(cudaMemcpy(base + b_pieces + b_child, f->chunk_pieces.data(),
                            f->chunk_pieces.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
        f->dirty = false;
    }
    char *base = reinterpret_cast<char *>(f->dev_tables);
    FanArgs a;
    memset(&a, 0, sizeof a);
    a.pieces = reinterpret_cast<const FanPiece *>(base);
    a.child_ptr = reinterpret_cast<const uint64_t *>(base + b_pieces);
    a.chunk_pieces = reinterpret_cast<const uint32_t *>(base + b_pieces + b_child);
    a.counters = f->counters;
    for (uint32_t c = 0; c < f->n_children; ++c) a.child_counters[c] = f->child_counters[c];
    a.n_pieces = np;
    a.n_chunks = (uint32_t)f->chunk_pieces.size();
    a.n_children = f->n_children;
    a.is_root = is_root ? 1u : 0u;
    a.run_index = ++f->run_index;
    a.timeout_ns = (uint64_t)(timeout_ms ? timeout_ms : 1000u) * 1000000ull;
    a.status = dv->status;
    if (np == 0) return MXB_OK;
    // all CTAs must be co-resident: they wait on data, never on each other, but a
    // CTA that is not scheduled cannot forward its pieces
    const bool bulk = f->engine == MXB_FANOUT_ENGINE_BULK;
    if (f->engine == MXB_FANOUT_ENGINE_DMA && is_root && f->n_children) {
        // Copy-engine push: every range to every child with one peer copy (children on streams
        // of their own, so their links run side by side), then one launch that announces all
        // chunks.  Nothing is announced before everything has arrived, which suits a root whose
        // children only receive; a node that waits for a parent keeps the store kernel.
        // Ranges that follow one another in memory on both sides travel as one copy; a payload
        // that still comes to many small copies (thousands of scattered tensors) costs more in
        // copy setup than the engines gain, and goes to the store kernel below instead.
        struct Run {
            uint64_t src, dst, len;
        };
        std::vector<Run> runs[MXB_FANOUT_MAX_CHILDREN];
        uint64_t total = 0, copies = 0;
        for (uint32_t c = 0; c < f->n_children; ++c) {
            Run cur{0, 0, 0};
            for (size_t p = 0; p < np; ++p) {
                if (f->piece_off[p] != 0) continue;  // the first piece of a range stands for the range
                const Run r{f->pieces[p].local, f->child_ptr[c][p], f->local[f->piece_range[p]].nbytes};
                if (cur.len && r.src == cur.src + cur.len && r.dst == cur.dst + cur.len) {
                    cur.len += r.len;
                    continue;
                }
                if (cur.len) runs[c].push_back(cur);
                cur = r;
            }
            if (cur.len) runs[c].push_back(cur);
            for (const Run &r : runs[c]) total += r.len;
            copies += runs[c].size();
        }
        if (copies && total / copies >= kDmaMinMeanCopy) {
            MXB_CUDA(cudaEventRecord(f->ev0, dv->stream));
            const uint32_t nchunks = (uint32_t)f->chunk_pieces.size();
            for (uint32_t c = 0; c < f->n_children; ++c) {
                if (!f->child_stream[c])
                    MXB_CUDA(cudaStreamCreateWithFlags(&f->child_stream[c], cudaStreamNonBlocking));
                if (!f->child_done[c])
                    MXB_CUDA(cudaEventCreateWithFlags(&f->child_done[c], cudaEventDisableTiming));
                MXB_CUDA(cudaStreamWaitEvent(f->child_stream[c], f->ev0, 0));
                for (const Run &r : runs[c])
                    MXB_CUDA(cudaMemcpyAsync(reinterpret_cast<void *>(r.dst), reinterpret_cast<const void *>(r.src),
                                             r.len, cudaMemcpyDeviceToDevice, f->child_stream[c]));
                MXB_CUDA(cudaEventRecord(f->child_done[c], f->child_stream[c]));
                MXB_CUDA(cudaStreamWaitEvent(dv->stream, f->child_done[c], 0));
            }
            fanout_announce_kernel<<<(nchunks + 255) / 256, 256, 0, dv->stream>>>(a, nchunks);
            MXB_CUDA(cudaGetLastError());
            MXB_CUDA(cudaEventRecord(f->ev1, dv->stream));
            f->ctx->launches.fetch_add(1);
            return MXB_OK;
        }
    }
    if (bulk)
        for (const FanPiece &pc : f->pieces)
            if (pc.nbytes > kFanPiece) {
                set_error("mxb_fanout_run: the bulk engine stages pieces of at most 64 KiB");
                return MXB_ERR_ARG;
            }
    MXB_CUDA(cudaEventRecord(f->ev0, dv->stream));
    if (bulk) {
        const size_t smem = (size_t)kFanStages * kFanPiece;
        // idempotent and cheap: set on every launch rather than keep a flag several threads share
        MXB_CUDA(cudaFuncSetAttribute(fanout_bulk_kernel,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        uint64_t grid = (uint64_t)dv->sm_count;
        if (grid > np) grid = np;
        fanout_bulk_kernel<<<(unsigned)grid, 32, smem, dv->stream>>>(a);
    } else {
        // 4 resident CTAs of 512 threads per SM: more warps posting stores keep the links fuller
        // than 2 per SM do
        int per_sm = 4;
        if (const char *g = getenv("MXB_FANOUT_CTAS_PER_SM")) per_sm = atoi(g) > 0 ? atoi(g) : 4;
        if (per_sm > 4) per_sm = 4;
        uint64_t grid = (uint64_t)dv->sm_count * per_sm;
        if (grid > np) grid = np;
        fanout_kernel<<<(unsigned)grid, kFanThreads, 0, dv->stream>>>(a);
    }
    MXB_CUDA(cudaGetLastError());
    MXB_CUDA(cudaEventRecord(f->ev1, dv->stream));
    f->ctx->launches.fetch_add(1);
    return MXB_OK;
}

int32_t mxb_fanout_wait(mxb_fanout *f, float *device_ms) {
    if (!f) return MXB_ERR_ARG;
    DeviceGuard g(f->dv->device);
    int32_t rc = check_status(f->dv);
    if (device_ms && f->run_index) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, f->ev0, f->ev1) == cudaSuccess) *device_ms = ms;
        else cudaGetLastError();
    }
    return rc;
}

int32_t mxb_fanout_destroy(mxb_fanout *f) {
    if (!f) return MXB_OK;
    DeviceGuard g(f->dv->device);
    cudaStreamSynchronize(f->dv->stream);
    for (int c = 0; c < MXB_FANOUT_MAX_CHILDREN; ++c) {
        if (f->child_stream[c]) {
            cudaStreamSynchronize(f->child_stream[c]);
            cudaStreamDestroy(f->child_stream[c]);
        }
        if (f->child_done[c]) cudaEventDestroy(f->child_done[c]);
    }
    if (f->counters) cudaFree(f->counters);
    if (f->dev_tables) cudaFree(f->dev_tables);
    if (f->ev0) cudaEventDestroy(f->ev0);
    if (f->ev1) cudaEventDestroy(f->ev1);
    delete f;
    return MXB_OK;
}

}  // extern "C"
