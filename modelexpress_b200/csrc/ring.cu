// Pinned staging ring: host checkpoint bytes -> HBM shards.
//
// mxb_place cuts the requested slices into chunks of one ring slot.  For every
// chunk the host threads gather exactly the bytes this rank keeps into the
// slot (densely packed, rows re-pitched so that the 16-byte vector path holds),
// the slot crosses PCIe once on the copy-engine stream, and one persistent
// scatter launch writes the shards from the device staging buffer.  Gathering
// chunk c+1 overlaps the copy of chunk c; the scatter of chunk c overlaps the
// copy of chunk c+1 (two device staging buffers).  In zero-copy mode the
// scatter kernel reads the pinned slot directly and the copy engine is idle.
#include <sys/mman.h>

#include <chrono>
#include <condition_variable>
#include <thread>

#include "common.cuh"

namespace mxb {

void stream_copy(void *dst, const void *src, size_t n);  // hostcopy.cpp
void stream_fence();

struct GatherOp {  // host memcpy work: rows of row_bytes from src (pitch) to slot offset
    const char *src;
    uint64_t slot_off;
    uint64_t rows, row_bytes, src_pitch, packed_pitch;
};

struct GatherPiece {
    const char *src;
    char *dst;
    uint64_t rows, row_bytes, src_pitch, dst_pitch;
};

struct Chunk {
    uint64_t op_begin = 0, op_end = 0;      // GatherOps
    uint64_t desc_begin = 0, desc_end = 0;  // scatter records
    uint64_t bytes = 0;                     // packed bytes used in the slot
};

// Minimal fork-join pool: run(pieces) executes them on the workers and the caller.
class GatherPool {
  public:
    explicit GatherPool(int threads) {
        for (int i = 1; i < threads; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~GatherPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    int size() const { return (int)workers_.size() + 1; }
    void run(const std::vector<GatherPiece> &pieces) {
        if (pieces.empty()) return;
        {
            std::lock_guard<std::mutex> lk(mu_);
            pieces_ = &pieces;
            next_.store(0);
            pending_ = (int)workers_.size();
            ++generation_;
        }
        cv_.notify_all();
        work();
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [this] { return pending_ == 0; });
        pieces_ = nullptr;
    }

  private:
    void work() {
        const std::vector<GatherPiece> &ps = *pieces_;
        for (;;) {
            size_t i = next_.fetch_add(1);
            if (i >= ps.size()) break;
            const GatherPiece &p = ps[i];
            if (p.src_pitch == p.row_bytes && p.dst_pitch == p.row_bytes) {
                stream_copy(p.dst, p.src, p.rows * p.row_bytes);
            } else {
                for (uint64_t r = 0; r < p.rows; ++r)
                    stream_copy(p.dst + r * p.dst_pitch, p.src + r * p.src_pitch, p.row_bytes);
            }
        }
        stream_fence();  // before the slot is handed to the copy engine / the kernel
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
            }
            work();
            {
                std::lock_guard<std::mutex> lk(mu_);
                --pending_;
            }
            done_cv_.notify_one();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    const std::vector<GatherPiece> *pieces_ = nullptr;
    std::atomic<size_t> next_{0};
    int pending_ = 0;
    uint64_t generation_ = 0;
    bool stop_ = false;
};

}  // namespace mxb

using namespace mxb;

struct mxb_ring {
    mxb_ctx *ctx = nullptr;
    DeviceState *dv = nullptr;
    uint64_t slot_bytes = 0;
    uint32_t slots = 0;
    char *host = nullptr;           // pinned, slots * slot_bytes
    void *host_map = nullptr;       // the mapping `host` lies in when it was pinned by registration
    size_t host_map_bytes = 0;
    char *staging[2] = {nullptr, nullptr};  // device
    std::vector<cudaEvent_t> slot_free;     // slot may be overwritten by the host
    cudaEvent_t stage_free[2] = {nullptr, nullptr};
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
    void *table_dev = nullptr, *table_host = nullptr;
    size_t table_bytes = 0;
    GatherPool *pool = nullptr;
    int pool_threads = 0;
};

namespace {

constexpr uint64_t kPackAlign = 256;
constexpr uint64_t kGatherPiece = 1ull << 20;  // bytes of host memcpy per work item

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Cut the items into chunks; emit gather ops and scatter records whose source
// is an offset into the slot (rebased per chunk by the caller).
int32_t plan_chunks(const mxb_desc2d *items, uint64_t n, uint64_t slot_bytes,
                    std::vector<Chunk> &chunks, std::vector<GatherOp> &ops,
                    std::vector<mxb_desc2d> &descs) {
    Chunk cur;
    uint64_t used = 0;
    auto close = [&]() {
        cur.op_end = ops.size();
        cur.desc_end = descs.size();
        cur.bytes = used;
        if (cur.op_end > cur.op_begin) chunks.push_back(cur);
        cur = Chunk();
        cur.op_begin = ops.size();
        cur.desc_begin = descs.size();
        used = 0;
    };
    for (uint64_t i = 0; i < n; ++i) {
        const mxb_desc2d &it = items[i];
        if (it.rows == 0 || it.row_bytes == 0) continue;
        // packed pitch keeps (packed row address - dst row address) constant mod 16
        uint64_t pp = it.row_bytes;
        if (it.rows > 1) pp = it.row_bytes + ((it.dst_pitch - it.row_bytes) & 15u);
        const bool row_fits_empty = (it.dst & 15u) + 15u + it.row_bytes <= slot_bytes;
        uint64_t row = 0, col = 0;  // progress inside the item
        while (row < it.rows) {
            // the packed copy starts at the same address phase (mod 16) as its destination
            const uint64_t phase = (it.dst + row * it.dst_pitch + col) & 15u;
            const uint64_t off = align_up(used, kPackAlign) + phase;
            const uint64_t room = off < slot_bytes ? slot_bytes - off : 0;
            if (col == 0 && row_fits_empty) {
                if (room < it.row_bytes) {  // the slot has data already: start a new chunk
                    close();
                    continue;
                }
                uint64_t fit = 1 + (room - it.row_bytes) / pp;
                uint64_t take = fit < it.rows - row ? fit : it.rows - row;
                ops.push_back({reinterpret_cast<const char *>(it.src) + row * it.src_pitch, off,
                               take, it.row_bytes, it.src_pitch, pp});
                descs.push_back({off, it.dst + row * it.dst_pitch, take, it.row_bytes, pp,
                                 it.dst_pitch});
                used = off + (take - 1) * pp + it.row_bytes;
                row += take;
            } else {
                // a row larger than a slot: split it by bytes into 256-byte multiples
                const uint64_t want = it.row_bytes - col;
                const uint64_t take = want <= room ? want : (room / kPackAlign) * kPackAlign;
                if (take == 0) {
                    close();
                    continue;
                }
                ops.push_back({reinterpret_cast<const char *>(it.src) + row * it.src_pitch + col,
                               off, 1, take, take, take});
                descs.push_back({off, it.dst + row * it.dst_pitch + col, 1, take, take, take});
                used = off + take;
                col += take;
                if (col == it.row_bytes) {
                    col = 0;
                    ++row;
                }
            }
            if (used + kPackAlign > slot_bytes) close();
        }
    }
    close();
    return MXB_OK;
}

}  // namespace

extern "C" {

int32_t mxb_ring_create(mxb_ctx *ctx, int32_t dev, uint64_t ring_bytes, uint32_t slots,
                        mxb_ring **out) {
    if (!ctx || !out || slots < 2 || ring_bytes / slots < (1u << 20)) {
        set_error("mxb_ring_create: need >= 2 slots of >= 1 MiB");
        return MXB_ERR_ARG;
    }
    DeviceState *dv = ctx->find(dev);
    if (!dv) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    DeviceGuard g(dev);
    mxb_ring *r = new mxb_ring();
    r->ctx = ctx;
    r->dv = dv;
    r->slots = slots;
    r->slot_bytes = (ring_bytes / slots) & ~uint64_t(4095);
    auto fail = [&](int32_t rc) {
        mxb_ring_destroy(r);
        return rc;
    };
    // Pinning sits inside a one-shot load's time to loaded weights.  cudaHostAlloc takes
    // 0.4-0.5 ms per MiB here; an anonymous mapping advised to use huge pages, touched by
    // several threads at once and then registered takes about a tenth of that and copies
    // to the device as fast.  MXB_RING_PIN=alloc selects cudaHostAlloc.
    const size_t ring_total = (size_t)r->slot_bytes * slots;
    const char *pin_mode = getenv("MXB_RING_PIN");
    if (!(pin_mode && !strcmp(pin_mode, "alloc"))) {
        const size_t huge = size_t(2) << 20;
        const size_t want = (ring_total + huge - 1) / huge * huge;
        void *map = mmap(nullptr, want + huge, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS,
                         -1, 0);
        if (map != MAP_FAILED) {
            char *base = reinterpret_cast<char *>(((uintptr_t)map + huge - 1) / huge * huge);
            madvise(base, want, MADV_HUGEPAGE);
            unsigned nt = std::thread::hardware_concurrency();
            nt = nt < 2 ? 2 : (nt > 16 ? 16 : nt);
            std::vector<std::thread> touch;
            for (unsigned t = 0; t < nt; ++t)
                touch.emplace_back([=]() {
                    const size_t lo = want / nt * t, hi = (t == nt - 1) ? want : want / nt * (t + 1);
                    for (size_t o = lo; o < hi; o += 4096) base[o] = 0;
                });
            for (auto &th : touch) th.join();
            if (cudaHostRegister(base, want, cudaHostRegisterPortable) == cudaSuccess) {
                r->host = base;
                r->host_map = map;
                r->host_map_bytes = want + huge;
            } else {
                cudaGetLastError();
                munmap(map, want + huge);
            }
        }
    }
    if (!r->host && cudaHostAlloc((void **)&r->host, ring_total, cudaHostAllocPortable) != cudaSuccess) {
        set_error("cudaHostAlloc(%llu) failed", (unsigned long long)ring_total);
        cudaGetLastError();
        return fail(MXB_ERR_NOMEM);
    }
    for (int i = 0; i < 2; ++i) {
        if (cudaMalloc((void **)&r->staging[i], r->slot_bytes) != cudaSuccess) {
            set_error("cudaMalloc(staging) failed");
            cudaGetLastError();
            return fail(MXB_ERR_NOMEM);
        }
        if (cudaEventCreateWithFlags(&r->stage_free[i], cudaEventDisableTiming) != cudaSuccess)
            return fail(MXB_ERR_CUDA);
    }
    r->slot_free.resize(slots, nullptr);
    for (uint32_t i = 0; i < slots; ++i)
        if (cudaEventCreateWithFlags(&r->slot_free[i], cudaEventDisableTiming) != cudaSuccess)
            return fail(MXB_ERR_CUDA);
    if (cudaEventCreate(&r->ev_begin) != cudaSuccess || cudaEventCreate(&r->ev_end) != cudaSuccess)
        return fail(MXB_ERR_CUDA);
    *out = r;
    return MXB_OK;
}

int32_t mxb_ring_destroy(mxb_ring *r) {
    if (!r) return MXB_OK;
    DeviceGuard g(r->dv->device);
    cudaStreamSynchronize(r->dv->stream);
    cudaStreamSynchronize(r->dv->copy_stream);
    delete r->pool;
    if (r->host_map) {
        cudaHostUnregister(r->host);
        munmap(r->host_map, r->host_map_bytes);
    } else if (r->host) {
        cudaFreeHost(r->host);
    }
    for (int i = 0; i < 2; ++i) {
        if (r->staging[i]) cudaFree(r->staging[i]);
        if (r->stage_free[i]) cudaEventDestroy(r->stage_free[i]);
    }
    for (cudaEvent_t e : r->slot_free)
        if (e) cudaEventDestroy(e);
    if (r->ev_begin) cudaEventDestroy(r->ev_begin);
    if (r->ev_end) cudaEventDestroy(r->ev_end);
    if (r->table_dev) cudaFree(r->table_dev);
    if (r->table_host) cudaFreeHost(r->table_host);
    delete r;
    return MXB_OK;
}

int32_t mxb_place(mxb_ring *r, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                  uint32_t mode, mxb_place_stats *stats) {
    using clk = std::chrono::steady_clock;
    if (!r || (!items && n) || mode > MXB_PLACE_ZERO_COPY) {
        set_error("mxb_place: bad arguments");
        return MXB_ERR_ARG;
    }
    const auto t0 = clk::now();
    // destinations are device addresses: check them like any scatter
    {
        int32_t rc = validate_descs(r->ctx, items, n);
        if (rc != MXB_OK) return rc;
    }
    DeviceState *dv = r->dv;
    DeviceGuard g(dv->device);
    std::lock_guard<std::mutex> lk(*dv->mu);
    if (host_threads < 1) host_threads = 1;
    if (!r->pool || r->pool_threads != host_threads) {
        delete r->pool;
        r->pool = new GatherPool(host_threads);
        r->pool_threads = host_threads;
    }

    std::vector<Chunk> chunks;
    std::vector<GatherOp> ops;
    std::vector<mxb_desc2d> descs;
    int32_t rc = plan_chunks(items, n, r->slot_bytes, chunks, ops, descs);
    if (rc != MXB_OK) return rc;
    const bool zero_copy = (mode == MXB_PLACE_ZERO_COPY);

    // rebase every record's source onto the buffer its chunk will be read from
    for (size_t c = 0; c < chunks.size(); ++c) {
        const char *base = zero_copy ? r->host + (c % r->slots) * r->slot_bytes
                                     : r->staging[c % 2];
        for (uint64_t i = chunks[c].desc_begin; i < chunks[c].desc_end; ++i)
            descs[i].src += (uint64_t)(uintptr_t)base;
    }
    // one table for all chunks, uploaded once
    const size_t tbytes = scatter_table_bytes(descs.data(), descs.size(), nullptr, nullptr);
    if (tbytes > r->table_bytes) {
        MXB_CUDA(cudaStreamSynchronize(dv->stream));
        if (r->table_dev) cudaFree(r->table_dev);
        if (r->table_host) cudaFreeHost(r->table_host);
        r->table_dev = r->table_host = nullptr;
        r->table_bytes = 0;
        size_t want = tbytes + tbytes / 2 + 4096;
        MXB_CUDA(cudaMalloc(&r->table_dev, want));
        MXB_CUDA(cudaHostAlloc(&r->table_host, want, cudaHostAllocDefault));
        r->table_bytes = want;
    }
    ScatterTable tb;
    std::vector<uint64_t> bulk_begin(descs.size() + 1, 0), vec_begin(descs.size() + 1, 0);
    if (!descs.empty()) {
        MXB_CUDA(cudaStreamSynchronize(dv->stream));
        rc = build_scatter_table(descs.data(), descs.size(), r->table_host, r->table_dev, &tb,
                                 bulk_begin.data(), vec_begin.data(), -1);
        if (rc != MXB_OK) return rc;
        MXB_CUDA(cudaMemcpyAsync(r->table_dev, r->table_host, tb.bytes, cudaMemcpyHostToDevice,
                                 dv->stream));
    }

    double gather_s = 0.0;
    uint64_t placed = 0, launches = 0;
    std::vector<GatherPiece> pieces;
    MXB_CUDA(cudaEventRecord(r->ev_begin, dv->stream));
    std::vector<bool> slot_used(r->slots, false);
    bool stage_used[2] = {false, false};
    for (size_t c = 0; c < chunks.size(); ++c) {
        const Chunk &ch = chunks[c];
        const uint32_t slot = (uint32_t)(c % r->slots);
        char *slot_base = r->host + (uint64_t)slot * r->slot_bytes;
        if (slot_used[slot]) MXB_CUDA(cudaEventSynchronize(r->slot_free[slot]));
        // gather
        const auto g0 = clk::now();
        pieces.clear();
        for (uint64_t i = ch.op_begin; i < ch.op_end; ++i) {
            const GatherOp &op = ops[i];
            placed += op.rows * op.row_bytes;
            uint64_t rows_per = op.row_bytes >= kGatherPiece ? 1 : kGatherPiece / op.row_bytes;
            for (uint64_t r0 = 0; r0 < op.rows; r0 += rows_per) {
                uint64_t take = rows_per < op.rows - r0 ? rows_per : op.rows - r0;
                if (take == 1 && op.row_bytes > kGatherPiece) {
                    for (uint64_t b = 0; b < op.row_bytes; b += kGatherPiece) {
                        uint64_t len = kGatherPiece < op.row_bytes - b ? kGatherPiece : op.row_bytes - b;
                        pieces.push_back({op.src + r0 * op.src_pitch + b,
                                          slot_base + op.slot_off + r0 * op.packed_pitch + b, 1, len,
                                          len, len});
                    }
                } else {
                    pieces.push_back({op.src + r0 * op.src_pitch,
                                      slot_base + op.slot_off + r0 * op.packed_pitch, take,
                                      op.row_bytes, op.src_pitch, op.packed_pitch});
                }
            }
        }
        r->pool->run(pieces);
        gather_s += std::chrono::duration<double>(clk::now() - g0).count();

        const uint64_t b0 = bulk_begin[ch.desc_begin], b1 = bulk_begin[ch.desc_end];
        const uint64_t v0 = vec_begin[ch.desc_begin], v1 = vec_begin[ch.desc_end];
        // the zero-copy source is pinned host memory: plain loads, not bulk copies
        const uint32_t eng = zero_copy ? MXB_SCATTER_VECTOR : MXB_SCATTER_DEFAULT;
        if (zero_copy) {
            rc = launch_scatter_tiles(r->ctx, dv, tb, b0, b1 - b0, v0, v1 - v0, eng, dv->stream);
            if (rc != MXB_OK) return rc;
            MXB_CUDA(cudaEventRecord(r->slot_free[slot], dv->stream));
        } else {
            const int st = (int)(c % 2);
            if (stage_used[st]) MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->stage_free[st], 0));
            if (c == 0) MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->ev_begin, 0));
            MXB_CUDA(cudaMemcpyAsync(r->staging[st], slot_base, ch.bytes, cudaMemcpyHostToDevice,
                                     dv->copy_stream));
            MXB_CUDA(cudaEventRecord(r->slot_free[slot], dv->copy_stream));
            MXB_CUDA(cudaStreamWaitEvent(dv->stream, r->slot_free[slot], 0));
            rc = launch_scatter_tiles(r->ctx, dv, tb, b0, b1 - b0, v0, v1 - v0, eng, dv->stream);
            if (rc != MXB_OK) return rc;
            MXB_CUDA(cudaEventRecord(r->stage_free[st], dv->stream));
            stage_used[st] = true;
        }
        slot_used[slot] = true;
        ++launches;
    }
    MXB_CUDA(cudaEventRecord(r->ev_end, dv->stream));
    rc = check_status(dv);
    if (rc != MXB_OK) return rc;
    if (stats) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r->ev_begin, r->ev_end);
        stats->bytes_placed = placed;
        stats->chunks = chunks.size();
        stats->launches = launches;
        stats->seconds_gather = gather_s;
        stats->seconds_device = ms * 1e-3;
        stats->seconds_total = std::chrono::duration<double>(clk::now() - t0).count();
    }
    return MXB_OK;
}

}  // extern "C"
