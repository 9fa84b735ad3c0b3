// Pinned staging ring: host checkpoint bytes -> HBM shards.
//
// mxb_place cuts the requested slices into chunks of one device staging buffer
// (densely packed, rows re-pitched so that the 16-byte vector path holds) and
// fills the two staging buffers alternately; one persistent scatter launch per
// chunk writes the shards while the other buffer is being filled.
//
// How a chunk is filled depends on where its source bytes live:
//   * sources inside memory pinned with mxb_host_register: the copy engine
//     gathers them straight from the source (one 1-D or 2-D cudaMemcpyAsync per
//     record); no host thread touches a byte;
//   * ordinary (pageable) host memory, e.g. a mapped checkpoint file: the chunk
//     is cut into units of a few MiB; each gather thread takes the next unit,
//     copies exactly the bytes this rank keeps into a pinned sub-slot of the
//     ring with streaming stores and sends that sub-slot over PCIe on its own
//     stream.  Threads never wait for one another, only for a sub-slot or a
//     staging buffer to come free.
#include <sys/mman.h>

#include <chrono>
#include <condition_variable>
#include <functional>
#include <thread>

#include "common.cuh"

namespace mxb {

void stream_copy(void *dst, const void *src, size_t n);  // hostcopy.cpp
void stream_fence();

struct GatherOp {  // rows of row_bytes from src (pitch) to an offset of the chunk's packed image
    const char *src;
    uint64_t slot_off;
    uint64_t rows, row_bytes, src_pitch, packed_pitch;
};

struct GatherPiece {  // a bounded amount of host copy work; dst_off is relative to the chunk
    const char *src;
    uint64_t dst_off;
    uint64_t rows, row_bytes, src_pitch, dst_pitch;
    uint64_t span() const { return (rows - 1) * dst_pitch + row_bytes; }
};

struct Chunk {
    uint64_t op_begin = 0, op_end = 0;      // GatherOps
    uint64_t desc_begin = 0, desc_end = 0;  // scatter records
    uint64_t bytes = 0;                     // packed bytes used in the staging buffer
    bool direct = false;                    // sources are pinned: the copy engine gathers
    uint64_t unit_begin = 0, unit_end = 0;  // Units (gathered chunks only)
};

struct Unit {  // one gather thread's job: a contiguous span of one chunk's packed image
    uint32_t chunk;
    uint64_t lo, hi;
    uint64_t piece_begin, piece_end;
};

// Persistent worker threads: start(fn) runs fn(worker index) on every worker, wait() joins the round.
class WorkerPool {
  public:
    explicit WorkerPool(int threads) {
        for (int i = 0; i < threads; ++i) workers_.emplace_back([this, i] { loop(i); });
    }
    ~WorkerPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    int size() const { return (int)workers_.size(); }
    void start(std::function<void(int)> fn) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = std::move(fn);
            pending_ = (int)workers_.size();
            ++generation_;
        }
        cv_.notify_all();
    }
    void wait() {
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [this] { return pending_ == 0; });
    }

  private:
    void loop(int index) {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
            }
            fn_(index);
            {
                std::lock_guard<std::mutex> lk(mu_);
                --pending_;
            }
            done_cv_.notify_all();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    std::function<void(int)> fn_;
    int pending_ = 0;
    uint64_t generation_ = 0;
    bool stop_ = false;
};

}  // namespace mxb

using namespace mxb;

struct mxb_ring {
    mxb_ctx *ctx = nullptr;
    DeviceState *dv = nullptr;
    uint64_t slot_bytes = 0;  // size of one device staging buffer (= one chunk)
    uint32_t slots = 0;
    char *host = nullptr;      // pinned, slots * slot_bytes, used as sub-slots of unit_bytes
    void *host_map = nullptr;  // the mapping `host` lies in when it was pinned by registration
    size_t host_map_bytes = 0;
    uint64_t unit_bytes = 0;
    uint32_t sub_slots = 0;
    char *staging[2] = {nullptr, nullptr};  // device
    std::vector<cudaEvent_t> sub_done;      // the copy out of a sub-slot has finished
    cudaEvent_t stage_free[2] = {nullptr, nullptr};
    cudaEvent_t dma_done[2] = {nullptr, nullptr};
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
    std::vector<cudaStream_t> streams;  // one copy stream per gather thread
    void *table_dev = nullptr, *table_host = nullptr;
    size_t table_bytes = 0;
    WorkerPool *pool = nullptr;
    int pool_threads = 0;
};

// A rank's slices kept in page-locked host memory exactly as they cross PCIe: the packed
// chunk images, one after the other.  Replaying it needs no host thread and no source file.
struct mxb_image {
    mxb_ring *ring = nullptr;
    char *host = nullptr;       // pinned
    void *host_map = nullptr;   // the mapping `host` lies in when it was pinned by registration
    size_t host_map_bytes = 0, host_bytes = 0;
    std::vector<Chunk> chunks;
    std::vector<uint64_t> chunk_off;   // byte offset of each chunk's image in `host`
    std::vector<mxb_desc2d> descs;     // sources already rebased onto the staging buffers
    std::vector<uint64_t> desc_item;   // which input item each record came from
    std::vector<uint64_t> desc_delta;  // record's destination minus its item's destination
    std::vector<mxb_desc2d> items;     // the items as last placed (geometry + destinations)
    std::vector<uint64_t> bulk_begin, vec_begin;
    void *table_dev = nullptr;
    std::vector<char> table_host;
    size_t table_cap = 0;
    ScatterTable tb;
    uint64_t bytes_placed = 0;
};

namespace {

constexpr uint64_t kPackAlign = 256;
constexpr uint64_t kGatherPiece = 1ull << 20;  // bytes of host memcpy per work item
constexpr uint64_t kUnitBytes = 4ull << 20;    // packed bytes one gather thread sends per copy

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Cut the items into chunks; emit gather ops and scatter records whose source
// is an offset into the chunk's packed image (rebased per chunk by the caller).
void plan_chunks(const mxb_desc2d *items, const std::vector<uint64_t> &which, uint64_t slot_bytes,
                 bool direct, std::vector<Chunk> &chunks, std::vector<GatherOp> &ops,
                 std::vector<mxb_desc2d> &descs, std::vector<uint64_t> *desc_item = nullptr) {
    Chunk cur;
    cur.direct = direct;
    cur.op_begin = ops.size();
    cur.desc_begin = descs.size();
    uint64_t used = 0;
    auto close = [&]() {
        cur.op_end = ops.size();
        cur.desc_end = descs.size();
        cur.bytes = used;
        if (cur.op_end > cur.op_begin) chunks.push_back(cur);
        cur = Chunk();
        cur.direct = direct;
        cur.op_begin = ops.size();
        cur.desc_begin = descs.size();
        used = 0;
    };
    for (uint64_t idx : which) {
        const mxb_desc2d &it = items[idx];
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
                if (room < it.row_bytes) {  // the chunk has data already: start a new one
                    close();
                    continue;
                }
                uint64_t fit = 1 + (room - it.row_bytes) / pp;
                uint64_t take = fit < it.rows - row ? fit : it.rows - row;
                ops.push_back({reinterpret_cast<const char *>(it.src) + row * it.src_pitch, off,
                               take, it.row_bytes, it.src_pitch, pp});
                descs.push_back({off, it.dst + row * it.dst_pitch, take, it.row_bytes, pp,
                                 it.dst_pitch});
                if (desc_item) desc_item->push_back(idx);
                used = off + (take - 1) * pp + it.row_bytes;
                row += take;
            } else {
                // a row larger than a chunk: split it by bytes into 256-byte multiples
                const uint64_t want = it.row_bytes - col;
                const uint64_t take = want <= room ? want : (room / kPackAlign) * kPackAlign;
                if (take == 0) {
                    close();
                    continue;
                }
                ops.push_back({reinterpret_cast<const char *>(it.src) + row * it.src_pitch + col,
                               off, 1, take, take, take});
                descs.push_back({off, it.dst + row * it.dst_pitch + col, 1, take, take, take});
                if (desc_item) desc_item->push_back(idx);
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
}

// Cut a gathered chunk's ops into pieces of about kGatherPiece bytes and group
// consecutive pieces into units whose packed span fits one sub-slot.
void plan_units(uint32_t chunk_index, Chunk &ch, const std::vector<GatherOp> &ops, uint64_t unit_bytes,
                std::vector<GatherPiece> &pieces, std::vector<Unit> &units) {
    ch.unit_begin = units.size();
    Unit cur{chunk_index, 0, 0, pieces.size(), pieces.size()};
    auto flush = [&]() {
        if (cur.piece_end > cur.piece_begin) units.push_back(cur);
        cur = Unit{chunk_index, 0, 0, pieces.size(), pieces.size()};
    };
    auto add = [&](const GatherPiece &p) {
        const uint64_t lo = p.dst_off & ~uint64_t(15), hi = p.dst_off + p.span();
        if (cur.piece_end > cur.piece_begin && hi - cur.lo > unit_bytes) flush();
        if (cur.piece_end == cur.piece_begin) cur.lo = lo;
        pieces.push_back(p);
        cur.piece_end = pieces.size();
        cur.hi = hi;
    };
    const uint64_t piece_cap = kGatherPiece < unit_bytes ? kGatherPiece : unit_bytes / 2;
    for (uint64_t i = ch.op_begin; i < ch.op_end; ++i) {
        const GatherOp &op = ops[i];
        if (op.row_bytes > piece_cap) {
            for (uint64_t r = 0; r < op.rows; ++r)
                for (uint64_t b = 0; b < op.row_bytes; b += piece_cap) {
                    const uint64_t len = piece_cap < op.row_bytes - b ? piece_cap : op.row_bytes - b;
                    add({op.src + r * op.src_pitch + b, op.slot_off + r * op.packed_pitch + b, 1, len,
                         len, len});
                }
        } else {
            uint64_t rows_per = piece_cap / op.packed_pitch;
            if (rows_per < 1) rows_per = 1;
            for (uint64_t r0 = 0; r0 < op.rows; r0 += rows_per) {
                const uint64_t take = rows_per < op.rows - r0 ? rows_per : op.rows - r0;
                add({op.src + r0 * op.src_pitch, op.slot_off + r0 * op.packed_pitch, take,
                     op.row_bytes, op.src_pitch, op.packed_pitch});
            }
        }
    }
    flush();
    ch.unit_end = units.size();
}

void gather_piece(const GatherPiece &p, char *dst) {
    if (p.src_pitch == p.row_bytes && p.dst_pitch == p.row_bytes) {
        stream_copy(dst, p.src, p.rows * p.row_bytes);
    } else {
        for (uint64_t r = 0; r < p.rows; ++r)
            stream_copy(dst + r * p.dst_pitch, p.src + r * p.src_pitch, p.row_bytes);
    }
}

// Page-locked host memory, the fast way: an anonymous mapping advised to use huge pages,
// touched by several threads at once and then registered is pinned several times faster
// than cudaHostAlloc pins the same amount, and copies to the device as fast.
// MXB_RING_PIN=alloc selects cudaHostAlloc.  *map_out is non-null when the memory must be
// released with cudaHostUnregister + munmap.
char *pinned_alloc(size_t bytes, void **map_out, size_t *map_bytes_out) {
    *map_out = nullptr;
    *map_bytes_out = 0;
    const char *pin_mode = getenv("MXB_RING_PIN");
    if (!(pin_mode && !strcmp(pin_mode, "alloc"))) {
        const size_t huge = size_t(2) << 20;
        const size_t want = (bytes + huge - 1) / huge * huge;
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
                *map_out = map;
                *map_bytes_out = want + huge;
                return base;
            }
            cudaGetLastError();
            munmap(map, want + huge);
        }
    }
    char *p = nullptr;
    if (cudaHostAlloc((void **)&p, bytes, cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void pinned_free(char *p, void *map, size_t map_bytes) {
    if (map) {
        cudaHostUnregister(p);
        munmap(map, map_bytes);
    } else if (p) {
        cudaFreeHost(p);
    }
}

// What the gather threads and the launching thread of one mxb_place call share.
struct PlaceShared {
    std::mutex mu;
    std::condition_variable cv;
    std::vector<uint8_t> issued;        // per unit: its copy has been queued
    std::vector<uint32_t> chunk_issued;  // per chunk: units queued so far
    uint64_t launched = 0;               // chunks whose scatter has been queued
    std::atomic<uint64_t> next_unit{0};
    std::atomic<int> error{MXB_OK};
    std::vector<double> busy;            // per thread: seconds spent copying
    char err_text[256] = "";
};

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
    // Pinning sits inside a one-shot load's time to loaded weights: see pinned_alloc.
    const size_t ring_total = (size_t)r->slot_bytes * slots;
    r->host = pinned_alloc(ring_total, &r->host_map, &r->host_map_bytes);
    if (!r->host) {
        set_error("pinning %llu bytes of host memory failed", (unsigned long long)ring_total);
        return fail(MXB_ERR_NOMEM);
    }
    // the pinned memory is handed out in sub-slots: one per copy a gather thread has in flight
    r->unit_bytes = kUnitBytes < r->slot_bytes ? kUnitBytes : r->slot_bytes;
    r->sub_slots = (uint32_t)(ring_total / r->unit_bytes);
    for (int i = 0; i < 2; ++i) {
        if (cudaMalloc((void **)&r->staging[i], r->slot_bytes) != cudaSuccess) {
            set_error("cudaMalloc(staging) failed");
            cudaGetLastError();
            return fail(MXB_ERR_NOMEM);
        }
        if (cudaEventCreateWithFlags(&r->stage_free[i], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&r->dma_done[i], cudaEventDisableTiming) != cudaSuccess)
            return fail(MXB_ERR_CUDA);
    }
    r->sub_done.resize(r->sub_slots, nullptr);
    for (uint32_t i = 0; i < r->sub_slots; ++i)
        if (cudaEventCreateWithFlags(&r->sub_done[i], cudaEventDisableTiming) != cudaSuccess)
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
    for (cudaStream_t st : r->streams)
        if (st) {
            cudaStreamSynchronize(st);
            cudaStreamDestroy(st);
        }
    pinned_free(r->host, r->host_map, r->host_map_bytes);
    for (int i = 0; i < 2; ++i) {
        if (r->staging[i]) cudaFree(r->staging[i]);
        if (r->stage_free[i]) cudaEventDestroy(r->stage_free[i]);
        if (r->dma_done[i]) cudaEventDestroy(r->dma_done[i]);
    }
    for (cudaEvent_t e : r->sub_done)
        if (e) cudaEventDestroy(e);
    if (r->ev_begin) cudaEventDestroy(r->ev_begin);
    if (r->ev_end) cudaEventDestroy(r->ev_end);
    if (r->table_dev) cudaFree(r->table_dev);
    if (r->table_host) cudaFreeHost(r->table_host);
    delete r;
    return MXB_OK;
}

}  // extern "C"

namespace {

void image_free(mxb_image *img) {
    if (!img) return;
    pinned_free(img->host, img->host_map, img->host_map_bytes);
    if (img->table_dev) cudaFree(img->table_dev);
    delete img;
}

// mxb_place, and with `retain` the first load of mxb_image_create: the same pipeline, except
// that every unit is gathered into its own place in a page-locked image that is kept.
int32_t place_impl(mxb_ring *r, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                   uint32_t mode, mxb_place_stats *stats, mxb_image **retain) {
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
    if (host_threads > 64) host_threads = 64;

    // ---- plan ---------------------------------------------------------------------------
    std::vector<uint64_t> pinned_items, paged_items;
    for (uint64_t i = 0; i < n; ++i) {
        const mxb_desc2d &it = items[i];
        if (it.rows == 0 || it.row_bytes == 0) continue;
        const uint64_t lo = it.src, hi = it.src + (it.rows - 1) * it.src_pitch + it.row_bytes;
        // a kept image holds every slice, wherever its source lives
        (!retain && host_range_pinned(lo, hi) ? pinned_items : paged_items).push_back(i);
    }
    const bool zero_copy = (mode == MXB_PLACE_ZERO_COPY) && !retain;
    std::vector<uint64_t> desc_item;
    std::vector<Chunk> chunks;
    std::vector<GatherOp> ops;
    std::vector<mxb_desc2d> descs;
    uint64_t direct_bytes = 0;
    for (uint64_t i : pinned_items) direct_bytes += items[i].rows * items[i].row_bytes;
    if (zero_copy) {
        // the kernel reads pinned sources where they lie: their records need no staging
        for (uint64_t i : pinned_items) descs.push_back(items[i]);
    } else {
        plan_chunks(items, pinned_items, r->slot_bytes, true, chunks, ops, descs);
    }
    const uint64_t zc_descs = zero_copy ? descs.size() : 0;
    plan_chunks(items, paged_items, r->slot_bytes, false, chunks, ops, descs, retain ? &desc_item : nullptr);
    std::vector<GatherPiece> pieces;
    std::vector<Unit> units;
    for (size_t c = 0; c < chunks.size(); ++c) {
        if (!chunks[c].direct) plan_units((uint32_t)c, chunks[c], ops, r->unit_bytes, pieces, units);
        // rebase every record's source onto the staging buffer its chunk goes through
        for (uint64_t i = chunks[c].desc_begin; i < chunks[c].desc_end; ++i)
            descs[i].src += (uint64_t)(uintptr_t)r->staging[c % 2];
    }
    mxb_image *img = nullptr;
    if (retain) {
        img = new mxb_image();
        img->ring = r;
        uint64_t total = 0;
        for (const Chunk &ch : chunks) {
            img->chunk_off.push_back(total);
            total += align_up(ch.bytes, 4096);
        }
        img->host_bytes = total ? total : 4096;
        img->host = pinned_alloc(img->host_bytes, &img->host_map, &img->host_map_bytes);
        if (!img->host) {
            set_error("pinning %llu bytes of host memory for the kept image failed",
                      (unsigned long long)img->host_bytes);
            image_free(img);
            return MXB_ERR_NOMEM;
        }
    }
    struct ImageGuard {  // an image that is not handed to the caller is released
        mxb_image *&img;
        bool keep = false;
        ~ImageGuard() {
            if (!keep && img) image_free(img);
        }
    } image_guard{img};
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
    int32_t rc = MXB_OK;
    if (!descs.empty()) {
        MXB_CUDA(cudaStreamSynchronize(dv->stream));
        rc = build_scatter_table(descs.data(), descs.size(), r->table_host, r->table_dev, &tb,
                                 bulk_begin.data(), vec_begin.data(), -1);
        if (rc != MXB_OK) return rc;
        MXB_CUDA(cudaMemcpyAsync(r->table_dev, r->table_host, tb.bytes, cudaMemcpyHostToDevice,
                                 dv->stream));
    }
    const bool gathering = !units.empty();
    if (gathering) {
        if (!r->pool || r->pool_threads != host_threads) {
            delete r->pool;
            r->pool = new WorkerPool(host_threads);
            r->pool_threads = host_threads;
        }
        while ((int)r->streams.size() < host_threads) {
            cudaStream_t st = nullptr;
            MXB_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
            r->streams.push_back(st);
        }
    }
    const double plan_s = std::chrono::duration<double>(clk::now() - t0).count();

    uint64_t placed = direct_bytes, launches = 0;
    for (const Unit &u : units)
        for (uint64_t p = u.piece_begin; p < u.piece_end; ++p)
            placed += pieces[p].rows * pieces[p].row_bytes;
    MXB_CUDA(cudaEventRecord(r->ev_begin, dv->stream));
    // every stream that writes a staging buffer starts behind whatever this ring's
    // earlier call still has in flight on the compute stream
    MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->ev_begin, 0));
    if (zero_copy && zc_descs) {
        rc = launch_scatter_tiles(r->ctx, dv, tb, bulk_begin[0], bulk_begin[zc_descs] - bulk_begin[0],
                                  vec_begin[0], vec_begin[zc_descs] - vec_begin[0], MXB_SCATTER_VECTOR,
                                  dv->stream);
        if (rc != MXB_OK) return rc;
        ++launches;
    }

    // ---- gather threads (pageable sources) ------------------------------------------------
    PlaceShared sh;
    sh.issued.assign(units.size(), 0);
    sh.chunk_issued.assign(chunks.size(), 0);
    sh.busy.assign(host_threads, 0.0);
    // a kept image gives every unit a place (and an event) of its own: no sub-slot is reused
    const uint32_t nsub = img ? (uint32_t)(units.size() ? units.size() : 1) : r->sub_slots;
    while (r->sub_done.size() < nsub) {
        cudaEvent_t e = nullptr;
        MXB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        r->sub_done.push_back(e);
    }
    if (gathering) {
        for (int t = 0; t < host_threads; ++t)
            MXB_CUDA(cudaStreamWaitEvent(r->streams[t], r->ev_begin, 0));
        const int device = dv->device;
        r->pool->start([&, device](int t) {
            cudaSetDevice(device);
            cudaStream_t st = r->streams[t];
            auto fail = [&](const char *what, cudaError_t e) {
                std::lock_guard<std::mutex> l(sh.mu);
                if (sh.error.load() == MXB_OK) {
                    snprintf(sh.err_text, sizeof sh.err_text, "%s: %s", what, cudaGetErrorString(e));
                    sh.error.store(MXB_ERR_CUDA);
                }
                sh.cv.notify_all();
            };
            for (;;) {
                const uint64_t u = sh.next_unit.fetch_add(1);
                if (u >= units.size() || sh.error.load() != MXB_OK) break;
                const Unit &un = units[u];
                const uint32_t sub = (uint32_t)(u % nsub);
                char *slot = img ? img->host + img->chunk_off[un.chunk] + un.lo
                                 : r->host + (uint64_t)sub * r->unit_bytes;
                if (u >= nsub) {  // the sub-slot's previous copy must have left it
                    {
                        std::unique_lock<std::mutex> l(sh.mu);
                        sh.cv.wait(l, [&] { return sh.issued[u - nsub] || sh.error.load() != MXB_OK; });
                    }
                    if (sh.error.load() != MXB_OK) break;
                    cudaError_t e = cudaEventSynchronize(r->sub_done[sub]);
                    if (e != cudaSuccess) {
                        fail("cudaEventSynchronize(sub-slot)", e);
                        break;
                    }
                }
                const auto g0 = clk::now();
                for (uint64_t p = un.piece_begin; p < un.piece_end; ++p)
                    gather_piece(pieces[p], slot + (pieces[p].dst_off - un.lo));
                stream_fence();  // before the sub-slot is handed to the copy engine
                sh.busy[t] += std::chrono::duration<double>(clk::now() - g0).count();
                const int stg = (int)(un.chunk % 2);
                if (un.chunk >= 2) {  // the scatter that last read this staging buffer must be queued
                    std::unique_lock<std::mutex> l(sh.mu);
                    sh.cv.wait(l, [&] { return sh.launched + 1 >= un.chunk || sh.error.load() != MXB_OK; });
                    if (sh.error.load() != MXB_OK) break;
                }
                cudaError_t e = cudaSuccess;
                if (un.chunk >= 2) e = cudaStreamWaitEvent(st, r->stage_free[stg], 0);
                if (e == cudaSuccess)
                    e = cudaMemcpyAsync(r->staging[stg] + un.lo, slot, un.hi - un.lo,
                                        cudaMemcpyHostToDevice, st);
                if (e == cudaSuccess) e = cudaEventRecord(r->sub_done[sub], st);
                if (e != cudaSuccess) {
                    fail("queueing a sub-slot copy", e);
                    break;
                }
                {
                    std::lock_guard<std::mutex> l(sh.mu);
                    sh.issued[u] = 1;
                    ++sh.chunk_issued[un.chunk];
                }
                sh.cv.notify_all();
            }
        });
    }

    // ---- the launching thread: one scatter per chunk -------------------------------------
    auto finish_workers = [&]() {
        if (gathering) r->pool->wait();
    };
    auto abort_with = [&](int32_t code) {
        {
            std::lock_guard<std::mutex> l(sh.mu);
            if (sh.error.load() == MXB_OK) sh.error.store(code);
        }
        sh.cv.notify_all();
        finish_workers();
        return code;
    };
#define MXB_PLACE_CUDA(call)                                                              \
    do {                                                                                  \
        cudaError_t _e = (call);                                                          \
        if (_e != cudaSuccess) {                                                          \
            set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), __FILE__,   \
                      __LINE__);                                                          \
            return abort_with(MXB_ERR_CUDA);                                              \
        }                                                                                 \
    } while (0)
    for (size_t c = 0; c < chunks.size(); ++c) {
        const Chunk &ch = chunks[c];
        const int stg = (int)(c % 2);
        if (ch.direct) {
            if (c >= 2) MXB_PLACE_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->stage_free[stg], 0));
            for (uint64_t i = ch.op_begin; i < ch.op_end; ++i) {
                const GatherOp &op = ops[i];
                char *dst = r->staging[stg] + op.slot_off;
                if (op.rows == 1 || (op.src_pitch == op.row_bytes && op.packed_pitch == op.row_bytes))
                    MXB_PLACE_CUDA(cudaMemcpyAsync(dst, op.src, op.rows * op.row_bytes,
                                                   cudaMemcpyHostToDevice, dv->copy_stream));
                else if (op.src_pitch < (1ull << 31))
                    MXB_PLACE_CUDA(cudaMemcpy2DAsync(dst, op.packed_pitch, op.src, op.src_pitch,
                                                     op.row_bytes, op.rows, cudaMemcpyHostToDevice,
                                                     dv->copy_stream));
                else  // a pitch the 2-D copy does not take: row by row
                    for (uint64_t row = 0; row < op.rows; ++row)
                        MXB_PLACE_CUDA(cudaMemcpyAsync(dst + row * op.packed_pitch,
                                                       op.src + row * op.src_pitch, op.row_bytes,
                                                       cudaMemcpyHostToDevice, dv->copy_stream));
            }
            MXB_PLACE_CUDA(cudaEventRecord(r->dma_done[stg], dv->copy_stream));
            MXB_PLACE_CUDA(cudaStreamWaitEvent(dv->stream, r->dma_done[stg], 0));
        } else {
            {
                std::unique_lock<std::mutex> l(sh.mu);
                sh.cv.wait(l, [&] {
                    return sh.chunk_issued[c] == ch.unit_end - ch.unit_begin || sh.error.load() != MXB_OK;
                });
            }
            if (sh.error.load() != MXB_OK) {
                set_error("%s", sh.err_text);
                return abort_with(sh.error.load());
            }
            // a sub-slot's event may already stand for a later copy out of the same sub-slot;
            // that copy was queued only after this chunk's had finished, so waiting on it is safe
            for (uint64_t u = ch.unit_begin; u < ch.unit_end; ++u)
                MXB_PLACE_CUDA(cudaStreamWaitEvent(dv->stream, r->sub_done[u % nsub], 0));
        }
        const uint64_t b0 = bulk_begin[ch.desc_begin], b1 = bulk_begin[ch.desc_end];
        const uint64_t v0 = vec_begin[ch.desc_begin], v1 = vec_begin[ch.desc_end];
        rc = launch_scatter_tiles(r->ctx, dv, tb, b0, b1 - b0, v0, v1 - v0, MXB_SCATTER_DEFAULT,
                                  dv->stream);
        if (rc != MXB_OK) return abort_with(rc);
        MXB_PLACE_CUDA(cudaEventRecord(r->stage_free[stg], dv->stream));
        {
            std::lock_guard<std::mutex> l(sh.mu);
            sh.launched = c + 1;
        }
        sh.cv.notify_all();
        ++launches;
    }
#undef MXB_PLACE_CUDA
    finish_workers();
    if (sh.error.load() != MXB_OK) {
        set_error("%s", sh.err_text);
        return sh.error.load();
    }
    MXB_CUDA(cudaEventRecord(r->ev_end, dv->stream));
    rc = check_status(dv);
    if (rc != MXB_OK) return rc;
    if (stats) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r->ev_begin, r->ev_end);
        double busiest = 0.0;
        for (double b : sh.busy) busiest = b > busiest ? b : busiest;
        stats->bytes_placed = placed;
        stats->chunks = chunks.size();
        stats->launches = launches;
        stats->seconds_gather = busiest;
        stats->seconds_device = ms * 1e-3;
        stats->seconds_total = std::chrono::duration<double>(clk::now() - t0).count();
        stats->bytes_direct = direct_bytes;
        stats->seconds_plan = plan_s;
    }
    if (img) {
        // keep what a replay needs: the chunk list, the records and a table of the image's own
        img->chunks = chunks;
        img->descs = descs;
        img->desc_item = desc_item;
        img->desc_delta.resize(descs.size());
        for (size_t i = 0; i < descs.size(); ++i) img->desc_delta[i] = descs[i].dst - items[desc_item[i]].dst;
        img->items.assign(items, items + n);
        img->bulk_begin = bulk_begin;
        img->vec_begin = vec_begin;
        img->bytes_placed = placed;
        if (tb.bytes) {
            img->table_cap = tb.bytes;
            img->table_host.assign(reinterpret_cast<char *>(r->table_host),
                                   reinterpret_cast<char *>(r->table_host) + tb.bytes);
            MXB_CUDA(cudaMalloc(&img->table_dev, tb.bytes));
            MXB_CUDA(cudaMemcpy(img->table_dev, r->table_dev, tb.bytes, cudaMemcpyDeviceToDevice));
            // same layout at another address: move the table's own pointers
            img->tb = tb;
            img->tb.descs = reinterpret_cast<const mxb_desc2d *>(img->table_dev);
            img->tb.tiles = reinterpret_cast<const char *>(img->table_dev) +
                            (reinterpret_cast<const char *>(tb.tiles) -
                             reinterpret_cast<const char *>(tb.descs));
        }
        image_guard.keep = true;
        *retain = img;
    }
    return MXB_OK;
}

}  // namespace

extern "C" {

int32_t mxb_place(mxb_ring *r, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                  uint32_t mode, mxb_place_stats *stats) {
    return place_impl(r, items, n, host_threads, mode, stats, nullptr);
}

int32_t mxb_image_create(mxb_ring *r, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                         mxb_image **out, mxb_place_stats *stats) {
    if (!out) {
        set_error("mxb_image_create: bad arguments");
        return MXB_ERR_ARG;
    }
    *out = nullptr;
    return place_impl(r, items, n, host_threads, MXB_PLACE_COPY_ENGINE, stats, out);
}

uint64_t mxb_image_bytes(mxb_image *img) { return img ? img->host_bytes : 0; }

int32_t mxb_image_destroy(mxb_image *img) {
    if (!img) return MXB_OK;
    DeviceState *dv = img->ring->dv;
    DeviceGuard g(dv->device);
    cudaStreamSynchronize(dv->stream);
    cudaStreamSynchronize(dv->copy_stream);
    image_free(img);
    return MXB_OK;
}

int32_t mxb_image_place(mxb_image *img, const mxb_desc2d *items, uint64_t n, mxb_place_stats *stats) {
    using clk = std::chrono::steady_clock;
    if (!img || (items && n != img->items.size())) {
        set_error("mxb_image_place: bad arguments (the image holds %llu slices)",
                  (unsigned long long)(img ? img->items.size() : 0));
        return MXB_ERR_ARG;
    }
    const auto t0 = clk::now();
    mxb_ring *r = img->ring;
    DeviceState *dv = r->dv;
    DeviceGuard g(dv->device);
    std::lock_guard<std::mutex> lk(*dv->mu);
    double plan_s = 0.0;
    if (items) {
        // new destinations: same slices, same packing (which follows the destination's address
        // phase and pitch), so only the records' destination addresses move
        bool moved = false;
        for (uint64_t i = 0; i < n; ++i) {
            const mxb_desc2d &a = items[i], &b = img->items[i];
            if (a.rows != b.rows || a.row_bytes != b.row_bytes || a.dst_pitch != b.dst_pitch ||
                ((a.dst ^ b.dst) & 15u) || (a.rows && a.row_bytes && !a.dst)) {
                set_error("mxb_image_place: slice %llu differs from the one the image was made for "
                          "(geometry or 16-byte phase of the destination); make a new image",
                          (unsigned long long)i);
                return MXB_ERR_STATE;
            }
            moved |= a.dst != b.dst;
        }
        if (moved) {
            int32_t rc = validate_descs(r->ctx, items, n);
            if (rc != MXB_OK) return rc;
            const size_t desc_bytes = img->descs.size() * sizeof(mxb_desc2d);
            mxb_desc2d *hd = reinterpret_cast<mxb_desc2d *>(img->table_host.data());
            // the table holds the live records in order; empty ones were never emitted
            for (size_t i = 0; i < img->descs.size(); ++i) {
                img->descs[i].dst = items[img->desc_item[i]].dst + img->desc_delta[i];
                hd[i].dst = img->descs[i].dst;
            }
            for (uint64_t i = 0; i < n; ++i) img->items[i].dst = items[i].dst;
            MXB_CUDA(cudaMemcpyAsync(img->table_dev, img->table_host.data(), desc_bytes,
                                     cudaMemcpyHostToDevice, dv->stream));
            MXB_CUDA(cudaStreamSynchronize(dv->stream));  // table_host may change again next call
        }
        plan_s = std::chrono::duration<double>(clk::now() - t0).count();
    }
    uint64_t launches = 0;
    MXB_CUDA(cudaEventRecord(r->ev_begin, dv->stream));
    MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->ev_begin, 0));
    for (size_t c = 0; c < img->chunks.size(); ++c) {
        const Chunk &ch = img->chunks[c];
        const int stg = (int)(c % 2);
        if (c >= 2) MXB_CUDA(cudaStreamWaitEvent(dv->copy_stream, r->stage_free[stg], 0));
        MXB_CUDA(cudaMemcpyAsync(r->staging[stg], img->host + img->chunk_off[c], ch.bytes,
                                 cudaMemcpyHostToDevice, dv->copy_stream));
        MXB_CUDA(cudaEventRecord(r->dma_done[stg], dv->copy_stream));
        MXB_CUDA(cudaStreamWaitEvent(dv->stream, r->dma_done[stg], 0));
        const uint64_t b0 = img->bulk_begin[ch.desc_begin], b1 = img->bulk_begin[ch.desc_end];
        const uint64_t v0 = img->vec_begin[ch.desc_begin], v1 = img->vec_begin[ch.desc_end];
        int32_t rc = launch_scatter_tiles(r->ctx, dv, img->tb, b0, b1 - b0, v0, v1 - v0,
                                          MXB_SCATTER_DEFAULT, dv->stream);
        if (rc != MXB_OK) return rc;
        MXB_CUDA(cudaEventRecord(r->stage_free[stg], dv->stream));
        ++launches;
    }
    MXB_CUDA(cudaEventRecord(r->ev_end, dv->stream));
    int32_t rc = check_status(dv);
    if (rc != MXB_OK) return rc;
    if (stats) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r->ev_begin, r->ev_end);
        stats->bytes_placed = img->bytes_placed;
        stats->chunks = img->chunks.size();
        stats->launches = launches;
        stats->seconds_gather = 0.0;
        stats->seconds_device = ms * 1e-3;
        stats->seconds_total = std::chrono::duration<double>(clk::now() - t0).count();
        stats->bytes_direct = img->bytes_placed;
        stats->seconds_plan = plan_s;
    }
    return MXB_OK;
}

}  // extern "C"
