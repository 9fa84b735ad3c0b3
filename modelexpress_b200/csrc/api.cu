// Context, memory, IPC and the host-side descriptor compiler of mxb200.
#include <chrono>
#include <thread>

#include "common.cuh"

namespace mxb {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int32_t ensure_table(DeviceState *d, size_t bytes) {
    if (bytes <= d->table_bytes) return MXB_OK;
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes + bytes / 2;
    MXB_CUDA(cudaStreamSynchronize(d->stream));
    if (d->table) cudaFree(d->table);
    if (d->table_host) cudaFreeHost(d->table_host);
    d->table = nullptr;
    d->table_host = nullptr;
    d->table_bytes = d->table_host_bytes = 0;
    d->table_tag = 0;
    MXB_CUDA(cudaMalloc(&d->table, want));
    MXB_CUDA(cudaHostAlloc(&d->table_host, want, cudaHostAllocDefault));
    d->table_bytes = d->table_host_bytes = want;
    return MXB_OK;
}

int32_t ensure_digest(DeviceState *d, size_t bytes) {
    if (bytes <= d->digest_bytes) return MXB_OK;
    size_t want = bytes < (1u << 16) ? (1u << 16) : bytes + bytes / 2;
    MXB_CUDA(cudaStreamSynchronize(d->stream));
    if (d->digest) cudaFree(d->digest);
    if (d->digest_host) cudaFreeHost(d->digest_host);
    d->digest = nullptr;
    d->digest_host = nullptr;
    d->digest_bytes = d->digest_host_bytes = 0;
    MXB_CUDA(cudaMalloc(&d->digest, want));
    MXB_CUDA(cudaHostAlloc(&d->digest_host, want, cudaHostAllocDefault));
    d->digest_bytes = d->digest_host_bytes = want;
    return MXB_OK;
}

int32_t check_status(DeviceState *d) {
    MXB_CUDA(cudaMemcpyAsync(d->status_host, d->status, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                             d->stream));
    MXB_CUDA(cudaStreamSynchronize(d->stream));
    if (*d->status_host == DEV_TIMEOUT) {
        uint32_t zero = 0;
        cudaMemcpyAsync(d->status, &zero, sizeof zero, cudaMemcpyHostToDevice, d->stream);
        cudaStreamSynchronize(d->stream);
        set_error("a device-side wait ran out on device %d", d->device);
        return MXB_ERR_TIMEOUT;
    }
    return MXB_OK;
}

// ---- pinned host ranges ---------------------------------------------------------------
// Process-wide (page-locked memory is a property of the process, not of a context): the
// ranges mxb_host_register pinned, disjoint and sorted by address.
namespace {
struct PinnedRange {
    uint64_t lo, hi;
};
std::mutex g_pin_mu;
std::vector<PinnedRange> g_pinned;
}  // namespace

bool host_range_pinned(uint64_t lo, uint64_t hi) {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    // ranges registered back to back count as one
    uint64_t need = lo;
    for (const PinnedRange &r : g_pinned) {
        if (r.hi <= need) continue;
        if (r.lo > need) return false;
        need = r.hi;
        if (need >= hi) return true;
    }
    return false;
}

uint64_t tiles_of(const mxb_desc2d &d) {
    if (d.rows == 0 || d.row_bytes == 0) return 0;
    if (d.row_bytes >= kTileBytes) return d.rows * ((d.row_bytes + kTileBytes - 1) / kTileBytes);
    uint64_t rows_per_tile = kTileBytes / d.row_bytes;
    return (d.rows + rows_per_tile - 1) / rows_per_tile;
}

int32_t validate_descs(mxb_ctx *ctx, const mxb_desc2d *descs, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) {
        const mxb_desc2d &d = descs[i];
        if (d.rows == 0 || d.row_bytes == 0) continue;
        if (d.src == 0 || d.dst == 0) {
            set_error("descriptor %llu has a null address", (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        if (d.rows > 1 && (d.src_pitch < d.row_bytes || d.dst_pitch < d.row_bytes)) {
            set_error("descriptor %llu: pitch smaller than row_bytes", (unsigned long long)i);
            return MXB_ERR_ARG;
        }
        if (!ctx->extents.empty()) {
            uint64_t lo = d.dst, hi = d.dst + (d.rows - 1) * d.dst_pitch + d.row_bytes;
            bool inside = false;
            for (const Extent &e : ctx->extents)
                if (lo >= e.base && hi <= e.end) {
                    inside = true;
                    break;
                }
            if (!inside) {
                set_error("descriptor %llu: destination [%llx, %llx) is outside the registered extents",
                          (unsigned long long)i, (unsigned long long)lo, (unsigned long long)hi);
                return MXB_ERR_BOUNDS;
            }
        }
    }
    return MXB_OK;
}

}  // namespace mxb

using namespace mxb;

extern "C" {

const char *mxb_last_error(void) { return g_err; }

int32_t mxb_version(void) { return 1; }

int32_t mxb_ctx_create(const int32_t *device_ids, int32_t n, mxb_ctx **out) {
    if (!device_ids || n <= 0 || !out) {
        set_error("mxb_ctx_create: bad arguments");
        return MXB_ERR_ARG;
    }
    int count = 0;
    MXB_CUDA(cudaGetDeviceCount(&count));
    for (int i = 0; i < n; ++i)
        if (device_ids[i] < 0 || device_ids[i] >= count) {
            set_error("mxb_ctx_create: device %d not present (%d devices)", device_ids[i], count);
            return MXB_ERR_ARG;
        }
    mxb_ctx *ctx = new mxb_ctx();
    ctx->devs.resize(n);
    int prev = 0;
    cudaGetDevice(&prev);
    int32_t rc = MXB_OK;
    for (int i = 0; i < n && rc == MXB_OK; ++i) {
        DeviceState &d = ctx->devs[i];
        d.device = device_ids[i];
        auto init = [&]() -> int32_t {
            MXB_CUDA(cudaSetDevice(d.device));
            cudaDeviceProp prop;
            MXB_CUDA(cudaGetDeviceProperties(&prop, d.device));
            if (prop.major != 10) {
                set_error("device %d is sm_%d%d; this library is built for sm_100a only", d.device,
                          prop.major, prop.minor);
                return MXB_ERR_CUDA;
            }
            d.sm_count = prop.multiProcessorCount;
            MXB_CUDA(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking));
            MXB_CUDA(cudaStreamCreateWithFlags(&d.copy_stream, cudaStreamNonBlocking));
            MXB_CUDA(cudaMalloc(&d.status, 256));
            MXB_CUDA(cudaMemset(d.status, 0, 256));
            MXB_CUDA(cudaHostAlloc(&d.status_host, 256, cudaHostAllocDefault));
            return MXB_OK;
        };
        rc = init();
    }
    // peer access between every pair of the context's devices
    for (int i = 0; i < n && rc == MXB_OK; ++i)
        for (int j = 0; j < n; ++j) {
            if (i == j) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, device_ids[i], device_ids[j]);
            if (!can) continue;
            cudaSetDevice(device_ids[i]);
            cudaError_t e = cudaDeviceEnablePeerAccess(device_ids[j], 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                set_error("cudaDeviceEnablePeerAccess(%d -> %d): %s", device_ids[i], device_ids[j],
                          cudaGetErrorString(e));
                rc = MXB_ERR_PEER;
            }
            cudaGetLastError();
        }
    cudaSetDevice(prev);
    if (rc != MXB_OK) {
        mxb_ctx_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return MXB_OK;
}

int32_t mxb_ctx_destroy(mxb_ctx *ctx) {
    if (!ctx) return MXB_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    for (DeviceState &d : ctx->devs) {
        if (d.device < 0) continue;
        cudaSetDevice(d.device);
        if (d.stream) cudaStreamSynchronize(d.stream);
        if (d.copy_stream) cudaStreamSynchronize(d.copy_stream);
        if (d.table) cudaFree(d.table);
        if (d.table_host) cudaFreeHost(d.table_host);
        if (d.digest) cudaFree(d.digest);
        if (d.digest_host) cudaFreeHost(d.digest_host);
        if (d.status) cudaFree(d.status);
        if (d.status_host) cudaFreeHost(d.status_host);
        for (cudaEvent_t e : d.events)
            if (e) cudaEventDestroy(e);
        if (d.fork_ev) cudaEventDestroy(d.fork_ev);
        if (d.join_ev) cudaEventDestroy(d.join_ev);
        if (d.stream) cudaStreamDestroy(d.stream);
        if (d.copy_stream) cudaStreamDestroy(d.copy_stream);
    }
    cudaSetDevice(prev);
    delete ctx;
    return MXB_OK;
}

int32_t mxb_sync(mxb_ctx *ctx, int32_t dev) {
    if (!ctx) return MXB_ERR_ARG;
    DeviceState *d = ctx->find(dev);
    if (!d) {
        set_error("device %d is not part of this context", dev);
        return MXB_ERR_ARG;
    }
    DeviceGuard g(dev);
    MXB_CUDA(cudaStreamSynchronize(d->copy_stream));
    return check_status(d);
}

int32_t mxb_event_record(mxb_ctx *ctx, int32_t dev, int32_t slot) {
    if (!ctx || slot < 0 || slot >= 16) return MXB_ERR_ARG;
    DeviceState *d = ctx->find(dev);
    if (!d) return MXB_ERR_ARG;
    DeviceGuard g(dev);
    if (!d->events[slot]) MXB_CUDA(cudaEventCreate(&d->events[slot]));
    MXB_CUDA(cudaEventRecord(d->events[slot], d->stream));
    return MXB_OK;
}

int32_t mxb_event_elapsed(mxb_ctx *ctx, int32_t dev, int32_t a, int32_t b, float *ms) {
    if (!ctx || !ms || a < 0 || a >= 16 || b < 0 || b >= 16) return MXB_ERR_ARG;
    DeviceState *d = ctx->find(dev);
    if (!d || !d->events[a] || !d->events[b]) {
        set_error("mxb_event_elapsed: event not recorded");
        return MXB_ERR_STATE;
    }
    DeviceGuard g(dev);
    MXB_CUDA(cudaEventSynchronize(d->events[b]));
    MXB_CUDA(cudaEventElapsedTime(ms, d->events[a], d->events[b]));
    return MXB_OK;
}

uint64_t mxb_launch_count(mxb_ctx *ctx) { return ctx ? ctx->launches.load() : 0; }

int32_t mxb_alloc(mxb_ctx *ctx, int32_t dev, uint64_t nbytes, uint64_t *out_ptr) {
    if (!ctx || !out_ptr || nbytes == 0) return MXB_ERR_ARG;
    if (!ctx->find(dev)) return MXB_ERR_ARG;
    DeviceGuard g(dev);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, nbytes);
    if (e != cudaSuccess) {
        set_error("cudaMalloc(%llu) on device %d: %s", (unsigned long long)nbytes, dev,
                  cudaGetErrorString(e));
        cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? MXB_ERR_NOMEM : MXB_ERR_CUDA;
    }
    *out_ptr = (uint64_t)(uintptr_t)p;
    return MXB_OK;
}

int32_t mxb_free(mxb_ctx *ctx, int32_t dev, uint64_t ptr) {
    if (!ctx || !ctx->find(dev)) return MXB_ERR_ARG;
    DeviceGuard g(dev);
    MXB_CUDA(cudaFree((void *)(uintptr_t)ptr));
    return MXB_OK;
}

int32_t mxb_host_alloc(uint64_t nbytes, uint64_t *out_ptr) {
    if (!out_ptr || nbytes == 0) return MXB_ERR_ARG;
    void *p = nullptr;
    MXB_CUDA(cudaHostAlloc(&p, nbytes, cudaHostAllocPortable));
    *out_ptr = (uint64_t)(uintptr_t)p;
    return MXB_OK;
}

int32_t mxb_host_free(uint64_t ptr) {
    MXB_CUDA(cudaFreeHost((void *)(uintptr_t)ptr));
    return MXB_OK;
}

int32_t mxb_host_register(uint64_t addr, uint64_t nbytes, uint64_t *out_base, uint64_t *out_bytes) {
    if (!addr || !nbytes) {
        set_error("mxb_host_register: empty range");
        return MXB_ERR_ARG;
    }
    const uint64_t page = 4096;
    const uint64_t lo = addr & ~(page - 1), hi = (addr + nbytes + page - 1) & ~(page - 1);
    {
        std::lock_guard<std::mutex> lk(g_pin_mu);
        for (const PinnedRange &r : g_pinned)
            if (lo < r.hi && r.lo < hi) {
                set_error("mxb_host_register: [%llx, %llx) overlaps the pinned range [%llx, %llx)",
                          (unsigned long long)lo, (unsigned long long)hi, (unsigned long long)r.lo,
                          (unsigned long long)r.hi);
                return MXB_ERR_STATE;
            }
    }
    // Page-locking a range that has never been touched through this mapping faults its pages
    // in one by one inside the driver call, several times slower than doing it up front on a
    // few threads: read one byte of every page first.
    const auto t_touch0 = std::chrono::steady_clock::now();
    {
        unsigned nt = std::thread::hardware_concurrency() / 2;
        nt = nt < 1 ? 1 : (nt > 8 ? 8 : nt);
        const uint64_t pages = (hi - lo) / page;
        if (pages < 4096) nt = 1;
        std::vector<std::thread> touch;
        for (unsigned t = 0; t < nt; ++t)
            touch.emplace_back([=]() {
                const uint64_t p0 = pages * t / nt, p1 = pages * (t + 1) / nt;
                const volatile char *base = reinterpret_cast<const volatile char *>((uintptr_t)lo);
                char sink = 0;
                for (uint64_t pg = p0; pg < p1; ++pg) sink += base[pg * page];
                (void)sink;
            });
        for (auto &th : touch) th.join();
    }
    // The device only ever reads these pages.  Saying so lets a private mapping of a file
    // that must not change be pinned without the kernel breaking copy-on-write page by page;
    // where the flag is refused the plain form is tried.
    const auto t_reg0 = std::chrono::steady_clock::now();
    cudaError_t e = cudaHostRegister((void *)(uintptr_t)lo, hi - lo,
                                     cudaHostRegisterPortable | cudaHostRegisterReadOnly);
    if (getenv("MXB_VERBOSE")) {
        const auto t_reg1 = std::chrono::steady_clock::now();
        fprintf(stderr, "[mxb200] cudaHostRegister(%llu bytes, portable|read-only): %s; touch %.1f ms, "
                        "register %.1f ms\n",
                (unsigned long long)(hi - lo), cudaGetErrorString(e),
                std::chrono::duration<double, std::milli>(t_reg0 - t_touch0).count(),
                std::chrono::duration<double, std::milli>(t_reg1 - t_reg0).count());
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        e = cudaHostRegister((void *)(uintptr_t)lo, hi - lo, cudaHostRegisterPortable);
    }
    if (e != cudaSuccess) {
        set_error("cudaHostRegister(%llx, %llu): %s (the range must be mapped readable and writable)",
                  (unsigned long long)lo, (unsigned long long)(hi - lo), cudaGetErrorString(e));
        cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? MXB_ERR_NOMEM : MXB_ERR_CUDA;
    }
    {
        std::lock_guard<std::mutex> lk(g_pin_mu);
        auto it = g_pinned.begin();
        while (it != g_pinned.end() && it->lo < lo) ++it;
        g_pinned.insert(it, {lo, hi});
    }
    if (out_base) *out_base = lo;
    if (out_bytes) *out_bytes = hi - lo;
    return MXB_OK;
}

int32_t mxb_host_unregister(uint64_t base) {
    {
        std::lock_guard<std::mutex> lk(g_pin_mu);
        auto it = g_pinned.begin();
        while (it != g_pinned.end() && it->lo != base) ++it;
        if (it == g_pinned.end()) {
            set_error("mxb_host_unregister: %llx is not the base of a pinned range",
                      (unsigned long long)base);
            return MXB_ERR_STATE;
        }
        g_pinned.erase(it);
    }
    MXB_CUDA(cudaHostUnregister((void *)(uintptr_t)base));
    return MXB_OK;
}

int32_t mxb_host_is_pinned(uint64_t addr, uint64_t nbytes) {
    if (!addr || !nbytes) return 0;
    return host_range_pinned(addr, addr + nbytes) ? 1 : 0;
}

int32_t mxb_register_extent(mxb_ctx *ctx, uint64_t base, uint64_t nbytes) {
    if (!ctx || base == 0 || nbytes == 0) return MXB_ERR_ARG;
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->extents.push_back({base, base + nbytes});
    return MXB_OK;
}

int32_t mxb_clear_extents(mxb_ctx *ctx) {
    if (!ctx) return MXB_ERR_ARG;
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->extents.clear();
    return MXB_OK;
}

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");

int32_t mxb_ipc_export(uint64_t ptr, uint8_t handle[64], uint64_t *offset) {
    if (!ptr || !handle || !offset) return MXB_ERR_ARG;
    // cudaIpcGetMemHandle names the whole allocation; find its base through
    // the driver-agnostic runtime query.
    cudaPointerAttributes attr;
    MXB_CUDA(cudaPointerGetAttributes(&attr, (void *)(uintptr_t)ptr));
    if (attr.type != cudaMemoryTypeDevice) {
        set_error("mxb_ipc_export: %llx is not device memory", (unsigned long long)ptr);
        return MXB_ERR_ARG;
    }
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, (void *)(uintptr_t)ptr);
    if (e != cudaSuccess) {
        set_error("cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return MXB_ERR_PEER;
    }
    memcpy(handle, &h, 64);
    // The handle names the whole allocation; the offset of ptr inside it comes
    // from the driver's range query, reached through the runtime so that the
    // library does not link the driver directly.
    typedef int (*range_fn)(unsigned long long *, size_t *, unsigned long long);
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn) {
        cudaGetLastError();
        set_error("cuMemGetAddressRange is unavailable");
        return MXB_ERR_PEER;
    }
    unsigned long long base = 0;
    size_t size = 0;
    if (((range_fn)fn)(&base, &size, (unsigned long long)ptr) != 0) {
        set_error("cuMemGetAddressRange failed for %llx", (unsigned long long)ptr);
        return MXB_ERR_PEER;
    }
    *offset = ptr - (uint64_t)base;
    return MXB_OK;
}

int32_t mxb_ipc_open(const uint8_t handle[64], uint64_t offset, uint64_t *out_ptr) {
    if (!handle || !out_ptr) return MXB_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        set_error("cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return MXB_ERR_PEER;
    }
    *out_ptr = (uint64_t)(uintptr_t)p + offset;
    return MXB_OK;
}

int32_t mxb_ipc_close(uint64_t ptr, uint64_t offset) {
    MXB_CUDA(cudaIpcCloseMemHandle((void *)(uintptr_t)(ptr - offset)));
    return MXB_OK;
}

int64_t mxb_coalesce_runs(const mxb_run *runs, uint64_t n, mxb_desc2d *out, uint64_t cap) {
    if ((!runs && n) || (!out && cap)) return MXB_ERR_ARG;
    uint64_t m = 0;
    uint64_t i = 0;
    while (i < n) {
        const mxb_run &r0 = runs[i];
        if (r0.nbytes == 0) {
            ++i;
            continue;
        }
        mxb_desc2d d{r0.src, r0.dst, 1, r0.nbytes, r0.nbytes, r0.nbytes};
        uint64_t j = i + 1;
        // skip empty runs when looking for the second row
        while (j < n && runs[j].nbytes == 0) ++j;
        if (j < n && runs[j].nbytes == r0.nbytes && runs[j].src > r0.src && runs[j].dst > r0.dst) {
            uint64_t sp = runs[j].src - r0.src, dp = runs[j].dst - r0.dst;
            if (sp >= r0.nbytes && dp >= r0.nbytes) {
                uint64_t rows = 2, k = j + 1;
                for (;;) {
                    while (k < n && runs[k].nbytes == 0) ++k;
                    if (k >= n) break;
                    if (runs[k].nbytes != r0.nbytes || runs[k].src != r0.src + rows * sp ||
                        runs[k].dst != r0.dst + rows * dp)
                        break;
                    ++rows;
                    ++k;
                }
                d.rows = rows;
                d.src_pitch = sp;
                d.dst_pitch = dp;
                j = k;
                // rows contiguous on both sides collapse to one long row
                if (sp == r0.nbytes && dp == r0.nbytes) {
                    d.row_bytes = rows * r0.nbytes;
                    d.rows = 1;
                    d.src_pitch = d.dst_pitch = d.row_bytes;
                }
            } else {
                j = i + 1;
            }
        } else {
            j = i + 1;
        }
        if (m < cap) out[m] = d;
        ++m;
        i = j;
    }
    if (m > cap) return -(int64_t)m;
    return (int64_t)m;
}

}  // extern "C"
