// Shared declarations of the mxb200 library (host side).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/mxb200.h"

namespace mxb {

void set_error(const char *fmt, ...);

#define MXB_CUDA(call)                                                                  \
    do {                                                                                \
        cudaError_t _e = (call);                                                        \
        if (_e != cudaSuccess) {                                                        \
            mxb::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e),      \
                           __FILE__, __LINE__);                                         \
            return MXB_ERR_CUDA;                                                        \
        }                                                                               \
    } while (0)

// Device-side status word values written by kernels whose waits ran out.
enum : uint32_t { DEV_OK = 0, DEV_TIMEOUT = 1 };

struct DeviceState {
    int device = -1;
    int sm_count = 0;
    cudaStream_t stream = nullptr;       // compute stream of the context
    cudaStream_t copy_stream = nullptr;  // copy-engine stream (H2D of ring slots)
    uint32_t *status = nullptr;          // device status word (one per device)
    uint32_t *status_host = nullptr;     // pinned mirror
    // scratch for descriptor tables, grown on demand
    void *table = nullptr;
    size_t table_bytes = 0;
    void *table_host = nullptr;  // pinned staging for the table upload
    size_t table_host_bytes = 0;
    uint64_t table_tag = 0;      // what the table holds: 0 = nothing reusable, else a digest span-list hash
    // scratch for digest accumulators
    void *digest = nullptr;
    size_t digest_bytes = 0;
    void *digest_host = nullptr;
    size_t digest_host_bytes = 0;
    cudaEvent_t events[16] = {};  // user timing events on `stream`
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;  // two-kernel scatter launches (stream <-> copy_stream)
    // serialises the entry points that share this device's scratch (tables, accumulators)
    std::unique_ptr<std::mutex> mu{new std::mutex()};
};

struct Extent {
    uint64_t base, end;
};

}  // namespace mxb

struct mxb_ctx {
    std::vector<mxb::DeviceState> devs;
    std::vector<mxb::Extent> extents;
    std::mutex mu;
    std::atomic<uint64_t> launches{0};

    mxb::DeviceState *find(int dev) {
        for (auto &d : devs)
            if (d.device == dev) return &d;
        return nullptr;
    }
};

namespace mxb {

// RAII device switch.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int32_t ensure_table(DeviceState *d, size_t bytes);
int32_t ensure_digest(DeviceState *d, size_t bytes);
int32_t check_status(DeviceState *d);

// Tiling of a descriptor table; shared by the scatter launcher and its tests.
constexpr uint64_t kTileBytes = 64 * 1024;
uint64_t tiles_of(const mxb_desc2d &d);

// A descriptor table cut into tiles, resident on the device.  The tiles of
// records that meet the bulk engine's rules come first, the rest after them.
struct ScatterTable {
    const mxb_desc2d *descs = nullptr;  // device
    const void *tiles = nullptr;        // device, Tile records: [bulk tiles | vector tiles]
    uint64_t n_bulk = 0, n_vec = 0;
    size_t bytes = 0;
};
size_t scatter_table_bytes(const mxb_desc2d *descs, uint64_t n, uint64_t *live_out,
                           uint64_t *tiles_out);
// Fill host_buf with the table image whose device copy will live at dev_buf.
// bulk_begin / vec_begin (n+1 entries each, optional) receive, per input record,
// its first tile in the bulk list and in the vector list.
// Records that touch another GPU's memory (as seen from `device`; -1 skips the check)
// always go to the vector list.
int32_t build_scatter_table(const mxb_desc2d *descs, uint64_t n, void *host_buf, void *dev_buf,
                            ScatterTable *out, uint64_t *bulk_begin, uint64_t *vec_begin,
                            int device);
// Launch the bulk engine over a range of the bulk list and the vector engine
// over a range of the vector list (MXB_SCATTER_VECTOR: vector engine for both).
int32_t launch_scatter_tiles(mxb_ctx *ctx, DeviceState *dv, const ScatterTable &tb,
                             uint64_t bulk_begin, uint64_t bulk_count, uint64_t vec_begin,
                             uint64_t vec_count, uint32_t flags, cudaStream_t stream);

// Launchers implemented in the kernel files.
int32_t launch_scatter(mxb_ctx *ctx, DeviceState *d, const mxb_desc2d *descs, uint64_t n,
                       uint32_t flags, cudaStream_t stream);
int32_t validate_descs(mxb_ctx *ctx, const mxb_desc2d *descs, uint64_t n);
// Whether every byte of the host range [lo, hi) lies in memory pinned by mxb_host_register.
bool host_range_pinned(uint64_t lo, uint64_t hi);

}  // namespace mxb
