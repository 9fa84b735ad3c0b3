// Library-owned device arena on CUDA virtual memory management.
//
// One reserved address range per arena; every allocation is one physical block
// (cuMemCreate, shareable as a POSIX file descriptor) mapped at the next free offset of the
// range.  Another process on the box imports the blocks at the same offsets of a range of its
// own, so a whole model's tensors cross the process boundary as one layout (an address is
// `their_base + offset`) instead of one IPC handle per allocation, and memory that torch
// allocates through the arena (the pluggable-allocator entry points at the end) stays
// exportable even where cudaIpcGetMemHandle refuses expandable segments.
// Follows the lifecycle of the reference's VmmArena (vmm/arena.py:155-350: reserve once, bump
// forward, one handle per malloc, free unmaps and releases that block, close releases the
// range); what the reference registers with its NIC once at the end of a load
// (arena.py:322-330) is here exported for NVLink peers.
//
// The driver's VMM calls are reached through cudaGetDriverEntryPoint, so the library still
// links the runtime only and loads on a machine without a driver.
#include <cuda.h>
#include <unistd.h>

#include <cstdio>
#include <map>
#include <vector>

#include "common.cuh"

namespace {

struct Driver {
    CUresult (*GetGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*AddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
    CUresult (*Export)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*Import)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType) = nullptr;
    bool ok = false;
};

template <typename F>
bool entry(const char *name, F *out) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
        cudaGetLastError();
        return false;
    }
    *out = reinterpret_cast<F>(fn);
    return true;
}

const Driver &driver() {
    static Driver d = [] {
        Driver x;
        x.ok = entry("cuMemGetAllocationGranularity", &x.GetGranularity) &&
               entry("cuMemAddressReserve", &x.AddressReserve) && entry("cuMemAddressFree", &x.AddressFree) &&
               entry("cuMemCreate", &x.Create) && entry("cuMemRelease", &x.Release) &&
               entry("cuMemMap", &x.Map) && entry("cuMemUnmap", &x.Unmap) &&
               entry("cuMemSetAccess", &x.SetAccess) &&
               entry("cuMemExportToShareableHandle", &x.Export) &&
               entry("cuMemImportFromShareableHandle", &x.Import);
        return x;
    }();
    return d;
}

CUmemAllocationProp block_prop(int dev) {
    CUmemAllocationProp p;
    memset(&p, 0, sizeof p);
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = dev;
    p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return p;
}

struct Block {
    uint64_t size = 0;
    CUmemGenericAllocationHandle handle = 0;
};

}  // namespace

struct mxb_arena {
    int dev = -1;           // device whose kernels use these addresses
    uint64_t base = 0;      // start of the reserved range
    uint64_t span = 0;      // bytes reserved
    uint64_t used = 0;      // bump offset (own arenas)
    uint64_t gran = 0;
    bool imported = false;  // blocks belong to another process
    std::map<uint64_t, Block> blocks;  // offset -> block
    std::mutex mu;
};

namespace {

std::mutex g_default_mu;
mxb_arena *g_default[64] = {};
std::vector<mxb_arena *> g_arenas;  // every live arena of the process (guarded by g_default_mu)

mxb_arena *arena_of(uint64_t ptr) {
    std::lock_guard<std::mutex> lk(g_default_mu);
    for (mxb_arena *a : g_arenas)
        if (ptr >= a->base && ptr < a->base + a->span) return a;
    return nullptr;
}

int32_t map_block(mxb_arena *a, uint64_t offset, uint64_t size, CUmemGenericAllocationHandle h) {
    const Driver &d = driver();
    if (d.Map((CUdeviceptr)(a->base + offset), size, 0, h, 0) != CUDA_SUCCESS) {
        mxb::set_error("cuMemMap failed at offset %llu", (unsigned long long)offset);
        return MXB_ERR_CUDA;
    }
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof acc);
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = a->dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (d.SetAccess((CUdeviceptr)(a->base + offset), size, &acc, 1) != CUDA_SUCCESS) {
        d.Unmap((CUdeviceptr)(a->base + offset), size);
        mxb::set_error("cuMemSetAccess failed for device %d (no peer access to the block's device?)", a->dev);
        return MXB_ERR_PEER;
    }
    return MXB_OK;
}

int32_t new_arena(int32_t dev, uint64_t span, bool imported, mxb_arena **out) {
    const Driver &d = driver();
    if (!d.ok) {
        mxb::set_error("the driver's virtual memory management entry points are unavailable");
        return MXB_ERR_CUDA;
    }
    mxb::DeviceGuard g(dev);
    if (!g.ok || cudaFree(nullptr) != cudaSuccess) {  // the device's primary context must exist
        cudaGetLastError();
        mxb::set_error("device %d cannot be selected", dev);
        return MXB_ERR_CUDA;
    }
    CUmemAllocationProp p = block_prop(dev);
    size_t gran = 0;
    if (d.GetGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || !gran) {
        mxb::set_error("cuMemGetAllocationGranularity failed");
        return MXB_ERR_CUDA;
    }
    span = (span + gran - 1) / gran * gran;
    CUdeviceptr base = 0;
    if (d.AddressReserve(&base, span, gran, 0, 0) != CUDA_SUCCESS) {
        mxb::set_error("cuMemAddressReserve of %llu bytes failed", (unsigned long long)span);
        return MXB_ERR_NOMEM;
    }
    mxb_arena *a = new mxb_arena();
    a->dev = dev;
    a->base = (uint64_t)base;
    a->span = span;
    a->gran = gran;
    a->imported = imported;
    {
        std::lock_guard<std::mutex> lk(g_default_mu);
        g_arenas.push_back(a);
    }
    *out = a;
    return MXB_OK;
}

}  // namespace

extern "C" {

int32_t mxb_arena_create(int32_t dev, uint64_t reserve_bytes, mxb_arena **out) {
    if (!out || !reserve_bytes || dev < 0 || dev >= 64) {
        mxb::set_error("mxb_arena_create: bad arguments");
        return MXB_ERR_ARG;
    }
    return new_arena(dev, reserve_bytes, false, out);
}

int32_t mxb_arena_malloc(mxb_arena *a, uint64_t nbytes, uint64_t *out_ptr) {
    if (!a || !out_ptr || !nbytes || a->imported) {
        mxb::set_error("mxb_arena_malloc: bad arguments (or an imported arena)");
        return MXB_ERR_ARG;
    }
    const Driver &d = driver();
    std::lock_guard<std::mutex> lk(a->mu);
    const uint64_t size = (nbytes + a->gran - 1) / a->gran * a->gran;
    if (a->used + size > a->span) {
        mxb::set_error("arena exhausted: %llu of %llu bytes used, %llu asked", (unsigned long long)a->used,
                       (unsigned long long)a->span, (unsigned long long)size);
        return MXB_ERR_NOMEM;
    }
    mxb::DeviceGuard g(a->dev);
    CUmemAllocationProp p = block_prop(a->dev);
    Block b;
    b.size = size;
    if (d.Create(&b.handle, size, &p, 0) != CUDA_SUCCESS) {
        mxb::set_error("cuMemCreate of %llu bytes failed", (unsigned long long)size);
        return MXB_ERR_NOMEM;
    }
    const int32_t rc = map_block(a, a->used, size, b.handle);
    if (rc != MXB_OK) {
        d.Release(b.handle);
        return rc;
    }
    a->blocks[a->used] = b;
    *out_ptr = a->base + a->used;
    a->used += size;  // offsets are never reused: an address names one block for the arena's life
    return MXB_OK;
}

int32_t mxb_arena_free(mxb_arena *a, uint64_t ptr) {
    if (!a || a->imported) return MXB_ERR_ARG;
    const Driver &d = driver();
    std::lock_guard<std::mutex> lk(a->mu);
    auto it = a->blocks.find(ptr - a->base);
    if (ptr < a->base || it == a->blocks.end()) {
        mxb::set_error("mxb_arena_free: %llx is not the start of a live block", (unsigned long long)ptr);
        return MXB_ERR_ARG;
    }
    mxb::DeviceGuard g(a->dev);
    d.Unmap((CUdeviceptr)ptr, it->second.size);
    d.Release(it->second.handle);
    a->blocks.erase(it);
    return MXB_OK;
}

int32_t mxb_arena_range(mxb_arena *a, uint64_t *base, uint64_t *used, uint64_t *span) {
    if (!a) return MXB_ERR_ARG;
    std::lock_guard<std::mutex> lk(a->mu);
    if (base) *base = a->base;
    if (used) *used = a->imported ? a->span : a->used;
    if (span) *span = a->span;
    return MXB_OK;
}

int32_t mxb_arena_blocks(mxb_arena *a, mxb_arena_block *out, uint64_t cap, uint64_t *n_out) {
    if (!a || !n_out || (!out && cap)) return MXB_ERR_ARG;
    std::lock_guard<std::mutex> lk(a->mu);
    uint64_t i = 0;
    for (const auto &kv : a->blocks) {
        if (i < cap) out[i] = {kv.first, kv.second.size};
        ++i;
    }
    *n_out = i;
    return i > cap ? MXB_ERR_NOMEM : MXB_OK;
}

int32_t mxb_arena_export_fd(mxb_arena *a, uint64_t offset, int32_t *fd_out) {
    if (!a || !fd_out || a->imported) return MXB_ERR_ARG;
    const Driver &d = driver();
    std::lock_guard<std::mutex> lk(a->mu);
    auto it = a->blocks.find(offset);
    if (it == a->blocks.end()) {
        mxb::set_error("mxb_arena_export_fd: no live block at offset %llu", (unsigned long long)offset);
        return MXB_ERR_ARG;
    }
    int fd = -1;
    if (d.Export(&fd, it->second.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS || fd < 0) {
        mxb::set_error("cuMemExportToShareableHandle failed");
        return MXB_ERR_PEER;
    }
    *fd_out = fd;
    return MXB_OK;
}

int32_t mxb_arena_import(int32_t dev, uint64_t span, const mxb_arena_block *blocks, const int32_t *fds,
                         uint64_t n, mxb_arena **out) {
    if (!out || !span || (!blocks && n) || (!fds && n) || dev < 0 || dev >= 64) {
        mxb::set_error("mxb_arena_import: bad arguments");
        return MXB_ERR_ARG;
    }
    mxb_arena *a = nullptr;
    int32_t rc = new_arena(dev, span, true, &a);
    if (rc != MXB_OK) return rc;
    const Driver &d = driver();
    mxb::DeviceGuard g(dev);
    for (uint64_t i = 0; i < n; ++i) {
        if (blocks[i].offset % a->gran || blocks[i].size % a->gran || blocks[i].offset + blocks[i].size > a->span) {
            mxb::set_error("mxb_arena_import: block %llu does not fit the range", (unsigned long long)i);
            rc = MXB_ERR_ARG;
            break;
        }
        CUmemGenericAllocationHandle h = 0;
        if (d.Import(&h, (void *)(uintptr_t)fds[i], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) {
            mxb::set_error("cuMemImportFromShareableHandle failed for block %llu", (unsigned long long)i);
            rc = MXB_ERR_PEER;
            break;
        }
        rc = map_block(a, blocks[i].offset, blocks[i].size, h);
        if (rc != MXB_OK) {
            d.Release(h);
            break;
        }
        a->blocks[blocks[i].offset] = {blocks[i].size, h};
    }
    if (rc != MXB_OK) {
        mxb_arena_destroy(a);
        return rc;
    }
    *out = a;
    return MXB_OK;
}

int32_t mxb_arena_destroy(mxb_arena *a) {
    if (!a) return MXB_OK;
    const Driver &d = driver();
    {
        std::lock_guard<std::mutex> lk(g_default_mu);
        for (auto &slot : g_default)
            if (slot == a) slot = nullptr;
        for (size_t i = 0; i < g_arenas.size(); ++i)
            if (g_arenas[i] == a) {
                g_arenas.erase(g_arenas.begin() + i);
                break;
            }
    }
    mxb::DeviceGuard g(a->dev);
    cudaDeviceSynchronize();
    for (auto &kv : a->blocks) {
        d.Unmap((CUdeviceptr)(a->base + kv.first), kv.second.size);
        d.Release(kv.second.handle);
    }
    d.AddressFree((CUdeviceptr)a->base, a->span);
    delete a;
    return MXB_OK;
}

int32_t mxb_arena_set_default(int32_t dev, mxb_arena *a) {
    if (dev < 0 || dev >= 64 || (a && (a->imported || a->dev != dev))) return MXB_ERR_ARG;
    std::lock_guard<std::mutex> lk(g_default_mu);
    g_default[dev] = a;
    return MXB_OK;
}

// torch.cuda.CUDAPluggableAllocator entry points: memory for `device` comes from the arena
// mxb_arena_set_default named for it (vmm/hook.py:82-109 routes torch's calls the same way).
void *mxb_arena_torch_malloc(ssize_t size, int device, void *) {
    mxb_arena *a = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_default_mu);
        if (device >= 0 && device < 64) a = g_default[device];
    }
    uint64_t p = 0;
    if (!a || size <= 0 || mxb_arena_malloc(a, (uint64_t)size, &p) != MXB_OK) {
        // the caller (torch's allocator) has no error channel but the null pointer: say why
        fprintf(stderr, "mxb arena: %zd bytes for device %d could not be allocated: %s\n", size, device,
                a ? mxb_last_error() : "no arena is set for the device");
        return nullptr;
    }
    return (void *)(uintptr_t)p;
}

void mxb_arena_torch_free(void *ptr, ssize_t, int, void *) {
    // the arena that owns the address, whichever is the default by now; a block whose arena is
    // gone went with it
    mxb_arena *a = ptr ? arena_of((uint64_t)(uintptr_t)ptr) : nullptr;
    if (a && !a->imported) mxb_arena_free(a, (uint64_t)(uintptr_t)ptr);
}

}  // extern "C"
