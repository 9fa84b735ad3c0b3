/*
 * mxb200 — C ABI of the B200 weight-placement data plane.
 *
 * Plain C: pointers and sizes only, no C++ or framework types.  Every device
 * address is a 64-bit integer valid in the calling process (a cudaMalloc'ed
 * pointer, a peer pointer opened with mxb_ipc_open, or pinned host memory).
 * All functions return an int32 status (MXB_OK or a negative MXB_ERR_*) unless
 * stated otherwise; mxb_last_error() gives the text of the last failure on the
 * calling thread.  Kernels and copies run on streams the context owns; work
 * the caller queued on its own streams for the same buffers must have
 * completed before a call, and a call that waits (everything except the
 * NO_SYNC / launch forms) returns with its results visible to any stream.
 * Nothing here falls back to the CPU: without a usable CUDA
 * device the compute entry points return MXB_ERR_CUDA.
 *
 * Each entry point cites the reference interface it stands in for, by path
 * inside the reference project (modelexpress_client/python/modelexpress/...).
 */
#ifndef MXB200_H
#define MXB200_H

#include <stddef.h>
#include <stdint.h>
#include <sys/types.h> /* ssize_t: the torch allocator entry points */

#ifdef __cplusplus
extern "C" {
#endif

#define MXB_OK 0
#define MXB_ERR_ARG (-1)     /* null pointer, zero size where one is needed, bad enum */
#define MXB_ERR_BOUNDS (-2)  /* a descriptor leaves the registered extents */
#define MXB_ERR_ALIGN (-3)   /* an address breaks an alignment the call requires */
#define MXB_ERR_CUDA (-4)    /* a CUDA runtime call failed; see mxb_last_error */
#define MXB_ERR_TIMEOUT (-5) /* a bounded device- or host-side wait ran out */
#define MXB_ERR_PEER (-6)    /* peer access / IPC mapping unavailable */
#define MXB_ERR_NOMEM (-7)
#define MXB_ERR_STATE (-8)   /* object used in the wrong state */
#define MXB_ERR_UNSUPPORTED (-9) /* geometry that is not a permuted box of its source
                                    (UnsupportedReshard, refit/reshard/types.py:21-24) */

typedef struct mxb_ctx mxb_ctx;
typedef struct mxb_ring mxb_ring;
typedef struct mxb_fanout mxb_fanout;
typedef struct mxb_table mxb_table;
typedef struct mxb_image mxb_image;

/* One contiguous byte run.  Mirrors ReadDescriptor(session, src_addr, dst_addr,
 * nbytes) of refit/reshard/transport/base.py:26-35 with the session resolved
 * to an address the caller can reach. */
typedef struct {
    uint64_t src;
    uint64_t dst;
    uint64_t nbytes;
} mxb_run;

/* One strided slice: `rows` runs of `row_bytes`, row r at src + r*src_pitch ->
 * dst + r*dst_pitch.  This is the closed form of the run list that
 * refit/reshard/slice_plan.py:259-294 (paired_runs) emits for one TP slice:
 * a row-parallel shard is one record instead of thousands of runs. */
typedef struct {
    uint64_t src;
    uint64_t dst;
    uint64_t rows;
    uint64_t row_bytes;
    uint64_t src_pitch;
    uint64_t dst_pitch;
} mxb_desc2d;

/* One byte range to digest. */
typedef struct {
    uint64_t ptr;
    uint64_t nbytes;
} mxb_span;

/* Per-span digest record written by mxb_digest. */
typedef struct {
    uint64_t nbytes;
    uint64_t row_sum;        /* sum of 4 KiB row sums (signed int32 words), mod 2^64 */
    uint64_t row_sum_w;      /* sum of row sums * (1-based row index) */
    uint64_t tail_sum;       /* words after the last whole row */
    uint64_t tail_sum_w;     /* ... weighted by 1-based word index */
    uint64_t ragged_sum;     /* bytes after the last whole word */
    uint64_t block_hash;     /* 64-bit block hash (MXB_DIGEST_BLOCK64) */
    uint32_t safe_checksum;  /* 32-bit position-weighted byte sum */
    uint32_t reserved;
} mxb_digest_out;

#define MXB_DIGEST_SAFE32 1u  /* tensor_utils.py:27-44 safe_checksum */
#define MXB_DIGEST_ROWS 2u    /* refit/reshard/verify.py:113-150 scalars of tensor_digest */
#define MXB_DIGEST_BLOCK64 4u /* 64-bit hash over 4 KiB blocks; no reference counterpart */

/* ---- context ----------------------------------------------------------- */

/* Create a context over `n` CUDA devices of this process and enable peer
 * access between every pair that supports it.  Replaces the per-worker agent
 * set-up of nixl_transfer.py:194-254 (NixlTransferManager.initialize). */
int32_t mxb_ctx_create(const int32_t *device_ids, int32_t n, mxb_ctx **out);
int32_t mxb_ctx_destroy(mxb_ctx *ctx);
/* Text of the last error raised on this thread ("" if none). */
const char *mxb_last_error(void);
/* ABI version of the loaded library. */
int32_t mxb_version(void);
/* Block the host until all work queued by this context on `dev` is done;
 * returns MXB_ERR_TIMEOUT if a kernel reported a wait that ran out. */
int32_t mxb_sync(mxb_ctx *ctx, int32_t dev);
/* Number of this library's kernels launched since the context was created. */
uint64_t mxb_launch_count(mxb_ctx *ctx);

/* Device memory owned by the library (plain cudaMalloc, so it can be exported
 * over CUDA IPC).  Replaces refit/reshard/cuda_pool.py:52-108. */
int32_t mxb_alloc(mxb_ctx *ctx, int32_t dev, uint64_t nbytes, uint64_t *out_ptr);
int32_t mxb_free(mxb_ctx *ctx, int32_t dev, uint64_t ptr);
/* Pinned host memory. */
int32_t mxb_host_alloc(uint64_t nbytes, uint64_t *out_ptr);
int32_t mxb_host_free(uint64_t ptr);
/* Pin host memory the caller already has (typically a mapped checkpoint file
 * that stays in host memory between loads) so that the copy engine and the
 * kernels can read it in place; mxb_place then moves slices of it with no host
 * copy at all.  The range is widened to page boundaries; the widened range is
 * returned and must be mapped readable AND writable (a private mapping of a
 * read-only file qualifies; the device only reads it).  Pinning costs host time
 * in proportion to the size, so it pays when the same bytes are loaded more
 * than once (several replicas or refits from one host image).  Process-wide;
 * ranges must not overlap.  Replaces the registration step the reference does
 * for its transfer buffers (nixl_transfer.py:302-585, gds_transfer.py:60-99). */
int32_t mxb_host_register(uint64_t addr, uint64_t nbytes, uint64_t *out_base, uint64_t *out_bytes);
/* `base` as returned by mxb_host_register.  No copy from the range may be in flight. */
int32_t mxb_host_unregister(uint64_t base);
/* 1 if every byte of [addr, addr + nbytes) is pinned by mxb_host_register, else 0. */
int32_t mxb_host_is_pinned(uint64_t addr, uint64_t nbytes);

/* Extents the scatter entry points check destinations (and device sources)
 * against; with none registered only structural checks run.  Replaces the
 * registration step of nixl_transfer.py:302-585. */
int32_t mxb_register_extent(mxb_ctx *ctx, uint64_t base, uint64_t nbytes);
int32_t mxb_clear_extents(mxb_ctx *ctx);

/* Cross-process peer mapping (one OS process per GPU rank).  `handle` is 64
 * opaque bytes; `offset` is ptr's distance from its allocation base.
 * Replaces the metadata exchange of nixl_transfer.py:680-712. */
int32_t mxb_ipc_export(uint64_t ptr, uint8_t handle[64], uint64_t *offset);
int32_t mxb_ipc_open(const uint8_t handle[64], uint64_t offset, uint64_t *out_ptr);
int32_t mxb_ipc_close(uint64_t ptr, uint64_t offset);

/* ---- device arena on CUDA virtual memory management --------------------- */

/* One reserved address range per arena; every allocation is one physical block
 * mapped at the next free offset (never reused).  Another process on the box
 * imports the blocks at the same offsets of a range of its own, so that an
 * address there is `its base + the same offset`: a whole model crosses the
 * process boundary as one layout instead of one IPC handle per allocation.
 * Lifecycle and names follow the reference's VmmArena (vmm/arena.py:155-350;
 * backend calls vmm/backend.py); what the reference registers with its NIC
 * once per load (arena.py:322-330, `registered_range`) is here exported to
 * NVLink peers.  Process-wide, no context needed. */
typedef struct mxb_arena mxb_arena;
typedef struct {
    uint64_t offset; /* from the arena's base; a multiple of the granularity */
    uint64_t size;   /* a multiple of the granularity */
} mxb_arena_block;

/* Reserve `reserve_bytes` of address space for device `dev` (no memory yet). */
int32_t mxb_arena_create(int32_t dev, uint64_t reserve_bytes, mxb_arena **out);
/* One new block of at least `nbytes` (rounded up to the granularity), mapped
 * read/write for the arena's device.  MXB_ERR_NOMEM when the range or the
 * device is exhausted. */
int32_t mxb_arena_malloc(mxb_arena *a, uint64_t nbytes, uint64_t *out_ptr);
/* `ptr` as returned by mxb_arena_malloc: unmaps and releases that block. */
int32_t mxb_arena_free(mxb_arena *a, uint64_t ptr);
/* Base address, bytes bumped through so far and bytes reserved. */
int32_t mxb_arena_range(mxb_arena *a, uint64_t *base, uint64_t *used, uint64_t *span);
/* The live blocks in address order; *n_out = how many there are
 * (MXB_ERR_NOMEM if `cap` is smaller). */
int32_t mxb_arena_blocks(mxb_arena *a, mxb_arena_block *out, uint64_t cap, uint64_t *n_out);
/* A POSIX file descriptor naming the block at `offset` (send it over a unix
 * socket with SCM_RIGHTS; the caller closes its copy). */
int32_t mxb_arena_export_fd(mxb_arena *a, uint64_t offset, int32_t *fd_out);
/* Map another process's blocks (descriptors received from it) at the same
 * offsets of a fresh range of `span` bytes, read/write for device `dev`
 * (MXB_ERR_PEER if `dev` has no peer access to the blocks' device).  The
 * result answers mxb_arena_range / mxb_arena_blocks / mxb_arena_destroy only. */
int32_t mxb_arena_import(int32_t dev, uint64_t span, const mxb_arena_block *blocks, const int32_t *fds,
                         uint64_t n, mxb_arena **out);
/* Unmaps and releases every block and the range.  No tensor or kernel may
 * still use the addresses. */
int32_t mxb_arena_destroy(mxb_arena *a);
/* Entry points for torch.cuda.CUDAPluggableAllocator(path, "mxb_arena_torch_malloc",
 * "mxb_arena_torch_free"): memory for a device comes from the arena that
 * mxb_arena_set_default named for it (NULL: none; allocations then fail), as
 * vmm/hook.py:82-109 routes torch's calls into the reference's arena. */
int32_t mxb_arena_set_default(int32_t dev, mxb_arena *a);
void *mxb_arena_torch_malloc(ssize_t size, int device, void *stream);
void mxb_arena_torch_free(void *ptr, ssize_t size, int device, void *stream);

/* ---- descriptor compiler (host) ---------------------------------------- */

#define MXB_MAX_DIMS 8

/* A strided window of a row-major source tensor and where it lands: what a
 * loader's chain of view ops (narrow, slicing, transpose, permute, select)
 * leaves of a checkpoint tensor, i.e. RecordedCopy after its op-chain has been
 * replayed (refit/reshard/types.py:57-70, slice_plan.py:136-168).  Offsets,
 * shapes and strides are in elements. */
typedef struct {
    int32_t ndim_src;                    /* rank of the full source tensor */
    int32_t ndim_win;                    /* rank of the window = rank of the destination view */
    int32_t keep_rank;                   /* 1: the window must have the source's rank (the
                                            reference's rule); 0: size-1 window dims are ignored
                                            and source dims the window does not walk have extent 1 */
    uint32_t elsize;                     /* bytes per element */
    int64_t global_shape[MXB_MAX_DIMS];  /* shape of the full source tensor */
    int64_t win_offset;                  /* first element of the window in the full tensor */
    int64_t win_shape[MXB_MAX_DIMS];
    int64_t win_stride[MXB_MAX_DIMS];    /* in elements of the full tensor */
    int64_t dst_offset;                  /* element offset from the destination base */
    int64_t dst_stride[MXB_MAX_DIMS];    /* destination stride of each window dim */
} mxb_window;

/* One published shard: a box of the full tensor held contiguously (row-major)
 * at `addr` (Shard, refit/reshard/slice_plan.py:54-70). */
typedef struct {
    int32_t ndim;
    int32_t reserved;
    int64_t offset[MXB_MAX_DIMS];
    int64_t shape[MXB_MAX_DIMS];
    uint64_t addr;
} mxb_shard;

/* Records that read exactly the window `w` out of `shards` and write it at
 * `dst_base` (+ w->dst_offset elements): the box of the window in source
 * coordinates, intersected with every shard box, one record per innermost
 * strided dimension; expanding the records row by row gives the run list of
 * plan_pull (refit/reshard/slice_plan.py:227-339: resolve_slice,
 * _view_to_box_perm, intersect, paired_runs) in the same order.  `out_shard`
 * (optional, cap entries) receives the index of the shard each record reads.
 * *n_out is the number of records the plan has; MXB_ERR_NOMEM if cap is
 * smaller (the first cap records are written), MXB_ERR_UNSUPPORTED if the
 * window is not a permuted box of the source. */
int32_t mxb_plan_pull(const mxb_window *w, const mxb_shard *shards, uint64_t n_shards,
                      uint64_t dst_base, mxb_desc2d *out, uint32_t *out_shard, uint64_t cap,
                      uint64_t *n_out);

/* The part of `n` strided regions of a flat tensor that one rank's contiguous
 * piece [shard_lo, shard_hi) of that tensor holds: regions[i].src is a byte
 * offset inside the full tensor, regions[i].dst the destination address of
 * the region's first byte.  Emitted records read from src_base + (byte -
 * shard_lo) and keep the region's destination layout; records larger than
 * max_record_bytes (0 = no limit) are cut into whole rows or 256-byte
 * multiples.  This is the push-side plan of the refit reshard for the flat
 * FSDP shard geometry of modelexpress_rl/train/engines/fsdp/publisher.py:71-147
 * (the reference plans the same slices as pulls, slice_plan.py:297-339). */
int32_t mxb_plan_reshard(const mxb_desc2d *regions, uint64_t n, uint64_t shard_lo, uint64_t shard_hi,
                         uint64_t src_base, uint64_t max_record_bytes, mxb_desc2d *out, uint64_t cap,
                         uint64_t *n_out);

/* Fold consecutive runs of equal length and constant src/dst stride into 2-D
 * records, preserving order.  Returns the number of records written (<= cap),
 * or the negated count needed if cap is too small.  The expansion of the
 * result is exactly the input run list (refit/reshard/slice_plan.py:297-339). */
int64_t mxb_coalesce_runs(const mxb_run *runs, uint64_t n, mxb_desc2d *out, uint64_t cap);

/* ---- kernel 1/3: descriptor-driven scatter ----------------------------- */

#define MXB_SCATTER_DEFAULT 0u /* bulk engine (cp.async.bulk) for records whose addresses,
                                  pitches and row sizes are multiples of 16 bytes with rows
                                  of at least 1 KiB; vector engine for the rest */
#define MXB_SCATTER_VECTOR 1u  /* vector engine (16-byte loads/stores) for everything */
#define MXB_SCATTER_NO_SYNC 2u /* return after enqueueing on the context stream */
#define MXB_SCATTER_OVERLAP 4u /* mxb_table_launch: run the bulk-engine and the vector-engine part
                                  of a table as two concurrent kernels (worth it when both have
                                  much to do, e.g. local copies next to peer stores) */

#define MXB_SCATTER_BULK_PART 8u    /* measurement aid: launch only the bulk-engine part of a table */
#define MXB_SCATTER_VECTOR_PART 16u /* measurement aid: launch only the vector-engine part */

/* One persistent launch on `dev` moves every record of the host table
 * `descs[0..n)`: sources and destinations may be local HBM, a peer GPU's HBM
 * or pinned host memory.  Stands in for Transport.read(descriptors)
 * (refit/reshard/transport/base.py:38-43), for the per-tensor narrow+copy_
 * loop reached from engines/vllm/adapter.py:316-329 and for the per-tensor
 * copy loop of engines/vllm/refit/installer.py:419-424. */
int32_t mxb_scatter(mxb_ctx *ctx, int32_t dev, const mxb_desc2d *descs, uint64_t n,
                    uint32_t flags);
/* Same, from a 1-D run list: coalesces, launches and waits.  Direct
 * equivalent of InMemoryReferenceTransport.read (transport/base.py:46-62). */
int32_t mxb_read_runs(mxb_ctx *ctx, int32_t dev, const mxb_run *runs, uint64_t n);

/* A descriptor table kept resident on the device, for plans that are replayed
 * (every refit cycle moves the same slices).  Stands in for the descriptor
 * cache of refit/reshard/receiver.py:795-854 and the resolve-once / copy-many
 * loop of engines/vllm/refit/installer.py:373-424. */
int32_t mxb_table_create(mxb_ctx *ctx, int32_t dev, const mxb_desc2d *descs, uint64_t n,
                         mxb_table **out);
/* One persistent launch over the whole table on the context stream; returns
 * without waiting (use mxb_sync). */
int32_t mxb_table_launch(mxb_table *t, uint32_t flags);
/* Bytes one launch moves. */
uint64_t mxb_table_bytes(mxb_table *t);
/* Tile engines a launch with `flags` uses: 0 = vector only, 1 = bulk only,
 * 2 = bulk for the qualifying records and vector for the rest (two kernels). */
int32_t mxb_table_engine(mxb_table *t, uint32_t flags);
int32_t mxb_table_destroy(mxb_table *t);

/* Measurement aid (no counterpart in the reference): `reps` launches of a plain
 * 16-byte load/store copy kernel from `src` to `dst` (multiples of 16 bytes)
 * on `dev`, timed with CUDA events; either side may be a peer GPU's memory.
 * Gives the rate a straightforward kernel reaches on the same memory path, the
 * yardstick the scatter, fan-out and reshard rates are reported against. */
int32_t mxb_copy_probe(mxb_ctx *ctx, int32_t dev, uint64_t src, uint64_t dst, uint64_t nbytes,
                       int32_t reps, float *ms_per_rep);

/* Timing on the context's compute stream of `dev`: record event `slot`
 * (0..15); elapsed waits for event `b` and returns b - a in milliseconds. */
int32_t mxb_event_record(mxb_ctx *ctx, int32_t dev, int32_t slot);
int32_t mxb_event_elapsed(mxb_ctx *ctx, int32_t dev, int32_t a, int32_t b, float *ms);

/* ---- staging ring: host bytes -> HBM shards ----------------------------- */

typedef struct {
    uint64_t bytes_placed;
    uint64_t chunks;
    uint64_t launches;
    double seconds_total;   /* wall time of the call */
    double seconds_gather;  /* host copy time of the busiest gather thread (overlaps the copies) */
    double seconds_device;  /* first H2D start to last scatter end, CUDA events */
    uint64_t bytes_direct;  /* of bytes_placed: read from pinned sources, no host copy */
    double seconds_plan;    /* chunking, table build and upload before the first copy */
} mxb_place_stats;

#define MXB_PLACE_COPY_ENGINE 0u /* host -> device staging by the copy engine, then scatter */
#define MXB_PLACE_ZERO_COPY 1u   /* slices whose source is pinned (mxb_host_register) are read by
                                    the scatter kernel where they lie: no staging, one launch;
                                    other sources go through the ring as in mode 0 */

/* A pinned host ring of ring_bytes in total plus two device staging buffers of
 * ring_bytes / slots each (one chunk = one staging buffer = one scatter launch). */
int32_t mxb_ring_create(mxb_ctx *ctx, int32_t dev, uint64_t ring_bytes, uint32_t slots,
                        mxb_ring **out);
int32_t mxb_ring_destroy(mxb_ring *ring);
/* Place `n` slices whose sources are host memory (a checkpoint file image) and
 * whose destinations are device addresses.  Only the bytes this rank keeps
 * cross PCIe.  Slices of pinned sources (mxb_host_register, mxb_host_alloc) are
 * gathered by the copy engine itself; for ordinary pageable memory
 * `host_threads` gather threads each copy a few MiB at a time into the pinned
 * ring and queue their own H2D copy.  Either way the bytes land densely packed
 * in a device staging buffer and one persistent scatter launch per chunk
 * writes the shards while the next chunk arrives.  Replaces the host-staged
 * path engines/vllm/adapter.py:316-329 and the file->GPU batches of
 * gds_loader.py:284-331 / gds_transfer.py:142-231. */
int32_t mxb_place(mxb_ring *ring, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                  uint32_t mode, mxb_place_stats *stats);

/* A rank's slices kept in page-locked host memory, packed exactly as they cross
 * PCIe (the pinned ring of the host-staged path, made as large as the rank's
 * shard and kept).  mxb_image_create is a load like mxb_place whose gather
 * threads write every chunk into its own place in the image instead of a ring
 * slot; from then on mxb_image_place loads the same slices again with one
 * contiguous copy-engine transfer and one scatter launch per chunk: no host
 * thread, no source file, nothing read from the page cache.  Meant for weights
 * that are loaded more than once from the same host (replicas started one
 * after the other, reloads after a weight swap, refits from a host copy).
 * `items` of mxb_image_place may carry new destination addresses for the same
 * slices (NULL keeps the previous ones); a destination whose address phase
 * (mod 16) or pitch changed needs a new image (MXB_ERR_STATE).  The image
 * uses its ring's staging buffers and must be destroyed before the ring.
 * Replaces the per-load re-read of the checkpoint files by
 * engines/vllm/adapter.py:316-329 for every load after the first. */
int32_t mxb_image_create(mxb_ring *ring, const mxb_desc2d *items, uint64_t n, int32_t host_threads,
                         mxb_image **out, mxb_place_stats *stats);
int32_t mxb_image_place(mxb_image *image, const mxb_desc2d *items, uint64_t n,
                        mxb_place_stats *stats);
/* Page-locked host bytes the image holds. */
uint64_t mxb_image_bytes(mxb_image *image);
int32_t mxb_image_destroy(mxb_image *image);

/* ---- kernel 4: integrity digests ---------------------------------------- */

/* Digest `n` device byte ranges in one launch; `out[i]` receives the record of
 * `spans[i]` (host memory).  `modes` is a bit set of MXB_DIGEST_*.  Replaces
 * tensor_utils.py:27-44 (safe_checksum) and the device half of
 * refit/reshard/verify.py:79-155 (tensor_digest; blake2b of the scalars stays
 * on the host). */
int32_t mxb_digest(mxb_ctx *ctx, int32_t dev, const mxb_span *spans, uint64_t n, uint32_t modes,
                   mxb_digest_out *out);
/* Per-4-KiB-block hashes of one range, written to device memory `out_blocks`
 * (ceil(nbytes/4096) uint64 values). */
int32_t mxb_block_hashes(mxb_ctx *ctx, int32_t dev, uint64_t ptr, uint64_t nbytes,
                         uint64_t out_blocks);

/* Digest without allocating anything (no counterpart in the reference).
 *
 * For callers that are not allowed to grow the process's device memory: a
 * serving engine that has already handed every free byte of HBM to its KV
 * cache (a cudaMalloc there fails, or succeeds by taking memory the engine
 * counted on), or a verification hook that runs where the framework's caching
 * allocator must not be disturbed.  Such a caller still wants to check the
 * weights it just received, so this variant of mxb_digest keeps its whole
 * scratch (range table, tile table, accumulators; about 148 KiB) in a fixed
 * array inside the library's device image.  It needs no context, creates no
 * stream and calls no cudaMalloc/cudaFree: work is queued on `stream` (a
 * cudaStream_t, NULL for the default stream) of device `dev` and the call
 * returns after that stream has drained, with out[i] filled for spans[i].
 *
 * Limits, checked before anything is queued (MXB_ERR_ARG with a message): at
 * most 256 ranges and at most 16384 tiles of 64 KiB (1 GiB) per call; larger
 * jobs are split by the caller.  The first call on a device looks up the
 * array's device address.  Every call copies its small tables from and to
 * ordinary host memory and waits for `stream` to drain, so no call may be made
 * while `stream` (or any stream of the device) is being captured.  All calls on
 * a device share the one array (it keeps the previous call's contents; the
 * accumulators a call uses are cleared by that call), so the library
 * serialises callers on the host; work that a caller queues on other streams
 * to run at the same time against this array would race. */
int32_t mxb_digest_noalloc(int32_t dev, const mxb_span *spans, uint64_t n, uint32_t modes,
                           mxb_digest_out *out, void *stream);

/* ---- box convert: staged boxes -> live parameters, transposed and cast ----- */

#define MXB_ELEM_RAW 0  /* `elem_bytes` bytes moved unchanged (1, 2, 4 or 8) */
#define MXB_ELEM_F32 1
#define MXB_ELEM_F16 2
#define MXB_ELEM_BF16 3

/* One box.  `src` holds the box row-major over extent[0..ndim) (the source
 * tensor's own dim order, element size given by `src_kind`), contiguously
 * unless `src_stride` says otherwise; the element at box index (i0, i1, ...) lands at
 * dst + sum(i_d * dst_stride[d]) destination elements (`dst_kind`).  This is the
 * copy the reference leaves to torch after a pull: `dst.copy_(staged)` for a
 * served dtype that differs from the parameter's (refit/reshard/receiver.py:964-971)
 * and the permuted boxes of refit/reshard/slice_plan.py:170-224. */
typedef struct {
    uint64_t src;
    uint64_t dst;
    uint32_t ndim;
    uint32_t src_kind;  /* MXB_ELEM_* */
    uint32_t dst_kind;  /* MXB_ELEM_*: equal to src_kind, or a float pair (F32, F16, BF16) */
    uint32_t elem_bytes; /* MXB_ELEM_RAW only */
    uint64_t extent[MXB_MAX_DIMS];
    int64_t dst_stride[MXB_MAX_DIMS]; /* destination elements, >= 0 */
    int64_t src_stride[MXB_MAX_DIMS]; /* source elements; all zero: the box is contiguous.  Otherwise the
                                       * innermost dim with extent > 1 must have stride 1 (a strided slice
                                       * of a shard read in place, e.g. straight from a peer's memory) */
} mxb_convert;

/* All `n` boxes on the context's stream of `dev`, one launch per conversion
 * (pair of kinds) present in the list; waits unless MXB_SCATTER_NO_SYNC.  Casts round to nearest even like torch's device copy.
 * *bytes_out (optional) = bytes read + written.  MXB_ERR_UNSUPPORTED for a pair
 * of kinds outside the table above or a box that needs more than four dims after
 * merging; MXB_ERR_ALIGN for an address not aligned to its element. */
int32_t mxb_convert_boxes(mxb_ctx *ctx, int32_t dev, const mxb_convert *items, uint64_t n,
                          uint32_t flags, uint64_t *bytes_out);

/* ---- kernel 2: serving-peer fan-out -------------------------------------- */

#define MXB_FANOUT_MAX_CHILDREN 7

/* One piece of a fan-out payload: `nbytes` (<= the piece size, 64 KiB by default) at `offset` inside range
 * `range`, belonging to chunk `chunk`. */
typedef struct {
    uint64_t range;
    uint64_t offset;
    uint32_t nbytes;
    uint32_t chunk;
} mxb_fanout_piece;

/* Host only: how a payload of `n` ranges is cut into pieces and chunks of
 * `chunk_bytes` (only the sizes of `local` matter, so every GPU of a broadcast
 * cuts alike).  chunk_pieces[c] is the number of pieces of chunk c: the value a
 * child's arrival counter c reaches per broadcast.  *n_pieces / *n_chunks give
 * the full counts; MXB_ERR_NOMEM if a cap is smaller.  This is the transfer
 * plan of the peer pull (nixl_transfer.py:769-952 posts one READ per matched
 * tensor; here a tensor is cut so that chunks can be forwarded while later
 * ones are still arriving). */
int32_t mxb_fanout_plan(const mxb_span *local, uint64_t n, uint64_t chunk_bytes,
                        mxb_fanout_piece *pieces, uint64_t piece_cap, uint64_t *n_pieces,
                        uint32_t *chunk_pieces, uint64_t chunk_cap, uint64_t *n_chunks);
/* The same with pieces of at most `piece_bytes` instead of 64 KiB (a multiple of
 * 16, 4 KiB .. MXB_FANOUT_PIECE_MAX).  A piece is what one CTA stores before it
 * releases a counter: larger pieces mean fewer system-scope fences per byte
 * (faster on a single hop), smaller ones let the next hop of a chain start
 * sooner.  Every node of a broadcast must use the same value; pieces above
 * 64 KiB run on the VECTOR engine only. */
#define MXB_FANOUT_PIECE_MAX (1u << 20)
int32_t mxb_fanout_plan_pieces(const mxb_span *local, uint64_t n, uint64_t chunk_bytes, uint64_t piece_bytes,
                               mxb_fanout_piece *pieces, uint64_t piece_cap, uint64_t *n_pieces,
                               uint32_t *chunk_pieces, uint64_t chunk_cap, uint64_t *n_chunks);

/* A fan-out node: this GPU's copy of the payload is the ranges
 * `local[0..n)`, cut into chunks of `chunk_bytes`.  The node waits for each
 * chunk to arrive from its parent (unless it is the root), stores it into
 * every child's ranges over NVLink and raises the child's per-chunk counter.
 * Replaces the name-matched whole-tensor pull of nixl_transfer.py:769-952 on
 * one box. */
int32_t mxb_fanout_create(mxb_ctx *ctx, int32_t dev, const mxb_span *local, uint64_t n,
                          uint64_t chunk_bytes, mxb_fanout **out);
/* The same with the piece size of mxb_fanout_plan_pieces. */
int32_t mxb_fanout_create_pieces(mxb_ctx *ctx, int32_t dev, const mxb_span *local, uint64_t n,
                                 uint64_t chunk_bytes, uint64_t piece_bytes, mxb_fanout **out);
/* Device address of this node's arrival counters (export it to the parent). */
uint64_t mxb_fanout_counters(mxb_fanout *f);
/* Ranges (same count and sizes as `local`) and counter address of child `k`,
 * as addresses valid in this process. */
int32_t mxb_fanout_set_child(mxb_fanout *f, int32_t k, const mxb_span *child, uint64_t n,
                             uint64_t child_counters);
/* How a node moves its chunks (default: VECTOR, or what the environment variable
 * MXB_FANOUT_ENGINE = "vector" | "bulk" | "dma" names when the node is created).
 *   VECTOR  one persistent kernel, 16-byte peer stores straight from HBM;
 *   BULK    one persistent kernel, pieces staged through shared memory with bulk copies;
 *   DMA     for a root: the copy engines move every range to every child (one peer copy
 *           each, children side by side), then one launch announces all chunks at once.
 *           Nothing is announced before everything has arrived, so it suits pushes whose
 *           children only receive (one hop); a node that has a parent runs VECTOR, and so
 *           does a root whose copies would average under 4 MiB (thousands of scattered
 *           tensors: copy setup would cost more than the engines gain).
 * All speak the same counters, so the nodes of one broadcast may differ.  The
 * reference has no counterpart: its pull is one RDMA READ per tensor with no
 * forwarding (nixl_transfer.py:769-952). */
#define MXB_FANOUT_ENGINE_VECTOR 0
#define MXB_FANOUT_ENGINE_BULK 1
#define MXB_FANOUT_ENGINE_DMA 2
int32_t mxb_fanout_set_engine(mxb_fanout *f, int32_t engine);
/* Launch this node's kernel for one broadcast.  `is_root`: has no parent.
 * `timeout_ms` bounds every device-side wait. */
int32_t mxb_fanout_run(mxb_fanout *f, int32_t is_root, uint32_t timeout_ms);
/* Wait for this node's kernel; MXB_ERR_TIMEOUT if a wait ran out. */
int32_t mxb_fanout_wait(mxb_fanout *f, float *device_ms);
int32_t mxb_fanout_destroy(mxb_fanout *f);

#ifdef __cplusplus
}
#endif
#endif /* MXB200_H */
