/*
 * CPU restatement of the ModelExpress byte-moving and digest arithmetic, in
 * plain C.  TEST INFRASTRUCTURE ONLY: the test-suite, the smoke entry and the
 * benchmark's CPU-baseline leg may load it as the checker; the shipped library
 * never links or calls it.
 *
 * Each function names the reference code it follows (paths relative to the
 * reference project's modelexpress_client/python/modelexpress/):
 *
 *   orc_memmove_runs        refit/reshard/transport/base.py:56-62
 *   orc_scatter2d           the same loop, with the runs of one strided slice
 *                           (refit/reshard/slice_plan.py:259-294 emits one run
 *                           per row) kept as a single rows x row_bytes record
 *   orc_safe_checksum       tensor_utils.py:27-44
 *   orc_digest_scalars      refit/reshard/verify.py:113-150
 *   orc_block_hashes64 /
 *   orc_block_hash64        no counterpart in the reference (parity unpinned);
 *                           same definition as ref_port.py:block_hashes64
 *
 * The *_mt variants split the work over OpenMP threads for the timed CPU
 * baseline; results are identical.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

typedef struct {
    uint64_t src, dst, nbytes;
} orc_run;

typedef struct {
    uint64_t src, dst, rows, row_bytes, src_pitch, dst_pitch;
} orc_desc2d;

void orc_memmove_runs(const orc_run *runs, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i)
        if (runs[i].nbytes)
            memmove((void *)(uintptr_t)runs[i].dst, (const void *)(uintptr_t)runs[i].src,
                    (size_t)runs[i].nbytes);
}

void orc_scatter2d(const orc_desc2d *d, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i)
        for (uint64_t r = 0; r < d[i].rows; ++r)
            memmove((void *)(uintptr_t)(d[i].dst + r * d[i].dst_pitch),
                    (const void *)(uintptr_t)(d[i].src + r * d[i].src_pitch),
                    (size_t)d[i].row_bytes);
}

void orc_scatter2d_mt(const orc_desc2d *d, uint64_t n) {
    /* flatten to (descriptor, row-block) work items so one huge tensor does
     * not serialise on a single thread */
#pragma omp parallel
    {
#pragma omp single
        for (uint64_t i = 0; i < n; ++i) {
            uint64_t rows = d[i].rows, rb = d[i].row_bytes;
            uint64_t per = rb ? (1u << 20) / rb : rows;
            if (per == 0) per = 1;
            for (uint64_t r0 = 0; r0 < rows; r0 += per) {
                uint64_t r1 = r0 + per < rows ? r0 + per : rows;
#pragma omp task firstprivate(i, r0, r1)
                for (uint64_t r = r0; r < r1; ++r)
                    memmove((void *)(uintptr_t)(d[i].dst + r * d[i].dst_pitch),
                            (const void *)(uintptr_t)(d[i].src + r * d[i].src_pitch),
                            (size_t)d[i].row_bytes);
            }
        }
    }
}

uint32_t orc_safe_checksum(const uint8_t *p, uint64_t n) {
    uint32_t acc = 0;
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t w = (uint32_t)(i * 2654435761ull + 1ull);
        acc += (uint32_t)p[i] * w;
    }
    return acc;
}

uint32_t orc_safe_checksum_mt(const uint8_t *p, uint64_t n) {
    uint32_t acc = 0;
#pragma omp parallel for reduction(+ : acc) schedule(static)
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t w = (uint32_t)(i * 2654435761ull + 1ull);
        acc += (uint32_t)p[i] * w;
    }
    return acc;
}

/* out[0..6] = n, sum(rows), sum(rows*(k+1)), sum(tail), sum(tail*(j+1)),
 * sum(ragged bytes), n%4; returns a bit mask of the groups that exist
 * (bit0 rows, bit1 tail, bit2 ragged) exactly as verify.py appends them. */
static inline int32_t load_i32(const uint8_t *p) {
    int32_t v;
    memcpy(&v, p, 4);
    return v;
}

uint32_t orc_digest_scalars(const uint8_t *p, uint64_t n, uint64_t out[7]) {
    uint64_t body = n - (n % 4), words = body / 4, rows = words / 1024;
    uint64_t s_rows = 0, s_rows_w = 0, s_tail = 0, s_tail_w = 0, s_rag = 0;
    for (uint64_t k = 0; k < rows; ++k) {
        int64_t rs = 0;
        const uint8_t *q = p + k * 4096;
        for (int j = 0; j < 1024; ++j) rs += load_i32(q + 4 * j);
        s_rows += (uint64_t)rs;
        s_rows_w += (uint64_t)rs * (k + 1);
    }
    uint64_t tail = words - rows * 1024;
    for (uint64_t j = 0; j < tail; ++j) {
        int64_t v = load_i32(p + rows * 4096 + 4 * j);
        s_tail += (uint64_t)v;
        s_tail_w += (uint64_t)v * (j + 1);
    }
    for (uint64_t j = body; j < n; ++j) s_rag += p[j];
    out[0] = n; out[1] = s_rows; out[2] = s_rows_w; out[3] = s_tail; out[4] = s_tail_w;
    out[5] = s_rag; out[6] = n % 4;
    return (rows ? 1u : 0u) | (tail ? 2u : 0u) | ((n % 4) ? 4u : 0u);
}

uint32_t orc_digest_scalars_mt(const uint8_t *p, uint64_t n, uint64_t out[7]) {
    uint64_t body = n - (n % 4), words = body / 4, rows = words / 1024;
    uint64_t s_rows = 0, s_rows_w = 0;
#pragma omp parallel for reduction(+ : s_rows, s_rows_w) schedule(static)
    for (uint64_t k = 0; k < rows; ++k) {
        int64_t rs = 0;
        const uint8_t *q = p + k * 4096;
        for (int j = 0; j < 1024; ++j) rs += load_i32(q + 4 * j);
        s_rows += (uint64_t)rs;
        s_rows_w += (uint64_t)rs * (k + 1);
    }
    uint64_t tmp[7];
    uint32_t mask = orc_digest_scalars(p + rows * 4096, n - rows * 4096, tmp);
    out[0] = n; out[1] = s_rows; out[2] = s_rows_w; out[3] = tmp[3]; out[4] = tmp[4];
    out[5] = tmp[5]; out[6] = n % 4;
    return (rows ? 1u : 0u) | (mask & 6u);
}

#define P1 0x9E3779B185EBCA87ull
#define P2 0xC2B2AE3D27D4EB4Full
#define P3 0x165667B19E3779F9ull
#define P4 0x85EBCA77C2B2AE63ull
#define P5 0x27D4EB2F165667C5ull

#define Q1 0x9E3779B1u
#define Q2 0x85EBCA77u
#define Q3 0xC2B2AE3Du
#define Q4 0x27D4EB2Fu
#define Q5 0x165667B1u
static inline uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }
static inline uint64_t avalanche(uint64_t h) {
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
    return h;
}

static uint64_t one_block(const uint8_t *p, uint64_t avail, uint64_t b) {
    uint8_t buf[4096];
    if (avail < 4096) {
        memset(buf, 0, sizeof buf);
        memcpy(buf, p, (size_t)avail);
        p = buf;
    }
    uint64_t h = 0;
    for (uint32_t lane = 0; lane < 32; ++lane) {
        uint32_t a[2] = {Q5 + lane * Q4, Q3 ^ (lane * Q1)};
        for (int step = 0; step < 8; ++step)
            for (int k = 0; k < 4; ++k) {
                uint32_t x;
                memcpy(&x, p + step * 512 + lane * 16 + k * 4, 4);
                a[k & 1] = rotl32(a[k & 1] + x * Q2, 13) * Q1;
            }
        uint64_t acc = ((uint64_t)a[0] << 32) | a[1];
        h += avalanche(acc + (b + 1) * P1); /* the lane's share of block b */
    }
    return h;
}

void orc_block_hashes64(const uint8_t *p, uint64_t n, uint64_t *out) {
    uint64_t nblk = (n + 4095) / 4096;
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nblk; ++b) {
        uint64_t off = b * 4096;
        out[b] = one_block(p + off, n - off, b);
    }
}

uint64_t orc_block_hash64(const uint8_t *p, uint64_t n) {
    uint64_t nblk = (n + 4095) / 4096, total = 0;
#pragma omp parallel for reduction(+ : total) schedule(static)
    for (uint64_t b = 0; b < nblk; ++b) {
        uint64_t off = b * 4096;
        total += one_block(p + off, n - off, b);
    }
    return total + avalanche(n * P5);
}
