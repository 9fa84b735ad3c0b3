// Host-side streaming copy used by the staging ring's gather threads.
//
// The ring slot is written once by the CPU and read once by the PCIe DMA, so
// pulling its cache lines into the CPU caches first (what an ordinary store
// does) only costs memory bandwidth: the gather, the read-for-ownership and
// the DMA read all compete for the same DRAM channels.  Non-temporal stores
// skip the read-for-ownership.  Falls back to memcpy on CPUs without AVX2 and
// for short or oddly aligned pieces.
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#if defined(__x86_64__)
#include <immintrin.h>
#define MXB_X86 1
#endif

namespace mxb {

#ifdef MXB_X86
__attribute__((target("avx2"))) static void stream_copy_avx2(char *d, const char *s, size_t n) {
    // head: bring the destination to a 32-byte boundary
    size_t head = (32 - (reinterpret_cast<uintptr_t>(d) & 31)) & 31;
    if (head > n) head = n;
    if (head) {
        memcpy(d, s, head);
        d += head;
        s += head;
        n -= head;
    }
    size_t i = 0;
    for (; i + 128 <= n; i += 128) {
        __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(s + i));
        __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(s + i + 32));
        __m256i c = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(s + i + 64));
        __m256i e = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(s + i + 96));
        _mm256_stream_si256(reinterpret_cast<__m256i *>(d + i), a);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(d + i + 32), b);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(d + i + 64), c);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(d + i + 96), e);
    }
    for (; i + 32 <= n; i += 32)
        _mm256_stream_si256(reinterpret_cast<__m256i *>(d + i),
                            _mm256_loadu_si256(reinterpret_cast<const __m256i *>(s + i)));
    if (i < n) memcpy(d + i, s + i, n - i);
}

static bool has_avx2() {
    static const bool ok = __builtin_cpu_supports("avx2");
    return ok;
}
#endif

// Copy n bytes; the destination will not be read by this CPU soon.
void stream_copy(void *dst, const void *src, size_t n) {
#ifdef MXB_X86
    // MXB_GATHER_MEMCPY=1 switches the streaming stores off (for A/B measurements)
    static const bool plain = getenv("MXB_GATHER_MEMCPY") != nullptr;
    if (!plain && n >= 256 && has_avx2()) {
        stream_copy_avx2(static_cast<char *>(dst), static_cast<const char *>(src), n);
        return;
    }
#endif
    memcpy(dst, src, n);
}

// Make streamed stores globally visible before another agent (the DMA engine,
// or a GPU reading pinned memory) is told to read them.
void stream_fence() {
#ifdef MXB_X86
    _mm_sfence();
#endif
}

}  // namespace mxb
