// Exact unsigned 32-bit division by a divisor fixed at descriptor-creation time.
// Plain C++ (no CUDA types) so that host tests can exercise it directly.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {

// Exact division of a 32-bit numerator by a fixed 32-bit divisor with one
// multiply-high and a shift (round-up method: n/d == (n * m) >> (32 + s) with a
// 33-bit multiplier handled through the add-back form).
struct FastDiv {
    uint32_t d, m, s;
    FastDiv() : d(1), m(0), s(0) {}
    explicit FastDiv(uint32_t div) : d(div) {
        if (div == 1) {
            m = 0;
            s = 0;
            return;
        }
        uint32_t l = 0;
        while ((1ull << l) < div) ++l;// ceil(log2 d)
        uint64_t mm = ((1ull << 32) * ((1ull << l) - div)) / div + 1;
        m = (uint32_t) mm;
        s = l;
    }
    B200_HD uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        uint32_t t = __umulhi(n, m);
#else
        uint32_t t = (uint32_t) (((uint64_t) n * m) >> 32);
#endif
        if (d == 1) return n;
        return (t + ((n - t) >> 1)) >> (s - 1);
    }
    B200_HD void divmod(uint32_t n, uint32_t &q, uint32_t &r) const {
        q = div(n);
        r = n - q * d;
    }
};


}// namespace b200
