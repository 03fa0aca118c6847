// Integer arithmetic of the serialization codes, usable from device code and
// (for the host-side self-check the tests build) from host code.
#pragma once
#include <stdint.h>
#if defined(__CUDACC__)
#define PTV3_HD __host__ __device__ __forceinline__
#else
#define PTV3_HD static inline
#endif

namespace ptv3 {

// bit i of v (i < 21) -> bit 3*i
PTV3_HD uint64_t spread3(uint32_t v32)
{
    uint64_t v = v32 & 0x1fffffu;
    v = (v | (v << 32)) & 0x001f00000000ffffull;
    v = (v | (v << 16)) & 0x001f0000ff0000ffull;
    v = (v | (v << 8)) & 0x100f00f00f00f00full;
    v = (v | (v << 4)) & 0x10c30c30c30c30c3ull;
    v = (v | (v << 2)) & 0x1249249249249249ull;
    return v;
}

PTV3_HD uint64_t morton3(uint32_t a, uint32_t b, uint32_t c)
{
    return (spread3(a) << 2) | (spread3(b) << 1) | spread3(c);
}

// Skilling's axes-to-transpose on the low `depth` bits, then interleave and
// Gray-decode.  All three axes live in registers; one iteration per level.
PTV3_HD uint64_t hilbert3(uint32_t x0, uint32_t x1, uint32_t x2, int depth)
{
    for (uint32_t q = 1u << (depth - 1); q > 1; q >>= 1) {
        const uint32_t p = q - 1;
        // dim 0: set -> invert own low bits; clear -> exchange with itself (nothing)
        if (x0 & q) x0 ^= p;
        // dim 1
        if (x1 & q) {
            x0 ^= p;
        } else {
            const uint32_t t = (x0 ^ x1) & p;
            x0 ^= t;
            x1 ^= t;
        }
        // dim 2
        if (x2 & q) {
            x0 ^= p;
        } else {
            const uint32_t t = (x0 ^ x2) & p;
            x0 ^= t;
            x2 ^= t;
        }
    }
    uint64_t g = morton3(x0, x1, x2);
    g ^= g >> 1;
    g ^= g >> 2;
    g ^= g >> 4;
    g ^= g >> 8;
    g ^= g >> 16;
    g ^= g >> 32;
    return g;
}

// inverse of spread3: bit 3 i of v -> bit i
PTV3_HD uint32_t compact3(uint64_t v)
{
    v &= 0x1249249249249249ull;
    v = (v | (v >> 2)) & 0x10c30c30c30c30c3ull;
    v = (v | (v >> 4)) & 0x100f00f00f00f00full;
    v = (v | (v >> 8)) & 0x001f0000ff0000ffull;
    v = (v | (v >> 16)) & 0x001f00000000ffffull;
    v = (v | (v >> 32)) & 0x1fffffull;
    return (uint32_t)v;
}

// Inverse of hilbert3: binary -> Gray, de-interleave, undo the transform from the
// lowest level up (serialization/hilbert.py:201-303).
PTV3_HD void hilbert3_inverse(uint64_t code, int depth, uint32_t& x0, uint32_t& x1, uint32_t& x2)
{
    const uint64_t g = code ^ (code >> 1);
    x0 = compact3(g >> 2);
    x1 = compact3(g >> 1);
    x2 = compact3(g);
    for (uint32_t q = 1; q < (1u << depth); q <<= 1) {
        const uint32_t p = q - 1;
        // dims 2, 1, 0 in that order
        if (x2 & q) {
            x0 ^= p;
        } else {
            const uint32_t t = (x0 ^ x2) & p;
            x0 ^= t;
            x2 ^= t;
        }
        if (x1 & q) {
            x0 ^= p;
        } else {
            const uint32_t t = (x0 ^ x1) & p;
            x0 ^= t;
            x1 ^= t;
        }
        if (x0 & q) x0 ^= p;
    }
}

}  // namespace ptv3
