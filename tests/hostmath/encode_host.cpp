// Host build of the integer arithmetic the CUDA encode kernel uses (the headers
// compile as plain C++), so that the bit tricks and the Hilbert state-machine
// tables can be checked against the oracle without a GPU.
#include <stdint.h>
#include "../../pointtransformerv3_b200/csrc/encode_math.cuh"
#include "../../pointtransformerv3_b200/csrc/hilbert_lut.cuh"

using namespace ptv3;
static constexpr hlut::Table1 T1 = hlut::make_table1();
static constexpr hlut::Table2 T2 = hlut::make_table2();

// same split-word arithmetic as hilbert_from_morton() in encode.cu
static uint64_t from_morton(uint64_t m64, int depth)
{
    const uint32_t mhi = (uint32_t)(m64 >> 24), mlo = (uint32_t)(m64 & 0xffffffu);
    const uint16_t* t1 = T1.v;
    const uint16_t* t2 = T2.v;
    uint32_t s = 0, gh = 0, gl = 0;
    int l = depth;
    if (l & 1) {
        --l;
        const uint32_t r = l >= 8 ? (mhi >> (3 * (l - 8))) & 7u : (mlo >> (3 * l)) & 7u;
        const uint32_t e = t1[s * 8 + r];
        if (l >= 8) gh = e & 7u; else gl = e & 7u;
        s = e >> 3;
    }
    for (; l > 8; l -= 2) {
        const uint32_t e = t2[s * 64 + ((mhi >> (3 * (l - 10))) & 63u)];
        gh = gh * 64u + (e & 63u);
        s = e >> 6;
    }
    for (; l > 0; l -= 2) {
        const uint32_t e = t2[s * 64 + ((mlo >> (3 * (l - 2))) & 63u)];
        gl = gl * 64u + (e & 63u);
        s = e >> 6;
    }
    gh ^= gh >> 1; gh ^= gh >> 2; gh ^= gh >> 4; gh ^= gh >> 8; gh ^= gh >> 16;
    gl ^= gl >> 1; gl ^= gl >> 2; gl ^= gl >> 4; gl ^= gl >> 8; gl ^= gl >> 16;
    gl ^= (0u - (gh & 1u)) & 0xffffffu;
    return ((uint64_t)gh << 24) | gl;
}

extern "C" void host_encode(const int32_t* grid, int64_t n, int depth, int order, int use_lut, int64_t* out)
{
    const uint32_t mask = (1u << depth) - 1u;
    for (int64_t i = 0; i < n; ++i) {
        uint32_t x = (uint32_t)grid[3 * i] & mask, y = (uint32_t)grid[3 * i + 1] & mask;
        const uint32_t z = (uint32_t)grid[3 * i + 2] & mask;
        if (order & 1) { const uint32_t t = x; x = y; y = t; }
        uint64_t c;
        if (order < 2) c = morton3(x, y, z);
        else c = use_lut ? from_morton(morton3(x, y, z), depth) : hilbert3(x, y, z, depth);
        out[i] = (int64_t)c;
    }
}

extern "C" void host_decode(const int64_t* code, int64_t n, int depth, int hilbert, int64_t* out)
{
    for (int64_t i = 0; i < n; ++i) {
        uint32_t x, y, z;
        const uint64_t c = (uint64_t)code[i] & ((1ull << (3 * depth)) - 1ull);
        if (hilbert) {
            hilbert3_inverse(c, depth, x, y, z);
        } else {
            x = compact3(c >> 2);
            y = compact3(c >> 1);
            z = compact3(c);
        }
        out[3 * i] = x;
        out[3 * i + 1] = y;
        out[3 * i + 2] = z;
    }
}
