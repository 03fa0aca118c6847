// Host build of the integer arithmetic the CUDA encode kernel uses (the headers
// compile as plain C++), so that the bit tricks and the Hilbert state-machine
// tables can be checked against the oracle without a GPU.
#include <stdint.h>
#include "../../pointtransformerv3_b200/csrc/encode_math.cuh"
#include "../../pointtransformerv3_b200/csrc/hilbert_lut.cuh"

using namespace ptv3;
static constexpr hlut::Table1 T1 = hlut::make_table1();
static constexpr hlut::Table2 T2 = hlut::make_table2();

static uint64_t from_morton(uint64_t m, int depth)
{
    uint32_t s = 0;
    uint64_t g = 0;
    int l = depth;
    if (l & 1) {
        --l;
        const uint32_t e = T1.v[s * 8 + (uint32_t)((m >> (3 * l)) & 7)];
        g = e & 7;
        s = e >> 3;
    }
    while (l > 0) {
        l -= 2;
        const uint32_t e = T2.v[s * 64 + (uint32_t)((m >> (3 * l)) & 63)];
        g = (g << 6) | (e & 63);
        s = e >> 6;
    }
    for (int sh = 1; sh < 64; sh <<= 1) g ^= g >> sh;
    return g;
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
