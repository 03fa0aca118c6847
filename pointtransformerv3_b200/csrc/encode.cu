// Space-filling-curve codes of a voxelised point cloud: one thread per point
// reads (x, y, z) and the scene id once and emits every requested order.
//
// Replaces serialization/default.py:8-24 (order dispatch, x/y swap, batch in
// the bits above 3*depth), serialization/z_order.py:66-101 (Morton key) and
// serialization/hilbert.py:91-198 (Skilling transform, dim 0 most significant,
// Gray decode).  The Hilbert transform runs as a 48-state machine over the
// Morton code, two levels per shared-memory table step, so that the kernel
// stays HBM-bound: 12 B + 8 B read and 8 B per order written.
#include "common.cuh"
#include "../../include/ptv3_b200.h"
#include "encode_math.cuh"
#include "hilbert_lut.cuh"

namespace ptv3 {

struct OrderList {
    int n;
    int id[PTV3_MAX_ORDERS];
};

// Hilbert transition tables (see hilbert_lut.cuh), evaluated at compile time
__device__ const hlut::Table1 g_hilbert_t1 = hlut::make_table1();
__device__ const hlut::Table2 g_hilbert_t2 = hlut::make_table2();

// The code is handled as two 24-bit words (levels 8..15 and 0..7) so that all
// arithmetic is 32-bit.  Hilbert code from the Morton words of the same point,
// two levels per table step.
struct Code48 {
    uint32_t hi, lo;
};

__device__ __forceinline__ Code48 hilbert_from_morton(Code48 m, int depth, const uint16_t* __restrict__ t1,
                                                      const uint16_t* __restrict__ t2)
{
    uint32_t s = 0, gh = 0, gl = 0;
    int l = depth;
    if (l & 1) {   // odd number of levels: the top one alone
        --l;
        const uint32_t r = l >= 8 ? (m.hi >> (3 * (l - 8))) & 7u : (m.lo >> (3 * l)) & 7u;
        const uint32_t e = t1[s * 8 + r];
        if (l >= 8) gh = e & 7u; else gl = e & 7u;
        s = e >> 3;
    }
    for (; l > 8; l -= 2) {
        const uint32_t e = t2[s * 64 + ((m.hi >> (3 * (l - 10))) & 63u)];
        gh = gh * 64u + (e & 63u);
        s = e >> 6;
    }
    for (; l > 0; l -= 2) {
        const uint32_t e = t2[s * 64 + ((m.lo >> (3 * (l - 2))) & 63u)];
        gl = gl * 64u + (e & 63u);
        s = e >> 6;
    }
    // Gray -> binary: prefix XOR from the top bit, done per word, then the parity of
    // the upper word carried into the lower one
    gh ^= gh >> 1; gh ^= gh >> 2; gh ^= gh >> 4; gh ^= gh >> 8; gh ^= gh >> 16;
    gl ^= gl >> 1; gl ^= gl >> 2; gl ^= gl >> 4; gl ^= gl >> 8; gl ^= gl >> 16;
    gl ^= (0u - (gh & 1u)) & 0xffffffu;
    return Code48{gh, gl};
}

__global__ void __launch_bounds__(256) encode_kernel(const int32_t* __restrict__ grid,
                                                     const int64_t* __restrict__ batch, int64_t n,
                                                     int depth, OrderList orders,
                                                     int64_t* __restrict__ codes)
{
    __shared__ uint16_t t1[48 * 8];
    __shared__ uint16_t t2[48 * 64];
    __shared__ uint32_t sp[256];   // bit i of a byte -> bit 3 i (as z_order.py:12-50 tabulates)
    for (int i = threadIdx.x; i < 48 * 8; i += blockDim.x) t1[i] = g_hilbert_t1.v[i];
    for (int i = threadIdx.x; i < 48 * 64; i += blockDim.x) t2[i] = g_hilbert_t2.v[i];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sp[i] = (uint32_t)spread3((uint32_t)i);
    __syncthreads();
    const uint32_t mask = (1u << depth) - 1u;   // depth <= 16
    const bool low_only = depth <= 8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t x = (uint32_t)grid[3 * i + 0] & mask;
        const uint32_t y = (uint32_t)grid[3 * i + 1] & mask;
        const uint32_t z = (uint32_t)grid[3 * i + 2] & mask;
        const uint64_t hi = batch ? ((uint64_t)batch[i] << (3 * depth)) : 0ull;
        const uint32_t xl = sp[x & 255u], yl = sp[y & 255u], zl = sp[z & 255u];
        uint32_t xh = 0, yh = 0, zh = 0;
        if (!low_only) {
            xh = sp[x >> 8];
            yh = sp[y >> 8];
            zh = sp[z >> 8];
        }
        const Code48 m{(xh << 2) | (yh << 1) | zh, (xl << 2) | (yl << 1) | zl};    // z order
        const Code48 mt{(yh << 2) | (xh << 1) | zh, (yl << 2) | (xl << 1) | zl};   // x and y exchanged
#pragma unroll
        for (int r = 0; r < PTV3_MAX_ORDERS; ++r) {
            if (r < orders.n) {
                Code48 c;
                switch (orders.id[r]) {
                    case PTV3_ORDER_Z: c = m; break;
                    case PTV3_ORDER_Z_TRANS: c = mt; break;
                    case PTV3_ORDER_HILBERT: c = hilbert_from_morton(m, depth, t1, t2); break;
                    default: c = hilbert_from_morton(mt, depth, t1, t2); break;
                }
                codes[(int64_t)r * n + i] = (int64_t)((((uint64_t)c.hi << 24) | c.lo) | hi);
            }
        }
    }
}

__global__ void __launch_bounds__(256) decode_kernel(const int64_t* __restrict__ codes, int64_t n, int depth,
                                                     int hilbert, int64_t* __restrict__ grid,
                                                     int64_t* __restrict__ batch)
{
    const uint64_t mask = (1ull << (3 * depth)) - 1ull;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint64_t c = (uint64_t)codes[i];
        if (batch) batch[i] = (int64_t)(c >> (3 * depth));
        const uint64_t low = c & mask;
        uint32_t x, y, z;
        if (hilbert) {
            hilbert3_inverse(low, depth, x, y, z);
        } else {
            x = compact3(low >> 2);
            y = compact3(low >> 1);
            z = compact3(low);
        }
        grid[3 * i + 0] = x;
        grid[3 * i + 1] = y;
        grid[3 * i + 2] = z;
    }
}

}  // namespace ptv3

extern "C" int ptv3_decode(const int64_t* codes, int64_t n, int depth, int order, int64_t* grid_coord,
                           int64_t* batch, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_decode: n < 0");
    PTV3_REQUIRE(depth >= 1 && depth <= 16, PTV3_ERR_INVALID_ARGUMENT, "ptv3_decode: depth %d outside [1, 16]",
                 depth);
    PTV3_REQUIRE(order == PTV3_ORDER_Z || order == PTV3_ORDER_HILBERT, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_decode: order %d (decodable: z = 0, hilbert = 2)", order);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(codes && grid_coord, PTV3_ERR_INVALID_ARGUMENT, "ptv3_decode: null pointer");
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    decode_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(codes, n, depth, order == PTV3_ORDER_HILBERT,
                                                                      grid_coord, batch);
    count_launches(1);
    return check_launch("ptv3_decode");
}

extern "C" int ptv3_encode(const int32_t* grid_coord, const int64_t* batch, int64_t n, int depth,
                           const int* orders, int n_orders, int64_t* codes, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_encode: n < 0");
    PTV3_REQUIRE(depth >= 1 && depth <= 16, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_encode: depth %d outside [1, 16]", depth);
    PTV3_REQUIRE(n_orders >= 1 && n_orders <= PTV3_MAX_ORDERS, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_encode: n_orders %d outside [1, %d]", n_orders, PTV3_MAX_ORDERS);
    PTV3_REQUIRE(orders != nullptr, PTV3_ERR_INVALID_ARGUMENT, "ptv3_encode: orders is null");
    OrderList ol;
    ol.n = n_orders;
    for (int r = 0; r < PTV3_MAX_ORDERS; ++r) ol.id[r] = 0;
    for (int r = 0; r < n_orders; ++r) {
        PTV3_REQUIRE(orders[r] >= 0 && orders[r] <= 3, PTV3_ERR_INVALID_ARGUMENT,
                     "ptv3_encode: unknown order id %d", orders[r]);
        ol.id[r] = orders[r];
    }
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(grid_coord && codes, PTV3_ERR_INVALID_ARGUMENT, "ptv3_encode: null pointer");
    const int threads = 256;
    int64_t blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    encode_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(grid_coord, batch, n, depth,
                                                                           ol, codes);
    count_launches(1);
    return check_launch("ptv3_encode");
}
