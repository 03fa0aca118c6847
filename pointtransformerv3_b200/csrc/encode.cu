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

// Hilbert code from the Morton code of the same point: two levels per table step
__device__ __forceinline__ uint64_t hilbert_from_morton(uint64_t m, int depth, const uint16_t* __restrict__ t1,
                                                        const uint16_t* __restrict__ t2)
{
    uint32_t s = 0;
    uint64_t g = 0;
    int l = depth;
    if (l & 1) {
        --l;
        const uint32_t e = t1[s * 8 + (uint32_t)((m >> (3 * l)) & 7)];
        g = e & 7;
        s = e >> 3;
    }
    while (l > 0) {
        l -= 2;
        const uint32_t e = t2[s * 64 + (uint32_t)((m >> (3 * l)) & 63)];
        g = (g << 6) | (e & 63);
        s = e >> 6;
    }
    g ^= g >> 1;
    g ^= g >> 2;
    g ^= g >> 4;
    g ^= g >> 8;
    g ^= g >> 16;
    g ^= g >> 32;
    return g;
}

__global__ void __launch_bounds__(256) encode_kernel(const int32_t* __restrict__ grid,
                                                     const int64_t* __restrict__ batch, int64_t n,
                                                     int depth, OrderList orders,
                                                     int64_t* __restrict__ codes)
{
    __shared__ uint16_t t1[48 * 8];
    __shared__ uint16_t t2[48 * 64];
    for (int i = threadIdx.x; i < 48 * 8; i += blockDim.x) t1[i] = g_hilbert_t1.v[i];
    for (int i = threadIdx.x; i < 48 * 64; i += blockDim.x) t2[i] = g_hilbert_t2.v[i];
    __syncthreads();
    const uint32_t mask = (depth >= 32) ? 0xffffffffu : ((1u << depth) - 1u);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t x = (uint32_t)grid[3 * i + 0] & mask;
        const uint32_t y = (uint32_t)grid[3 * i + 1] & mask;
        const uint32_t z = (uint32_t)grid[3 * i + 2] & mask;
        const uint64_t hi = batch ? ((uint64_t)batch[i] << (3 * depth)) : 0ull;
        const uint64_t sx = spread3(x), sy = spread3(y), sz = spread3(z);
        const uint64_t m = (sx << 2) | (sy << 1) | sz;    // z order
        const uint64_t mt = (sy << 2) | (sx << 1) | sz;   // z order with x and y exchanged
#pragma unroll
        for (int r = 0; r < PTV3_MAX_ORDERS; ++r) {
            if (r < orders.n) {
                uint64_t c;
                switch (orders.id[r]) {
                    case PTV3_ORDER_Z: c = m; break;
                    case PTV3_ORDER_Z_TRANS: c = mt; break;
                    case PTV3_ORDER_HILBERT: c = hilbert_from_morton(m, depth, t1, t2); break;
                    default: c = hilbert_from_morton(mt, depth, t1, t2); break;
                }
                codes[(int64_t)r * n + i] = (int64_t)(c | hi);
            }
        }
    }
}

}  // namespace ptv3

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
