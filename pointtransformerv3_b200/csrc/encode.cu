// Space-filling-curve codes of a voxelised point cloud: one thread per point
// reads (x, y, z) and the scene id once and emits every requested order.
//
// Replaces serialization/default.py:8-24 (order dispatch, x/y swap, batch in
// the bits above 3*depth), serialization/z_order.py:66-101 (Morton key) and
// serialization/hilbert.py:91-198 (Skilling transform, dim 0 most significant,
// Gray decode).  HBM-bound: 12 B + 8 B read and 8 B per order written.
#include "common.cuh"
#include "../../include/ptv3_b200.h"
#include "encode_math.cuh"

namespace ptv3 {

struct OrderList {
    int n;
    int id[PTV3_MAX_ORDERS];
};

__global__ void __launch_bounds__(256) encode_kernel(const int32_t* __restrict__ grid,
                                                     const int64_t* __restrict__ batch, int64_t n,
                                                     int depth, OrderList orders,
                                                     int64_t* __restrict__ codes)
{
    const uint32_t mask = (depth >= 32) ? 0xffffffffu : ((1u << depth) - 1u);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t x = (uint32_t)grid[3 * i + 0] & mask;
        const uint32_t y = (uint32_t)grid[3 * i + 1] & mask;
        const uint32_t z = (uint32_t)grid[3 * i + 2] & mask;
        const uint64_t hi = batch ? ((uint64_t)batch[i] << (3 * depth)) : 0ull;
#pragma unroll
        for (int r = 0; r < PTV3_MAX_ORDERS; ++r) {
            if (r < orders.n) {
                uint64_t c;
                switch (orders.id[r]) {
                    case PTV3_ORDER_Z: c = morton3(x, y, z); break;
                    case PTV3_ORDER_Z_TRANS: c = morton3(y, x, z); break;
                    case PTV3_ORDER_HILBERT: c = hilbert3(x, y, z, depth); break;
                    default: c = hilbert3(y, x, z, depth); break;
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
