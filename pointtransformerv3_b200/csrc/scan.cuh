// Device-wide exclusive scan of per-element 0/1 flags in three launches
// (tile sums -> scan of the sums -> apply), for rows of a (k, n) problem.
// The flag of an element and what is done with its scanned position are
// functors, so that flags are recomputed instead of stored.
#pragma once
#include "common.cuh"

namespace ptv3 {

constexpr int SC_THREADS = 256;
constexpr int SC_ITEMS = 8;
constexpr int SC_TILE = SC_THREADS * SC_ITEMS;

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums,
                                                         uint32_t& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    __syncthreads();
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    uint32_t base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < SC_THREADS / 32; ++w) {
        const uint32_t s = warp_sums[w];
        if (w < warp) base += s;
        tot += s;
    }
    total = tot;
    return base + inc - v;
}

// tile_sums[row][tile] = number of set flags in the tile
template <typename Flag>
__global__ void __launch_bounds__(SC_THREADS) scan_tile_sums_kernel(Flag flag, int64_t n, int ntiles,
                                                                   uint32_t* __restrict__ tile_sums)
{
    __shared__ uint32_t warp_sums[SC_THREADS / 32];
    const int row = blockIdx.y;
    const int64_t base = (int64_t)blockIdx.x * SC_TILE + (int64_t)threadIdx.x * SC_ITEMS;
    uint32_t c = 0;
#pragma unroll
    for (int it = 0; it < SC_ITEMS; ++it) {
        const int64_t j = base + it;
        if (j < n) c += flag(row, j) ? 1u : 0u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t s = 0;
        for (int w = 0; w < SC_THREADS / 32; ++w) s += warp_sums[w];
        tile_sums[(int64_t)row * ntiles + blockIdx.x] = s;
    }
}

// in-place exclusive scan of tile_sums[row][0..ntiles); totals[row] = sum
static __global__ void __launch_bounds__(SC_THREADS) scan_sums_kernel(uint32_t* __restrict__ tile_sums,
                                                              int ntiles,
                                                              uint32_t* __restrict__ totals)
{
    __shared__ uint32_t warp_sums[SC_THREADS / 32];
    const int row = blockIdx.x;
    uint32_t* s = tile_sums + (int64_t)row * ntiles;
    uint32_t carry = 0;
    for (int base = 0; base < ntiles; base += SC_THREADS) {
        const int t = base + threadIdx.x;
        const uint32_t v = t < ntiles ? s[t] : 0u;
        uint32_t total;
        const uint32_t ex = block_exclusive_scan(v, warp_sums, total);
        if (t < ntiles) s[t] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) totals[row] = carry;
}

// calls sink(row, j, position, flag) for every element; position = number of
// set flags before j in the row
template <typename Flag, typename Sink>
__global__ void __launch_bounds__(SC_THREADS) scan_apply_kernel(Flag flag, Sink sink, int64_t n,
                                                               int ntiles,
                                                               const uint32_t* __restrict__ tile_sums)
{
    __shared__ uint32_t warp_sums[SC_THREADS / 32];
    const int row = blockIdx.y;
    const int64_t base = (int64_t)blockIdx.x * SC_TILE + (int64_t)threadIdx.x * SC_ITEMS;
    bool f[SC_ITEMS];
    uint32_t c = 0;
#pragma unroll
    for (int it = 0; it < SC_ITEMS; ++it) {
        const int64_t j = base + it;
        f[it] = (j < n) && flag(row, j);
        c += f[it] ? 1u : 0u;
    }
    uint32_t total;
    uint32_t pos = block_exclusive_scan(c, warp_sums, total) +
                   tile_sums[(int64_t)row * ntiles + blockIdx.x];
#pragma unroll
    for (int it = 0; it < SC_ITEMS; ++it) {
        const int64_t j = base + it;
        if (j < n) sink(row, j, pos, f[it]);
        pos += f[it] ? 1u : 0u;
    }
}

}  // namespace ptv3
