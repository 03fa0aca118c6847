// Stable LSD radix argsort of k rows of n non-negative int64 codes, restricted
// to the significant low bits, with the inverse permutation written by the last
// pass.  Replaces torch.argsort + scatter_ at model.py:118-126 and :667-674
// (ties are resolved by original index, the canonical order).
//
// Per pass (8-bit digits, spread evenly over the significant bits): tile histogram ->
// per-digit scan over tiles -> stable scatter.  The first pass reads the caller's codes and takes the value
// of an element to be its index; the last pass writes order/inverse as int64
// and drops the keys.  HBM-bound: 8 B key + 4 B value read and written per
// element and pass.
#include "common.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

constexpr int RS_THREADS = 256;
constexpr int RS_WARPS = RS_THREADS / 32;
constexpr int RS_ITEMS = 8;
constexpr int RS_TILE = RS_THREADS * RS_ITEMS;  // 2048 elements per CTA
constexpr int RS_MAX_BITS = 11;
constexpr int RS_MAX_BINS = 1 << RS_MAX_BITS;

// tile_hist[row][digit][tile]; digit_total[row][digit]
__global__ void __launch_bounds__(RS_THREADS) rs_hist_kernel(const uint64_t* __restrict__ keys,
                                                            int64_t n, int shift, uint32_t mask,
                                                            int ntiles,
                                                            uint32_t* __restrict__ tile_hist,
                                                            uint32_t* __restrict__ digit_total)
{
    __shared__ uint32_t hist[RS_MAX_BINS];
    const int bins = (int)mask + 1;
    const int row = blockIdx.y, tile = blockIdx.x;
    for (int b = threadIdx.x; b < bins; b += RS_THREADS) hist[b] = 0;
    __syncthreads();
    const uint64_t* k = keys + (int64_t)row * n;
    const int64_t base = (int64_t)tile * RS_TILE;
#pragma unroll
    for (int it = 0; it < RS_ITEMS; ++it) {
        const int64_t idx = base + it * RS_THREADS + threadIdx.x;
        if (idx < n) atomicAdd(&hist[(uint32_t)(k[idx] >> shift) & mask], 1u);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < bins; b += RS_THREADS) {
        const uint32_t c = hist[b];
        tile_hist[((int64_t)row * bins + b) * ntiles + tile] = c;
        if (c) atomicAdd(&digit_total[row * RS_MAX_BINS + b], c);
    }
}

// One CTA per (digit, row): exclusive scan of that digit's tile counts, offset
// by the number of elements with a smaller digit.
__global__ void __launch_bounds__(RS_THREADS) rs_scan_kernel(uint32_t* __restrict__ tile_hist,
                                                            const uint32_t* __restrict__ digit_total,
                                                            int ntiles)
{
    __shared__ uint32_t warp_sums[RS_WARPS];
    __shared__ uint32_t carry;
    const int digit = blockIdx.x, row = blockIdx.y, bins = gridDim.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // digit base: sum of totals of smaller digits
    uint32_t v = 0;
    for (int b = threadIdx.x; b < digit; b += RS_THREADS) v += digit_total[row * RS_MAX_BINS + b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) warp_sums[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t s = 0;
        for (int w = 0; w < RS_WARPS; ++w) s += warp_sums[w];
        carry = s;
    }
    __syncthreads();
    uint32_t* h = tile_hist + ((int64_t)row * bins + digit) * ntiles;
    for (int base = 0; base < ntiles; base += RS_THREADS) {
        const int t = base + threadIdx.x;
        const uint32_t c = (t < ntiles) ? h[t] : 0u;
        uint32_t inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += u;
        }
        __syncthreads();  // carry/warp_sums of the previous round are consumed
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < warp; ++w) wbase += warp_sums[w];
        const uint32_t excl = carry + wbase + inc - c;
        if (t < ntiles) h[t] = excl;
        __syncthreads();
        if (threadIdx.x == RS_THREADS - 1) carry = excl + c;
    }
}

// Stable scatter of one tile.  Element order inside a tile is warp-major:
// warp w owns [w*256, (w+1)*256), visited 32 consecutive elements at a time.
template <bool FIRST, bool LAST>
__global__ void __launch_bounds__(RS_THREADS) rs_scatter_kernel(
    const uint64_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
    uint64_t* __restrict__ keys_out, int32_t* __restrict__ vals_out, int64_t* __restrict__ order,
    int64_t* __restrict__ inverse, const uint32_t* __restrict__ tile_off, int64_t n, int shift,
    uint32_t mask, int ntiles)
{
    extern __shared__ uint32_t rs_smem[];
    const int bins = (int)mask + 1;
    uint32_t* whist = rs_smem;                    // [RS_WARPS][bins]
    uint32_t* goff = rs_smem + RS_WARPS * bins;   // [bins]
    const int row = blockIdx.y, tile = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < RS_WARPS * bins; i += RS_THREADS) whist[i] = 0;
    __syncthreads();

    const int64_t rbase = (int64_t)row * n;
    const int64_t wbase = (int64_t)tile * RS_TILE + warp * (32 * RS_ITEMS);
    uint64_t key[RS_ITEMS];
    uint32_t rank[RS_ITEMS];
    uint32_t dig[RS_ITEMS];
    const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
    for (int it = 0; it < RS_ITEMS; ++it) {
        const int64_t idx = wbase + it * 32 + lane;
        const bool valid = idx < n;
        key[it] = valid ? keys_in[rbase + idx] : ~0ull;
        // padding elements sit behind every real element of the tile and use
        // the last bin, so they never move a real element's rank
        const uint32_t d = valid ? ((uint32_t)(key[it] >> shift) & mask) : mask;
        dig[it] = d;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(peers) - 1;
        uint32_t cnt = 0;
        if (lane == leader) {
            cnt = whist[warp * bins + d];
            whist[warp * bins + d] = cnt + __popc(peers);
        }
        cnt = __shfl_sync(0xffffffffu, cnt, leader);
        rank[it] = cnt + __popc(peers & lt);
        __syncwarp();
    }
    __syncthreads();
    for (int d = threadIdx.x; d < bins; d += RS_THREADS) {
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < RS_WARPS; ++w) {
            const uint32_t c = whist[w * bins + d];
            whist[w * bins + d] = run;
            run += c;
        }
        goff[d] = tile_off[((int64_t)row * bins + d) * ntiles + tile];
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < RS_ITEMS; ++it) {
        const int64_t idx = wbase + it * 32 + lane;
        if (idx < n) {
            const uint32_t d = dig[it];
            const int64_t dst = (int64_t)goff[d] + whist[warp * bins + d] + rank[it];
            const int32_t v = FIRST ? (int32_t)idx : vals_in[rbase + idx];
            if (LAST) {
                order[rbase + dst] = v;
                inverse[rbase + v] = dst;
            } else {
                keys_out[rbase + dst] = key[it];
                vals_out[rbase + dst] = v;
            }
        }
    }
}

struct SortPlan {
    int passes;
    int bits;      // digit width of every pass but possibly the last
    int ntiles;
    size_t bytes;
};

static SortPlan sort_plan(int k, int64_t n, int sig_bits)
{
    SortPlan p;
    // The kernels take digits of up to RS_MAX_BITS bits; measured on B200, 10-bit digits (5 instead
    // of 7 passes at 49 bits) are no faster at 16 M keys and slower at 0.4 M, because the per-tile
    // histogram table grows with the digit while a tile stays 2048 keys: 8-bit digits are used.
    constexpr int kDigitBits = 8;
    p.passes = sig_bits <= 0 ? 1 : (sig_bits + kDigitBits - 1) / kDigitBits;
    p.bits = sig_bits <= 0 ? 8 : (sig_bits + p.passes - 1) / p.passes;   // spread evenly
    p.ntiles = ceil_div(n, RS_TILE);
    size_t b = 0;
    b += 2 * align_up((size_t)k * n * sizeof(uint64_t), 256);   // key ping-pong
    b += 2 * align_up((size_t)k * n * sizeof(int32_t), 256);    // value ping-pong
    b += align_up((size_t)k * RS_MAX_BINS * p.ntiles * sizeof(uint32_t), 256);
    b += align_up((size_t)p.passes * k * RS_MAX_BINS * sizeof(uint32_t), 256);
    p.bytes = b;
    return p;
}

}  // namespace ptv3

extern "C" size_t ptv3_argsort_workspace_bytes(int k, int64_t n, int sig_bits)
{
    if (k <= 0 || n <= 0) return 0;
    return ptv3::sort_plan(k, n, sig_bits).bytes;
}

extern "C" int ptv3_argsort_inverse(const int64_t* codes, int k, int64_t n, int sig_bits,
                                    int64_t* order, int64_t* inverse, void* workspace,
                                    size_t workspace_bytes, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(k >= 1 && n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_argsort_inverse: bad k/n");
    PTV3_REQUIRE(sig_bits >= 0 && sig_bits <= 63, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_argsort_inverse: sig_bits %d outside [0, 63]", sig_bits);
    PTV3_REQUIRE(n < (1ll << 31) - RS_TILE, PTV3_ERR_UNSUPPORTED,
                 "ptv3_argsort_inverse: n too large for 32-bit indices");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(codes && order && inverse && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_argsort_inverse: null pointer");
    const SortPlan p = sort_plan(k, n, sig_bits);
    PTV3_REQUIRE(workspace_bytes >= p.bytes, PTV3_ERR_WORKSPACE,
                 "ptv3_argsort_inverse: workspace %zu < %zu bytes", workspace_bytes, p.bytes);
    cudaStream_t stream = (cudaStream_t)stream_;
    Carver cv(workspace);
    uint64_t* kbuf[2] = {cv.take<uint64_t>((size_t)k * n), cv.take<uint64_t>((size_t)k * n)};
    int32_t* vbuf[2] = {cv.take<int32_t>((size_t)k * n), cv.take<int32_t>((size_t)k * n)};
    uint32_t* tile_hist = cv.take<uint32_t>((size_t)k * RS_MAX_BINS * p.ntiles);
    uint32_t* totals = cv.take<uint32_t>((size_t)p.passes * k * RS_MAX_BINS);
    if (cudaMemsetAsync(totals, 0, (size_t)p.passes * k * RS_MAX_BINS * sizeof(uint32_t), stream) !=
        cudaSuccess)
        return check_launch("ptv3_argsort_inverse: memset");

    const dim3 grid(p.ntiles, k);
    const uint64_t* kin = reinterpret_cast<const uint64_t*>(codes);
    const int32_t* vin = nullptr;
    int cur = 0;
    const size_t scatter_smem = (size_t)(RS_WARPS + 1) * RS_MAX_BINS * sizeof(uint32_t);
    {
        auto set = [&](const void* f) {
            return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scatter_smem);
        };
        if (set((const void*)rs_scatter_kernel<true, true>) != cudaSuccess ||
            set((const void*)rs_scatter_kernel<true, false>) != cudaSuccess ||
            set((const void*)rs_scatter_kernel<false, true>) != cudaSuccess ||
            set((const void*)rs_scatter_kernel<false, false>) != cudaSuccess)
            return check_launch("ptv3_argsort_inverse: shared memory attribute");
    }
    for (int pass = 0; pass < p.passes; ++pass) {
        const int shift = pass * p.bits;
        const int left = sig_bits - shift;
        const int bits = left >= p.bits ? p.bits : (left <= 0 ? p.bits : left);
        const uint32_t mask = (1u << bits) - 1u;
        const int bins = 1 << bits;
        const size_t smem = (size_t)(RS_WARPS + 1) * bins * sizeof(uint32_t);
        uint32_t* tot = totals + (size_t)pass * k * RS_MAX_BINS;
        rs_hist_kernel<<<grid, RS_THREADS, 0, stream>>>(kin, n, shift, mask, p.ntiles, tile_hist, tot);
        rs_scan_kernel<<<dim3(bins, k), RS_THREADS, 0, stream>>>(tile_hist, tot, p.ntiles);
        const bool first = pass == 0, last = pass == p.passes - 1;
        uint64_t* kout = kbuf[cur];
        int32_t* vout = vbuf[cur];
#define RS_LAUNCH(F, L)                                                                          \
    rs_scatter_kernel<F, L><<<grid, RS_THREADS, smem, stream>>>(kin, vin, kout, vout, order, inverse, \
                                                             tile_hist, n, shift, mask, p.ntiles)
        if (first && last) RS_LAUNCH(true, true);
        else if (first) RS_LAUNCH(true, false);
        else if (last) RS_LAUNCH(false, true);
        else RS_LAUNCH(false, false);
#undef RS_LAUNCH
        kin = kout;
        vin = vout;
        cur ^= 1;
    }
    count_launches(3 * p.passes);
    return check_launch("ptv3_argsort_inverse");
}
