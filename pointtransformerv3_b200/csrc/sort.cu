// Stable LSD radix argsort of k rows of n non-negative int64 codes, restricted
// to the significant low bits, with the inverse permutation written by the last
// pass.  Replaces torch.argsort + scatter_ at model.py:118-126 and :667-674
// (ties are resolved by original index, the canonical order).
//
// One-sweep form: one kernel reads every key once and builds the digit
// histograms of ALL passes; after that every pass is a single kernel.  A tile of
// a pass ranks its keys by digit in shared memory, publishes its per-digit counts
// in a status table and obtains its global offsets by looking back over the
// status words of the tiles before it (decoupled look-back), so a pass reads and
// writes every element exactly once.  Digits are up to 10 bits wide and spread
// evenly over the significant bits (29 bits -> 3 passes, 49 bits -> 5 passes).
// The first pass reads the caller's codes and takes an element's value to be its
// index; the last pass writes order / inverse as int64 and drops the keys.
//
// Bytes per element: 8 (histograms) + 8 + 12 (first pass) + 24 per middle pass +
// 12 + 16 (last pass).  Measured on B200 a pass runs at 50-60 G elements per second
// (16 M x 4 rows of 49 significant bits: 6.5 ms): a tile's life is a chain of short
// phases separated by barriers, and the scattered shared-memory accesses of the
// ranking and the reordering (several bank conflicts per access on random digits)
// take a third of it, so the kernel sits far below the HBM bound of its 24 bytes.
//
// Tiles take their number from a counter when they start, so every tile a tile
// waits for is already running or finished; all the same every wait is bounded
// and a wait that runs out sets PTV3_STATUS_WAIT_LIMIT.
#include "common.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

constexpr int OS_THREADS = 512;
constexpr int OS_WARPS = OS_THREADS / 32;
constexpr int OS_ITEMS = 8;
constexpr int OS_TILE = OS_THREADS * OS_ITEMS;   // 4096 keys per tile
constexpr int OS_MAX_BITS = 10;
constexpr int OS_MAX_BINS = 1 << OS_MAX_BITS;
constexpr int OS_DPT = OS_MAX_BINS / OS_THREADS;  // digits a thread looks after
constexpr int OS_MAX_PASSES = 7;                  // 63 bits / 10 -> 7
constexpr uint32_t OS_COUNT_MASK = (1u << 28) - 1u;
constexpr uint32_t OS_SPIN_LIMIT = 1u << 20;
constexpr int OS_WINDOW = 8;                     // earlier tiles inspected per round trip

struct SortPlan {
    int passes;
    int bits;      // digit width of every pass but possibly the last
    int ntiles;
    size_t bytes;
};

// Digit histograms of every pass in one read of the keys: hist[row][pass][digit].
__global__ void __launch_bounds__(OS_THREADS) os_hist_kernel(const uint64_t* __restrict__ keys, int64_t n,
                                                            int sig_bits, int bits, int passes,
                                                            uint32_t* __restrict__ hist)
{
    extern __shared__ uint32_t os_smem[];      // [passes][OS_MAX_BINS]
    const int row = blockIdx.y;
    for (int i = threadIdx.x; i < passes * OS_MAX_BINS; i += OS_THREADS) os_smem[i] = 0;
    __syncthreads();
    const uint64_t* k = keys + (int64_t)row * n;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t idx = (int64_t)blockIdx.x * OS_THREADS + threadIdx.x; idx < n;
         idx += (int64_t)gridDim.x * OS_THREADS) {
        const uint64_t key = k[idx];
        for (int p = 0; p < passes; ++p)
            atomicAdd(&os_smem[p * OS_MAX_BINS + ((uint32_t)(key >> (p * bits)) & mask)], 1u);
    }
    __syncthreads();
    uint32_t* out = hist + (size_t)row * OS_MAX_PASSES * OS_MAX_BINS;
    for (int i = threadIdx.x; i < passes * OS_MAX_BINS; i += OS_THREADS) {
        const uint32_t c = os_smem[i];
        if (c) atomicAdd(&out[i], c);
    }
}

// exclusive scan over the block of one value per thread (two 32-bit sums packed in 64 bits)
__device__ __forceinline__ uint64_t os_block_excl_scan(uint64_t v, uint64_t* warp_sums)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint64_t u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    uint64_t base = 0;
#pragma unroll
    for (int w = 0; w < OS_WARPS; ++w)
        if (w < warp) base += warp_sums[w];
    return base + inc - v;
}

// lanes of the warp whose digit equals this lane's, among the lanes in `vmask`: one ballot per
// digit bit, all independent of each other (the match.any instruction takes about a thousand
// cycles on many distinct values)
__device__ __forceinline__ uint32_t os_match(uint32_t d, int bits, uint32_t vmask)
{
    uint32_t peers = vmask;
#pragma unroll
    for (int b = 0; b < OS_MAX_BITS; ++b) {
        if (b < bits) {     // uniform over the grid
            const bool bit = (d >> b) & 1u;
            const uint32_t bal = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? bal : ~bal;
        }
    }
    return peers;
}

// One pass over one tile.  Element order inside a tile is warp-major: warp w owns
// [w * 256, (w + 1) * 256), visited 32 consecutive elements at a time, so that
// (warp, item, lane) order is index order and ranks taken in that order are stable.
//
// Order of the steps: counts first (a histogram with shared-memory atomics) and their
// publication; then the ranking and the reordering in shared memory; the look-back last.  By
// then the tiles before this one, which started earlier, have mostly finished their own
// look-back, so the walk finds an inclusive prefix after one or two tiles.  (With the look-back
// first, a tile meets hundreds of tiles in the "counts only" state; that walk then takes longer
// than everything else and keeps itself long.)
template <bool FIRST, bool LAST>
__global__ void __launch_bounds__(OS_THREADS, 2) os_pass_kernel(
    const uint64_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
    uint64_t* __restrict__ keys_out, int32_t* __restrict__ vals_out, int64_t* __restrict__ order,
    int64_t* __restrict__ inverse, const uint32_t* __restrict__ hist, uint32_t* __restrict__ tile_status,
    uint32_t* __restrict__ tile_counter, uint32_t* __restrict__ status, int64_t n, int shift, int bits,
    int pass, int ntiles, int k_rows)
{
    extern __shared__ __align__(16) unsigned char os_raw[];
    const int bins = 1 << bits;
    uint64_t* skeys = reinterpret_cast<uint64_t*>(os_raw);                       // [OS_TILE]
    int32_t* svals = reinterpret_cast<int32_t*>(skeys + OS_TILE);                // [OS_TILE]
    uint16_t* whist = reinterpret_cast<uint16_t*>(svals + OS_TILE);              // [OS_WARPS][bins]
    uint32_t* local_off = reinterpret_cast<uint32_t*>(whist + OS_WARPS * bins);  // [bins + 1]
    uint32_t* gprefix = local_off + bins + 1;                                    // [bins]
    __shared__ uint64_t warp_sums[OS_WARPS];
    __shared__ uint32_t tile_s;
    __shared__ int give_up;

    // rows take turns over the grid, so every row has the same share of the running tiles (a
    // tile waits only for tiles of its own row)
    const int row = blockIdx.x % k_rows;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t mask = (uint32_t)bins - 1u;
    if (threadIdx.x == 0) {
        tile_s = atomicAdd(&tile_counter[pass * k_rows + row], 1u);
        give_up = 0;
    }
    // (bins >= 2: the 16-bit counters are cleared and counted in pairs)
    for (int i = threadIdx.x; i < OS_WARPS * bins / 2; i += OS_THREADS) reinterpret_cast<uint32_t*>(whist)[i] = 0;
    __syncthreads();
    const int tile = (int)tile_s;
    if (tile >= ntiles) return;    // cannot happen with a grid of ntiles blocks per row

    const int64_t rbase = (int64_t)row * n;
    const int64_t tbase = (int64_t)tile * OS_TILE;
    const int64_t wbase = tbase + warp * (32 * OS_ITEMS);
    const int tile_count = (int)min((int64_t)OS_TILE, n - tbase);

    // ---- load; count the digits per warp ------------------------------------------------------
    uint64_t key[OS_ITEMS];
    int32_t val[OS_ITEMS];
    uint16_t* wh = whist + warp * bins;
#pragma unroll
    for (int it = 0; it < OS_ITEMS; ++it) {
        const int64_t idx = wbase + it * 32 + lane;
        key[it] = idx < n ? keys_in[rbase + idx] : ~0ull;
        val[it] = FIRST ? (int32_t)idx : (idx < n ? vals_in[rbase + idx] : 0);
    }
    {
        // a warp holds at most 256 elements, so two 16-bit counters share a word without carries
        uint32_t* wh32 = reinterpret_cast<uint32_t*>(wh);
#pragma unroll
        for (int it = 0; it < OS_ITEMS; ++it) {
            const int64_t idx = wbase + it * 32 + lane;
            if (idx < n) {
                const uint32_t d = (uint32_t)(key[it] >> shift) & mask;
                atomicAdd(&wh32[d >> 1], (d & 1u) ? 0x10000u : 1u);
            }
        }
    }
    __syncthreads();

    // ---- per digit: offsets of the warps and of the digit inside the tile -----------------------
    // For the scans thread t owns the contiguous digits t * dpt .. t * dpt + dpt - 1; for the
    // status table (below) it owns the interleaved digits t, t + 256, ..., so that a warp's
    // status reads and writes are contiguous in memory.  The two views meet in shared memory.
    const int dpt = bins > OS_THREADS ? bins / OS_THREADS : 1;
    const bool has_digit = threadIdx.x * dpt < bins;
    uint32_t* st_row = tile_status + ((size_t)row * ntiles) * OS_MAX_BINS;
    const uint32_t code_agg = (uint32_t)(2 * pass + 1) << 28, code_inc = (uint32_t)(2 * pass + 2) << 28;
    {
        uint32_t cnt[OS_DPT], gcnt[OS_DPT];
        uint32_t mine = 0, gmine = 0;
        const uint32_t* gh = hist + ((size_t)row * OS_MAX_PASSES + pass) * OS_MAX_BINS;
#pragma unroll
        for (int j = 0; j < OS_DPT; ++j) {
            cnt[j] = gcnt[j] = 0;
            if (j < dpt && has_digit) {
                const int d = threadIdx.x * dpt + j;
                uint32_t run = 0;
#pragma unroll
                for (int w = 0; w < OS_WARPS; ++w) {
                    const uint32_t c = whist[w * bins + d];
                    whist[w * bins + d] = (uint16_t)run;
                    run += c;
                }
                cnt[j] = run;
                mine += run;
                gcnt[j] = gh[d];
                gmine += gcnt[j];
            }
        }
        // exclusive prefixes over the digits: of the tile's counts (low word) and of the global
        // histogram (high word: start of every digit's range in the output)
        const uint64_t both = os_block_excl_scan(((uint64_t)gmine << 32) | mine, warp_sums);
        uint32_t excl = (uint32_t)both, gexcl = (uint32_t)(both >> 32);
#pragma unroll
        for (int j = 0; j < OS_DPT; ++j) {
            if (j < dpt && has_digit) {
                const int d = threadIdx.x * dpt + j;
                local_off[d] = excl;
                gprefix[d] = gexcl;          // the look-back adds the earlier tiles' counts
                excl += cnt[j];
                gexcl += gcnt[j];
            }
        }
        if (threadIdx.x == 0) local_off[bins] = (uint32_t)tile_count;
    }
    __syncthreads();

    // ---- publish the tile's counts (the first tile's counts are inclusive prefixes already) ----
    uint32_t cnt[OS_DPT], look[OS_DPT];
#pragma unroll
    for (int j = 0; j < OS_DPT; ++j) {
        const int d = j * OS_THREADS + threadIdx.x;
        cnt[j] = look[j] = 0;
        if (d < bins) {
            cnt[j] = local_off[d + 1] - local_off[d];
            *reinterpret_cast<volatile uint32_t*>(&st_row[(size_t)tile * OS_MAX_BINS + d]) =
                (tile == 0 ? code_inc : code_agg) | cnt[j];
        }
    }

    // ---- rank inside the warp and order the tile by digit in shared memory ------------------------
    {
        const uint32_t lt = (1u << lane) - 1u;
        // the matches of all items first (independent ballots), then the chain through the
        // per-warp running offsets
        uint32_t peers[OS_ITEMS];
#pragma unroll
        for (int it = 0; it < OS_ITEMS; ++it) {
            const int64_t idx = wbase + it * 32 + lane;
            const uint32_t d = (uint32_t)(key[it] >> shift) & mask;
            const uint32_t vmask = __ballot_sync(0xffffffffu, idx < n);
            peers[it] = os_match(d, bits, vmask);
        }
#pragma unroll
        for (int it = 0; it < OS_ITEMS; ++it) {
            const int64_t idx = wbase + it * 32 + lane;
            const bool valid = idx < n;
            const uint32_t d = (uint32_t)(key[it] >> shift) & mask;
            // every lane takes part in one shuffle with its own source lane (a shuffle per group
            // of equal digits would run the groups one after the other)
            const int leader = valid ? __ffs(peers[it]) - 1 : lane;
            uint32_t base = 0;
            if (valid && lane == leader) {
                base = wh[d];
                wh[d] = (uint16_t)(base + __popc(peers[it]));
            }
            base = __shfl_sync(0xffffffffu, base, leader);
            if (valid) {
                const uint32_t pos = local_off[d] + base + __popc(peers[it] & lt);
                skeys[pos] = key[it];
                svals[pos] = val[it];
            }
            __syncwarp();
        }
    }
    // ---- look back over the earlier tiles: all of this thread's digits at once, and a window of
    //      tiles per digit and round trip (the loads of a window do not depend on each other)
    if (tile > 0) {
        int back[OS_DPT];
        bool done[OS_DPT];
#pragma unroll
        for (int j = 0; j < OS_DPT; ++j) {
            back[j] = tile - 1;
            done[j] = j * OS_THREADS + threadIdx.x >= bins;
        }
        uint32_t spins = 0;
        bool all = false;
        while (!all) {
            uint32_t s[OS_DPT][OS_WINDOW];
#pragma unroll
            for (int j = 0; j < OS_DPT; ++j) {
                const int d = j * OS_THREADS + threadIdx.x;
#pragma unroll
                for (int q = 0; q < OS_WINDOW; ++q) {
                    const int tb = back[j] - q;
                    s[j][q] = code_inc;      // before the first tile: an inclusive prefix of zero
                    if (!done[j] && tb >= 0)
                        s[j][q] = *reinterpret_cast<volatile uint32_t*>(&st_row[(size_t)tb * OS_MAX_BINS + d]);
                }
            }
            all = true;
#pragma unroll
            for (int j = 0; j < OS_DPT; ++j) {
                if (done[j]) continue;
                bool stop = false;
#pragma unroll
                for (int q = 0; q < OS_WINDOW; ++q) {
                    const uint32_t code = s[j][q] & ~OS_COUNT_MASK;
                    if (stop || done[j]) continue;
                    if (code == code_inc) {
                        look[j] += s[j][q] & OS_COUNT_MASK;
                        done[j] = true;
                    } else if (code == code_agg) {
                        look[j] += s[j][q] & OS_COUNT_MASK;
                        --back[j];
                    } else {
                        stop = true;        // not published yet: ask again from this tile on
                    }
                }
                if (!done[j]) all = false;
            }
            if (!all && (++spins > OS_SPIN_LIMIT || *reinterpret_cast<volatile int*>(&give_up))) {
                give_up = 1;
                break;
            }
        }
    }
    // publish the inclusive prefixes; global offset of the tile's share of every digit
#pragma unroll
    for (int j = 0; j < OS_DPT; ++j) {
        const int d = j * OS_THREADS + threadIdx.x;
        if (d < bins) {
            if (tile > 0)
                *reinterpret_cast<volatile uint32_t*>(&st_row[(size_t)tile * OS_MAX_BINS + d]) =
                    code_inc | ((look[j] + cnt[j]) & OS_COUNT_MASK);
            gprefix[d] += look[j];
        }
    }
    __syncthreads();
    if (give_up) {
        if (threadIdx.x == 0 && status) atomicOr(status, PTV3_STATUS_WAIT_LIMIT);
        return;
    }

    // ---- write out: neighbours in shared memory with the same digit are neighbours in global
    for (int i = threadIdx.x; i < tile_count; i += OS_THREADS) {
        const uint64_t kx = skeys[i];
        const uint32_t d = (uint32_t)(kx >> shift) & mask;
        const int64_t dst = (int64_t)gprefix[d] + (i - (int)local_off[d]);
        const int32_t v = svals[i];
        if (LAST) {
            order[rbase + dst] = v;
            inverse[rbase + v] = dst;
        } else {
            keys_out[rbase + dst] = kx;
            vals_out[rbase + dst] = v;
        }
    }
}

static size_t os_pass_smem(int bits)
{
    const size_t bins = (size_t)1 << bits;
    return (size_t)OS_TILE * 12 + OS_WARPS * bins * 2 + (2 * bins + 1) * 4;
}

static SortPlan sort_plan(int k, int64_t n, int sig_bits)
{
    SortPlan p;
    p.passes = sig_bits <= 0 ? 1 : (sig_bits + OS_MAX_BITS - 1) / OS_MAX_BITS;
    p.bits = sig_bits <= 0 ? 8 : (sig_bits + p.passes - 1) / p.passes;   // spread evenly
    p.ntiles = ceil_div(n, OS_TILE);
    size_t b = 0;
    b += 2 * align_up((size_t)k * n * sizeof(uint64_t), 256);   // key ping-pong
    b += 2 * align_up((size_t)k * n * sizeof(int32_t), 256);    // value ping-pong
    // zeroed region: histograms, tile counters, tile status
    b += align_up((size_t)k * OS_MAX_PASSES * OS_MAX_BINS * sizeof(uint32_t), 256);
    b += align_up((size_t)k * OS_MAX_PASSES * sizeof(uint32_t), 256);
    b += align_up((size_t)k * p.ntiles * OS_MAX_BINS * sizeof(uint32_t), 256);
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
                                    int64_t* order, int64_t* inverse, uint32_t* status, void* workspace,
                                    size_t workspace_bytes, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(k >= 1 && k <= 65535 && n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_argsort_inverse: bad k/n");
    PTV3_REQUIRE(sig_bits >= 0 && sig_bits <= 63, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_argsort_inverse: sig_bits %d outside [0, 63]", sig_bits);
    PTV3_REQUIRE(n <= (int64_t)OS_COUNT_MASK, PTV3_ERR_UNSUPPORTED,
                 "ptv3_argsort_inverse: more than 2^28 - 1 elements per row");
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
    char* zero_lo = cv.base + cv.off;
    uint32_t* hist = cv.take<uint32_t>((size_t)k * OS_MAX_PASSES * OS_MAX_BINS);
    uint32_t* counters = cv.take<uint32_t>((size_t)k * OS_MAX_PASSES);
    uint32_t* tile_status = cv.take<uint32_t>((size_t)k * p.ntiles * OS_MAX_BINS);
    if (cudaMemsetAsync(zero_lo, 0, (size_t)(cv.base + cv.off - zero_lo), stream) != cudaSuccess)
        return check_launch("ptv3_argsort_inverse: memset");

    const uint64_t* kin = reinterpret_cast<const uint64_t*>(codes);
    {
        const int hb = (int)std::min<int64_t>(ceil_div(n, OS_THREADS * 8), 4 * 148);
        os_hist_kernel<<<dim3(hb, k), OS_THREADS, (size_t)p.passes * OS_MAX_BINS * sizeof(uint32_t), stream>>>(
            kin, n, sig_bits, p.bits, p.passes, hist);
    }
    const size_t max_smem = os_pass_smem(OS_MAX_BITS);
    {
        auto set = [&](const void* f) {
            return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)max_smem);
        };
        if (set((const void*)os_pass_kernel<true, true>) != cudaSuccess ||
            set((const void*)os_pass_kernel<true, false>) != cudaSuccess ||
            set((const void*)os_pass_kernel<false, true>) != cudaSuccess ||
            set((const void*)os_pass_kernel<false, false>) != cudaSuccess)
            return check_launch("ptv3_argsort_inverse: shared memory attribute");
    }
    const dim3 grid((unsigned)((size_t)p.ntiles * k));
    const int32_t* vin = nullptr;
    int cur = 0;
    for (int pass = 0; pass < p.passes; ++pass) {
        const int shift = pass * p.bits;
        // the histogram kernel cuts every digit with the full width; the last digit then only
        // holds the bits that are left, which is the same value (nothing is set above sig_bits)
        const int bits = p.bits;
        const size_t smem = os_pass_smem(bits);
        const bool first = pass == 0, last = pass == p.passes - 1;
        uint64_t* kout = kbuf[cur];
        int32_t* vout = vbuf[cur];
#define OS_LAUNCH(F, L)                                                                              \
    os_pass_kernel<F, L><<<grid, OS_THREADS, smem, stream>>>(kin, vin, kout, vout, order, inverse, hist, \
                                                           tile_status, counters, status, n, shift, bits, \
                                                           pass, p.ntiles, k)
        if (first && last) OS_LAUNCH(true, true);
        else if (first) OS_LAUNCH(true, false);
        else if (last) OS_LAUNCH(false, true);
        else OS_LAUNCH(false, false);
#undef OS_LAUNCH
        kin = kout;
        vin = vout;
        cur ^= 1;
    }
    count_launches(1 + p.passes);
    return check_launch("ptv3_argsort_inverse");
}
