// Offset-sorted pair list of a kernel map, and the convolution over it.
//
// The list holds, for every kernel offset o in turn, the (input row, output row)
// pairs nbr[o][j] >= 0.  It is built from the neighbour table with one flagged
// scan per offset (no sort).  Replaces, together with conv_mma.cu, the
// gather-GEMM-scatter form of spconv.SubMConv3d (model.py:546-552) on the coarse
// levels of the hierarchy.
#include "common.cuh"
#include "conv_mma.cuh"
#include "scan.cuh"

namespace ptv3 {

struct PairFlag {
    const int32_t* nbr;
    int64_t n;
    __device__ bool operator()(int o, int64_t j) const { return nbr[(int64_t)o * n + j] >= 0; }
};

struct PairSink {
    const int32_t* nbr;
    const int64_t* row_order;
    const int32_t* off_start;
    int64_t n;
    int32_t* pair_in;
    int32_t* pair_out;
    __device__ void operator()(int o, int64_t j, uint32_t pos, bool f) const
    {
        if (!f) return;
        const int64_t p = (int64_t)off_start[o] + pos;
        pair_in[p] = nbr[(int64_t)o * n + j];
        pair_out[p] = (int32_t)(row_order ? row_order[j] : j);
    }
};

// totals[o] pairs per offset -> prefix sums of pairs and of 128-pair tiles
__global__ void pair_meta_kernel(const uint32_t* __restrict__ totals, int kvol, int32_t* __restrict__ off_start,
                                 int32_t* __restrict__ tile_start)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int32_t p = 0, t = 0;
        for (int o = 0; o < kvol; ++o) {
            off_start[o] = p;
            tile_start[o] = t;
            p += (int32_t)totals[o];
            t += ((int32_t)totals[o] + 127) / 128;
        }
        off_start[kvol] = p;
        tile_start[kvol] = t;
    }
}

static size_t pairs_ws_bytes(int kvol, int64_t n)
{
    const int ntiles = ceil_div(n, SC_TILE);
    return align_up((size_t)kvol * ntiles * sizeof(uint32_t), 256) + align_up((size_t)kvol * sizeof(uint32_t), 256);
}

}  // namespace ptv3

extern "C" size_t ptv3_conv_pairs_workspace_bytes(int64_t n, int kernel_volume)
{
    return n > 0 ? ptv3::pairs_ws_bytes(kernel_volume, n) : 0;
}

extern "C" int ptv3_conv_pairs_build(const int32_t* nbr, const int64_t* row_order, int64_t n,
                                     int kernel_volume, int32_t* pair_in, int32_t* pair_out,
                                     int32_t* off_start, int32_t* tile_start, void* workspace,
                                     size_t workspace_bytes, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && kernel_volume >= 1 && kernel_volume <= 343, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_conv_pairs_build: bad sizes");
    PTV3_REQUIRE(n * (int64_t)kernel_volume < (1ll << 31), PTV3_ERR_UNSUPPORTED,
                 "ptv3_conv_pairs_build: more than 2^31 candidate pairs");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(nbr && pair_in && pair_out && off_start && tile_start && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_conv_pairs_build: null pointer");
    PTV3_REQUIRE(workspace_bytes >= pairs_ws_bytes(kernel_volume, n), PTV3_ERR_WORKSPACE,
                 "ptv3_conv_pairs_build: workspace too small");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int ntiles = ceil_div(n, SC_TILE);
    Carver cv(workspace);
    uint32_t* tile_sums = cv.take<uint32_t>((size_t)kernel_volume * ntiles);
    uint32_t* totals = cv.take<uint32_t>(kernel_volume);
    PairFlag pf{nbr, n};
    PairSink ps{nbr, row_order, off_start, n, pair_in, pair_out};
    scan_tile_sums_kernel<<<dim3(ntiles, kernel_volume), SC_THREADS, 0, stream>>>(pf, n, ntiles, tile_sums);
    scan_sums_kernel<<<kernel_volume, SC_THREADS, 0, stream>>>(tile_sums, ntiles, totals);
    pair_meta_kernel<<<1, 32, 0, stream>>>(totals, kernel_volume, off_start, tile_start);
    scan_apply_kernel<<<dim3(ntiles, kernel_volume), SC_THREADS, 0, stream>>>(pf, ps, n, ntiles, tile_sums);
    count_launches(4);
    return check_launch("ptv3_conv_pairs_build");
}

extern "C" int ptv3_subm_conv_pairs_fwd(const void* feat, const int32_t* pair_in, const int32_t* pair_out,
                                        const int32_t* off_start, const int32_t* tile_start,
                                        const void* weight, const void* bias, void* out, void* workspace,
                                        size_t workspace_bytes, int64_t n, int c_in, int c_out,
                                        int kernel_volume, int dtype, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && c_in >= 1 && c_out >= 1, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_pairs_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_BF16 && conv_pairs_supported(c_in, c_out, kernel_volume),
                 PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_pairs_fwd: needs bf16, <= 27 offsets, C_in %% 64 == 0, C_out %% 128 == 0");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(feat && pair_in && pair_out && off_start && tile_start && weight && out && workspace,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_subm_conv_pairs_fwd: null pointer");
    PTV3_REQUIRE(workspace_bytes >= (size_t)n * c_out * sizeof(long long), PTV3_ERR_WORKSPACE,
                 "ptv3_subm_conv_pairs_fwd: workspace %zu < %zu bytes", workspace_bytes,
                 (size_t)n * c_out * sizeof(long long));
    PTV3_REQUIRE((((uintptr_t)feat | (uintptr_t)weight | (uintptr_t)workspace) & 15) == 0,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_subm_conv_pairs_fwd: tensors must be 16-byte aligned");
    // every offset ends with at most one partial tile
    const int64_t max_tiles = (n * kernel_volume + 127) / 128 + kernel_volume;
    return launch_conv_pairs(feat, pair_in, pair_out, off_start, tile_start, max_tiles, weight, bias, out,
                             static_cast<long long*>(workspace), n, c_in, c_out, kernel_volume,
                             (cudaStream_t)stream);
}
