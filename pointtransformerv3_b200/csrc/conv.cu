// Submanifold sparse convolution over a prebuilt kernel map:
//   out[i] = bias + sum_o W[:, o, :] . in[nbr[o][i]]      (nbr < 0 contributes 0)
// Replaces spconv.SubMConv3d.forward at model.py:546-552 (xCPE, 27 offsets) and
// model.py:767-774 (stem, 125 offsets).  Weight layout [C_out, k, k, k, C_in].
//
// This file holds the CUDA-core (fp32 FMA) path, used for fp32 features and as
// the baseline the tensor-core path is checked against: a CTA owns 64 voxels x
// TN output channels, skips offsets no voxel of the tile has a neighbour for,
// and gathers the input rows of each remaining offset into shared memory.
#include "common.cuh"
#include "convert.cuh"
#include "conv_mma.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

constexpr int CF_TM = 64;
constexpr int CF_TK = 16;
constexpr int CF_THREADS = 256;

template <typename T, int TN>
__global__ void __launch_bounds__(CF_THREADS) conv_fma_kernel(
    const T* __restrict__ feat, const int32_t* __restrict__ nbr, const T* __restrict__ weight,
    const T* __restrict__ bias, T* __restrict__ out, const int64_t* __restrict__ row_order, int64_t n,
    int cin, int cout, int kvol)
{
    constexpr int CN = TN / 16;  // output columns per thread
    __shared__ float As[CF_TK][CF_TM + 4];
    __shared__ float Bs[CF_TK][TN + 4];
    __shared__ int32_t rows[CF_TM];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int64_t row0 = (int64_t)blockIdx.x * CF_TM;
    const int col0 = blockIdx.y * TN;
    float acc[4][CN];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < CN; ++b) acc[a][b] = 0.f;

    for (int o = 0; o < kvol; ++o) {
        int32_t mine = -1;
        if (tid < CF_TM) {
            const int64_t i = row0 + tid;
            mine = i < n ? nbr[(int64_t)o * n + i] : -1;
        }
        __syncthreads();   // previous offset's reads of rows/As/Bs are done
        if (tid < CF_TM) rows[tid] = mine;
        if (!__syncthreads_or(mine >= 0)) continue;
        for (int kc = 0; kc < cin; kc += CF_TK) {
            // A: 64 rows x 16 k, 4 elements per thread
#pragma unroll
            for (int e = 0; e < (CF_TM * CF_TK) / CF_THREADS; ++e) {
                const int idx = e * CF_THREADS + tid;
                const int r = idx / CF_TK, kk = idx % CF_TK;
                const int32_t src = rows[r];
                float v = 0.f;
                if (src >= 0 && kc + kk < cin) v = to_f<T>(feat[(int64_t)src * cin + kc + kk]);
                As[kk][r] = v;
            }
#pragma unroll
            for (int e = 0; e < (TN * CF_TK) / CF_THREADS; ++e) {
                const int idx = e * CF_THREADS + tid;
                const int c = idx / CF_TK, kk = idx % CF_TK;
                float v = 0.f;
                if (col0 + c < cout && kc + kk < cin)
                    v = to_f<T>(weight[((int64_t)(col0 + c) * kvol + o) * cin + kc + kk]);
                Bs[kk][c] = v;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < CF_TK; ++kk) {
                float a[4], b[CN];
#pragma unroll
                for (int x = 0; x < 4; ++x) a[x] = As[kk][ty * 4 + x];
#pragma unroll
                for (int y = 0; y < CN; ++y) b[y] = Bs[kk][tx * CN + y];
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < CN; ++y) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
            }
            __syncthreads();
        }
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        int64_t i = row0 + ty * 4 + x;
        if (i >= n) continue;
        if (row_order) i = row_order[i];
#pragma unroll
        for (int y = 0; y < CN; ++y) {
            const int c = col0 + tx * CN + y;
            if (c < cout) {
                const float bv = bias ? to_f<T>(bias[c]) : 0.f;
                out[i * cout + c] = from_f<T>(acc[x][y] + bv);
            }
        }
    }
}

template <typename T>
static int launch_conv_fma(const void* feat, const int32_t* nbr, const void* weight, const void* bias,
                           void* out, const int64_t* row_order, int64_t n, int cin, int cout, int kvol,
                           cudaStream_t stream)
{
    const unsigned gx = (unsigned)((n + CF_TM - 1) / CF_TM);
    if (cout <= 32) {
        conv_fma_kernel<T, 32><<<dim3(gx, (cout + 31) / 32), CF_THREADS, 0, stream>>>(
            (const T*)feat, nbr, (const T*)weight, (const T*)bias, (T*)out, row_order, n, cin, cout, kvol);
    } else {
        conv_fma_kernel<T, 64><<<dim3(gx, (cout + 63) / 64), CF_THREADS, 0, stream>>>(
            (const T*)feat, nbr, (const T*)weight, (const T*)bias, (T*)out, row_order, n, cin, cout, kvol);
    }
    count_launches(1);
    return check_launch("ptv3_subm_conv_fwd");
}

}  // namespace ptv3

extern "C" int ptv3_subm_conv_fwd(const void* feat, const int32_t* nbr, const void* weight,
                                  const void* bias, void* out, const int64_t* row_order, int64_t n,
                                  int c_in, int c_out, int kernel_volume, int dtype, int algo,
                                  uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && c_in >= 1 && c_out >= 1 && kernel_volume >= 1, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_fwd: dtype %d", dtype);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(feat && nbr && weight && out, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_fwd: null pointer");
    PTV3_REQUIRE(algo >= 0 && algo <= 3, PTV3_ERR_INVALID_ARGUMENT, "ptv3_subm_conv_fwd: algo %d", algo);
    const bool mma_ok = dtype == PTV3_DTYPE_BF16 && conv_mma_supported(c_in, c_out, kernel_volume) &&
                        ((uintptr_t)feat & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                        ((uintptr_t)out & 3) == 0;
    PTV3_REQUIRE(algo != 2 || mma_ok, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_fwd: the tensor-core path needs bf16, <= 27 offsets, channels 32->32 or "
                 "C_in %% 64 == 0 with C_out 64 or a multiple of 128, and 16-byte aligned tensors");
    const bool tc_ok = dtype == PTV3_DTYPE_BF16 && conv_tc05_supported(c_in, c_out, kernel_volume) && status &&
                       n < (1ll << 31) && ((uintptr_t)feat & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                       ((uintptr_t)out & 15) == 0;
    PTV3_REQUIRE(algo != 3 || tc_ok, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_fwd: the tcgen05 path needs bf16, <= 27 offsets, channels 32->32 or multiples of "
                 "64, a status word and 16-byte aligned tensors");
    // automatic choice: tensor memory for 64 channels and more; at 32 channels a stage of the tcgen05
    // pipeline is too small for its fixed cost and the mma.sync kernel is faster
    if (tc_ok && (algo == 3 || (algo == 0 && c_in >= 64)))
        return launch_conv_tc05(feat, nbr, weight, bias, out, row_order, n, c_in, c_out, kernel_volume, status,
                                (cudaStream_t)stream);
    if (mma_ok && algo != 1)
        return launch_conv_mma(feat, nbr, weight, bias, out, row_order, n, c_in, c_out, kernel_volume,
                               (cudaStream_t)stream);
    if (dtype == PTV3_DTYPE_F32)
        return launch_conv_fma<float>(feat, nbr, weight, bias, out, row_order, n, c_in, c_out,
                                      kernel_volume, (cudaStream_t)stream);
    return launch_conv_fma<__nv_bfloat16>(feat, nbr, weight, bias, out, row_order, n, c_in, c_out,
                                          kernel_volume, (cudaStream_t)stream);
}
