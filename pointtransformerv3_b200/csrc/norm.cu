// Row-wise residual + LayerNorm fusion for the glue between the GEMMs of a block:
//
//     t   = ln1 ? LayerNorm1(x) : x
//     sum = residual ? residual + t : t          -> sum_out   (optional)
//     y   = LayerNorm2(sum)                      -> norm_out  (optional)
//
// which covers `feat = shortcut + LN(Linear(conv))` followed by the pre-norm of
// the attention (model.py:553-554,589-592), `feat = shortcut + proj(attn)`
// followed by the pre-norm of the MLP (model.py:594,598-600), the plain residual
// add after the MLP (model.py:602) and a stand-alone LayerNorm.  Every
// intermediate that the unfused sequence would write is rounded to the element
// type exactly where that sequence rounds it.  HBM-bound: each tensor is read
// or written once, with 16-byte accesses; a row is owned by 4..32 lanes.
#include "common.cuh"
#include "vec.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

template <int LANES>
__device__ __forceinline__ float group_sum(float v)
{
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// LANES lanes own a row; each lane holds VPL vectors (VPL * Vec<T>::N channels)
template <typename T, int LANES, int VPL>
__global__ void __launch_bounds__(256) add_ln_kernel(
    const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ g1,
    const T* __restrict__ b1, float eps1, T* __restrict__ sum_out, const T* __restrict__ g2,
    const T* __restrict__ b2, float eps2, T* __restrict__ norm_out, int64_t n, int C)
{
    pdl_launch_next();
    pdl_wait();
    using V = Vec<T>;
    constexpr int E = VPL * V::N;
    const int lane_in_row = threadIdx.x % LANES;
    const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) / LANES;
    const bool active = row < n;
    const float inv_c = 1.f / (float)C;
    float v[E];
    // channel of element e of this lane: vectors are interleaved over the lanes
    auto ch = [&](int k) { return (k * LANES + lane_in_row) * V::N; };
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        if (active) {
            V::unpack(*reinterpret_cast<const typename V::Raw*>(x + row * C + ch(k)), v + k * V::N);
        } else {
#pragma unroll
            for (int i = 0; i < V::N; ++i) v[k * V::N + i] = 0.f;
        }
    }
    auto layer_norm = [&](const T* g, const T* b, float eps) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) s += v[e];
        const float mean = group_sum<LANES>(s) * inv_c;
        float q = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) q += (v[e] - mean) * (v[e] - mean);
        const float rstd = rsqrtf(group_sum<LANES>(q) * inv_c + eps);
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
            float gg[V::N], bb[V::N];
            V::unpack(*reinterpret_cast<const typename V::Raw*>(g + ch(k)), gg);
            V::unpack(*reinterpret_cast<const typename V::Raw*>(b + ch(k)), bb);
#pragma unroll
            for (int i = 0; i < V::N; ++i)
                v[k * V::N + i] = V::round(fmaf((v[k * V::N + i] - mean) * rstd, gg[i], bb[i]));
        }
    };
    if (g1) layer_norm(g1, b1, eps1);
    if (residual) {
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
            float r[V::N];
            if (active) {
                V::unpack(*reinterpret_cast<const typename V::Raw*>(residual + row * C + ch(k)), r);
#pragma unroll
                for (int i = 0; i < V::N; ++i) v[k * V::N + i] = V::round(r[i] + v[k * V::N + i]);
            }
        }
    }
    if (sum_out && active) {
#pragma unroll
        for (int k = 0; k < VPL; ++k)
            *reinterpret_cast<typename V::Raw*>(sum_out + row * C + ch(k)) = V::pack(v + k * V::N);
    }
    if (norm_out) {
        layer_norm(g2, b2, eps2);
        if (active) {
#pragma unroll
            for (int k = 0; k < VPL; ++k)
                *reinterpret_cast<typename V::Raw*>(norm_out + row * C + ch(k)) = V::pack(v + k * V::N);
        }
    }
}

template <typename T, int LANES, int VPL>
static void launch_add_ln(const void* x, const void* residual, const void* g1, const void* b1, float eps1,
                          void* sum_out, const void* g2, const void* b2, float eps2, void* norm_out,
                          int64_t n, int C, cudaStream_t stream)
{
    const int64_t threads = n * LANES;
    launch_dependent(add_ln_kernel<T, LANES, VPL>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream,
                     (const T*)x, (const T*)residual, (const T*)g1, (const T*)b1, eps1, (T*)sum_out, (const T*)g2,
                     (const T*)b2, eps2, (T*)norm_out, n, C);
}

template <typename T>
static int dispatch_add_ln(const void* x, const void* residual, const void* g1, const void* b1, float eps1,
                           void* sum_out, const void* g2, const void* b2, float eps2, void* norm_out,
                           int64_t n, int C, cudaStream_t stream)
{
    const int vectors = C / Vec<T>::N;   // per row
#define ALN(L, V) launch_add_ln<T, L, V>(x, residual, g1, b1, eps1, sum_out, g2, b2, eps2, norm_out, n, C, stream)
    switch (vectors) {
        case 1: ALN(1, 1); break;
        case 2: ALN(2, 1); break;
        case 4: ALN(4, 1); break;
        case 8: ALN(8, 1); break;
        case 16: ALN(16, 1); break;
        case 32: ALN(32, 1); break;
        case 64: ALN(32, 2); break;
        case 128: ALN(32, 4); break;
        case 256: ALN(32, 8); break;
        case 6: ALN(2, 3); break;
        case 12: ALN(4, 3); break;
        case 24: ALN(8, 3); break;
        case 48: ALN(16, 3); break;
        case 96: ALN(32, 3); break;
        default:
            set_error("ptv3_add_layernorm_fwd: %d channels are not supported (need a power of two or 3 x a "
                      "power of two, times %d, up to %d)", C, Vec<T>::N, 256 * Vec<T>::N);
            return PTV3_ERR_UNSUPPORTED;
    }
#undef ALN
    count_launches(1);
    return check_launch("ptv3_add_layernorm_fwd");
}

}  // namespace ptv3

extern "C" int ptv3_add_layernorm_fwd(const void* x, const void* residual, const void* ln1_weight,
                                      const void* ln1_bias, float ln1_eps, void* sum_out,
                                      const void* ln2_weight, const void* ln2_bias, float ln2_eps,
                                      void* norm_out, int64_t n, int channels, int dtype, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && channels >= 1, PTV3_ERR_INVALID_ARGUMENT, "ptv3_add_layernorm_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_add_layernorm_fwd: dtype %d", dtype);
    if (n == 0) return PTV3_OK;   // empty tensors carry null pointers
    PTV3_REQUIRE((ln1_weight == nullptr) == (ln1_bias == nullptr) &&
                     (ln2_weight == nullptr) == (ln2_bias == nullptr),
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_add_layernorm_fwd: weight and bias go together");
    PTV3_REQUIRE((norm_out == nullptr) == (ln2_weight == nullptr), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_add_layernorm_fwd: norm_out goes with the second LayerNorm");
    PTV3_REQUIRE(sum_out || norm_out, PTV3_ERR_INVALID_ARGUMENT, "ptv3_add_layernorm_fwd: no output");
    const int vn = dtype == PTV3_DTYPE_F32 ? 4 : 8;
    PTV3_REQUIRE(channels % vn == 0, PTV3_ERR_UNSUPPORTED,
                 "ptv3_add_layernorm_fwd: channels %d not a multiple of %d", channels, vn);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(x, PTV3_ERR_INVALID_ARGUMENT, "ptv3_add_layernorm_fwd: null input");
    if (dtype == PTV3_DTYPE_F32)
        return dispatch_add_ln<float>(x, residual, ln1_weight, ln1_bias, ln1_eps, sum_out, ln2_weight,
                                      ln2_bias, ln2_eps, norm_out, n, channels, (cudaStream_t)stream);
    return dispatch_add_ln<__nv_bfloat16>(x, residual, ln1_weight, ln1_bias, ln1_eps, sum_out, ln2_weight,
                                          ln2_bias, ln2_eps, norm_out, n, channels, (cudaStream_t)stream);
}
