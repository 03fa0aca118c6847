// Feature side of serialized pooling / unpooling.
//
// pool:   out[c] = GELU(BN(max over the points of cluster c of x))   and the
//         mean coordinate of the cluster.  Replaces torch_scatter.segment_csr at
//         model.py:684-689 together with the BatchNorm1d(eval) + GELU that follow
//         (model.py:707-710).  The points of a cluster are contiguous in the
//         sorted order the plan was built from, so a segment is a run of that
//         order; one warp owns a cluster and reads whole rows with 16-byte loads.
// unpool: out[i] = GELU(BN_s(skip[i])) + GELU(BN_c(child[cluster[i]])), and the
//         first term alone as a second output.  Replaces model.py:726-735,
//         :744-746 after the two Linear layers.
// BatchNorm in eval mode is passed as per-channel scale/shift (fp32).
#include "common.cuh"
#include "convert.cuh"
#include "vec.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

// GELU in its erf form.  fp32 features take the library erff; bf16 features the tanh-based
// form (fit + hardware tanh, relative error ~5e-4, below the bf16 rounding that follows),
// which costs a quarter of the instructions: with erff these kernels are bound by
// arithmetic, not by memory.
template <typename T>
__device__ __forceinline__ float gelu_for(float x)
{
    if (sizeof(T) == 2) return gelu_tanh_erf(x);
    return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
}

// LANES lanes own a cluster (LANES * Vec<T>::N channels per pass); the first three
// lanes of a group also average the coordinates.  C must be a multiple of Vec<T>::N.
// REDUCE: 0 max, 1 min, 2 sum, 3 mean (torch_scatter.segment_csr's reduce argument)
template <typename T, int LANES, int REDUCE>
__global__ void __launch_bounds__(256, 4) pool_max_kernel(const T* __restrict__ x, const float* __restrict__ coord,
                                                       const int64_t* __restrict__ indices,
                                                       const int64_t* __restrict__ idx_ptr, int64_t m, int C,
                                                       const float* __restrict__ scale,
                                                       const float* __restrict__ shift, T* __restrict__ out,
                                                       float* __restrict__ coord_out)
{
    pdl_launch_next();
    pdl_wait();
    using V = Vec<T>;
    const int sub = threadIdx.x % LANES;
    const int64_t c = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) / LANES;
    if (c >= m) return;
    const int64_t lo = idx_ptr[c], hi = idx_ptr[c + 1];
    constexpr int CHUNK = 4;     // members fetched together (a stride-2 cluster has 4 on average, at most 8)
    float cacc = 0.f;
    for (int ch = sub * V::N; ch < C; ch += LANES * V::N) {
        float best[V::N];
#pragma unroll
        for (int i = 0; i < V::N; ++i) best[i] = REDUCE == 0 ? -INFINITY : (REDUCE == 1 ? INFINITY : 0.f);
        for (int64_t j0 = lo; j0 < hi; j0 += CHUNK) {
            // the member indices first, then all their rows: independent loads, one latency each
            int64_t p[CHUNK];
#pragma unroll
            for (int k = 0; k < CHUNK; ++k) p[k] = j0 + k < hi ? indices[j0 + k] : -1;
            typename V::Raw raw[CHUNK];
#pragma unroll
            for (int k = 0; k < CHUNK; ++k)
                if (p[k] >= 0) raw[k] = *reinterpret_cast<const typename V::Raw*>(x + p[k] * C + ch);
            if (coord_out && sub < 3 && ch == sub * V::N) {
#pragma unroll
                for (int k = 0; k < CHUNK; ++k)
                    if (p[k] >= 0) cacc += coord[3 * p[k] + sub];
            }
#pragma unroll
            for (int k = 0; k < CHUNK; ++k) {
                if (p[k] < 0) continue;
                float f[V::N];
                V::unpack(raw[k], f);
#pragma unroll
                for (int i = 0; i < V::N; ++i)
                    best[i] = REDUCE == 0 ? fmaxf(best[i], f[i])
                                          : (REDUCE == 1 ? fminf(best[i], f[i]) : best[i] + f[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < V::N; ++i) {
            float v = best[i];
            if (REDUCE == 3) v = v / (float)(hi - lo);
            if (REDUCE >= 2) v = to_f<T>(from_f<T>(v));   // the reduction's output is rounded before the norm
            if (scale) v = gelu_for<T>(fmaf(v, scale[ch + i], shift[ch + i]));
            best[i] = v;
        }
        *reinterpret_cast<typename V::Raw*>(out + c * C + ch) = V::pack(best);
    }
    if (coord_out && sub < 3) {
        if (sub * V::N >= C) {     // fewer channel groups than coordinate lanes: not reached above
            for (int64_t j = lo; j < hi; ++j) cacc += coord[3 * indices[j] + sub];
        }
        coord_out[3 * c + sub] = cacc / (float)(hi - lo);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) unpool_kernel(const T* __restrict__ skip,
                                                     const T* __restrict__ child,
                                                     const int64_t* __restrict__ cluster, int64_t n,
                                                     int C, const float* __restrict__ s_scale,
                                                     const float* __restrict__ s_shift,
                                                     const float* __restrict__ c_scale,
                                                     const float* __restrict__ c_shift,
                                                     T* __restrict__ out, T* __restrict__ skip_act)
{
    pdl_launch_next();
    pdl_wait();
    using V = Vec<T>;
    const int vec_per_row = C / V::N;
    const int vpr_shift = (vec_per_row & (vec_per_row - 1)) == 0 ? __ffs(vec_per_row) - 1 : -1;
    const int64_t total = n * vec_per_row;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        int64_t i;
        int ch;
        if (vpr_shift >= 0) {
            i = t >> vpr_shift;
            ch = (int)(t & (vec_per_row - 1)) * V::N;
        } else {
            i = t / vec_per_row;
            ch = (int)(t % vec_per_row) * V::N;
        }
        const int64_t cl = cluster[i];
        float a[V::N], b[V::N], o[V::N];
        V::unpack(*reinterpret_cast<const typename V::Raw*>(skip + i * C + ch), a);
        V::unpack(*reinterpret_cast<const typename V::Raw*>(child + cl * C + ch), b);
        // per-channel parameters with 16-byte loads (ch is a multiple of 4)
        float ss[V::N], sh[V::N], cs[V::N], csh[V::N];
#pragma unroll
        for (int k = 0; k < V::N; k += 4) {
            *reinterpret_cast<float4*>(ss + k) = *reinterpret_cast<const float4*>(s_scale + ch + k);
            *reinterpret_cast<float4*>(sh + k) = *reinterpret_cast<const float4*>(s_shift + ch + k);
            *reinterpret_cast<float4*>(cs + k) = *reinterpret_cast<const float4*>(c_scale + ch + k);
            *reinterpret_cast<float4*>(csh + k) = *reinterpret_cast<const float4*>(c_shift + ch + k);
        }
#pragma unroll
        for (int k = 0; k < V::N; ++k) {
            a[k] = gelu_for<T>(fmaf(a[k], ss[k], sh[k]));
            // both branches are rounded to the element type before the sum, as
            // two separate modules would
            a[k] = to_f<T>(from_f<T>(a[k]));
            const float bb = to_f<T>(from_f<T>(gelu_for<T>(fmaf(b[k], cs[k], csh[k]))));
            o[k] = a[k] + bb;
        }
        *reinterpret_cast<typename V::Raw*>(out + i * C + ch) = V::pack(o);
        if (skip_act) *reinterpret_cast<typename V::Raw*>(skip_act + i * C + ch) = V::pack(a);
    }
}

}  // namespace ptv3

extern "C" int ptv3_pool_fwd(const void* x, const float* coord, const int64_t* indices,
                             const int64_t* idx_ptr, int64_t m, int channels, const float* bn_scale,
                             const float* bn_shift, void* out, float* coord_out, int reduce, int dtype,
                             void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(reduce >= 0 && reduce <= 3, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_pool_fwd: reduce %d (0 max, 1 min, 2 sum, 3 mean)", reduce);
    PTV3_REQUIRE(m >= 0 && channels >= 1, PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_pool_fwd: dtype %d", dtype);
    const int vn = dtype == PTV3_DTYPE_F32 ? 4 : 8;
    PTV3_REQUIRE(channels % vn == 0, PTV3_ERR_UNSUPPORTED,
                 "ptv3_pool_fwd: channels %d not a multiple of %d", channels, vn);
    PTV3_REQUIRE((bn_scale == nullptr) == (bn_shift == nullptr), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_pool_fwd: bn_scale and bn_shift go together");
    if (m == 0) return PTV3_OK;
    PTV3_REQUIRE(x && indices && idx_ptr && out, PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_fwd: null pointer");
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool with_coord = coord && coord_out;
    const int vectors = channels / vn;
    int lanes = 4;   // at least 3 for the coordinate lanes
    while (lanes < 32 && lanes < vectors) lanes *= 2;
    const unsigned blocks = (unsigned)((m * lanes + 255) / 256);
#define PTV3_POOL_LAUNCH(T, L)                                                                          \
    do {                                                                                                 \
        auto args = [&](auto kern) {                                                                     \
            launch_dependent(kern, dim3(blocks), dim3(256), 0, stream, (const T*)x,                      \
                             with_coord ? coord : (const float*)nullptr, indices, idx_ptr, m, channels,  \
                             bn_scale, bn_shift, (T*)out, with_coord ? coord_out : (float*)nullptr);     \
        };                                                                                               \
        switch (reduce) {                                                                                \
            case 0: args(pool_max_kernel<T, L, 0>); break;                                               \
            case 1: args(pool_max_kernel<T, L, 1>); break;                                               \
            case 2: args(pool_max_kernel<T, L, 2>); break;                                               \
            default: args(pool_max_kernel<T, L, 3>); break;                                              \
        }                                                                                                \
    } while (0)
#define PTV3_POOL_DISPATCH(T)                      \
    switch (lanes) {                               \
        case 4: PTV3_POOL_LAUNCH(T, 4); break;     \
        case 8: PTV3_POOL_LAUNCH(T, 8); break;     \
        case 16: PTV3_POOL_LAUNCH(T, 16); break;   \
        default: PTV3_POOL_LAUNCH(T, 32); break;   \
    }
    if (dtype == PTV3_DTYPE_F32) {
        PTV3_POOL_DISPATCH(float)
    } else {
        PTV3_POOL_DISPATCH(__nv_bfloat16)
    }
#undef PTV3_POOL_DISPATCH
#undef PTV3_POOL_LAUNCH
    count_launches(1);
    return check_launch("ptv3_pool_fwd");
}

extern "C" int ptv3_unpool_fwd(const void* skip, const void* child, const int64_t* cluster, int64_t n,
                               int channels, const float* skip_scale, const float* skip_shift,
                               const float* child_scale, const float* child_shift, void* out,
                               void* skip_act, int dtype, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && channels >= 1, PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_unpool_fwd: dtype %d", dtype);
    const int vn = dtype == PTV3_DTYPE_F32 ? 4 : 8;
    PTV3_REQUIRE(channels % vn == 0, PTV3_ERR_UNSUPPORTED,
                 "ptv3_unpool_fwd: channels %d not a multiple of %d", channels, vn);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(skip && child && cluster && skip_scale && skip_shift && child_scale && child_shift && out,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_fwd: null pointer");
    cudaStream_t stream = (cudaStream_t)stream_;
    int64_t blocks = (n * (channels / vn) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PTV3_DTYPE_F32)
        launch_dependent(unpool_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)skip,
                         (const float*)child, cluster, n, channels, skip_scale, skip_shift, child_scale,
                         child_shift, (float*)out, (float*)skip_act);
    else
        launch_dependent(unpool_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream,
                         (const __nv_bfloat16*)skip, (const __nv_bfloat16*)child, cluster, n, channels,
                         skip_scale, skip_shift, child_scale, child_shift, (__nv_bfloat16*)out,
                         (__nv_bfloat16*)skip_act);
    count_launches(1);
    return check_launch("ptv3_unpool_fwd");
}
