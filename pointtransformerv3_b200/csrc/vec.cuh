// 16-byte vector access to rows of fp32 / bf16 features.
#pragma once
#include "mma_util.cuh"
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace ptv3 {

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    using Raw = float4;
    __device__ static void unpack(const Raw& r, float* f) { f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
    __device__ static Raw pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
    __device__ static float round(float v) { return v; }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    using Raw = uint4;
    __device__ static void unpack(const Raw& r, float* f)
    {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __bfloat1622float2(h[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    __device__ static Raw pack(const float* f)
    {
        Raw r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return r;
    }
    // value after a round trip through the element type
    __device__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// GELU in its erf form, 0.5 x (1 + erf(x / sqrt 2)), with erf(z) = tanh(c1 z + c3 z^3 + c5 z^5)
// (|error| < 4.1e-5 for the fit, z^2 clamped at 16 where erf is 1 to eight digits) and the
// hardware tanh (relative error about 2^-11).  The result is rounded to bf16 (relative
// 2^-9) right after, and the library erff costs 2.5x the instructions in an epilogue that
// is bound by instruction issue.
__device__ __forceinline__ float gelu_tanh_erf(float x)
{
    // coefficients of the fit in z, rescaled to x = z sqrt 2
    const float c1 = 1.12812329f * 0.70710678f, c3 = 0.10414445f * 0.35355339f, c5 = -0.00181548f * 0.17677670f;
    const float x2 = fminf(x * x, 32.f);
    const float p = fmaf(fmaf(c5, x2, c3), x2, c1) * x;
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(p));
    const float hx = 0.5f * x;
    return fmaf(hx, th, hx);
}
// the same for a pair of values (packed fp32 arithmetic; the same operations in the same order)
__device__ __forceinline__ uint64_t gelu_tanh_erf2(uint64_t x)
{
    const float c1 = 1.12812329f * 0.70710678f, c3 = 0.10414445f * 0.35355339f, c5 = -0.00181548f * 0.17677670f;
    float a, b;
    unpack2(fma2(x, x, 0ull), a, b);
    const uint64_t x2 = pack2(fminf(a, 32.f), fminf(b, 32.f));
    const uint64_t p = fma2(fma2(fma2(pack2(c5, c5), x2, pack2(c3, c3)), x2, pack2(c1, c1)), x, 0ull);
    unpack2(p, a, b);
    float ta, tb;
    asm("tanh.approx.f32 %0, %1;" : "=f"(ta) : "f"(a));
    asm("tanh.approx.f32 %0, %1;" : "=f"(tb) : "f"(b));
    const uint64_t hx = fma2(x, pack2(0.5f, 0.5f), 0ull);
    return fma2(hx, pack2(ta, tb), hx);
}

}  // namespace ptv3
