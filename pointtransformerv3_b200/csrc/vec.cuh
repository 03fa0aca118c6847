// 16-byte vector access to rows of fp32 / bf16 features.
#pragma once
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

}  // namespace ptv3
