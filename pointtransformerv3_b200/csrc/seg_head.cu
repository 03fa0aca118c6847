// Segmentation head, the step after the backbone: logits = feat W^T + b over a small
// number of classes and the per-point arg max, in one pass over the features
// (the backbone's output rows are read once; the logits need not be stored).
//
// The reference file stops at the backbone (model.py:966-982 returns the Point); the
// head is a Linear(dec_channels[0], num_classes) in the segmentor that wraps it.
// A CTA stages 128 feature rows in shared memory with coalesced, independent 16-byte
// loads (rows padded by 16 bytes so that the row-per-thread reads that follow are free
// of bank conflicts); then one thread owns one point.  The weight matrix sits in shared
// memory as fp32 (class-major), accumulation is fp32.  Ties go to the lowest class index,
// as torch.argmax does on CUDA for equal values.
#include "common.cuh"
#include "convert.cuh"
#include "vec.cuh"

namespace ptv3 {

constexpr int SH_THREADS = 128;
constexpr int SH_MAX_CLASSES = 64;
constexpr int SH_MAX_CHANNELS = 512;

// KMAX: compile-time bound of the class count (the accumulators live in registers)
template <typename T, int KMAX>
__global__ void __launch_bounds__(SH_THREADS) seg_head_kernel(const T* __restrict__ feat, const T* __restrict__ weight,
                                                              const T* __restrict__ bias, T* __restrict__ logits,
                                                              int64_t* __restrict__ labels, int64_t n, int C, int K)
{
    extern __shared__ __align__(16) float w_s[];   // K x C, then K biases
    float* b_s = w_s + (size_t)K * C;
    for (int i = threadIdx.x; i < K * C; i += SH_THREADS) w_s[i] = to_f<T>(weight[i]);
    for (int i = threadIdx.x; i < K; i += SH_THREADS) b_s[i] = bias ? to_f<T>(bias[i]) : 0.f;
    __syncthreads();
    // stage the CTA's rows: chunk idx -> (row, 16-byte piece), consecutive threads on consecutive pieces
    using Raw = typename Vec<T>::Raw;
    unsigned char* stage = reinterpret_cast<unsigned char*>(b_s + ((K + 3) & ~3));
    const int cpr = C / Vec<T>::N;                    // 16-byte pieces per row
    const int pitch = cpr * 16 + 16;
    const int64_t row0 = blockIdx.x * (int64_t)SH_THREADS;
    const Raw* src = reinterpret_cast<const Raw*>(feat + row0 * C);
    const int64_t pieces = min((int64_t)SH_THREADS, n - row0) * cpr;
    for (int idx = threadIdx.x; idx < SH_THREADS * cpr; idx += SH_THREADS)
        if (idx < pieces) *reinterpret_cast<Raw*>(stage + (idx / cpr) * pitch + (idx % cpr) * 16) = src[idx];
    __syncthreads();
    const int64_t row = row0 + threadIdx.x;
    if (row >= n) return;
    float acc[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) acc[k] = 0.f;
    const unsigned char* my = stage + threadIdx.x * pitch;
    for (int c0 = 0; c0 < C; c0 += Vec<T>::N) {
        float x[Vec<T>::N];
        Vec<T>::unpack(*reinterpret_cast<const Raw*>(my + (c0 / Vec<T>::N) * 16), x);
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
                // same address warp-wide: one 16-byte broadcast load per four weights
                const float4* w = reinterpret_cast<const float4*>(w_s + (size_t)k * C + c0);
#pragma unroll
                for (int q = 0; q < Vec<T>::N / 4; ++q) {
                    const float4 wv = w[q];
                    acc[k] = fmaf(x[4 * q + 0], wv.x, acc[k]);
                    acc[k] = fmaf(x[4 * q + 1], wv.y, acc[k]);
                    acc[k] = fmaf(x[4 * q + 2], wv.z, acc[k]);
                    acc[k] = fmaf(x[4 * q + 3], wv.w, acc[k]);
                }
            }
        }
    }
    float best = 0.f;
    int arg = 0;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
        if (k < K) {
            // compare what a caller would see: the logit rounded to the feature type
            const float v = Vec<T>::round(acc[k] + b_s[k]);
            if (logits) logits[row * K + k] = from_f<T>(v);
            if (k == 0 || v > best) {
                best = v;
                arg = k;
            }
        }
    }
    if (labels) labels[row] = arg;
}

template <typename T>
static int launch_seg_head(const void* feat, const void* weight, const void* bias, void* logits, int64_t* labels,
                           int64_t n, int C, int K, cudaStream_t stream)
{
    const int vec = Vec<T>::N;
    const size_t smem = ((size_t)K * C + ((K + 3) & ~3)) * sizeof(float) + (size_t)SH_THREADS * (C / vec * 16 + 16);
    const unsigned blocks = (unsigned)((n + SH_THREADS - 1) / SH_THREADS);
#define SH_LAUNCH(KMAX)                                                                                          \
    do {                                                                                                         \
        auto kern = seg_head_kernel<T, KMAX>;                                                                    \
        if (smem > 48 * 1024 &&                                                                                  \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)   \
            return check_launch("ptv3_seg_head_fwd: shared memory attribute");                                   \
        kern<<<blocks, SH_THREADS, smem, stream>>>((const T*)feat, (const T*)weight, (const T*)bias, (T*)logits, \
                                                   labels, n, C, K);                                             \
    } while (0)
    if (K <= 16)
        SH_LAUNCH(16);
    else if (K <= 32)
        SH_LAUNCH(32);
    else
        SH_LAUNCH(64);
#undef SH_LAUNCH
    count_launches(1);
    return check_launch("ptv3_seg_head_fwd");
}

}  // namespace ptv3

extern "C" int ptv3_seg_head_fwd(const void* feat, const void* weight, const void* bias, void* logits,
                                 int64_t* labels, int64_t n, int channels, int classes, int dtype, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_seg_head_fwd: n < 0");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_seg_head_fwd: dtype %d", dtype);
    const int vec = dtype == PTV3_DTYPE_F32 ? 4 : 8;
    PTV3_REQUIRE(classes >= 1 && classes <= SH_MAX_CLASSES && channels >= vec && channels <= SH_MAX_CHANNELS &&
                     channels % vec == 0,
                 PTV3_ERR_UNSUPPORTED, "ptv3_seg_head_fwd: %d classes (1..%d), %d channels (multiple of %d, up to %d)",
                 classes, SH_MAX_CLASSES, channels, vec, SH_MAX_CHANNELS);
    PTV3_REQUIRE(((size_t)classes * channels + classes + 4) * 4 + 128 * ((size_t)channels / vec * 16 + 16) <= 200 * 1024,
                 PTV3_ERR_UNSUPPORTED, "ptv3_seg_head_fwd: %d classes x %d channels do not fit shared memory", classes,
                 channels);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(feat && weight && (logits || labels), PTV3_ERR_INVALID_ARGUMENT, "ptv3_seg_head_fwd: null pointer");
    PTV3_REQUIRE(((uintptr_t)feat & 15) == 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_seg_head_fwd: feat must be 16-byte aligned");
    if (dtype == PTV3_DTYPE_F32)
        return launch_seg_head<float>(feat, weight, bias, logits, labels, n, channels, classes, (cudaStream_t)stream);
    return launch_seg_head<__nv_bfloat16>(feat, weight, bias, logits, labels, n, channels, classes,
                                          (cudaStream_t)stream);
}
