// Patch attention over a serialized order: for every sequence (patch) of the
// padded serialized layout and every head, softmax(q k^T * scale) v, with rows
// gathered straight from the point-major qkv tensor and results scattered
// straight back to point-major rows.
//
// Replaces model.py:452-484 of SerializedAttention.forward (the row gather
// qkv[order[pad]], the per-patch attention, and the un-pad/un-serialize gather
// feat[unpad[inverse]]).  Row P of the padded layout reads point
// order[pad[P]]; it owns that point's output iff unpad[pad[P]] == P (borrowed
// rows of a last patch take part as keys and queries but write nothing).
//
// This file holds the CUDA-core path (fp32 arithmetic for either element type):
// one thread per query row, keys/values staged through shared memory in chunks
// with a per-chunk running-max rescale, so any sequence length works.
#include "common.cuh"
#include "convert.cuh"
#include "attention_mma.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

constexpr int AF_QT = 128;   // queries (threads) per CTA

// Relative position bias (model.py:297-316, 372-380, 468-469): for query i and key j of a
// patch, bias[h] = sum over the three axes a of table[clamp(g_i[a] - g_j[a], +-bnd) + bnd + a * num][h].
struct RpeArgs {
    const int32_t* grid_coord;   // n x 3, or NULL when no bias is used
    const float* table;          // (3 * num) x heads, fp32
    int pos_bnd, num, heads;
};

constexpr int AF_RPE_MAX = 3 * 129;   // table rows held in shared memory (pos_bnd <= 64)

template <typename T, int D>
__global__ void __launch_bounds__(AF_QT) attn_fma_kernel(
    const T* __restrict__ qkv, const int64_t* __restrict__ order, const int64_t* __restrict__ pad,
    const int64_t* __restrict__ unpad, const int32_t* __restrict__ cu_seqlens, T* __restrict__ out,
    int C, float scale, RpeArgs rpe, uint32_t* __restrict__ status)
{
    constexpr int AF_KC = D <= 32 ? 128 : 64;   // keys per staged chunk
    __shared__ float Ks[AF_KC][D];
    __shared__ float Vs[AF_KC][D];
    __shared__ int64_t ksrc[AF_KC];
    __shared__ int kg[AF_KC][3];          // grid coordinates of the staged keys (bias only)
    __shared__ float tab[AF_RPE_MAX];     // this head's column of the bias table
    const int seq = blockIdx.y, h = blockIdx.z, tid = threadIdx.x;
    const bool use_rpe = rpe.grid_coord != nullptr;
    if (use_rpe)
        for (int i = tid; i < 3 * rpe.num; i += AF_QT) tab[i] = rpe.table[i * rpe.heads + h];
    const int64_t start = cu_seqlens[seq];
    const int L = (int)(cu_seqlens[seq + 1] - start);
    const int q0 = blockIdx.x * AF_QT;
    // the grid covers max_seqlen queries per sequence: a longer sequence would leave rows of
    // the output unwritten, so it is reported instead
    if (blockIdx.x == 0 && tid == 0 && status && L > (int)gridDim.x * AF_QT)
        atomicOr(status, PTV3_STATUS_BAD_INDEX);
    if (q0 >= L) return;
    const int qi = q0 + tid;
    const bool valid = qi < L;
    int64_t src = 0;
    bool primary = false;
    float q[D], acc[D];
    int qg[3] = {0, 0, 0};
    if (valid) {
        const int64_t P = start + qi;
        const int64_t pd = pad[P];
        src = order[pd];
        primary = unpad[pd] == P;
        if (use_rpe) {
            qg[0] = rpe.grid_coord[3 * src] + rpe.pos_bnd;
            qg[1] = rpe.grid_coord[3 * src + 1] + rpe.pos_bnd + rpe.num;
            qg[2] = rpe.grid_coord[3 * src + 2] + rpe.pos_bnd + 2 * rpe.num;
        }
        const T* qp = qkv + src * (3 * (int64_t)C) + h * D;
#pragma unroll
        for (int d = 0; d < D; ++d) q[d] = to_f<T>(qp[d]) * scale;
    } else {
#pragma unroll
        for (int d = 0; d < D; ++d) q[d] = 0.f;
    }
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int c0 = 0; c0 < L; c0 += AF_KC) {
        const int nk = min(AF_KC, L - c0);
        __syncthreads();
        if (tid < nk) {
            const int64_t ks = order[pad[start + c0 + tid]];
            ksrc[tid] = ks;
            if (use_rpe) {
                kg[tid][0] = rpe.grid_coord[3 * ks];
                kg[tid][1] = rpe.grid_coord[3 * ks + 1];
                kg[tid][2] = rpe.grid_coord[3 * ks + 2];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < nk * D; idx += AF_QT) {
            const int j = idx / D, d = idx % D;
            const T* base = qkv + ksrc[j] * (3 * (int64_t)C) + h * D + d;
            Ks[j][d] = to_f<T>(base[C]);
            Vs[j][d] = to_f<T>(base[2 * C]);
        }
        __syncthreads();
        // bias of key j for this thread's query: table rows are pre-offset per axis
        auto bias = [&](int j) {
            const int lo0 = rpe.pos_bnd, lo1 = rpe.pos_bnd + rpe.num, lo2 = rpe.pos_bnd + 2 * rpe.num;
            const int i0 = min(max(qg[0] - kg[j][0], lo0 - rpe.pos_bnd), lo0 + rpe.pos_bnd);
            const int i1 = min(max(qg[1] - kg[j][1], lo1 - rpe.pos_bnd), lo1 + rpe.pos_bnd);
            const int i2 = min(max(qg[2] - kg[j][2], lo2 - rpe.pos_bnd), lo2 + rpe.pos_bnd);
            return tab[i0] + tab[i1] + tab[i2];
        };
        float cm = -INFINITY;
        for (int j = 0; j < nk; ++j) {
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) s = fmaf(q[d], Ks[j][d], s);
            if (use_rpe) s += bias(j);
            cm = fmaxf(cm, s);
        }
        const float mn = fmaxf(m, cm);
        const float corr = __expf(m - mn);   // m = -inf on the first chunk -> 0
        l *= corr;
#pragma unroll
        for (int d = 0; d < D; ++d) acc[d] *= corr;
        for (int j = 0; j < nk; ++j) {
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) s = fmaf(q[d], Ks[j][d], s);
            if (use_rpe) s += bias(j);
            const float p = __expf(s - mn);
            l += p;
#pragma unroll
            for (int d = 0; d < D; ++d) acc[d] = fmaf(p, Vs[j][d], acc[d]);
        }
        m = mn;
    }
    if (valid && primary) {
        const float inv = 1.f / l;
        T* op = out + src * (int64_t)C + h * D;
#pragma unroll
        for (int d = 0; d < D; ++d) op[d] = from_f<T>(acc[d] * inv);
    }
}

template <typename T>
static int launch_attn_fma(const void* qkv, const int64_t* order, const int64_t* pad,
                           const int64_t* unpad, const int32_t* cu, void* out, int n_seq,
                           int max_seqlen, int C, int H, float scale, RpeArgs rpe, uint32_t* status,
                           cudaStream_t stream)
{
    const int D = C / H;
    const dim3 grid((max_seqlen + AF_QT - 1) / AF_QT, n_seq, H);
#define AF_LAUNCH(DD)                                                                         \
    attn_fma_kernel<T, DD><<<grid, AF_QT, 0, stream>>>((const T*)qkv, order, pad, unpad, cu, \
                                                       (T*)out, C, scale, rpe, status)
    switch (D) {
        case 8: AF_LAUNCH(8); break;
        case 16: AF_LAUNCH(16); break;
        case 32: AF_LAUNCH(32); break;
        case 64: AF_LAUNCH(64); break;
        default:
            set_error("ptv3_attention_fwd: head dim %d (supported: 8, 16, 32, 64)", D);
            return PTV3_ERR_UNSUPPORTED;
    }
#undef AF_LAUNCH
    count_launches(1);
    return check_launch("ptv3_attention_fwd");
}

}  // namespace ptv3

static int attention_impl(const void* qkv, const int64_t* order, const int64_t* pad, const int64_t* unpad,
                          const int32_t* cu_seqlens, void* out, int64_t n, int n_seq, int max_seqlen,
                          int channels, int heads, float scale, int dtype, int algo, ptv3::RpeArgs rpe,
                          uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n_seq >= 0 && max_seqlen >= 1 && channels >= 1 && heads >= 1 &&
                     channels % heads == 0,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_attention_fwd: bad sizes");
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_attention_fwd: dtype %d", dtype);
    PTV3_REQUIRE(heads <= 65535 && n_seq <= 65535, PTV3_ERR_UNSUPPORTED,
                 "ptv3_attention_fwd: more than 65535 sequences or heads");
    if (n == 0 || n_seq == 0) return PTV3_OK;
    PTV3_REQUIRE(qkv && order && pad && unpad && cu_seqlens && out, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_attention_fwd: null pointer");
    PTV3_REQUIRE(algo >= 0 && algo <= 4, PTV3_ERR_INVALID_ARGUMENT, "ptv3_attention_fwd: algo %d", algo);
    const bool mma_ok = rpe.grid_coord == nullptr && dtype == PTV3_DTYPE_BF16 &&
                        attn_mma_supported(channels, heads, max_seqlen) &&
                        n <= 2147483647ll && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)out & 3) == 0;
    const bool tc05_ok = mma_ok && status != nullptr && attn_tc05_supported(channels, heads, max_seqlen) &&
                         ((uintptr_t)out & 15) == 0;
    PTV3_REQUIRE(algo != 4 || tc05_ok, PTV3_ERR_UNSUPPORTED,
                 "ptv3_attention_fwd: the tcgen05 path needs bf16, head dim 16, max_seqlen <= %d, 16-byte "
                 "aligned qkv and out, and a status word", ATTN_TC05_MAX_SEQLEN);
    if (algo == 4)
        return launch_attn_tc05(qkv, order, pad, unpad, cu_seqlens, out, n_seq, max_seqlen, channels,
                                heads, scale, status, (cudaStream_t)stream);
    PTV3_REQUIRE(algo < 2 || mma_ok, PTV3_ERR_UNSUPPORTED,
                 "ptv3_attention_fwd: the tensor-core path needs bf16, head dim 16, max_seqlen <= %d and "
                 "16-byte aligned qkv", ATTN_MMA_MAX_SEQLEN);
    if (mma_ok && algo != 1)
        return launch_attn_mma(qkv, order, pad, unpad, cu_seqlens, out, n_seq, max_seqlen, channels,
                               heads, scale, algo == 3, status, (cudaStream_t)stream);
    if (dtype == PTV3_DTYPE_F32)
        return launch_attn_fma<float>(qkv, order, pad, unpad, cu_seqlens, out, n_seq, max_seqlen,
                                      channels, heads, scale, rpe, status, (cudaStream_t)stream);
    return launch_attn_fma<__nv_bfloat16>(qkv, order, pad, unpad, cu_seqlens, out, n_seq, max_seqlen,
                                          channels, heads, scale, rpe, status, (cudaStream_t)stream);
}

extern "C" int ptv3_attention_fwd(const void* qkv, const int64_t* order, const int64_t* pad,
                                  const int64_t* unpad, const int32_t* cu_seqlens, void* out,
                                  int64_t n, int n_seq, int max_seqlen, int channels, int heads,
                                  float scale, int dtype, int algo, uint32_t* status, void* stream)
{
    return attention_impl(qkv, order, pad, unpad, cu_seqlens, out, n, n_seq, max_seqlen, channels, heads,
                          scale, dtype, algo, ptv3::RpeArgs{nullptr, nullptr, 0, 0, 0}, status, stream);
}

extern "C" int ptv3_attention_rpe_fwd(const void* qkv, const int64_t* order, const int64_t* pad,
                                      const int64_t* unpad, const int32_t* cu_seqlens,
                                      const int32_t* grid_coord, const float* rpe_table, int pos_bnd,
                                      void* out, int64_t n, int n_seq, int max_seqlen, int channels,
                                      int heads, float scale, int dtype, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(grid_coord && rpe_table, PTV3_ERR_INVALID_ARGUMENT, "ptv3_attention_rpe_fwd: null pointer");
    PTV3_REQUIRE(pos_bnd >= 0 && 3 * (2 * pos_bnd + 1) <= AF_RPE_MAX, PTV3_ERR_UNSUPPORTED,
                 "ptv3_attention_rpe_fwd: pos_bnd %d outside [0, 64]", pos_bnd);
    return attention_impl(qkv, order, pad, unpad, cu_seqlens, out, n, n_seq, max_seqlen, channels, heads,
                          scale, dtype, 1, RpeArgs{grid_coord, rpe_table, pos_bnd, 2 * pos_bnd + 1, heads},
                          nullptr, stream);
}
