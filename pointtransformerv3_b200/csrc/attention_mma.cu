// Tensor-core path of the patch attention core for bf16 features and head
// dimension 16 (every stage of the default backbone).
//
// One CTA owns one (sequence, head) pair (optionally a slice of its queries):
// the keys and values of the whole sequence are gathered once into shared
// memory with cp.async, straight from the point-major qkv tensor through
// order[pad[.]].  Each warp then walks 16-query tiles: S = Q K^T for 64 keys at
// a time by mma.sync (k = head_dim = 16, one instruction per 16x8 tile), an
// online softmax on the accumulator registers (exp2 with the running maximum),
// P rounded to bf16 in the same registers re-used as the A operand of P V.
// Nothing but q, k, v and the output rows touches global memory; scores never
// leave registers.  Rows are written back to out[order[pad[.]]] only by the
// padded row that owns the point (borrowed rows of a last patch are dropped).
//
// Replaces model.py:452-484 for the bf16 case (see attention.cu for the
// contract).  Work per (sequence, head): 4 L^2 16 tensor FLOPs and L^2 exps;
// at head_dim 16 the exp unit, not the tensor pipe, is the limiter.
#include "common.cuh"
#include "attention_mma.cuh"
#include "mma_util.cuh"

namespace ptv3 {

constexpr int AM_THREADS = 256;
constexpr int AM_WARPS = AM_THREADS / 32;
constexpr int AM_KC = 64;           // keys per online-softmax step
constexpr int AM_D = 16;
constexpr float AM_LOG2E = 1.4426950408889634f;
constexpr float AM_LAZY = 8.f;       // slack of the running maximum, in powers of two

// byte offset of 16-byte chunk c (0/1) of row r in a [rows][16] bf16 tile whose
// chunks are swapped in rows 4..7 (mod 8) so that 8-row ldmatrix reads hit 32
// distinct banks
__device__ __forceinline__ uint32_t kv_offset(int r, int c)
{
    return (uint32_t)(r * 32 + ((c ^ ((r >> 2) & 1)) << 4));
}

__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t v, float s)
{
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
    return pack_bf16(f.x * s, f.y * s);
}

template <bool PACKED>
__global__ void __launch_bounds__(AM_THREADS, 3) attn_mma_d16_kernel(
    const __nv_bfloat16* __restrict__ qkv, const int64_t* __restrict__ order,
    const int64_t* __restrict__ pad, const int64_t* __restrict__ unpad,
    const int32_t* __restrict__ cu_seqlens, __nv_bfloat16* __restrict__ out, int C, float scale,
    int lpad_max, uint32_t* __restrict__ status)
{
    pdl_launch_next();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* Ks = smem;
    unsigned char* Vs = smem + (size_t)lpad_max * 32;
    // point row of every padded row of the sequence, negated - 1 where the padded row does not own
    // its point (borrowed rows): the gather walks pad -> order for every row anyway, and the query
    // tiles then need one dependent load instead of three
    int32_t* src_s = reinterpret_cast<int32_t*>(smem + (size_t)lpad_max * 64);

    // heads and query slices vary fastest over the grid (blockIdx.x = slice * heads + head): the
    // CTAs of one patch run together, so the rows they all gather from (a row holds every head's
    // q, k and v side by side) are fetched from DRAM once
    const int n_heads = C / 16;
    const int seq = blockIdx.y, h = blockIdx.x % n_heads;
    const int slice = blockIdx.x / n_heads, n_slices = gridDim.x / n_heads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t start = cu_seqlens[seq];
    const int L = (int)(cu_seqlens[seq + 1] - start);
    if (L <= 0) return;
    // shared memory was sized from the caller's max_seqlen: a longer sequence (a plan made
    // for a larger patch) is reported and skipped, uniformly over the CTA, before any write
    if (L > lpad_max) {
        if (tid == 0 && status) atomicOr(status, PTV3_STATUS_BAD_INDEX);
        return;
    }
    const int Lp = (L + AM_KC - 1) / AM_KC * AM_KC;   // <= lpad_max
    const int ntiles = (L + 15) / 16;
    const int tiles_per_slice = (ntiles + n_slices - 1) / n_slices;
    const int tile_lo = slice * tiles_per_slice;
    const int tile_hi = min(ntiles, tile_lo + tiles_per_slice);
    if (tile_lo >= tile_hi) return;
    const int64_t row_stride = 3 * (int64_t)C;

    // ---- gather K and V of the whole sequence ------------------------------
    for (int r = tid; r < Lp; r += AM_THREADS) {
        const uint32_t k0 = smem_u32(Ks) + kv_offset(r, 0), k1 = smem_u32(Ks) + kv_offset(r, 1);
        const uint32_t v0 = smem_u32(Vs) + kv_offset(r, 0), v1 = smem_u32(Vs) + kv_offset(r, 1);
        if (r < L) {
            const int64_t pd = pad[start + r];
            const int64_t src = order[pd];
            src_s[r] = unpad[pd] == start + r ? (int32_t)src : -(int32_t)src - 1;
            const __nv_bfloat16* kp = qkv + src * row_stride + C + h * AM_D;
            cp_async16(k0, kp);
            cp_async16(k1, kp + 8);
            cp_async16(v0, kp + C);
            cp_async16(v1, kp + C + 8);
        } else {
            const uint4 z = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(Ks + kv_offset(r, 0)) = z;
            *reinterpret_cast<uint4*>(Ks + kv_offset(r, 1)) = z;
            *reinterpret_cast<uint4*>(Vs + kv_offset(r, 0)) = z;
            *reinterpret_cast<uint4*>(Vs + kv_offset(r, 1)) = z;
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const int g = lane >> 2, t = lane & 3;
    // ldmatrix row/chunk this lane addresses inside a 16-key group
    const int k_row = (lane & 7) + ((lane >> 4) << 3), k_chunk = (lane >> 3) & 1;   // K: keys x d
    const int v_row = (lane & 7) + (((lane >> 3) & 1) << 3), v_chunk = lane >> 4;   // V (transposed)
    const uint32_t ks_base = smem_u32(Ks), vs_base = smem_u32(Vs);
    const float sl2 = AM_LOG2E;

    // query rows of a warp's tile, fetched one tile ahead (the row numbers are in shared memory,
    // so this is a single load per row)
    auto fetch_q = [&](int tile, uint32_t (&q)[4]) {
        const int r0 = tile * 16 + g, r1 = r0 + 8;
        q[0] = q[1] = q[2] = q[3] = 0u;
        if (tile < tile_hi && r0 < L) {
            const int32_t e = src_s[r0];
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(qkv + (int64_t)(e >= 0 ? e : -(e + 1)) * row_stride + h * AM_D);
            q[0] = qp[t];
            q[2] = qp[4 + t];
        }
        if (tile < tile_hi && r1 < L) {
            const int32_t e = src_s[r1];
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(qkv + (int64_t)(e >= 0 ? e : -(e + 1)) * row_stride + h * AM_D);
            q[1] = qp[t];
            q[3] = qp[4 + t];
        }
    };
    uint32_t qn[4];
    fetch_q(tile_lo + warp, qn);
    for (int tile = tile_lo + warp; tile < tile_hi; tile += AM_WARPS) {
        const int r0 = tile * 16 + g, r1 = r0 + 8;
        const bool ok0 = r0 < L, ok1 = r1 < L;
        const uint32_t qa[4] = {scale_bf16x2(qn[0], scale), scale_bf16x2(qn[1], scale), scale_bf16x2(qn[2], scale),
                                scale_bf16x2(qn[3], scale)};
        fetch_q(tile + AM_WARPS, qn);
        float m0 = -INFINITY, m1 = -INFINITY, l0, l1;
        float o[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float osum[4] = {0.f, 0.f, 0.f, 0.f};   // row sums of the rounded probabilities: a ones column of V

        for (int kc = 0; kc < Lp; kc += AM_KC) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t kb[4];
                ldmatrix_x4(kb, ks_base + kv_offset(kc + 16 * j + k_row, k_chunk));
                mma_bf16(s[2 * j], qa, kb[0], kb[1]);
                mma_bf16(s[2 * j + 1], qa, kb[2], kb[3]);
            }
            if (kc + AM_KC > L) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = kc + 8 * j + 2 * t;
                    if (col >= L) s[j][0] = s[j][2] = -INFINITY;
                    if (col + 1 >= L) s[j][1] = s[j][3] = -INFINITY;
                }
            }
            // three-input maxima (one instruction each on this architecture)
            float mx0 = fmaxf(s[0][0], s[0][1]), mx1 = fmaxf(s[0][2], s[0][3]);
#pragma unroll
            for (int j = 1; j < 8; ++j) {
                mx0 = fmaxf(fmaxf(mx0, s[j][0]), s[j][1]);
                mx1 = fmaxf(fmaxf(mx1, s[j][2]), s[j][3]);
            }
            // Lazy reference: the running "maximum" m only has to keep the exponentials in
            // range, so it is raised (and the output rescaled) only when some score of the
            // chunk exceeds it by more than AM_LAZY in the exp2 domain; probabilities then
            // stay below 2^AM_LAZY, exact in bf16's range and harmless in the fp32 sums.
            // After the first chunks of a sequence this is rare, and the common path needs
            // neither the cross-lane reduction nor the rescaling.
            if (__any_sync(0xffffffffu, (mx0 - m0) * sl2 > AM_LAZY || (mx1 - m1) * sl2 > AM_LAZY)) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                // every chunk holds at least one real key, so mn is finite
                const float c0 = fast_exp2((m0 - mn0) * sl2), c1 = fast_exp2((m1 - mn1) * sl2);
                m0 = mn0;
                m1 = mn1;
                osum[0] *= c0;
                osum[2] *= c1;
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    o[n][0] *= c0;
                    o[n][1] *= c0;
                    o[n][2] *= c1;
                    o[n][3] *= c1;
                }
            }
            const float mn0 = m0, mn1 = m1;
            const float b0 = mn0 * sl2, b1 = mn1 * sl2;
            uint32_t pa[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (PACKED) {
                    // exponent argument rounded to bf16, two exps per instruction, the result
                    // already is the bf16 pair the next MMA consumes
                    pa[j][0] = exp2_bf16x2(pack_bf16(fmaf(s[j][0], sl2, -b0), fmaf(s[j][1], sl2, -b0)));
                    pa[j][1] = exp2_bf16x2(pack_bf16(fmaf(s[j][2], sl2, -b1), fmaf(s[j][3], sl2, -b1)));
                } else {
                    const float p0 = fast_exp2(fmaf(s[j][0], sl2, -b0));
                    const float p1 = fast_exp2(fmaf(s[j][1], sl2, -b0));
                    const float p2 = fast_exp2(fmaf(s[j][2], sl2, -b1));
                    const float p3 = fast_exp2(fmaf(s[j][3], sl2, -b1));
                    pa[j][0] = pack_bf16(p0, p1);
                    pa[j][1] = pack_bf16(p2, p3);
                }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t a[4] = {pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1]};
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, vs_base + kv_offset(kc + 16 * kk + v_row, v_chunk));
                mma_bf16(o[0], a, vb[0], vb[1]);
                mma_bf16(o[1], a, vb[2], vb[3]);
                // a column of ones appended to V: the tensor core sums the rounded probabilities
                mma_bf16(osum, a, 0x3f803f80u, 0x3f803f80u);
            }
        }
        l0 = osum[0];
        l1 = osum[2];
        const int32_t e0 = ok0 ? src_s[r0] : -1, e1 = ok1 ? src_s[r1] : -1;     // >= 0: the row owns its point
        if (e0 >= 0) {
            const float inv = 1.f / l0;
            uint32_t* op = reinterpret_cast<uint32_t*>(out + e0 * (int64_t)C + h * AM_D);
            op[t] = pack_bf16(o[0][0] * inv, o[0][1] * inv);
            op[4 + t] = pack_bf16(o[1][0] * inv, o[1][1] * inv);
        }
        if (e1 >= 0) {
            const float inv = 1.f / l1;
            uint32_t* op = reinterpret_cast<uint32_t*>(out + e1 * (int64_t)C + h * AM_D);
            op[t] = pack_bf16(o[0][2] * inv, o[0][3] * inv);
            op[4 + t] = pack_bf16(o[1][2] * inv, o[1][3] * inv);
        }
    }
}

bool attn_mma_supported(int channels, int heads, int max_seqlen)
{
    return channels % heads == 0 && channels / heads == AM_D && channels % 8 == 0 &&
           max_seqlen <= ATTN_MMA_MAX_SEQLEN;
}

int launch_attn_mma(const void* qkv, const int64_t* order, const int64_t* pad, const int64_t* unpad,
                    const int32_t* cu, void* out, int n_seq, int max_seqlen, int C, int H, float scale,
                    bool packed_exp, uint32_t* status, cudaStream_t stream)
{
    const int lpad = (max_seqlen + AM_KC - 1) / AM_KC * AM_KC;
    const size_t smem = (size_t)lpad * 68;      // K, V and the row numbers
    // per device and cheap, so it is simply repeated on every call
    auto kern = packed_exp ? attn_mma_d16_kernel<true> : attn_mma_d16_kernel<false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ATTN_MMA_MAX_SEQLEN * 68) !=
        cudaSuccess)
        return check_launch("ptv3_attention_fwd: shared memory attribute");
    // slice the queries of a sequence over several CTAs when there are few (sequence, head) pairs
    int qsplit = 1;
    const int pairs = n_seq * H;
    const int tiles = (max_seqlen + 15) / 16;
    // three CTAs fit on an SM; aim at several waves so that the last one costs little
    while (pairs * qsplit < 4 * 3 * 148 && qsplit * 2 * AM_WARPS <= tiles) qsplit *= 2;
    const dim3 grid(H * qsplit, n_seq);
    launch_dependent(kern, grid, dim3(AM_THREADS), smem, stream, (const __nv_bfloat16*)qkv, order, pad, unpad, cu,
                     (__nv_bfloat16*)out, C, scale, lpad, status);
    count_launches(1);
    return check_launch("ptv3_attention_fwd");
}

}  // namespace ptv3
