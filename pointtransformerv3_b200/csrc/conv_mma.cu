// Tensor-core path of the submanifold convolution for bf16 features:
// an implicit GEMM, output-stationary over tiles of 128 voxels.
//
// For its tile a CTA first stages the 27 x 128 neighbour rows in shared memory
// and drops the offsets for which no voxel of the tile has a neighbour.  For
// each remaining offset o and each 32/64-wide slice of the input channels it
// gathers the neighbour rows (zero rows where there is none) and the matching
// slice of W[:, o, :] with cp.async into a double-buffered, bank-swizzled
// shared-memory stage, and accumulates out_tile += A_o . W_o^T with mma.sync
// (bf16 operands, fp32 accumulators in registers).  Bias is added in the
// epilogue.  An optional voxel permutation lets tiles follow a space-filling
// curve, which makes most offsets of a tile empty on surface-like data.
//
// Replaces spconv.SubMConv3d.forward at model.py:546-552 for bf16.
// Useful work: 2 . pairs . C_in . C_out FLOP.
#include "common.cuh"
#include "conv_mma.cuh"
#include "mma_util.cuh"

namespace ptv3 {

constexpr int CM_MAX_KVOL = 27;
constexpr int CM_STAGES = 3;
constexpr float CM_FIXED_ONE = 4294967296.f;    // 2^32: scale of the fixed-point accumulation

// physical 16-byte chunk of logical chunk c in row r for rows of NCH chunks
template <int NCH>
__device__ __forceinline__ int swz(int r, int c)
{
    if (NCH == 8) return c ^ (r & 7);
    if (NCH == 4) return c ^ ((r >> 1) & 3);
    return c;
}

// CM_TM: voxels per CTA; CN: output channels per CTA; KC: input channels per
// stage; WM x WN warps
// PAIRS: instead of 128 output voxels and all their offsets, a CTA owns 128
// (input row, output row) pairs of ONE offset from an offset-sorted pair list and
// adds its products into an accumulation buffer with atomics (no zero rows are
// multiplied; used for the coarse levels, where tiles are not planar and most of
// the 27 offsets of an output-stationary tile would be half empty).  The buffer
// holds 64-bit fixed-point numbers (32 fractional bits): integer addition is
// associative, so the sum does not depend on the order in which the CTAs arrive
// and the result is the same bit for bit on every run.  Every tile's fp32 product
// is rounded to 2^-32 once (absolute error below 1.2e-10 per contribution; values
// up to 2^31 in magnitude are representable, beyond that the conversion saturates).
struct PairList {
    const int32_t* pair_in;     // input row of every pair, sorted by offset
    const int32_t* pair_out;    // output row of every pair
    const int32_t* off_start;   // kvol + 1: first pair of every offset
    const int32_t* tile_start;  // kvol + 1: first 128-pair tile of every offset
    long long* acc;             // n x cout fixed-point accumulation buffer (zeroed by the launcher)
};

template <int CM_TM, int CN, int KC, int WM, int WN, bool PAIRS>
__global__ void __launch_bounds__(WM * WN * 32) conv_mma_kernel(
    const __nv_bfloat16* __restrict__ feat, const int32_t* __restrict__ nbr,
    const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ bias,
    __nv_bfloat16* __restrict__ out, const int64_t* __restrict__ row_order, int64_t n, int cin,
    int cout, int kvol, PairList pl)
{
    pdl_launch_next();
    pdl_wait();
    constexpr int CM_THREADS = WM * WN * 32;
    constexpr int NCH = KC / 8;              // 16-byte chunks per staged row
    constexpr int ROWB = KC * 2;             // bytes per staged row
    constexpr int WTM = CM_TM / WM;          // rows per warp
    constexpr int WTN = CN / WN;             // cols per warp
    constexpr int MT = WTM / 16, NT = WTN / 8;
    static_assert(NT % 2 == 0, "n tiles are loaded in pairs");
    constexpr int A_BYTES = CM_TM * ROWB, B_BYTES = CN * ROWB;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* As = smem;                                  // CM_STAGES stages
    unsigned char* Bs = smem + CM_STAGES * A_BYTES;            // CM_STAGES stages
    int32_t* nbr_s = reinterpret_cast<int32_t*>(smem + CM_STAGES * (A_BYTES + B_BYTES));   // kvol x CM_TM
    int* act = reinterpret_cast<int*>(nbr_s + CM_MAX_KVOL * CM_TM);                   // kvol + 1
    int64_t* rows_s = reinterpret_cast<int64_t*>(act + 32);                          // 128

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;
    const int64_t row0 = (int64_t)blockIdx.x * CM_TM;
    const int col0 = blockIdx.y * CN;

    if (PAIRS) {
        // which offset this tile of pairs belongs to
        const int tile = blockIdx.x;
        if (tile >= pl.tile_start[kvol]) return;
        int o = 0;
        while (o + 1 < kvol && pl.tile_start[o + 1] <= tile) ++o;
        const int p0 = pl.off_start[o] + (tile - pl.tile_start[o]) * CM_TM;
        const int cnt = min(CM_TM, pl.off_start[o + 1] - p0);
        if (tid < CM_TM) {
            rows_s[tid] = tid < cnt ? pl.pair_out[p0 + tid] : -1;
            nbr_s[tid] = tid < cnt ? pl.pair_in[p0 + tid] : -1;
        }
        if (tid == 0) {
            act[0] = 1;
            act[1] = o;
        }
        __syncthreads();
    } else {
        // ---- voxels of this tile and their neighbour rows ----------------------
        if (tid < CM_TM) {
            const int64_t i = row0 + tid;
            rows_s[tid] = i < n ? (row_order ? row_order[i] : i) : -1;
        }
        __syncthreads();
        {
            // a warp stages whole offsets (coalesced rows of 32 entries), all of its loads issued
            // before the first store, and notes in the same pass whether the tile has the offset
            constexpr int NW = CM_THREADS / 32, OPW = (CM_MAX_KVOL + NW - 1) / NW, RPL = CM_TM / 32;
            int32_t v[OPW][RPL];
#pragma unroll
            for (int j = 0; j < OPW; ++j) {
                const int o = warp + j * NW;
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    const int r = lane + 32 * i;
                    v[j][i] = (o < kvol && row0 + r < n) ? __ldg(nbr + (int64_t)o * n + row0 + r) : -1;
                }
            }
#pragma unroll
            for (int j = 0; j < OPW; ++j) {
                const int o = warp + j * NW;
                if (o < kvol) {
                    bool any = false;
#pragma unroll
                    for (int i = 0; i < RPL; ++i) {
                        nbr_s[o * CM_TM + lane + 32 * i] = v[j][i];
                        any |= v[j][i] >= 0;
                    }
                    const unsigned b = __ballot_sync(0xffffffffu, any);
                    if (lane == 0) act[1 + o] = b != 0;
                }
            }
        }
        __syncthreads();
        if (warp == 0) {
            // the offsets in use, in ascending order: act[1 ..], their number in act[0]
            const int flag = lane < kvol ? act[1 + lane] : 0;
            const unsigned m = __ballot_sync(0xffffffffu, flag != 0);
            if (flag) act[1 + __popc(m & ((1u << lane) - 1))] = lane;
            if (lane == 0) act[0] = __popc(m);
        }
        __syncthreads();
    }
    const int n_act = act[0];
    const int kchunks = cin / KC;
    const int nit = n_act * kchunks;

    float acc[MT][NT][4];
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;

    auto prefetch = [&](int it, int buf) {
        const int o = act[1 + it / kchunks];
        const int kc = (it % kchunks) * KC;
        const uint32_t a_base = smem_u32(As + buf * A_BYTES);
        const uint32_t b_base = smem_u32(Bs + buf * B_BYTES);
        for (int idx = tid; idx < CM_TM * NCH; idx += CM_THREADS) {
            const int r = idx / NCH, c = idx % NCH;
            const int32_t src = nbr_s[(PAIRS ? 0 : o) * CM_TM + r];
            const uint32_t dst = a_base + r * ROWB + swz<NCH>(r, c) * 16;
            if (src >= 0) {
                cp_async16(dst, feat + (int64_t)src * cin + kc + c * 8);
            } else {
                *reinterpret_cast<uint4*>(As + buf * A_BYTES + r * ROWB + swz<NCH>(r, c) * 16) =
                    make_uint4(0, 0, 0, 0);
            }
        }
        for (int idx = tid; idx < CN * NCH; idx += CM_THREADS) {
            const int r = idx / NCH, c = idx % NCH;
            const uint32_t dst = b_base + r * ROWB + swz<NCH>(r, c) * 16;
            cp_async16(dst, weight + ((int64_t)(col0 + r) * kvol + o) * cin + kc + c * 8);
        }
    };

    // ldmatrix lane roles
    const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3), a_ch = lane >> 4;
    const int b_row = (lane & 7) + ((lane >> 4) << 3), b_ch = (lane >> 3) & 1;

    // one cp.async group per iteration (empty past the end) keeps the wait uniform
#pragma unroll
    for (int st = 0; st < CM_STAGES - 1; ++st) {
        if (st < nit) prefetch(st, st);
        cp_async_commit();
    }
    for (int it = 0; it < nit; ++it) {
        const int buf = it % CM_STAGES;
        cp_async_wait<CM_STAGES - 2>();
        __syncthreads();   // stage `buf` has landed; stage (it - 1) % CM_STAGES is free again
        if (it + CM_STAGES - 1 < nit) prefetch(it + CM_STAGES - 1, (it + CM_STAGES - 1) % CM_STAGES);
        cp_async_commit();
        const uint32_t a_base = smem_u32(As + buf * A_BYTES);
        const uint32_t b_base = smem_u32(Bs + buf * B_BYTES);
#pragma unroll
        for (int ks = 0; ks < KC / 16; ++ks) {
            uint32_t af[MT][4];
#pragma unroll
            for (int a = 0; a < MT; ++a) {
                const int r = wm * WTM + a * 16 + a_row;
                ldmatrix_x4(af[a], a_base + r * ROWB + swz<NCH>(r, ks * 2 + a_ch) * 16);
            }
#pragma unroll
            for (int b = 0; b < NT / 2; ++b) {
                uint32_t bf[4];
                const int r = wn * WTN + b * 16 + b_row;
                ldmatrix_x4(bf, b_base + r * ROWB + swz<NCH>(r, ks * 2 + b_ch) * 16);
#pragma unroll
                for (int a = 0; a < MT; ++a) {
                    mma_bf16(acc[a][2 * b], af[a], bf[0], bf[1]);
                    mma_bf16(acc[a][2 * b + 1], af[a], bf[2], bf[3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- epilogue: + bias, round, store -------------------------------------
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int a = 0; a < MT; ++a) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * WTM + a * 16 + g + half * 8;
            const int64_t v = rows_s[r];
            if (v < 0) continue;
            if (PAIRS) {
                long long* op64 = pl.acc + v * (int64_t)cout + col0 + wn * WTN;
#pragma unroll
                for (int b = 0; b < NT; ++b) {
                    const long long f0 = __float2ll_rn(acc[a][b][half * 2] * CM_FIXED_ONE);
                    const long long f1 = __float2ll_rn(acc[a][b][half * 2 + 1] * CM_FIXED_ONE);
                    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(op64 + b * 8 + 2 * t), "l"(f0) : "memory");
                    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(op64 + b * 8 + 2 * t + 1), "l"(f1) : "memory");
                }
                continue;
            }
            __nv_bfloat16* op = out + v * (int64_t)cout + col0 + wn * WTN;
#pragma unroll
            for (int b = 0; b < NT; ++b) {
                const int c = b * 8 + 2 * t;
                float x0 = acc[a][b][half * 2], x1 = acc[a][b][half * 2 + 1];
                if (bias) {
                    x0 += __bfloat162float(bias[col0 + wn * WTN + c]);
                    x1 += __bfloat162float(bias[col0 + wn * WTN + c + 1]);
                }
                *reinterpret_cast<uint32_t*>(op + c) = pack_bf16(x0, x1);
            }
        }
    }
}

template <int CM_TM, int CN, int KC>
constexpr size_t conv_mma_smem()
{
    return CM_STAGES * ((size_t)CM_TM * KC * 2 + (size_t)CN * KC * 2) + (size_t)CM_MAX_KVOL * CM_TM * 4 +
           32 * 4 + CM_TM * 8;
}

bool conv_mma_supported(int c_in, int c_out, int kernel_volume)
{
    if (kernel_volume > CM_MAX_KVOL) return false;
    if (c_in == 32 && c_out == 32) return true;
    return c_in % 64 == 0 && (c_out == 64 || c_out % 128 == 0);
}

template <int CM_TM, int CN, int KC, int WM, int WN>
static int launch_one(const void* feat, const int32_t* nbr, const void* weight, const void* bias, void* out,
                      const int64_t* row_order, int64_t n, int cin, int cout, int kvol, cudaStream_t stream)
{
    constexpr size_t smem = conv_mma_smem<CM_TM, CN, KC>();
    auto kern = conv_mma_kernel<CM_TM, CN, KC, WM, WN, false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("ptv3_subm_conv_fwd: shared memory attribute");
    const dim3 grid((unsigned)((n + CM_TM - 1) / CM_TM), cout / CN);
    launch_dependent(kern, grid, dim3(WM * WN * 32), smem, stream, (const __nv_bfloat16*)feat, nbr,
                     (const __nv_bfloat16*)weight, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, row_order, n, cin,
                     cout, kvol, PairList{});
    count_launches(1);
    return check_launch("ptv3_subm_conv_fwd");
}

// out = bf16(acc * 2^-32 + bias)
__global__ void __launch_bounds__(256) conv_pairs_finalize_kernel(const long long* __restrict__ acc,
                                                                  const __nv_bfloat16* __restrict__ bias,
                                                                  __nv_bfloat16* __restrict__ out, int64_t total,
                                                                  int cout)
{
    const int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    const longlong2 lo = *reinterpret_cast<const longlong2*>(acc + i);
    const longlong2 hi = *reinterpret_cast<const longlong2*>(acc + i + 2);
    constexpr float inv = 1.f / CM_FIXED_ONE;
    // (the integer is split so that the conversion to fp32 rounds once, at 24 bits of the value)
    const float4 v = make_float4((float)((double)lo.x * inv), (float)((double)lo.y * inv),
                                 (float)((double)hi.x * inv), (float)((double)hi.y * inv));
    const int c = (int)(i % cout);
    float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
    if (bias) {
        b0 = __bfloat162float(bias[c]);
        b1 = __bfloat162float(bias[c + 1]);
        b2 = __bfloat162float(bias[c + 2]);
        b3 = __bfloat162float(bias[c + 3]);
    }
    uint2 o;
    o.x = pack_bf16(v.x + b0, v.y + b1);
    o.y = pack_bf16(v.z + b2, v.w + b3);
    *reinterpret_cast<uint2*>(out + i) = o;
}

bool conv_pairs_supported(int c_in, int c_out, int kernel_volume)
{
    return kernel_volume <= CM_MAX_KVOL && c_in % 64 == 0 && c_out % 128 == 0;
}

int launch_conv_pairs(const void* feat, const int32_t* pair_in, const int32_t* pair_out,
                      const int32_t* off_start, const int32_t* tile_start, int64_t max_tiles,
                      const void* weight, const void* bias, void* out, long long* acc, int64_t n, int c_in,
                      int c_out, int kvol, cudaStream_t stream)
{
    constexpr size_t smem = conv_mma_smem<128, 128, 64>();
    auto kern = conv_mma_kernel<128, 128, 64, 4, 2, true>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("ptv3_subm_conv_pairs_fwd: shared memory attribute");
    if (cudaMemsetAsync(acc, 0, (size_t)n * c_out * sizeof(long long), stream) != cudaSuccess)
        return check_launch("ptv3_subm_conv_pairs_fwd: memset");
    const PairList pl{pair_in, pair_out, off_start, tile_start, acc};
    launch_dependent(kern, dim3((unsigned)max_tiles, c_out / 128), dim3(256), smem, stream,
                     (const __nv_bfloat16*)feat, (const int32_t*)nullptr, (const __nv_bfloat16*)weight,
                     (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)nullptr, (const int64_t*)nullptr, n, c_in, c_out,
                     kvol, pl);
    const int64_t total = n * (int64_t)c_out;
    conv_pairs_finalize_kernel<<<(unsigned)((total / 4 + 255) / 256), 256, 0, stream>>>(
        acc, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, total, c_out);
    count_launches(2);
    return check_launch("ptv3_subm_conv_pairs_fwd");
}

int launch_conv_mma(const void* feat, const int32_t* nbr, const void* weight, const void* bias, void* out,
                    const int64_t* row_order, int64_t n, int c_in, int c_out, int kvol, cudaStream_t stream)
{
#define CM_ARGS feat, nbr, weight, bias, out, row_order, n, c_in, c_out, kvol, stream
    if (c_in == 32 && c_out == 32) return launch_one<128, 32, 32, 8, 1>(CM_ARGS);
    // few voxels: 64 x 64 tiles on 4 warps so that enough CTAs exist to fill the GPU
    const int64_t big_ctas = ((n + 127) / 128) * ((c_out + 127) / 128);
    if (c_out == 64) {
        if (big_ctas * 2 < 2 * 148) return launch_one<64, 64, 64, 2, 2>(CM_ARGS);
        return launch_one<128, 64, 64, 4, 2>(CM_ARGS);
    }
    if (big_ctas < 2 * 148) return launch_one<64, 64, 64, 2, 2>(CM_ARGS);
    return launch_one<128, 128, 64, 4, 2>(CM_ARGS);
#undef CM_ARGS
}

}  // namespace ptv3
