// Linear layers whose weights do not fit in shared memory at once (input width 256 and
// more, or more than 384 outputs), on the 5th-generation tensor cores:
//
//     out = [residual +] act(x W^T + b),    act = identity or GELU (erf form)
//
// which is what the two coarsest levels (C = 256, 512), the MLP of C = 128 and the pooling /
// unpooling projections between them need (model.py:456, 487, 510-516, 684, 726-735).
//
// A persistent CTA per SM walks 128-row x BN-column tiles (BN = 256 or 128).  Warp 0 streams
// 64-wide K chunks of x and W through a ring of stages in shared memory with TMA (128-byte
// swizzle), warp 1 issues four tcgen05.mma (K = 16 each) per chunk into one of TWO accumulators
// in tensor memory and releases a stage with tcgen05.commit, warps 2..5 take a finished
// accumulator (tcgen05.ld, thread = row), add the bias, apply GELU, add the residual row and
// store bf16 while the next tile is already being multiplied into the other accumulator.
// The roundings are those of the unfused sequence (GEMM output rounded to bf16, then GELU or
// the residual sum rounded again).  Every mbarrier wait is bounded and reports through the
// status word.
#include "common.cuh"
#include "tc05.cuh"
#include "vec.cuh"

namespace ptv3 {

using namespace tc05;

constexpr int GM_BM = 128;
constexpr int GM_BK = 64;                       // bf16 columns per stage: one 128-byte swizzle span
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;   // 16 KiB
constexpr int GM_THREADS = 192;

struct GemmArgs {
    const __nv_bfloat16* bias;       // n_out or NULL
    const __nv_bfloat16* residual;   // n x n_out or NULL
    __nv_bfloat16* out;              // n x n_out
    int64_t n;
    int k, n_out;
    int gelu;
    int row_tiles, col_tiles;
    uint32_t* status;
};

__device__ __forceinline__ float gm_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int BN, int STAGES>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  const GemmArgs a)
{
    pdl_launch_next();
    constexpr int B_BYTES = BN * GM_BK * 2;
    constexpr int STAGE_BYTES = GM_A_BYTES + B_BYTES;
    constexpr int NBAR = 2 * STAGES + 4;      // full, empty per stage; accumulator full / empty x 2
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32_generic(smem);
    const int off_bias = STAGES * STAGE_BYTES;            // 2 x BN floats (one set per accumulator)
    const int off_bar = off_bias + 2 * BN * 4;
    float* bias_s = reinterpret_cast<float*>(smem + off_bias);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t full0 = sbase + off_bar, empty0 = full0 + 8 * STAGES, accfull0 = empty0 + 8 * STAGES,
                   accempty0 = accfull0 + 16;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = a.k / GM_BK;
    const int ntiles = a.row_tiles * a.col_tiles;

    if (tid == 0) {
        for (int i = 0; i < 2 * STAGES + 2; ++i) mbar_init(full0 + 8 * i, 1);
        mbar_init(accempty0, 4);          // one arrival per epilogue warp
        mbar_init(accempty0 + 8, 4);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) tmem_alloc(sbase + off_bar + 8 * NBAR, 2 * BN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    // barriers, tensor memory and descriptors are set up; everything the kernel before this one in
    // the stream may have written is touched after this wait
    pdl_wait();

    // tile t -> (row tile, column tile); column tiles of a row tile run on neighbouring CTAs, so
    // the x rows they share are fetched from DRAM once
    if (warp == 0) {
        // ---- producer: K chunks of the x tile and of the W tile, tile after tile -----------------
        if (lane == 0) {
            int it = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
                const int row0 = (t / a.col_tiles) * GM_BM, col0 = (t % a.col_tiles) * BN;
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % STAGES;
                    // a stage is free once the products that read it have completed (the first pass
                    // over the ring finds every stage free: waiting for the phase before the first)
                    ok &= mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort);
                    const uint32_t sa = sbase + s * STAGE_BYTES, sb = sa + GM_A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(sa, &map_x, kc * GM_BK, row0, full0 + 8 * s);
                    tma_load_2d(sb, &map_w, kc * GM_BK, col0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- issuer -----------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(GM_BM, BN);
            int it = 0, j = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++j) {
                const int buf = j & 1;
                // the epilogue has read the accumulator's previous tile (first use: free)
                ok &= mbar_wait(accempty0 + 8 * buf, ((j >> 1) & 1) ^ 1, abort);
                fence_after_sync();
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % STAGES;
                    ok &= mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort);
                    fence_after_sync();
                    const uint32_t sa = sbase + s * STAGE_BYTES, sb = sa + GM_A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < GM_BK / 16; ++k4) {
                        const uint64_t da = umma_desc_kmajor(sa + k4 * 32, 128);
                        const uint64_t db = umma_desc_kmajor(sb + k4 * 32, 128);
                        umma_bf16(tmem_base + buf * BN, da, db, idesc, kc > 0 || k4 > 0);
                    }
                    umma_commit(empty0 + 8 * s);       // the stage may be refilled when these have run
                }
                umma_commit(accfull0 + 8 * buf);       // the accumulator is complete
            }
        }
    } else {
        // ---- epilogue: thread = row of the tile ------------------------------------------------
        const int q = warp & 3;                    // the warp's quarter of the tensor-memory lanes
        const int r = q * 32 + lane;
        const int et = tid - 64;                   // 0..127 among the epilogue threads
        int j = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++j) {
            const int buf = j & 1;
            const int64_t row = (int64_t)(t / a.col_tiles) * GM_BM + r;
            const int col0 = (t % a.col_tiles) * BN;
            const bool live = row < a.n;
            // this tile's bias as floats (the set of the other accumulator may still be in use)
            float* bs = bias_s + buf * BN;
            for (int c = et; c < BN; c += 128) bs[c] = a.bias ? __bfloat162float(a.bias[col0 + c]) : 0.f;
            named_barrier(1, 128);
            ok &= mbar_wait(accfull0 + 8 * buf, (j >> 1) & 1, abort);
            fence_after_sync();
            const uint32_t tm = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            __nv_bfloat16* orow = a.out + row * a.n_out + col0;
            const __nv_bfloat16* rrow = a.residual ? a.residual + row * a.n_out + col0 : nullptr;
#pragma unroll 2
            for (int c = 0; c < BN / 32; ++c) {
                uint4 res4[4] = {};
                if (rrow && live) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) res4[g] = *reinterpret_cast<const uint4*>(rrow + c * 32 + g * 8);
                }
                uint32_t v[32];
                tmem_ld32(tm + c * 32, v);
                tmem_ld_wait();
                if (!live) continue;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float y = gm_round(__uint_as_float(v[g * 8 + i]) + bs[c * 32 + g * 8 + i]);
                        if (a.gelu) y = gelu_tanh_erf(y);
                        f[i] = y;
                    }
                    if (rrow) {
                        float res[8];
                        Vec<__nv_bfloat16>::unpack(res4[g], res);
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] += res[i];
                    }
                    *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = Vec<__nv_bfloat16>::pack(f);
                }
            }
            // the accumulator may be overwritten
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_one(accempty0 + 8 * buf);
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
    if (lane == 0 && (!ok || (tid == 0 && *abort))) atomicOr(a.status, PTV3_STATUS_WAIT_LIMIT);
}

static bool gemm_shape_ok(int k, int n_out)
{
    return k >= 64 && k % 64 == 0 && k <= 8192 && n_out >= 128 && n_out % 128 == 0 && n_out <= 8192;
}

template <int BN, int STAGES>
static int launch_gemm_as(const CUtensorMap& mx, const CUtensorMap& mw, GemmArgs a, cudaStream_t stream)
{
    const size_t smem = (size_t)STAGES * (GM_A_BYTES + (size_t)BN * GM_BK * 2) + 2 * BN * 4 + 8 * (2 * STAGES + 4) +
                        16 + 1024;
    auto kern = gemm_tc05_kernel<BN, STAGES>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("ptv3_gemm_fwd: shared memory attribute");
    a.col_tiles = a.n_out / BN;
    const int64_t tiles = (int64_t)a.row_tiles * a.col_tiles;
    launch_dependent(kern, dim3((unsigned)(tiles < 148 ? tiles : 148)), dim3(GM_THREADS), smem, stream, mx, mw, a);
    count_launches(1);
    return check_launch("ptv3_gemm_fwd");
}

static int launch_gemm(const void* x, const void* w, GemmArgs a, cudaStream_t stream)
{
    a.row_tiles = (int)((a.n + GM_BM - 1) / GM_BM);
    // 256-column tiles halve the traffic of x; 128-column tiles when those would leave SMs idle
    int bn = a.n_out % 256 == 0 ? 256 : 128;
    if (bn == 256 && (int64_t)a.row_tiles * (a.n_out / 256) < 148) bn = 128;
    CUtensorMap mx, mw;
    int rc = make_tensor_map_bf16(&mx, x, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.k * 2, GM_BM, GM_BK);
    if (rc) return rc;
    rc = make_tensor_map_bf16(&mw, w, (uint64_t)a.n_out, (uint64_t)a.k, (uint64_t)a.k * 2, bn, GM_BK);
    if (rc) return rc;
    if (bn == 256) return launch_gemm_as<256, 4>(mx, mw, a, stream);
    return launch_gemm_as<128, 6>(mx, mw, a, stream);
}

}  // namespace ptv3

extern "C" int ptv3_gemm_supported(int k, int n_out, int dtype)
{
    return dtype == PTV3_DTYPE_BF16 && ptv3::gemm_shape_ok(k, n_out);
}

extern "C" int ptv3_gemm_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* out,
                             int64_t n, int k, int n_out, int gelu, int dtype, uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_gemm_fwd: bad n");
    PTV3_REQUIRE(ptv3_gemm_supported(k, n_out, dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_gemm_fwd: supported: bf16, k a multiple of 64, n_out a multiple of 128 (got %d, %d)", k, n_out);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(x && weight && out && status, PTV3_ERR_INVALID_ARGUMENT, "ptv3_gemm_fwd: null pointer");
    PTV3_REQUIRE((((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out | (uintptr_t)bias | (uintptr_t)residual) & 15) == 0,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_gemm_fwd: tensors must be 16-byte aligned");
    GemmArgs a{};
    a.bias = (const __nv_bfloat16*)bias;
    a.residual = (const __nv_bfloat16*)residual;
    a.out = (__nv_bfloat16*)out;
    a.n = n;
    a.k = k;
    a.n_out = n_out;
    a.gelu = gelu ? 1 : 0;
    a.status = status;
    return launch_gemm(x, weight, a, (cudaStream_t)stream);
}
