// Fused MLP of a block on the 5th-generation tensor cores:
//     out = residual + fc2(GELU(fc1(x) + b1)) + b2          (model.py:510-516, 601-602)
// for bf16 features with C = 32 or 64 channels (hidden = 4 C), i.e. the stages that
// hold almost all points.  The hidden activation (the largest tensor of the
// backbone) never leaves the SM.
//
// A CTA is persistent and holds both weight matrices in shared memory (TMA, loaded
// once).  Its 512 threads form four independent groups of 128 (so that the
// tensor-memory loads, GELU arithmetic and stores of different tiles overlap);
// each group walks its own 128-row tiles, 64 hidden columns at a time:
//   TMA    x tile (128 x C, 64/128-byte swizzle)                 -> shared memory
//   UMMA   D1[128 x 64] = x . W1_chunk^T     (tcgen05.mma, accumulator in TMEM)
//   warps  tcgen05.ld D1 -> + b1 -> GELU -> bf16 -> shared memory in the UMMA
//          K-major 128-byte-swizzled layout (the A operand of the second GEMM)
//   UMMA   D2[128 x C] += h_chunk . W2_chunk^T
//   warps  tcgen05.ld D2 -> + b2 -> + residual -> global
// Completion is tracked with mbarriers (TMA transaction bytes, tcgen05.commit);
// every wait is bounded and reports through the status word instead of hanging.
#include "common.cuh"
#include "tc05.cuh"
#include "vec.cuh"

namespace ptv3 {

using namespace tc05;

template <int C>
struct MlpCfg {
    static constexpr int HD = 4 * C;                  // hidden width
    static constexpr int HC = 64;                     // hidden columns per round
    static constexpr int NG = 4;                      // independent 128-thread groups per CTA
    static constexpr int NCH = HD / HC;
    static constexpr int SWX = C * 2;                 // bytes per row of x / W1 (= swizzle span)
    static constexpr int W1_BYTES = HD * SWX;
    static constexpr int W2_BLOCK = C * 128;          // one 64-wide K block of W2
    static constexpr int W2_BYTES = (HD / 64) * W2_BLOCK;
    static constexpr int X_BYTES = 128 * SWX;
    static constexpr int H_BLOCK = 128 * 128;         // one 64-wide K block of the activation
    static constexpr int H_BYTES = (HC / 64) * H_BLOCK;
    static constexpr int OFF_W1 = 0;
    static constexpr int OFF_W2 = OFF_W1 + W1_BYTES;
    static constexpr int OFF_G = OFF_W2 + W2_BYTES;   // per group: x tile, activation
    static constexpr int G_BYTES = X_BYTES + H_BYTES;
    static constexpr int OFF_B1 = OFF_G + NG * G_BYTES;
    static constexpr int OFF_B2 = OFF_B1 + HD * 4;
    static constexpr int OFF_BAR = OFF_B2 + C * 4;    // 1 + 3 NG mbarriers, tmem pointer, abort flag
    static constexpr int NBAR = 1 + 3 * NG;
    // + slack for the 1 KiB alignment; at least 120 KiB so that two CTAs (each wanting all of
    // tensor memory) never share an SM
    static constexpr int SMEM_NEED = OFF_BAR + 8 * NBAR + 64 + 1024;
    static constexpr int SMEM = SMEM_NEED < 120 * 1024 ? 120 * 1024 : SMEM_NEED;
    static constexpr int TMEM_D1 = 0, TMEM_D2 = 64, TMEM_GROUP = 128;
};

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int C>
__global__ void __launch_bounds__(128 * MlpCfg<C>::NG, 1) mlp_tc05_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
    const __grid_constant__ CUtensorMap map_w2, const __nv_bfloat16* __restrict__ b1,
    const __nv_bfloat16* __restrict__ b2, const __nv_bfloat16* __restrict__ residual,
    __nv_bfloat16* __restrict__ out, int64_t n, uint32_t* __restrict__ status)
{
    pdl_launch_next();
    using Cfg = MlpCfg<C>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32_generic(smem);
    float* b1s = reinterpret_cast<float*>(smem + Cfg::OFF_B1);
    float* b2s = reinterpret_cast<float*>(smem + Cfg::OFF_B2);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NBAR);
    constexpr int NT = 128 * Cfg::NG;
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int g = tid >> 7, t = tid & 127;
    const uint32_t wbar = sbase + Cfg::OFF_BAR;
    const uint32_t xbar = wbar + 8 * (1 + g), m1bar = wbar + 8 * (1 + Cfg::NG + g),
                   m2bar = wbar + 8 * (1 + 2 * Cfg::NG + g);

    if (tid == 0) {
        for (int i = 0; i < Cfg::NBAR; ++i) mbar_init(wbar + 8 * i, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w1);
        prefetch_tensormap(&map_w2);
    }
    for (int i = tid; i < Cfg::HD; i += NT) b1s[i] = __bfloat162float(b1[i]);
    for (int i = tid; i < C; i += NT) b2s[i] = __bfloat162float(b2[i]);
    if (warp == 0) tmem_alloc(sbase + Cfg::OFF_BAR + 8 * Cfg::NBAR, 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (tid == 0) {   // weights: once per CTA
        mbar_expect_tx(wbar, Cfg::W1_BYTES + Cfg::W2_BYTES);
        constexpr int W1_ROWS_PER_BOX = Cfg::HD > 256 ? 256 : Cfg::HD;
        for (int r = 0; r < Cfg::HD; r += W1_ROWS_PER_BOX)
            tma_load_2d(sbase + Cfg::OFF_W1 + r * Cfg::SWX, &map_w1, 0, r, wbar);
        for (int kb = 0; kb < Cfg::HD / 64; ++kb)
            tma_load_2d(sbase + Cfg::OFF_W2 + kb * Cfg::W2_BLOCK, &map_w2, kb * 64, 0, wbar);
    }
    // up to here only weights and biases were read: everything the kernel before this one in the
    // stream may have written is touched after this wait
    pdl_wait();
    bool ok = mbar_wait(wbar, 0, abort);

    const uint32_t xs = sbase + Cfg::OFF_G + g * Cfg::G_BYTES;
    const uint32_t hs = xs + Cfg::X_BYTES;
    unsigned char* hs_ptr = smem + Cfg::OFF_G + g * Cfg::G_BYTES + Cfg::X_BYTES;
    const uint32_t tm_lane = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tm_d1 = tmem_base + tm_lane + g * Cfg::TMEM_GROUP + Cfg::TMEM_D1;
    const uint32_t tm_d2 = tmem_base + tm_lane + g * Cfg::TMEM_GROUP + Cfg::TMEM_D2;
    const uint32_t tm_d1_mma = tmem_base + g * Cfg::TMEM_GROUP + Cfg::TMEM_D1;
    const uint32_t tm_d2_mma = tmem_base + g * Cfg::TMEM_GROUP + Cfg::TMEM_D2;
    constexpr uint32_t IDESC1 = umma_idesc_bf16(128, Cfg::HC);
    constexpr uint32_t IDESC2 = umma_idesc_bf16(128, C);
    uint32_t xph = 0, m1ph = 0, m2ph = 0;

    auto issue_gemm1 = [&](int ch) {
#pragma unroll
        for (int k = 0; k < C / 16; ++k) {
            const uint64_t da = umma_desc_kmajor(xs + k * 32, Cfg::SWX);
            const uint64_t db = umma_desc_kmajor(sbase + Cfg::OFF_W1 + ch * Cfg::HC * Cfg::SWX + k * 32, Cfg::SWX);
            umma_bf16(tm_d1_mma, da, db, IDESC1, k > 0);
        }
    };
    auto issue_gemm2 = [&](int ch) {
#pragma unroll
        for (int kb = 0; kb < Cfg::HC / 64; ++kb) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t da = umma_desc_kmajor(hs + kb * Cfg::H_BLOCK + k * 32, 128);
                const uint64_t db = umma_desc_kmajor(
                    sbase + Cfg::OFF_W2 + (ch * (Cfg::HC / 64) + kb) * Cfg::W2_BLOCK + k * 32, 128);
                umma_bf16(tm_d2_mma, da, db, IDESC2, !(ch == 0 && kb == 0 && k == 0));
            }
        }
    };

    const int64_t ntiles = (n + 127) / 128;
    const int64_t tile_step = (int64_t)gridDim.x * Cfg::NG;
    const int64_t tile0 = (int64_t)blockIdx.x * Cfg::NG + g;
    if (t == 0 && tile0 < ntiles) {
        mbar_expect_tx(xbar, Cfg::X_BYTES);
        tma_load_2d(xs, &map_x, 0, (int)(tile0 * 128), xbar);
    }
    for (int64_t tile = tile0; tile < ntiles; tile += tile_step) {
        const int64_t row0 = tile * 128;
        ok &= mbar_wait(xbar, xph, abort);
        xph ^= 1;
        if (t == 0) {
            fence_after_sync();
            issue_gemm1(0);
            umma_commit(m1bar);
        }
#pragma unroll 1
        for (int ch = 0; ch < Cfg::NCH; ++ch) {
            ok &= mbar_wait(m1bar, m1ph, abort);
            m1ph ^= 1;
            fence_after_sync();
            // the x tile has been consumed once the last first-GEMM is done: fetch the next one
            // while this tile's activation, second GEMM and output are still in progress
            if (t == 0 && ch == Cfg::NCH - 1 && tile + tile_step < ntiles) {
                mbar_expect_tx(xbar, Cfg::X_BYTES);
                tma_load_2d(xs, &map_x, 0, (int)((tile + tile_step) * 128), xbar);
            }
            // D1 -> + b1 -> GELU -> bf16 -> activation tile (K-major, 128-byte swizzle)
#pragma unroll 1
            for (int cg = 0; cg < Cfg::HC / 32; ++cg) {
                uint32_t v[32];
                tmem_ld32(tm_d1 + cg * 32, v);
                tmem_ld_wait();
                const float* bb = b1s + ch * Cfg::HC + cg * 32;
                unsigned char* blk = hs_ptr + (cg >> 1) * Cfg::H_BLOCK + t * 128;
                // pairs of channels: packed fp32 arithmetic, parameters two pairs per load
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t ow[4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const ulonglong2 b2 = *reinterpret_cast<const ulonglong2*>(bb + q * 8 + h * 4);
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int i = q * 8 + h * 4 + e * 2;
                            uint32_t pk;
                            const uint64_t y = round2(add2(pack2u(v[i], v[i + 1]), e ? b2.y : b2.x), pk);
                            float lo, hi;
                            unpack2(gelu_tanh_erf2(y), lo, hi);
                            ow[h * 2 + e] = pack_bf16(lo, hi);
                        }
                    }
                    const int c = (cg & 1) * 4 + q;
                    *reinterpret_cast<uint4*>(blk + ((c ^ (t & 7)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
            }
            fence_proxy_async();
            fence_before_sync();
            named_barrier(1 + g, 128);
            if (t == 0) {
                fence_after_sync();
                issue_gemm2(ch);
                if (ch + 1 < Cfg::NCH) {
                    issue_gemm1(ch + 1);
                    umma_commit(m1bar);
                } else {
                    umma_commit(m2bar);
                }
            }
        }
        ok &= mbar_wait(m2bar, m2ph, abort);
        m2ph ^= 1;
        fence_after_sync();
        // D2 -> + b2 -> + residual -> out.  The activation tile is free now and serves as a
        // staging tile (same 128-byte-pitch swizzle): the residual comes in and the result goes
        // out with coalesced 16-byte pieces, the row-per-thread arithmetic runs on shared memory.
        constexpr int PIECES = C / 8;   // 16-byte pieces per row
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int idx = i * 128 + t, r = idx / PIECES, c = idx % PIECES;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row0 + r < n) v = *reinterpret_cast<const uint4*>(residual + (row0 + r) * C + c * 8);
            *reinterpret_cast<uint4*>(hs_ptr + r * 128 + ((c ^ (r & 7)) << 4)) = v;
        }
        named_barrier(1 + g, 128);
#pragma unroll 1
        for (int cg = 0; cg < C / 32; ++cg) {
            uint32_t v[32];
            tmem_ld32(tm_d2 + cg * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                unsigned char* slot = hs_ptr + t * 128 + (((cg * 4 + q) ^ (t & 7)) << 4);
                const uint4 rr = *reinterpret_cast<const uint4*>(slot);
                const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
                uint32_t ow[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const ulonglong2 b2 = *reinterpret_cast<const ulonglong2*>(b2s + cg * 32 + q * 8 + h * 4);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int i = q * 8 + h * 4 + e * 2;
                        uint32_t pk;
                        const uint64_t y = round2(add2(pack2u(v[i], v[i + 1]), e ? b2.y : b2.x), pk);
                        float lo, hi;
                        unpack2(add2(unpack_bf16x2(rw[h * 2 + e]), y), lo, hi);
                        ow[h * 2 + e] = pack_bf16(lo, hi);
                    }
                }
                *reinterpret_cast<uint4*>(slot) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
        named_barrier(1 + g, 128);
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int idx = i * 128 + t, r = idx / PIECES, c = idx % PIECES;
            if (row0 + r < n)
                *reinterpret_cast<uint4*>(out + (row0 + r) * C + c * 8) =
                    *reinterpret_cast<const uint4*>(hs_ptr + r * 128 + ((c ^ (r & 7)) << 4));
        }
        fence_before_sync();
        named_barrier(1 + g, 128);
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && (*abort || !ok)) atomicOr(status, PTV3_STATUS_WAIT_LIMIT);
}

template <int C>
static int launch_mlp(const void* x, const void* w1, const void* b1, const void* w2, const void* b2,
                      const void* residual, void* out, int64_t n, uint32_t* status, cudaStream_t stream)
{
    using Cfg = MlpCfg<C>;
    CUtensorMap mx, mw1, mw2;
    int rc = make_tensor_map_bf16(&mx, x, (uint64_t)n, C, (uint64_t)C * 2, 128, C);
    if (rc) return rc;
    rc = make_tensor_map_bf16(&mw1, w1, Cfg::HD, C, (uint64_t)C * 2, Cfg::HD > 256 ? 256 : Cfg::HD, C);
    if (rc) return rc;
    rc = make_tensor_map_bf16(&mw2, w2, C, Cfg::HD, (uint64_t)Cfg::HD * 2, C, 64);
    if (rc) return rc;
    auto kern = mlp_tc05_kernel<C>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
        return check_launch("ptv3_mlp_fwd: shared memory attribute");
    const int64_t ntiles = (n + 127) / 128;
    int64_t grid = (ntiles + Cfg::NG - 1) / Cfg::NG;
    if (grid > 148) grid = 148;
    launch_dependent(kern, dim3((unsigned)grid), dim3(128 * Cfg::NG), Cfg::SMEM, stream, mx, mw1, mw2,
                     (const __nv_bfloat16*)b1, (const __nv_bfloat16*)b2, (const __nv_bfloat16*)residual,
                     (__nv_bfloat16*)out, n, status);
    count_launches(1);
    return check_launch("ptv3_mlp_fwd");
}

}  // namespace ptv3

extern "C" int ptv3_mlp_supported(int channels, int hidden, int dtype)
{
    return dtype == PTV3_DTYPE_BF16 && hidden == 4 * channels && (channels == 32 || channels == 64);
}

extern "C" int ptv3_mlp_fwd(const void* x, const void* fc1_weight, const void* fc1_bias,
                            const void* fc2_weight, const void* fc2_bias, const void* residual, void* out,
                            int64_t n, int channels, int hidden, int dtype, uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_mlp_fwd: bad n");
    PTV3_REQUIRE(ptv3_mlp_supported(channels, hidden, dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_mlp_fwd: supported: bf16, channels 32 or 64, hidden = 4 x channels");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(x && fc1_weight && fc1_bias && fc2_weight && fc2_bias && residual && out && status,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_mlp_fwd: null pointer");
    PTV3_REQUIRE((((uintptr_t)x | (uintptr_t)fc1_weight | (uintptr_t)fc2_weight | (uintptr_t)residual |
                   (uintptr_t)out) & 15) == 0,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_mlp_fwd: tensors must be 16-byte aligned");
    if (channels == 32)
        return launch_mlp<32>(x, fc1_weight, fc1_bias, fc2_weight, fc2_bias, residual, out, n, status,
                              (cudaStream_t)stream);
    return launch_mlp<64>(x, fc1_weight, fc1_bias, fc2_weight, fc2_bias, residual, out, n, status,
                          (cudaStream_t)stream);
}
