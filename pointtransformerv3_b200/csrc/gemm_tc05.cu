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
// in tensor memory and releases a stage with tcgen05.commit, warps 2..9 take a finished
// accumulator (tcgen05.ld, thread = row; two warps per quarter of the tensor-memory lanes, half of
// the tile's columns each), add the bias, apply GELU, add the residual row and write bf16 while
// the next tile is already being multiplied into the other accumulator.
// The output leaves through shared memory: each epilogue warp packs 64 columns of its 32 rows
// into a 4 KiB staging tile (128-byte swizzle, so the 16-byte stores of a warp do not collide)
// and one lane hands the tile to TMA, which writes whole 128-byte lines; a thread that stored
// its own row directly touched 32 lines per instruction, and that store path, not the tensor
// pipe or DRAM, set the pace of long inputs (10 000 cycles per 128 x 256 tile).
// The roundings are those of the unfused sequence (GEMM output rounded to bf16, then GELU or
// the residual sum rounded again).  Every mbarrier wait is bounded and reports through the
// status word.
#include "common.cuh"
#include "tc05.cuh"
#include "vec.cuh"
#include "mma_util.cuh"

namespace ptv3 {

using namespace tc05;

constexpr int GM_BM = 128;
constexpr int GM_BK = 64;                       // bf16 columns per stage: one 128-byte swizzle span
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;   // 16 KiB
constexpr int GM_EPI_WARPS = 8;                              // two per quarter of the tensor-memory lanes
constexpr int GM_THREADS = 64 + GM_EPI_WARPS * 32;
constexpr int GM_OUT_COLS = 64;                              // columns of a staging tile
constexpr int GM_OUT_BYTES = 32 * GM_OUT_COLS * 2;           // per epilogue warp: 4 KiB
constexpr int GM_OUT_TOTAL = GM_EPI_WARPS * GM_OUT_BYTES;

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


// MODE: bit 0 = GELU after the bias, bit 1 = residual added last.
// WRES: the CTA keeps its column tile of W (all K chunks) in shared memory for the whole launch and
// walks row tiles of that one column tile; only x goes through the ring.  Without it every tile
// fetches its W chunks again (from L2), which is what paces long inputs once the output path is out
// of the way: 192 KiB per 128 x 256 tile at K = 256, against 64 KiB of x.
template <int BN, int STAGES, int MODE, bool WRES>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_o,
                                                                  const GemmArgs a)
{
    pdl_launch_next();
    constexpr int B_BYTES = BN * GM_BK * 2;
    constexpr int STAGE_BYTES = WRES ? GM_A_BYTES : GM_A_BYTES + B_BYTES;
    constexpr int NBAR = 2 * STAGES + 5;      // full, empty per stage; accumulator full / empty x 2; W
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32_generic(smem);
    const int nk = a.k / GM_BK;
    const int w_bytes = WRES ? nk * B_BYTES : 0;          // the resident column tile of W comes first
    const uint32_t ring = sbase + w_bytes;
    const int off_out = w_bytes + STAGES * STAGE_BYTES;   // staging tiles of the output
    const int off_bias = off_out + GM_OUT_TOTAL;          // BN floats
    const int off_bar = off_bias + BN * 4;
    float* bias_s = reinterpret_cast<float*>(smem + off_bias);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t full0 = sbase + off_bar, empty0 = full0 + 8 * STAGES, accfull0 = empty0 + 8 * STAGES,
                   accempty0 = accfull0 + 16, wbar = accempty0 + 16;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ntiles = a.row_tiles * a.col_tiles;
    // i-th tile of this CTA.  Column tiles of a row tile run on neighbouring CTAs at the same time, so
    // the x rows they share are fetched from DRAM once.
    auto tile_at = [&](int i, int& row0, int& col0) -> bool {
        if (WRES) {
            const int rt = (int)blockIdx.x / a.col_tiles + i * ((int)gridDim.x / a.col_tiles);
            row0 = rt * GM_BM;
            col0 = ((int)blockIdx.x % a.col_tiles) * BN;
            return rt < a.row_tiles;
        }
        const int t = (int)blockIdx.x + i * (int)gridDim.x;
        row0 = (t / a.col_tiles) * GM_BM;
        col0 = (t % a.col_tiles) * BN;
        return t < ntiles;
    };

    if (tid == 0) {
        for (int i = 0; i < 2 * STAGES + 2; ++i) mbar_init(full0 + 8 * i, 1);
        mbar_init(accempty0, GM_EPI_WARPS);          // one arrival per epilogue warp
        mbar_init(accempty0 + 8, GM_EPI_WARPS);
        mbar_init(wbar, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_o);
    }
    if (warp == 1) tmem_alloc(sbase + off_bar + 8 * NBAR, 2 * BN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    if (WRES && tid == 0) {
        // the weights are not written by the launch before this one: fetched ahead of the wait below
        int row0, col0;
        tile_at(0, row0, col0);
        mbar_expect_tx(wbar, (uint32_t)w_bytes);
        for (int kc = 0; kc < nk; ++kc) tma_load_2d(sbase + kc * B_BYTES, &map_w, kc * GM_BK, col0, wbar);
    }
    // barriers, tensor memory and descriptors are set up; everything the kernel before this one in
    // the stream may have written is touched after this wait
    pdl_wait();

    if (warp == 0) {
        // ---- producer: K chunks of the x tile and of the W tile, tile after tile -----------------
        if (lane == 0) {
            int it = 0, row0, col0;
            for (int i = 0; tile_at(i, row0, col0); ++i) {
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % STAGES;
                    // a stage is free once the products that read it have completed (the first pass
                    // over the ring finds every stage free: waiting for the phase before the first)
                    ok &= mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort);
                    const uint32_t sa = ring + s * STAGE_BYTES;
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(sa, &map_x, kc * GM_BK, row0, full0 + 8 * s);
                    if (!WRES) tma_load_2d(sa + GM_A_BYTES, &map_w, kc * GM_BK, col0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- issuer -----------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(GM_BM, BN);
            int it = 0, row0, col0;
            if (WRES) ok &= mbar_wait(wbar, 0, abort);
            for (int j = 0; tile_at(j, row0, col0); ++j) {
                const int buf = j & 1;
                // the epilogue has read the accumulator's previous tile (first use: free)
                ok &= mbar_wait(accempty0 + 8 * buf, ((j >> 1) & 1) ^ 1, abort);
                fence_after_sync();
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % STAGES;
                    ok &= mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort);
                    fence_after_sync();
                    const uint32_t sa = ring + s * STAGE_BYTES, sb = WRES ? sbase + kc * B_BYTES : sa + GM_A_BYTES;
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
        const int half = (warp - 2) >> 2;          // which half of the tile's columns
        const int et = tid - 64;                   // index among the epilogue threads
        const ulonglong2* bias4 = reinterpret_cast<const ulonglong2*>(bias_s);
        const uint32_t so = sbase + off_out + (warp - 2) * GM_OUT_BYTES;
        const uint32_t my_row = lane * 128, sw = lane & 7;
        int row0, col0;
        for (int j = 0; tile_at(j, row0, col0); ++j) {
            const int buf = j & 1;
            const int64_t row = (int64_t)row0 + r;
            const bool live = row < a.n;
            if (j == 0 || (!WRES && a.col_tiles > 1)) {
                // this tile's bias as floats, once every warp has finished the tile before
                if (j) named_barrier(1, GM_EPI_WARPS * 32);
                for (int c = et; c < BN; c += GM_EPI_WARPS * 32) bias_s[c] = a.bias ? __bfloat162float(a.bias[col0 + c]) : 0.f;
                named_barrier(1, GM_EPI_WARPS * 32);
            }
            ok &= mbar_wait(accfull0 + 8 * buf, (j >> 1) & 1, abort);
            fence_after_sync();
            const uint32_t tm = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            const __nv_bfloat16* rrow = (MODE & 2) ? a.residual + row * a.n_out + col0 : nullptr;
            constexpr int NCH = BN / GM_OUT_COLS / 2;      // 64-column chunks of this warp
            for (int c = half * NCH; c < (half + 1) * NCH; ++c) {
                uint32_t v[2][32];
                tmem_ld32(tm + c * 64, v[0]);
                tmem_ld32(tm + c * 64 + 32, v[1]);
                uint4 res4[(MODE & 2) ? 8 : 1] = {};
                if ((MODE & 2) && live) {
#pragma unroll
                    for (int g = 0; g < 8; ++g) res4[g] = *reinterpret_cast<const uint4*>(rrow + c * 64 + g * 8);
                }
                // the copy of the chunk before has finished reading the staging tile
                if (lane == 0) bulk_wait_read<0>();
                __syncwarp();
                tmem_ld_wait();
                tmem_ld_fence(v[0]);
                tmem_ld_fence(v[1]);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const uint32_t* vv = &v[g >> 2][(g & 3) * 8];
                    const uint4 r4 = res4[(MODE & 2) ? g : 0];
                    const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
                    uint32_t o[4];
#pragma unroll
                    for (int p2 = 0; p2 < 4; ++p2) {
                        const ulonglong2 b4 = bias4[c * 16 + g * 2 + (p2 >> 1)];
                        uint64_t y = add2(pack2u(vv[2 * p2], vv[2 * p2 + 1]), (p2 & 1) ? b4.y : b4.x);
                        float lo, hi;
                        unpack2(y, lo, hi);
                        uint32_t packed = pack_bf16(lo, hi);     // the Linear's own output in bf16
                        if (MODE != 0) {
                            y = unpack_bf16x2(packed);
                            if (MODE & 1) y = gelu_tanh_erf2(y);
                            if (MODE & 2) y = add2(y, unpack_bf16x2(rw[p2]));
                            unpack2(y, lo, hi);
                            packed = pack_bf16(lo, hi);
                        }
                        o[p2] = packed;
                    }
                    // (no memory clobber: the bias loads of the next columns may be scheduled above it;
                    // volatile keeps it before the proxy fence below)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(so + my_row + ((g ^ sw) << 4)),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]));
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && row0 + q * 32 < a.n) {
                    tma_store_2d(&map_o, col0 + c * GM_OUT_COLS, row0 + q * 32, so);
                    bulk_commit();
                }
            }
            // the accumulator may be overwritten
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_one(accempty0 + 8 * buf);
        }
        // shared memory stays allocated until the last copies have read it
        if (lane == 0) bulk_wait_read<0>();
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

// W stays in shared memory when a column tile of it fits beside the ring, the ring of four x chunks
// still holds a whole tile (K <= 256: with K = 512 the streamed form measured faster) and a CTA has
// enough tiles to repay loading it
static bool gemm_w_resident(const GemmArgs& a, int bn)
{
    return a.k <= 256 && (size_t)a.k * bn * 2 <= 131072 && (int64_t)a.row_tiles * (a.n_out / bn) >= 3 * 148;
}

template <int BN, int STAGES, int MODE, bool WRES>
static int launch_gemm_mode(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, GemmArgs a,
                            cudaStream_t stream)
{
    const size_t b_bytes = (size_t)BN * GM_BK * 2;
    const size_t smem = (WRES ? (size_t)(a.k / GM_BK) * b_bytes + (size_t)STAGES * GM_A_BYTES
                              : (size_t)STAGES * (GM_A_BYTES + b_bytes)) +
                        GM_OUT_TOTAL + BN * 4 + 8 * (2 * STAGES + 5) + 16 + 1024;
    auto kern = gemm_tc05_kernel<BN, STAGES, MODE, WRES>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("ptv3_gemm_fwd: shared memory attribute");
    a.col_tiles = a.n_out / BN;
    const int64_t tiles = (int64_t)a.row_tiles * a.col_tiles;
    // resident W: the same number of CTAs on every column tile
    const unsigned grid = WRES ? (unsigned)(148 / a.col_tiles * a.col_tiles) : (unsigned)(tiles < 148 ? tiles : 148);
    launch_dependent(kern, dim3(grid), dim3(GM_THREADS), smem, stream, mx, mw, mo, a);
    count_launches(1);
    return check_launch("ptv3_gemm_fwd");
}

template <int BN, int STAGES, bool WRES>
static int launch_gemm_as(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const GemmArgs& a,
                          cudaStream_t stream)
{
    switch ((a.gelu ? 1 : 0) | (a.residual ? 2 : 0)) {
    case 0: return launch_gemm_mode<BN, STAGES, 0, WRES>(mx, mw, mo, a, stream);
    case 1: return launch_gemm_mode<BN, STAGES, 1, WRES>(mx, mw, mo, a, stream);
    case 2: return launch_gemm_mode<BN, STAGES, 2, WRES>(mx, mw, mo, a, stream);
    default: return launch_gemm_mode<BN, STAGES, 3, WRES>(mx, mw, mo, a, stream);
    }
}

static int launch_gemm(const void* x, const void* w, GemmArgs a, cudaStream_t stream)
{
    a.row_tiles = (int)((a.n + GM_BM - 1) / GM_BM);
    // 256-column tiles halve the traffic of x; 128-column tiles when those would leave SMs idle
    int bn = a.n_out % 256 == 0 ? 256 : 128;
    if (bn == 256 && (int64_t)a.row_tiles * (a.n_out / 256) < 148) bn = 128;
    CUtensorMap mx, mw, mo;
    int rc = make_tensor_map_bf16(&mx, x, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.k * 2, GM_BM, GM_BK);
    if (rc) return rc;
    rc = make_tensor_map_bf16(&mw, w, (uint64_t)a.n_out, (uint64_t)a.k, (uint64_t)a.k * 2, bn, GM_BK);
    if (rc) return rc;
    rc = make_tensor_map_bf16(&mo, a.out, (uint64_t)a.n, (uint64_t)a.n_out, (uint64_t)a.n_out * 2, 32, GM_OUT_COLS);
    if (rc) return rc;
    if (gemm_w_resident(a, bn))
        return bn == 256 ? launch_gemm_as<256, 4, true>(mx, mw, mo, a, stream)
                         : launch_gemm_as<128, 4, true>(mx, mw, mo, a, stream);
    if (bn == 256) return launch_gemm_as<256, 4, false>(mx, mw, mo, a, stream);
    return launch_gemm_as<128, 6, false>(mx, mw, mo, a, stream);
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
