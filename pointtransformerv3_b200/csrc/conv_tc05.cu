// Submanifold convolution (3x3x3) for bf16 features on the 5th-generation tensor cores:
// an implicit GEMM, output-stationary over tiles of 128 voxels, accumulated in tensor memory.
//
// A CTA owns 128 voxels (consecutive in the tile order, which follows a space-filling curve) and
// BN output channels.  It stages the 27 x 128 neighbour rows of its tile in shared memory and
// drops the offsets for which no voxel of the tile has a neighbour.  Then, for each remaining
// offset o and each KC-wide slice of the input channels,
//   warps 0..3  each fill every fourth stage: the 128 neighbour rows (zero rows where there is none)
//               gathered with cp.async into the 128-byte (64-byte for KC = 32) swizzled K-major
//               operand layout, and the matching BN x KC slice of W[:, o, :] fetched with TMA into
//               the same layout,
//   warp 4      issues KC / 16 tcgen05.mma (M = 128, N = BN, K = 16) that add A_o W_o^T to the
//               accumulator in tensor memory, and releases the stage with tcgen05.commit,
// through a ring of stages guarded by mbarriers.  When the last product has completed, warps 0..3
// read the accumulator (thread = voxel), add the bias, round to bf16 and store their rows.
//
// Two threads issue the products, taking the stages in turn, each into its own accumulator (one
// thread can start a stage only every ~450 cycles: looking at a stage's barrier costs it as much as
// issuing the stage's four products); the epilogue adds the two partial sums.  Every sum is taken
// in one fixed order, so the result is the same bit for bit on every run, on every level: no
// atomics, no pair lists, no second pass.  Products with zero rows are not skipped (on coarse
// levels about two thirds of the rows of an active offset are empty): the tensor pipe has time to
// spare.  What bounds the kernel is the length of a slot's cycle, not a throughput: once a slot is
// free its warp issues the weight load and 32 copies per lane (~1100 cycles), the rows land (~1200),
// the warp fences and arrives, an issuer notices, issues, the products complete and the commit
// frees the slot (~1500 more): ~4000 cycles for six slots, one stage per ~700 cycles.  Counters of
// one launch: tensor pipe 22 % active, shared-memory pipe 29 % (16 % operand reads of the tensor
// core, 13 % copies and loads), L2 19 %, DRAM 5 %; leaving out the gather copies or the weight
// loads altogether changes the time by 10 % and 2 %.
//
// Replaces spconv.SubMConv3d.forward at model.py:546-552 for bf16.
// Useful work: 2 . pairs . C_in . C_out FLOP.  Every mbarrier wait is bounded and reports through
// the status word.
#include "common.cuh"
#include "conv_mma.cuh"
#include "mma_util.cuh"
#include "tc05.cuh"

namespace ptv3 {

using namespace tc05;

constexpr int CT_TM = 128;         // voxels per tile
constexpr int CT_MAX_KVOL = 27;
constexpr int CT_GATHER_WARPS = 8;


struct ConvTcArgs {
    const __nv_bfloat16* feat;
    const int32_t* nbr;            // kvol x n, columns in tile order
    const __nv_bfloat16* bias;     // cout or NULL
    __nv_bfloat16* out;
    const int64_t* row_order;      // voxel of every tile position, or NULL
    int64_t n;
    int cin, cout, kvol;
    uint32_t* status;
};

template <int BN, int KC, int STAGES, int NI>
__global__ void __launch_bounds__((CT_GATHER_WARPS + NI) * 32) conv_tc05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                               const ConvTcArgs a)
{
    pdl_launch_next();
    constexpr int ROWB = KC * 2;                    // bytes per staged row: one swizzle span (128 or 64)
    constexpr int NCH = ROWB / 16;                  // 16-byte chunks per row
    constexpr int A_BYTES = CT_TM * ROWB, B_BYTES = BN * ROWB, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int CT_THREADS = (CT_GATHER_WARPS + NI) * 32;
    // NI issuing threads, each with its own accumulator in tensor memory (columns rounded up to a power
    // of two for the allocation).  A slot of the ring must always be consumed by the same issuer
    // (STAGES a multiple of NI): an issuer that met a slot whose previous use another, slower issuer had
    // not consumed yet would take the parity of that older phase for its own.
    constexpr int TM_USED = NI * BN;
    constexpr int TM_COLS = TM_USED <= 32 ? 32 : TM_USED <= 64 ? 64 : TM_USED <= 128 ? 128 : TM_USED <= 256 ? 256 : 512;
    static_assert(TM_USED <= 512 && STAGES % NI == 0, "issuers and accumulators");
    static_assert(STAGE_BYTES % 1024 == 0 && A_BYTES % 1024 == 0, "operand tiles start on a swizzle atom");
    // Warps that gather: at most one per stage of the ring.  A parity wait on an mbarrier can only tell
    // the current phase from the one before it, so a warp must never be two uses ahead of a slot: its
    // stages are NGW apart, and having been given a slot for stage X (stage X - STAGES consumed) it may
    // ask for the slot of stage X + NGW only if stage X + NGW - 2 STAGES is known to be consumed,
    // i.e. NGW <= STAGES (the products run in order).
    constexpr int NGW = STAGES < CT_GATHER_WARPS ? STAGES : CT_GATHER_WARPS;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32_generic(smem);
    constexpr int OFF_NBR = STAGES * STAGE_BYTES;                   // kvol x 128 int32
    constexpr int OFF_ROWS = OFF_NBR + CT_MAX_KVOL * CT_TM * 4;     // 128 int64
    constexpr int OFF_ACT = OFF_ROWS + CT_TM * 8;                   // 32 int
    constexpr int OFF_BIAS = OFF_ACT + 32 * 4;                      // BN float
    constexpr int OFF_BAR = OFF_BIAS + BN * 4;                      // full, empty per stage; accumulator full
    int32_t* nbr_s = reinterpret_cast<int32_t*>(smem + OFF_NBR);
    int64_t* rows_s = reinterpret_cast<int64_t*>(smem + OFF_ROWS);
    int* act = reinterpret_cast<int*>(smem + OFF_ACT);
    float* bias_s = reinterpret_cast<float*>(smem + OFF_BIAS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 8 * (2 * STAGES + 1));
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t full0 = sbase + OFF_BAR, empty0 = full0 + 8 * STAGES, accfull = empty0 + 8 * STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t row0 = (int64_t)blockIdx.x * CT_TM;
    const int col0 = blockIdx.y * BN;
    const int kvol = a.kvol;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 2);        // the gathering warp of the stage + its weight load
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accfull, NI);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_w);
    }
    if (warp == CT_GATHER_WARPS) tmem_alloc(smem_u32_generic(tmem_slot), TM_COLS);
    // (only the set-up above runs beside the kernel before this one in the stream)
    pdl_wait();

    // ---- voxels of this tile, their neighbour rows, the offsets in use -------------------------
    if (tid < CT_TM) {
        const int64_t i = row0 + tid;
        rows_s[tid] = i < a.n ? (a.row_order ? a.row_order[i] : i) : -1;
    }
    for (int c = tid; c < BN; c += CT_THREADS) bias_s[c] = a.bias ? __bfloat162float(a.bias[col0 + c]) : 0.f;
    {
        // A warp stages whole offsets (four coalesced rows of 32 entries each), all of its loads issued
        // before the first store, and notes in the same pass whether the tile has the offset at all.
        constexpr int NW = CT_THREADS / 32, OPW = (CT_MAX_KVOL + NW - 1) / NW;
        int32_t v[OPW][4];
#pragma unroll
        for (int j = 0; j < OPW; ++j) {
            const int o = warp + j * NW;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = lane + 32 * i;
                v[j][i] = (o < kvol && row0 + r < a.n) ? __ldg(a.nbr + (int64_t)o * a.n + row0 + r) : -1;
            }
        }
#pragma unroll
        for (int j = 0; j < OPW; ++j) {
            const int o = warp + j * NW;
            if (o < kvol) {
                bool any = false;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    nbr_s[o * CT_TM + lane + 32 * i] = v[j][i];
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
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int n_act = act[0];
    const int kchunks = a.cin / KC;
    const int nit = n_act * kchunks;
    bool ok = true;

    if (warp < CT_GATHER_WARPS) {
        // ---- gather: warp w < NGW fills stages w, w + NGW, ...: the 128 neighbour rows of offset
        // act[it / kchunks], channels of chunk it % kchunks, and (lane 0) the matching slice of W.
        // The warps run independent pipelines, so the fixed cost of a stage (barrier waits, the TMA
        // issue, the proxy fence) and the latency of its copies overlap with the other warps' stages.
        constexpr int RPP = 32 / NCH;                     // rows per pass of the warp
        const int c = lane % NCH, rr = lane / NCH;        // this lane's chunk and first row
        for (int it = warp < NGW ? warp : nit; it < nit; it += NGW) {
            const int s = it % STAGES;
            if (lane == 0) {
                if (it >= STAGES) ok &= mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort);
            }
            __syncwarp();
            const int o = act[1 + it / kchunks];
            const int kc = (it % kchunks) * KC;
            const uint32_t sa = sbase + s * STAGE_BYTES;
            const __nv_bfloat16* src0 = a.feat + kc + c * 8;
            const int32_t* nb = nbr_s + o * CT_TM + rr;
#pragma unroll
            for (int j0 = 0; j0 < CT_TM / RPP; j0 += 8) {
                int32_t src[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) src[j] = nb[(j0 + j) * RPP];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = rr + (j0 + j) * RPP;
                    const int pc = NCH == 8 ? (c ^ (r & 7)) : (c ^ ((r >> 1) & 3));
                    cp_async16_zfill(sa + r * ROWB + pc * 16, src0 + (int64_t)(src[j] < 0 ? 0 : src[j]) * a.cin,
                                     src[j] >= 0);
                }
            }
            cp_async_commit();
            // (the weight load is issued after the copies: its issue costs lane 0 ~350 cycles, during
            // which the rows are already on their way)
            if (lane == 0) {
                mbar_expect_tx(full0 + 8 * s, B_BYTES);
                tma_load_2d(sa + A_BYTES, &map_w, o * a.cin + kc, col0, full0 + 8 * s);
            }
            cp_async_wait<0>();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_one(full0 + 8 * s);
        }

        // ---- epilogue: thread = voxel ----------------------------------------------------------
        if (nit > 0) {
            ok &= mbar_wait(accfull, 0, abort);
            fence_after_sync();
        }
        const bool read_acc = nit > 0 && __all_sync(0xffffffffu, ok);    // tcgen05.ld is warp-wide
        const int q = warp & 3, half = warp >> 2;      // lane quarter of tensor memory, half of the columns
        const int64_t v = rows_s[q * 32 + lane];
        const uint32_t tm = tmem_base + ((uint32_t)(q * 32) << 16);
        __nv_bfloat16* orow = a.out + v * a.cout + col0;
        constexpr int NCB = BN / 32;                   // 32-column blocks, split between the two halves
#pragma unroll 1
        for (int cb = half * ((NCB + 1) / 2); cb < (half == 0 ? (NCB + 1) / 2 : NCB); ++cb) {
            uint32_t acc[32];
            if (read_acc) {
                tmem_ld32(tm + cb * 32, acc);
                tmem_ld_wait();
                // the other issuers' partial sums, added in a fixed order
#pragma unroll 1
                for (int i = 1; i < NI && i < nit; ++i) {
                    uint32_t more[32];
                    tmem_ld32(tm + i * BN + cb * 32, more);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        acc[e] = __float_as_uint(__uint_as_float(acc[e]) + __uint_as_float(more[e]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = 0;
            }
            if (v < 0) continue;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint4 o4;
                uint32_t* o = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    o[i] = pack_bf16(__uint_as_float(acc[g * 8 + 2 * i]) + bias_s[cb * 32 + g * 8 + 2 * i],
                                     __uint_as_float(acc[g * 8 + 2 * i + 1]) + bias_s[cb * 32 + g * 8 + 2 * i + 1]);
                *reinterpret_cast<uint4*>(orow + cb * 32 + g * 8) = o4;
            }
        }
    } else {
        // ---- issuers: thread i takes stages i, i + NI, ... in order and accumulates them in
        // its own accumulator.  One thread can start a stage's products only every ~450 cycles (a look
        // at the stage's barrier costs it as much as the four products), which is what bounded the
        // kernel with a single issuer; the partial sums are added in the epilogue.
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(CT_TM, BN);
            const int me = warp - CT_GATHER_WARPS;
            const uint32_t tm_acc = tmem_base + me * BN;
            for (int it = me; it < nit; it += NI) {
                const int s = it % STAGES;
                ok &= mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort);
                fence_after_sync();
                const uint32_t sa = sbase + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                for (int k4 = 0; k4 < KC / 16; ++k4)
                    umma_bf16(tm_acc, umma_desc_kmajor(sa + k4 * 32, ROWB), umma_desc_kmajor(sb + k4 * 32, ROWB),
                              idesc, it >= NI || k4 > 0);
                umma_commit(empty0 + 8 * s);
            }
            if (nit > me) umma_commit(accfull);
            else if (nit > 0) mbar_arrive_one(accfull);
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == CT_GATHER_WARPS) {
        fence_after_sync();
        tmem_dealloc(tmem_base, TM_COLS);
    }
    if (lane == 0 && (!ok || (tid == 0 && *abort))) atomicOr(a.status, PTV3_STATUS_WAIT_LIMIT);
}

bool conv_tc05_supported(int c_in, int c_out, int kernel_volume)
{
    if (kernel_volume > CT_MAX_KVOL) return false;
    if (c_in == 32 && c_out == 32) return true;
    return c_in % 64 == 0 && c_in <= 4096 && c_out % 64 == 0 && c_out <= 4096;
}

template <int BN, int KC, int STAGES, int NI>
static int launch_conv_tc05_as(const void* weight, const ConvTcArgs& a, cudaStream_t stream)
{
    CUtensorMap mw;
    const uint64_t wcols = (uint64_t)a.kvol * a.cin;
    const int rc = make_tensor_map_bf16(&mw, weight, (uint64_t)a.cout, wcols, wcols * 2, BN, KC);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (CT_TM + BN) * KC * 2 + CT_MAX_KVOL * CT_TM * 4 + CT_TM * 8 + 32 * 4 +
                            BN * 4 + 8 * (2 * STAGES + 1) + 16 + 1024;
    auto kern = conv_tc05_kernel<BN, KC, STAGES, NI>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("ptv3_subm_conv_fwd: shared memory attribute");
    const dim3 grid((unsigned)((a.n + CT_TM - 1) / CT_TM), a.cout / BN);
    launch_dependent(kern, grid, dim3((CT_GATHER_WARPS + NI) * 32), smem, stream, mw, a);
    count_launches(1);
    return check_launch("ptv3_subm_conv_fwd");
}

int launch_conv_tc05(const void* feat, const int32_t* nbr, const void* weight, const void* bias, void* out,
                     const int64_t* row_order, int64_t n, int c_in, int c_out, int kvol, uint32_t* status,
                     cudaStream_t stream)
{
    ConvTcArgs a{};
    a.feat = (const __nv_bfloat16*)feat;
    a.nbr = nbr;
    a.bias = (const __nv_bfloat16*)bias;
    a.out = (__nv_bfloat16*)out;
    a.row_order = row_order;
    a.n = n;
    a.cin = c_in;
    a.cout = c_out;
    a.kvol = kvol;
    a.status = status;
    if (c_in == 32) return launch_conv_tc05_as<32, 32, 6, 2>(weight, a, stream);
    // 128 output channels per CTA halve the gathers of a tile; 64 when that would leave SMs idle
    const int64_t tiles = (n + CT_TM - 1) / CT_TM;
    // long inputs with wide outputs: 256 output channels per CTA (the gathers of a tile once more halved,
    // every product twice as wide), four stages of 48 KiB
    if (c_out % 256 == 0 && tiles * (c_out / 256) >= 148) return launch_conv_tc05_as<256, 64, 4, 2>(weight, a, stream);
    if (c_out % 128 == 0 && tiles * (c_out / 128) >= 120) return launch_conv_tc05_as<128, 64, 6, 2>(weight, a, stream);
    // many tiles: two CTAs per SM, so that one tile's prologue and epilogue run beside another's products
    if (tiles * (c_out / 64) >= 2 * 148) return launch_conv_tc05_as<64, 64, 4, 2>(weight, a, stream);
    return launch_conv_tc05_as<64, 64, 8, 2>(weight, a, stream);
}

}  // namespace ptv3
