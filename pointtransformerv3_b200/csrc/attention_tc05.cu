// Patch attention core on the 5th-generation tensor cores (tcgen05 + tensor memory)
// for bf16 features, head dimension 16 and patches of up to 1024 rows: the shape
// of every stage of the default backbone (model.py:452-484).  Selected with algo 4.
//
// At head dimension 16 a score costs 64 tensor FLOPs and one exponential, so the
// exponential unit bounds the kernel.  With tcgen05 the two matrix products cost
// the CUDA cores nothing (one thread issues one instruction per block instead of an
// ldmatrix + mma.sync stream in every warp), and a thread owns a whole score row
// (tensor-memory lane = query row), so row maxima and the running output need no
// shuffles.
//
// One CTA owns one (patch, head) pair (optionally a slice of its query tiles):
//   gather  K and V of the whole patch, through order[pad[.]], with cp.async into
//           the no-swizzle UMMA operand layout: planes [d chunk][key] of 16-byte
//           chunks, which is K-major for K (B of Q K^T) and MN-major for V (B of P V).
//           V carries a third plane holding a column of ones, so that P V' also
//           yields the row sums of the rounded probabilities.
//   four softmax groups of 128 threads, each walking 128-query tiles on its own, and
//   one issuing warp per group; they talk through mbarriers only:
//     issuer   S[128 x 64] = Q K_j^T                (one tcgen05.mma, K = 16)
//     softmax  tcgen05.ld S -> registers, arrive "S free" (the issuer starts S_j+1),
//              row maximum, exp2, P rounded to bf16 -> tensor memory (tcgen05.st),
//              arrive "P ready"
//     issuer   R|l [128 x 32] = P V'_j              (A from tensor memory, 4 instructions)
//     softmax  O = O * exp2(m_old - m_new) + R on the 16 + 1 registers of the row
//   The groups fill each other's latencies on the exponential unit.  Tensor memory
//   (512 columns: 64 S + 32 P + 32 R per group) is what limits a CTA to four groups.
// Every mbarrier wait is bounded; a wait that runs out sets PTV3_STATUS_WAIT_LIMIT.
//
// Measured on B200 (407 000 points, C = 64, 4 heads): 0.65 ms against 0.57 ms of the
// mma.sync kernel (attention_mma.cu), i.e. 2.6e12 against 2.9e12 exponentials per
// second of the unit's 4.5e12.  Cycle stamps of one thread show why: a key block takes
// a group ~2600 cycles, of which the exponentials are 1100-1300 (512 alone); every
// round trip through an mbarrier (try_wait on a completed phase) or tensor memory
// (tcgen05.ld / st + wait) costs 100-300 cycles, there are seven of them per block, and
// only four groups fit in the 512 columns to hide them.  With the exponentials removed
// altogether the kernel still takes 0.52 ms; moving a third of them to the FMA pipe or
// staggering the groups changes nothing.  A CTA also spends ~15 % of its life in the
// exposed K / V gather, which three co-resident CTAs hide in the mma.sync kernel.  The
// automatic choice therefore stays with the mma.sync kernel.
#include "common.cuh"
#include "attention_mma.cuh"
#include "mma_util.cuh"
#include "tc05.cuh"

namespace ptv3 {

using namespace tc05;

constexpr int AT_WG = 4;                    // softmax groups of 128 threads
constexpr int AT_SOFTMAX_THREADS = 128 * AT_WG;
constexpr int AT_THREADS = AT_SOFTMAX_THREADS + 32 * AT_WG;   // + one issuing warp per group
constexpr int AT_BM = 128;                  // query rows per tile
constexpr int AT_BK = 64;                   // keys per block
constexpr int AT_D = 16;
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr int AT_Q_BYTES = 128 * AT_D * 2;
// tensor-memory columns of a group: S (fp32), P (bf16 pairs), R (16) + l (16)
constexpr int AT_TM_S = 0, AT_TM_P = AT_BK, AT_TM_R = AT_BK + AT_BK / 2, AT_TMEM_GROUP = AT_TM_R + 32;
static_assert(AT_TMEM_GROUP * AT_WG <= 512, "tensor memory holds 512 columns");
// columns a CTA allocates (a power of two); 512 / AT_TMEM_COLS CTAs share an SM
constexpr int AT_TMEM_COLS = AT_TMEM_GROUP * AT_WG <= 256 ? 256 : 512;
constexpr int AT_CTAS_PER_SM = 512 / AT_TMEM_COLS;
// mbarriers of a group
constexpr int AT_BAR_Q = 0, AT_BAR_S = 1, AT_BAR_SFREE = 2, AT_BAR_P = 3, AT_BAR_PV = 4, AT_BARS_PER_WG = 5;
constexpr int AT_NBAR = AT_BARS_PER_WG * AT_WG;

// shared-memory map for a patch padded to lpad keys
struct AtLayout {
    int off_k, off_v, off_q, off_bar, total;
    __host__ __device__ explicit AtLayout(int lpad)
    {
        off_k = 0;                      // 2 planes of lpad 16-byte chunks
        off_v = off_k + lpad * 32;      // 4 planes: V d 0-7, V d 8-15, the ones column, zeros
        off_q = off_v + lpad * 64;
        off_bar = off_q + AT_WG * AT_Q_BYTES;
        total = off_bar + 8 * AT_NBAR + 16;
    }
};

// Descriptor of a no-swizzle operand: `lbo` / `sbo` are the leading / stride byte
// offsets of the canonical layouts (K-major: lbo between the two 8-element halves of
// K = 16, sbo between 8-row groups; MN-major: lbo between 8-deep K groups, sbo
// between 8-element chunks along M/N).
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// D[tmem] (+)= A[tmem] * B[smem]^T: A holds 128 rows (lanes) x 16 bf16 (8 columns of pairs)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             bool accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t at_scale_bf16x2(uint32_t v, float s)
{
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
    return pack_bf16(f.x * s, f.y * s);
}

__device__ __forceinline__ float max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

__global__ void __launch_bounds__(AT_THREADS, AT_CTAS_PER_SM) attn_tc05_d16_kernel(
    const __nv_bfloat16* __restrict__ qkv, const int64_t* __restrict__ order,
    const int64_t* __restrict__ pad, const int64_t* __restrict__ unpad,
    const int32_t* __restrict__ cu_seqlens, __nv_bfloat16* __restrict__ out, int C, float scale,
    int lpad_max, uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    const AtLayout lay(lpad_max);
    const uint32_t sbase = smem_u32_generic(smem);

    // heads and query slices vary fastest over the grid (blockIdx.x = slice * heads + head): the
    // CTAs of one patch run together, so the rows they all gather from (a row holds every head's
    // q, k and v side by side) are fetched from DRAM once
    const int n_heads = C / 16;
    const int seq = blockIdx.y, h = blockIdx.x % n_heads;
    const int slice = blockIdx.x / n_heads, n_slices = gridDim.x / n_heads;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int start = cu_seqlens[seq];
    const int L = cu_seqlens[seq + 1] - start;
    // uniform over the CTA, and before anything is allocated
    if (L <= 0) return;
    if (L > lpad_max) {   // the caller's max_seqlen does not cover this patch
        if (tid == 0) atomicOr(status, PTV3_STATUS_BAD_INDEX);
        return;
    }
    const int ntiles = (L + AT_BM - 1) / AT_BM;      // query tiles
    const int nb = (L + AT_BK - 1) / AT_BK;          // key blocks
    const int Lp = ntiles * AT_BM;                   // rows of the zero-padded K / V planes
    const int tiles_per_slice = (ntiles + n_slices - 1) / n_slices;
    const int tile_lo = slice * tiles_per_slice;
    const int tile_hi = min(ntiles, tile_lo + tiles_per_slice);
    if (tile_lo >= tile_hi) return;
    const int64_t row_stride = 3 * (int64_t)C;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + lay.off_bar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AT_NBAR);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = sbase + lay.off_bar;

    if (tid == 0) {
        for (int g = 0; g < AT_WG; ++g) {
            const uint32_t b = bar0 + 8 * AT_BARS_PER_WG * g;
            mbar_init(b + 8 * AT_BAR_Q, 128);
            mbar_init(b + 8 * AT_BAR_S, 1);
            mbar_init(b + 8 * AT_BAR_SFREE, 128);
            mbar_init(b + 8 * AT_BAR_P, 128);
            mbar_init(b + 8 * AT_BAR_PV, 1);
        }
        *abort = 0;
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(sbase + lay.off_bar + 8 * AT_NBAR, AT_TMEM_COLS);

    // ---- gather K and V of the whole patch into [d half][key] planes ------------
    const uint32_t ks = sbase + lay.off_k, vs = sbase + lay.off_v;
    const uint32_t plane = (uint32_t)Lp * 16;
    const bool issuer = tid >= AT_SOFTMAX_THREADS;
    const int wg = issuer ? warp - AT_SOFTMAX_THREADS / 32 : tid >> 7;
    const int t = tid & 127;

    // ---- gather K and V of the whole patch into [d chunk][key] planes; the chain
    //      pad -> order -> row of every thread's (at most two) key rows and of its first
    //      query row is walked level by level, so the loads of a level overlap --------------
    static_assert(2 * AT_THREADS >= ATTN_TC05_MAX_SEQLEN, "two key rows per thread cover a patch");
    const int r0 = tid, r1 = tid + AT_THREADS;
    const bool g0 = r0 < L, g1 = r1 < L;
    const int rq = (tile_lo + wg) * AT_BM + t;
    const bool gq = !issuer && tile_lo + wg < tile_hi && rq < L;
    // row numbers fit 32 bits (cu_seqlens is 32-bit); kept narrow to spare registers
    const int pd0 = g0 ? (int)pad[start + r0] : 0, pd1 = g1 ? (int)pad[start + r1] : 0;
    const int pdq = gq ? (int)pad[start + rq] : 0;
    const int s0 = g0 ? (int)order[pd0] : 0, s1 = g1 ? (int)order[pd1] : 0;
    const int sq = gq ? (int)order[pdq] : 0;
    uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
    if (gq) {
        const uint4* qp = reinterpret_cast<const uint4*>(qkv + (int64_t)sq * row_stride + h * AT_D);
        q0 = qp[0];
        q1 = qp[1];
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int r = k ? r1 : r0;
        if (r >= Lp) continue;
        // V is extended by a column of ones (and seven of zeros, then a plane of zeros): the
        // product P V' also yields the row sums of the rounded probabilities
        *reinterpret_cast<uint4*>(smem + lay.off_v + 2 * plane + r * 16) = make_uint4(0x3f80u, 0, 0, 0);
        *reinterpret_cast<uint4*>(smem + lay.off_v + 3 * plane + r * 16) = make_uint4(0, 0, 0, 0);
        if (r < L) {
            const __nv_bfloat16* kp = qkv + (int64_t)(k ? s1 : s0) * row_stride + C + h * AT_D;
            cp_async16(ks + r * 16, kp);
            cp_async16(ks + plane + r * 16, kp + 8);
            cp_async16(vs + r * 16, kp + C);
            cp_async16(vs + plane + r * 16, kp + C + 8);
        } else {
            const uint4 z = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(smem + lay.off_k + r * 16) = z;
            *reinterpret_cast<uint4*>(smem + lay.off_k + plane + r * 16) = z;
            *reinterpret_cast<uint4*>(smem + lay.off_v + r * 16) = z;
            *reinterpret_cast<uint4*>(smem + lay.off_v + plane + r * 16) = z;
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t wbar = bar0 + 8 * AT_BARS_PER_WG * wg;
    const uint32_t qbar = wbar + 8 * AT_BAR_Q, sbar = wbar + 8 * AT_BAR_S, sfree = wbar + 8 * AT_BAR_SFREE,
                   pbar = wbar + 8 * AT_BAR_P, pvbar = wbar + 8 * AT_BAR_PV;
    const uint32_t tm_group = tmem_base + wg * AT_TMEM_GROUP;

    // The issuing warps (one whole warpgroup) need few registers; they hand theirs to the
    // softmax warpgroups, which hold a block of scores per thread.  The kernel starts with
    // 96 registers per thread (640 threads); the increase must fit in what the decrease
    // releases, or it would wait for ever: 128 x (96 - 40) = 7168 >= 512 x (104 - 96) = 4096.
    static_assert(AT_THREADS == 640, "the setmaxnreg budget below assumes 640 threads at 96 registers");
    static_assert(AT_WG == 4, "the issuing warps must form one warpgroup for setmaxnreg");
    if (issuer) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        // ---- one warp per group: waits for the group's mbarriers, lane 0 issues ----------
        const bool lead = (tid & 31) == 0;
        constexpr uint32_t IDESC_S = umma_idesc_bf16(128, AT_BK);
        constexpr uint32_t IDESC_R = umma_idesc_bf16(128, 32) | (1u << 16);   // B is MN-major
        // S = Q K_j^T: A = Q planes [d half][row], B = K planes [d half][key]
        const uint64_t desc_q = umma_desc_plain(sbase + lay.off_q + wg * AT_Q_BYTES, AT_BM * 16, 128);
        const uint64_t desc_k = umma_desc_plain(ks, plane, 128);
        // R|l = P V': A = P (tensor memory), B = V' planes [d chunk][key]
        const uint64_t desc_v = umma_desc_plain(vs, 128, plane);
        uint32_t qph = 0, fph = 0, pph = 0;
        for (int tile = tile_lo + wg; tile < tile_hi; tile += AT_WG) {
            mbar_wait(qbar, qph, abort);
            qph ^= 1;
            if (lead) {
                fence_after_sync();
                umma_bf16(tm_group + AT_TM_S, desc_q, desc_k, IDESC_S, false);
                umma_commit(sbar);
            }
            for (int j = 0; j < nb; ++j) {
                mbar_wait(sfree, fph, abort);   // S_j is in the group's registers
                fph ^= 1;
                if (lead && j + 1 < nb) {
                    fence_after_sync();
                    // a descriptor's low word holds the address / 16: blocks are AT_BK chunks apart
                    umma_bf16(tm_group + AT_TM_S, desc_q, desc_k + (uint64_t)((j + 1) * AT_BK), IDESC_S, false);
                    umma_commit(sbar);
                }
                mbar_wait(pbar, pph, abort);    // P_j is in tensor memory, R_j-1 has been read
                pph ^= 1;
                if (lead) {
                    fence_after_sync();
                    const uint64_t dv = desc_v + (uint64_t)(j * AT_BK);
#pragma unroll
                    for (int i = 0; i < AT_BK / 16; ++i)
                        umma_bf16_ts(tm_group + AT_TM_R, tm_group + AT_TM_P + 8 * i, dv + 16 * i, IDESC_R, i > 0);
                    umma_commit(pvbar);
                }
                __syncwarp();
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
        // ---- softmax groups: thread t owns query row t of the tile ---------------------
        unsigned char* qs_ptr = smem + lay.off_q + wg * AT_Q_BYTES;
        const uint32_t tm_lane = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s = tm_group + tm_lane + AT_TM_S, tm_p = tm_group + tm_lane + AT_TM_P,
                       tm_r = tm_group + tm_lane + AT_TM_R;
        uint32_t sph = 0, pvph = 0;

        int pd = pdq, src = sq;                      // of this tile's row
        int pd_next = 0, src_next = 0;               // of the group's next tile, fetched ahead
        for (int tile = tile_lo + wg; tile < tile_hi; tile += AT_WG) {
            const int r = tile * AT_BM + t;
            const bool ok = r < L;
            if (tile != tile_lo + wg) {
                pd = pd_next;
                src = src_next;
                q0 = q1 = make_uint4(0, 0, 0, 0);
                if (ok) {
                    const uint4* qp = reinterpret_cast<const uint4*>(qkv + (int64_t)src * row_stride + h * AT_D);
                    q0 = qp[0];
                    q1 = qp[1];
                }
            }
            // used at the end of the tile only
            const bool own = ok && unpad[pd] == start + r;
            const int rn = r + AT_WG * AT_BM;
            const bool okn = tile + AT_WG < tile_hi && rn < L;
            if (okn) pd_next = (int)pad[start + rn];
            if (ok) {
                q0.x = at_scale_bf16x2(q0.x, scale); q0.y = at_scale_bf16x2(q0.y, scale);
                q0.z = at_scale_bf16x2(q0.z, scale); q0.w = at_scale_bf16x2(q0.w, scale);
                q1.x = at_scale_bf16x2(q1.x, scale); q1.y = at_scale_bf16x2(q1.y, scale);
                q1.z = at_scale_bf16x2(q1.z, scale); q1.w = at_scale_bf16x2(q1.w, scale);
            }
            // every product that read the previous tile's Q has completed (its R was awaited)
            *reinterpret_cast<uint4*>(qs_ptr + t * 16) = q0;
            *reinterpret_cast<uint4*>(qs_ptr + 2048 + t * 16) = q1;
            fence_proxy_async();
            mbar_arrive(qbar);

            float m = -INFINITY, alpha_prev = 1.f, lsum = 0.f;
            float o[AT_D];
#pragma unroll
            for (int i = 0; i < AT_D; ++i) o[i] = 0.f;

            for (int j = 0; j < nb; ++j) {
                mbar_wait(sbar, sph, abort);
                sph ^= 1;
                fence_after_sync();
                float v[AT_BK];
                {
                    uint32_t (&u)[AT_BK] = reinterpret_cast<uint32_t (&)[AT_BK]>(v);
#pragma unroll
                    for (int c = 0; c < AT_BK / 32; ++c)
                        tmem_ld32(tm_s + 32 * c, reinterpret_cast<uint32_t (&)[32]>(u[32 * c]));
                    tmem_ld_wait();
                }
                // the scores are in registers: the next block's product may overwrite them
                fence_before_sync();
                mbar_arrive(sfree);
                const int valid = L - j * AT_BK;
                if (valid < AT_BK) {
#pragma unroll
                    for (int i = 0; i < AT_BK; ++i)
                        if (i >= valid) v[i] = -INFINITY;
                }
                float mx0 = v[0], mx1 = v[1], mx2 = v[2], mx3 = v[3];
#pragma unroll
                for (int i = 4; i < AT_BK; i += 8) {
                    mx0 = max3(mx0, v[i], v[i + 1]);
                    mx1 = max3(mx1, v[i + 2], v[i + 3]);
                    if (i + 4 < AT_BK) {
                        mx2 = max3(mx2, v[i + 4], v[i + 5]);
                        mx3 = max3(mx3, v[i + 6], v[i + 7]);
                    }
                }
                // every block holds at least one real key, so the new maximum is finite
                const float mn = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m);
                const float alpha = fast_exp2((m - mn) * AT_LOG2E);
                m = mn;
                const float mb = m * AT_LOG2E;
                uint32_t pk[AT_BK / 2];
#pragma unroll
                for (int i = 0; i < AT_BK / 2; ++i)
                    pk[i] = pack_bf16(fast_exp2(fmaf(v[2 * i], AT_LOG2E, -mb)),
                                      fast_exp2(fmaf(v[2 * i + 1], AT_LOG2E, -mb)));
                if (j > 0) {
                    // the previous block's P V has finished: its result can be read and the
                    // probability columns rewritten
                    mbar_wait(pvbar, pvph, abort);
                    pvph ^= 1;
                    fence_after_sync();
                    uint32_t rr[32];
                    tmem_ld32(tm_r, rr);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < AT_D; ++i) o[i] = fmaf(o[i], alpha_prev, __uint_as_float(rr[i]));
                    lsum = fmaf(lsum, alpha_prev, __uint_as_float(rr[16]));
                }
                alpha_prev = alpha;
#pragma unroll
                for (int c = 0; c < AT_BK / 64; ++c)
                    tmem_st32(tm_p + 32 * c, reinterpret_cast<const uint32_t (&)[32]>(pk[32 * c]));
                tmem_st_wait();
                fence_before_sync();
                mbar_arrive(pbar);
                // walk the next tile's pad -> order -> row chain one level per key block
                if (j == 0 && okn) src_next = (int)order[pd_next];
                if (j == 1 && okn)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(qkv + (int64_t)src_next * row_stride + h * AT_D));
            }
            mbar_wait(pvbar, pvph, abort);
            pvph ^= 1;
            fence_after_sync();
            {
                uint32_t rr[32];
                tmem_ld32(tm_r, rr);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < AT_D; ++i) o[i] = fmaf(o[i], alpha_prev, __uint_as_float(rr[i]));
                lsum = fmaf(lsum, alpha_prev, __uint_as_float(rr[16]));
            }
            if (ok && own) {
                const float inv = 1.f / lsum;
                uint4 w0, w1;
                w0.x = pack_bf16(o[0] * inv, o[1] * inv);   w0.y = pack_bf16(o[2] * inv, o[3] * inv);
                w0.z = pack_bf16(o[4] * inv, o[5] * inv);   w0.w = pack_bf16(o[6] * inv, o[7] * inv);
                w1.x = pack_bf16(o[8] * inv, o[9] * inv);   w1.y = pack_bf16(o[10] * inv, o[11] * inv);
                w1.z = pack_bf16(o[12] * inv, o[13] * inv); w1.w = pack_bf16(o[14] * inv, o[15] * inv);
                uint4* op = reinterpret_cast<uint4*>(out + (int64_t)src * C + h * AT_D);
                op[0] = w0;
                op[1] = w1;
            }
        }
    }

    fence_before_sync();
    __syncthreads();
    if (tid == 0 && *abort) atomicOr(status, PTV3_STATUS_WAIT_LIMIT);
    if (warp == 0) {
        fence_after_sync();
        tmem_dealloc(tmem_base, AT_TMEM_COLS);
    }
}

bool attn_tc05_supported(int channels, int heads, int max_seqlen)
{
    return channels % heads == 0 && channels / heads == AT_D && channels % 16 == 0 &&
           max_seqlen <= ATTN_TC05_MAX_SEQLEN;
}

int launch_attn_tc05(const void* qkv, const int64_t* order, const int64_t* pad, const int64_t* unpad,
                     const int32_t* cu, void* out, int n_seq, int max_seqlen, int C, int H, float scale,
                     uint32_t* status, cudaStream_t stream)
{
    const int lpad = (max_seqlen + AT_BM - 1) / AT_BM * AT_BM;
    const AtLayout lay(lpad);
    // Each CTA takes 1 / AT_CTAS_PER_SM of tensor memory: ask for enough shared memory that no
    // more than that many CTAs share an SM (one more would wait in tcgen05.alloc).
    const size_t floor_smem = (size_t)(228 * 1024 / (AT_CTAS_PER_SM + 1) + 1024);
    const size_t smem = lay.total + 128 < floor_smem ? floor_smem : (size_t)lay.total + 128;
    if (cudaFuncSetAttribute(attn_tc05_d16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
        return check_launch("ptv3_attention_fwd: shared memory attribute");
    // Query tiles of a patch can be sliced over CTAs (each gathers K and V again).  Pick the
    // slicing with the shortest estimated time: waves of 148 CTAs, each taking one gather
    // (about 0.3 of a tile pair) plus its tile pairs.
    const int tiles = lpad / AT_BM;
    const long pairs = (long)n_seq * H;
    int qsplit = 1;
    double best = 0;
    for (int q = 1; q <= tiles; q *= 2) {
        const long waves = (pairs * q + 147) / 148;
        const int tile_pairs = ((tiles + q - 1) / q + AT_WG - 1) / AT_WG;
        const double cost = (double)waves * (tile_pairs + 0.3);
        if (q == 1 || cost < best) {
            best = cost;
            qsplit = q;
        }
    }
    const dim3 grid(H * qsplit, n_seq);
    attn_tc05_d16_kernel<<<grid, AT_THREADS, smem, stream>>>(
        (const __nv_bfloat16*)qkv, order, pad, unpad, cu, (__nv_bfloat16*)out, C, scale, lpad, status);
    count_launches(1);
    return check_launch("ptv3_attention_fwd");
}

}  // namespace ptv3
