// Patch attention core on the 5th-generation tensor cores (tcgen05 + tensor memory)
// for bf16 features, head dimension 16 and patches of up to 1024 rows: the shape
// of every stage of the default backbone (model.py:452-484).
//
// At head dimension 16 a score costs 64 tensor FLOPs and one exponential, so the
// exponential unit bounds the kernel, not the tensor pipe.  With tcgen05 the two
// matrix products cost the CUDA cores nothing (one thread issues one instruction
// per block instead of an ldmatrix + mma.sync stream in every warp), and a thread
// owns a whole score row (tensor-memory lane = query row), so row maxima need no
// shuffles.  What is left per score on the CUDA cores is half a max, half a packed
// multiply-add, the exponential and half a conversion.
//
// One CTA owns one (patch, head) pair (optionally a slice of its query tiles).
//   gather   K and V of the whole patch, through order[pad[.]], with cp.async into
//            the no-swizzle UMMA operand layout: planes [d chunk][key] of 16-byte
//            chunks, which is K-major for K (B of Q K^T) and MN-major for V (B of P V).
//            V carries a third plane holding a column of ones, so that P V' also
//            yields the row sums of the rounded probabilities.  The gather is issued
//            by the four issuing warps in blocks of 128 keys, each with its own
//            mbarrier, so the first products start when the first block has landed.
//   four softmax groups of 128 threads, each walking 128-query tiles on its own, and
//   one issuing warp per group; they talk through mbarriers only.  Per 48-key block:
//     issuer   S[128 x 48] = Q K_j^T into one of two score buffers (one tcgen05.mma, K = 16),
//              always one block ahead of the group
//     softmax  tcgen05.ld S -> registers, block maximum, P = exp2(S - m) rounded to bf16
//              and written over the first half of that S (tcgen05.st), arrive "P ready"
//     issuer   O|l [128 x 32] += P V'_j  (A from tensor memory, accumulating over all key
//              blocks), then S_j+2 into the buffer P_j occupied
//   and at the end of a tile the group reads O|l once, divides and writes its rows.
//   With two score buffers the next S is ready when a group has finished a block, so the
//   groups never wait in step and the exponential unit always has a group to serve.
//   The output stays in tensor memory for the whole tile.  The reference value m of the
//   exponentials is raised lazily (only when a score exceeds it by 2^8); in that rare case
//   the group waits for the product before it and rescales O|l in place.
//   A share of the exponentials (AT_POLY of every 8 pairs) is evaluated on the FMA pipe
//   (range reduction + cubic), the rest on the exponential unit: with the products off
//   the CUDA cores there are issue slots to spare, and the exponential unit is the
//   bottleneck otherwise.
// Tensor memory: 128 columns per group (S_0 in 0..47, S_1 in 48..95, each P over the first 24
// columns of its S; O|l in 96..127).
// Every mbarrier wait is bounded; a wait that runs out sets PTV3_STATUS_WAIT_LIMIT.
//
// Measured on B200 (240 000 points, C = 64, 4 heads): 0.41 ms against 0.31 ms of the mma.sync
// kernel (attention_mma.cu), which therefore stays the automatic choice.  Cycle stamps of one
// group against its issuer show what bounds this kernel: a key block takes a group ~2400
// cycles whatever the softmax does (all exponentials on the exponential unit, three of eight
// on the FMA pipe, or none at all), and the next S is seen one block period after the product
// that makes it was issued.  The period is the asynchronous tensor path working through the
// 16 products of a round of the four groups (3 x P V' + 1 x Q K^T each): at head dimension 16
// every product is tiny (128 x 32 x 16 or 128 x 48 x 16), K is 16 per instruction by the
// instruction set, so a (patch, head) pair needs ~690 of them at ~150 cycles each, whatever
// their size.  The arithmetic is not what takes the time: the profiler shows the tensor pipe
// 12 % active, the exponential unit 41 % and instruction issue 65 %; the time goes to the
// latency of each product through that path (issue, operand fetch from shared and tensor
// memory, commit), which at this size is not hidden by the next product.  The mma.sync kernel
// pays for its products with issue slots of the CUDA cores instead, which it has.
// Earlier forms of this kernel (scores read back every block with the output in registers;
// two passes with the exact maximum first; one score buffer) all ran at 0.42-0.49 ms for
// the same reason.
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
constexpr int AT_BK = 48;                   // keys per block (two score buffers of 48 columns)
constexpr int AT_POLY = 3;                  // of every 8 pairs of exponentials, this many on the FMA pipe
constexpr float AT_LAZY = 8.f;              // slack of the reference value, in powers of two
constexpr int AT_D = 16;
constexpr int AT_KV_BLOCK = 128;            // keys per gather block (one mbarrier each)
constexpr int AT_KV_BLOCKS = ATTN_TC05_MAX_SEQLEN / AT_KV_BLOCK;
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr int AT_Q_BYTES = 128 * AT_D * 2;
// tensor-memory columns of a group: two score buffers (P re-uses the first half of its S), O|l
constexpr int AT_TM_S = 0, AT_TM_O = 2 * AT_BK, AT_TMEM_GROUP = 128;
static_assert(AT_TM_O + 32 <= AT_TMEM_GROUP, "two score buffers and the output fit a group's columns");
constexpr int AT_PAD_ROWS = AT_BK;          // zero rows behind the last 128-row block (key blocks of 48)
constexpr int AT_TMEM_COLS = AT_TMEM_GROUP * AT_WG;
static_assert(AT_TMEM_COLS == 512, "the CTA takes the whole tensor memory of its SM");
// mbarriers of a group
constexpr int AT_BAR_Q = 0, AT_BAR_S = 1 /* two */, AT_BAR_P = 3, AT_BAR_PV = 4, AT_BARS_PER_WG = 5;
constexpr int AT_NBAR = AT_BARS_PER_WG * AT_WG + AT_KV_BLOCKS;

// shared-memory map for a patch padded to lpad keys
struct AtLayout {
    int off_k, off_v, off_q, off_bar, total;
    __host__ __device__ explicit AtLayout(int lpad)
    {
        const int rows = lpad + AT_PAD_ROWS;
        off_k = 0;                      // 2 planes of 16-byte chunks
        off_v = off_k + rows * 32;      // 4 planes: V d 0-7, V d 8-15, the ones column, zeros
        off_q = off_v + rows * 64;
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

// waits until this thread's cp.async groups, except the newest `pending`, have landed
__device__ __forceinline__ void cp_async_wait_pending(int pending)
{
    switch (pending) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        case 6: cp_async_wait<6>(); break;
        default: cp_async_wait<7>(); break;
    }
}

__global__ void __launch_bounds__(AT_THREADS, 1) attn_tc05_d16_kernel(
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
    const int nkv = ntiles;                          // gather blocks (128 keys, zero padded)
    const int nb = (L + AT_BK - 1) / AT_BK;          // key blocks of pass 2
    const int Lp = ntiles * AT_BM;                   // rows covered by the gather blocks
    const int Lk = max(Lp, nb * AT_BK);              // rows of the zero-padded K / V planes
    const int tiles_per_slice = (ntiles + n_slices - 1) / n_slices;
    const int tile_lo = slice * tiles_per_slice;
    const int tile_hi = min(ntiles, tile_lo + tiles_per_slice);
    if (tile_lo >= tile_hi) return;
    const int64_t row_stride = 3 * (int64_t)C;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + lay.off_bar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AT_NBAR);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = sbase + lay.off_bar;
    const uint32_t kvbar0 = bar0 + 8 * AT_BARS_PER_WG * AT_WG;

    if (tid == 0) {
        for (int g = 0; g < AT_WG; ++g) {
            const uint32_t b = bar0 + 8 * AT_BARS_PER_WG * g;
            mbar_init(b + 8 * AT_BAR_Q, 4);      // one arrival per warp of the group
            mbar_init(b + 8 * AT_BAR_S, 1);
            mbar_init(b + 8 * (AT_BAR_S + 1), 1);
            mbar_init(b + 8 * AT_BAR_PV, 1);
            mbar_init(b + 8 * AT_BAR_P, 4);
        }
        for (int b = 0; b < AT_KV_BLOCKS; ++b) mbar_init(kvbar0 + 8 * b, 32 * AT_WG);
        *abort = 0;
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(sbase + lay.off_bar + 8 * AT_NBAR, AT_TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t ks = sbase + lay.off_k, vs = sbase + lay.off_v;
    const uint32_t plane = (uint32_t)Lk * 16;
    const bool issuer = tid >= AT_SOFTMAX_THREADS;
    const int wg = issuer ? warp - AT_SOFTMAX_THREADS / 32 : tid >> 7;
    const int t = tid & 127;

    const uint32_t wbar = bar0 + 8 * AT_BARS_PER_WG * wg;
    const uint32_t qbar = wbar + 8 * AT_BAR_Q, sbar = wbar + 8 * AT_BAR_S, pbar = wbar + 8 * AT_BAR_P,
                   pvbar = wbar + 8 * AT_BAR_PV;
    const uint32_t tm_group = tmem_base + wg * AT_TMEM_GROUP;

    // The issuing warps (one whole warpgroup) need few registers; they hand theirs to the
    // softmax warpgroups.  The kernel starts with 96 registers per thread (640 threads); the
    // increase must fit in what the decrease releases, or it would wait for ever:
    // 128 x (96 - 64) = 4096 >= 512 x (104 - 96) = 4096.
    static_assert(AT_THREADS == 640, "the setmaxnreg budget below assumes 640 threads at 96 registers");
    static_assert(AT_WG == 4, "the issuing warps must form one warpgroup for setmaxnreg");
    if (issuer) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        // ---- gather: the 128 issuer threads own one key row of every 128-key block -----------
        const int a = tid - AT_SOFTMAX_THREADS;     // 0..127
        {
            int src[AT_KV_BLOCKS];
#pragma unroll
            for (int b = 0; b < AT_KV_BLOCKS; ++b) {
                const int r = b * AT_KV_BLOCK + a;
                src[b] = (b < nkv && r < L) ? (int)pad[start + r] : -1;
            }
#pragma unroll
            for (int b = 0; b < AT_KV_BLOCKS; ++b)
                if (src[b] >= 0) src[b] = (int)order[src[b]];
#pragma unroll
            for (int b = 0; b < AT_KV_BLOCKS; ++b) {
                if (b < nkv) {
                    const int r = b * AT_KV_BLOCK + a;
                    // V is extended by a column of ones (and seven of zeros, then a plane of zeros):
                    // the product P V' also yields the row sums of the rounded probabilities
                    *reinterpret_cast<uint4*>(smem + lay.off_v + 2 * plane + r * 16) = make_uint4(0x3f80u, 0, 0, 0);
                    *reinterpret_cast<uint4*>(smem + lay.off_v + 3 * plane + r * 16) = make_uint4(0, 0, 0, 0);
                    if (src[b] >= 0) {
                        const __nv_bfloat16* kp = qkv + (int64_t)src[b] * row_stride + C + h * AT_D;
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
                cp_async_commit();      // one group per block, empty ones included
            }
            // key blocks are 48 rows: the last one may reach behind the last gather block
            if (Lp + a < Lk) {
                const int r = Lp + a;
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int pl = 0; pl < 2; ++pl) *reinterpret_cast<uint4*>(smem + lay.off_k + pl * plane + r * 16) = z;
#pragma unroll
                for (int pl = 0; pl < 4; ++pl) *reinterpret_cast<uint4*>(smem + lay.off_v + pl * plane + r * 16) = z;
            }
        }
        // ---- one warp per group: waits for the group's mbarriers, lane 0 issues ----------
        const bool lead = (tid & 31) == 0;
        constexpr uint32_t IDESC_S = umma_idesc_bf16(128, AT_BK);
        constexpr uint32_t IDESC_R = umma_idesc_bf16(128, 32) | (1u << 16);   // B is MN-major
        // S = Q K_j^T: A = Q planes [d half][row], B = K planes [d half][key]
        const uint64_t desc_q = umma_desc_plain(sbase + lay.off_q + wg * AT_Q_BYTES, AT_BM * 16, 128);
        const uint64_t desc_k = umma_desc_plain(ks, plane, 128);
        // O|l += P V': A = P (tensor memory), B = V' planes [d chunk][key]
        const uint64_t desc_v = umma_desc_plain(vs, 128, plane);
        uint32_t qph = 0, pph = 0;
        int landed = 0;      // gather blocks handed over so far
        // this thread's copies of the gather blocks up to the one holding key row `row` have
        // landed: tell the tensor-core proxy and the other issuing warps, then wait for theirs
        auto land_upto = [&](int row) {
            const int need = min(row / AT_KV_BLOCK, nkv - 1);
            while (landed <= need) {
                cp_async_wait_pending(AT_KV_BLOCKS - 1 - landed);
                fence_proxy_async();
                mbar_arrive(kvbar0 + 8 * landed);
                mbar_wait(kvbar0 + 8 * landed, 0, abort);
                ++landed;
            }
        };
        auto issue_s = [&](int jj) {      // S_jj = Q K_jj^T into buffer jj & 1
            // a descriptor's low word holds the address / 16: blocks are AT_BK chunks apart
            umma_bf16(tm_group + AT_TM_S + (jj & 1) * AT_BK, desc_q, desc_k + (uint64_t)(jj * AT_BK), IDESC_S, false);
            umma_commit(sbar + 8 * (jj & 1));
        };
        for (int tile = tile_lo + wg; tile < tile_hi; tile += AT_WG) {
            mbar_wait(qbar, qph, abort);
            qph ^= 1;
            land_upto(min(2, nb) * AT_BK - 1);
            if (lead) {
                fence_after_sync();
                issue_s(0);
                if (nb > 1) issue_s(1);
            }
            __syncwarp();
            for (int j = 0; j < nb; ++j) {
                mbar_wait(pbar, pph, abort);    // P_j is in tensor memory (over the first half of S_j)
                pph ^= 1;
                if (j + 2 < nb) land_upto((j + 3) * AT_BK - 1);
                if (lead) {
                    fence_after_sync();
                    const uint64_t dv = desc_v + (uint64_t)(j * AT_BK);
                    const uint32_t tm_p = tm_group + AT_TM_S + (j & 1) * AT_BK;
#pragma unroll
                    for (int i = 0; i < AT_BK / 16; ++i)
                        umma_bf16_ts(tm_group + AT_TM_O, tm_p + 8 * i, dv + 16 * i, IDESC_R, j > 0 || i > 0);
                    umma_commit(pvbar);
                    // the next product into this buffer runs after the ones above, which read it
                    if (j + 2 < nb) issue_s(j + 2);
                }
                __syncwarp();
            }
        }
        const bool kv_landed = landed >= nkv;
        if (!kv_landed) {
            // a warp whose group has no tile in this CTA (or a patch shorter than its planes): its
            // share of the gather still has to be handed over, the other issuing warps wait for it
            for (int jb = landed; jb < nkv; ++jb) {
                cp_async_wait_pending(AT_KV_BLOCKS - 1 - jb);
                fence_proxy_async();
                mbar_arrive(kvbar0 + 8 * jb);
            }
        }
        cp_async_wait<0>();
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
        // ---- softmax groups: thread t owns query row t of the tile ---------------------
        unsigned char* qs_ptr = smem + lay.off_q + wg * AT_Q_BYTES;
        const uint32_t tm_lane = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s0 = tm_group + tm_lane + AT_TM_S, tm_o = tm_group + tm_lane + AT_TM_O;
        uint32_t sph0 = 0, sph1 = 0, pvph = 0;
        const Exp2Const kexp;

        // pad -> order -> q row of this thread's row in the group's NEXT tile is walked one level
        // per key block while the current tile is computed
        int pd = 0, src = 0, pd_next = 0, src_next = 0;
        {
            const int r = (tile_lo + wg) * AT_BM + t;
            if (tile_lo + wg < tile_hi && r < L) {
                pd = (int)pad[start + r];
                src = (int)order[pd];
            }
        }
        for (int tile = tile_lo + wg; tile < tile_hi; tile += AT_WG) {
            const int r = tile * AT_BM + t;
            const bool ok = r < L;
            if (tile != tile_lo + wg) {
                pd = pd_next;
                src = src_next;
            }
            uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
            if (ok) {
                const uint4* qp = reinterpret_cast<const uint4*>(qkv + (int64_t)src * row_stride + h * AT_D);
                q0 = qp[0];
                q1 = qp[1];
                q0.x = at_scale_bf16x2(q0.x, scale); q0.y = at_scale_bf16x2(q0.y, scale);
                q0.z = at_scale_bf16x2(q0.z, scale); q0.w = at_scale_bf16x2(q0.w, scale);
                q1.x = at_scale_bf16x2(q1.x, scale); q1.y = at_scale_bf16x2(q1.y, scale);
                q1.z = at_scale_bf16x2(q1.z, scale); q1.w = at_scale_bf16x2(q1.w, scale);
            }
            // used at the end of the tile only
            const bool own = ok && unpad[pd] == start + r;
            const int rn = r + AT_WG * AT_BM;
            const bool okn = tile + AT_WG < tile_hi && rn < L;
            if (okn) pd_next = (int)pad[start + rn];
            // every product that read the previous tile's Q has completed (its O was awaited)
            *reinterpret_cast<uint4*>(qs_ptr + t * 16) = q0;
            *reinterpret_cast<uint4*>(qs_ptr + 2048 + t * 16) = q1;
            fence_proxy_async();
            // one arrival per warp: 128 arrivals on one mbarrier are 128 updates of one shared-memory
            // word, one after the other
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(qbar);

            float m = -INFINITY;     // reference value of the exponentials (raw score units)
            float mb = 0.f;          // -m * log2(e)
            for (int j = 0; j < nb; ++j) {
                const int buf = j & 1;
                const uint32_t tm_s = tm_s0 + buf * AT_BK;
                if (buf) {
                    mbar_wait(sbar + 8, sph1, abort);
                    sph1 ^= 1;
                } else {
                    mbar_wait(sbar, sph0, abort);
                    sph0 ^= 1;
                }
                fence_after_sync();
                float v[AT_BK];
                {
                    uint32_t* u = reinterpret_cast<uint32_t*>(v);
#pragma unroll
                    for (int c = 0; c < AT_BK / 16; ++c) tmem_ld16(tm_s + 16 * c, u + 16 * c);
                    tmem_ld_wait();
                }
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
                // every block holds at least one real key, so the block maximum is finite
                const float bm = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                const bool raise = (bm - m) * AT_LOG2E > AT_LAZY;     // always on the first block
                // tensor-memory loads and stores are warp-wide: the rare rescaling is taken by the
                // whole warp, with factor 1 for the rows that keep their reference value
                bool pv_awaited = j == 0;
                if (__any_sync(0xffffffffu, raise)) {
                    const float mn = raise ? bm : m;
                    if (j > 0) {
                        // the product P_j-1 V' may still be running
                        mbar_wait(pvbar, pvph, abort);
                        pvph ^= 1;
                        pv_awaited = true;
                        fence_after_sync();
                        const float alpha = raise ? fast_exp2((m - mn) * AT_LOG2E) : 1.f;
                        uint32_t rr[32];
                        tmem_ld32(tm_o, rr);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i <= AT_D; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
                        tmem_st32(tm_o, rr);
                    }
                    m = mn;
                    mb = -m * AT_LOG2E;
                }
                uint32_t pk[AT_BK / 2];
                const uint64_t mb2 = pack2(mb, mb);
#pragma unroll
                for (int i = 0; i < AT_BK / 2; ++i) {
                    const uint64_t x2 = fma2(pack2(v[2 * i], v[2 * i + 1]), kexp.log2e, mb2);
                    if ((i & 7) < AT_POLY) {
                        pk[i] = exp2_poly2_bf16(x2, kexp);
                    } else {
                        float x, y;
                        unpack2(x2, x, y);
                        pk[i] = pack_bf16(fast_exp2(x), fast_exp2(y));
                    }
                }
                // every block consumes one completion of the "P V done" barrier (of the block before
                // it), here in the common case, where that product has long finished
                if (!pv_awaited) {
                    mbar_wait(pvbar, pvph, abort);
                    pvph ^= 1;
                }
                // P over the first half of S_j (all of S_j is in registers)
#pragma unroll
                for (int c = 0; c < AT_BK / 16; ++c) tmem_st8(tm_s + 8 * c, pk + 8 * c);
                tmem_st_wait();
                fence_before_sync();
                __syncwarp();
                if ((tid & 31) == 0) mbar_arrive(pbar);
                // walk the next tile's pad -> order -> row chain one level per key block
                if (j == 0 && okn) src_next = (int)order[pd_next];
                if (j == 1 && okn)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(qkv + (int64_t)src_next * row_stride + h * AT_D));
            }
            mbar_wait(pvbar, pvph, abort);      // the last product of the tile
            pvph ^= 1;
            fence_after_sync();
            {
                uint32_t rr[32];
                tmem_ld32(tm_o, rr);
                tmem_ld_wait();
                // the next tile's first product overwrites these columns; it is issued only after
                // this thread's arrival on the Q barrier, which comes after this load
                fence_before_sync();
                if (own) {
                    const float inv = 1.f / __uint_as_float(rr[16]);
                    uint4 w0, w1;
#define AT_O(i) (__uint_as_float(rr[i]) * inv)
                    w0.x = pack_bf16(AT_O(0), AT_O(1));   w0.y = pack_bf16(AT_O(2), AT_O(3));
                    w0.z = pack_bf16(AT_O(4), AT_O(5));   w0.w = pack_bf16(AT_O(6), AT_O(7));
                    w1.x = pack_bf16(AT_O(8), AT_O(9));   w1.y = pack_bf16(AT_O(10), AT_O(11));
                    w1.z = pack_bf16(AT_O(12), AT_O(13)); w1.w = pack_bf16(AT_O(14), AT_O(15));
#undef AT_O
                    uint4* op = reinterpret_cast<uint4*>(out + (int64_t)src * C + h * AT_D);
                    op[0] = w0;
                    op[1] = w1;
                }
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
    // A CTA takes the whole tensor memory of its SM: ask for enough shared memory that no
    // second CTA shares the SM (it would wait in tcgen05.alloc).
    const size_t floor_smem = (size_t)(228 * 1024 / 2 + 1024);
    const size_t smem = lay.total + 128 < floor_smem ? floor_smem : (size_t)lay.total + 128;
    if (cudaFuncSetAttribute(attn_tc05_d16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
        return check_launch("ptv3_attention_fwd: shared memory attribute");
    // Query tiles of a patch can be sliced over CTAs (each gathers K and V again).  Pick the
    // slicing with the shortest estimated time: waves of 148 CTAs, each taking one gather
    // (about 0.2 of a tile round) plus its rounds of up to four tiles.
    const int tiles = lpad / AT_BM;
    const long pairs = (long)n_seq * H;
    int qsplit = 1;
    double best = 0;
    for (int q = 1; q <= tiles; q *= 2) {
        const long waves = (pairs * q + 147) / 148;
        const int rounds = ((tiles + q - 1) / q + AT_WG - 1) / AT_WG;
        const double cost = (double)waves * (rounds + 0.2);
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

