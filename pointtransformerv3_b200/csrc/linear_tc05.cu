// Linear layers of a block on the 5th-generation tensor cores, with the row-wise
// glue that follows them fused into the epilogue:
//
//   plain      out = x W^T + b                                  (qkv, model.py:456)
//   residual   y   = x W^T + b
//              t   = ln1 ? LayerNorm(y; ln1) : y
//              s   = residual + t                   -> sum_out
//              out = LayerNorm(s; ln2)              -> norm_out
//     which is  cpe.1 + cpe.2 + shortcut + norm1     (model.py:553-554, 589-592)
//     and       attn.proj + shortcut + norm2         (model.py:487, 594, 598-600)
//
// bf16, input width K in {32, 64, 128}.  A persistent CTA keeps W in shared memory
// (TMA, once) and runs up to four independent 128-thread groups; a group loads a
// 128-row x tile by TMA, issues K/16 tcgen05.mma into its slice of tensor memory and
// owns one accumulator row per thread, so LayerNorm statistics are thread-local
// (no shuffles).  The residual sum is parked in tensor memory (tcgen05.st) between the
// pass that forms it and the pass that normalises it.  Every intermediate the unfused
// sequence would round to bf16 is rounded at the same place.  Waits are bounded.
#include "common.cuh"
#include "mma_util.cuh"
#include "tc05.cuh"
#include "vec.cuh"

namespace ptv3 {

using namespace tc05;

struct LinearArgs {
    const __nv_bfloat16* bias;       // n_out or NULL
    __nv_bfloat16* out;              // plain mode: n x n_out
    const __nv_bfloat16* residual;   // residual mode: n x n_out
    const __nv_bfloat16* ln1_w;      // optional
    const __nv_bfloat16* ln1_b;
    const __nv_bfloat16* ln2_w;      // required in residual mode
    const __nv_bfloat16* ln2_b;
    __nv_bfloat16* sum_out;
    __nv_bfloat16* norm_out;
    float eps1, eps2;
    int64_t n;
    int n_out;
    int groups;       // 128-thread groups that work (1..4)
    int nacc;         // accumulators per group in tensor memory (2 where 2 x groups x columns fit in 512)
    int w_box_rows;   // rows per TMA box of W
    int residual_mode;
    int out_box;      // plain mode: columns per staging tile and TMA store (64, or 32 when n_out % 64 != 0)
    uint32_t* status;
};

__device__ __forceinline__ float lin_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Staging tile of a group: 128 rows x 64 bf16 columns, rows 144 bytes apart, so that
// both the row-per-thread accesses of the epilogue and the coalesced copies to and
// from global memory (consecutive threads on consecutive 16-byte pieces) are free of
// bank conflicts.  Global rows are `pitch` elements wide; `col0` is the slab's column.
constexpr int LIN_STAGE_ROW = 144;
constexpr int LIN_STAGE_BYTES = 128 * LIN_STAGE_ROW;

// A warp copies the 32 rows its own threads filled (t = thread of the group; rows (t / 32) * 32 ...), so
// that only the warp has to be in step, not the group.
__device__ __forceinline__ void stage_to_global(const unsigned char* stage, __nv_bfloat16* dst, int64_t row0,
                                                int64_t n, int pitch, int col0, int t)
{
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 3), c = idx & 7;
        if (row0 + r < n)
            *reinterpret_cast<uint4*>(dst + (row0 + r) * pitch + col0 + c * 8) =
                *reinterpret_cast<const uint4*>(stage + r * LIN_STAGE_ROW + c * 16);
    }
}

__device__ __forceinline__ void global_to_stage(unsigned char* stage, const __nv_bfloat16* src, int64_t row0,
                                                int64_t n, int pitch, int col0, int t)
{
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 3), c = idx & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row0 + r < n) v = *reinterpret_cast<const uint4*>(src + (row0 + r) * pitch + col0 + c * 8);
        *reinterpret_cast<uint4*>(stage + r * LIN_STAGE_ROW + c * 16) = v;
    }
}

template <int K>
__global__ void __launch_bounds__(512, 1) linear_tc05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_o,
                                                             const LinearArgs a)
{
    pdl_launch_next();
    constexpr int SW = K >= 64 ? 128 : 64;       // bytes per shared-memory row (swizzle span)
    constexpr int KB = K >= 64 ? K / 64 : 1;     // 64-wide K blocks
    constexpr int KCOLS = K >= 64 ? 64 : K;      // columns per K block
    constexpr int X_BLOCK = 128 * SW;            // one K block of an x tile
    constexpr int X_BYTES = KB * X_BLOCK;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32_generic(smem);
    const int n_out = a.n_out;
    const int w_block = n_out * SW;              // one K block of W
    const int off_x = KB * w_block;              // x tiles of the groups
    const int off_stage = off_x + 2 * a.groups * X_BYTES;   // (x tiles are double buffered) one staging tile per group
    const int off_par = off_stage + a.groups * LIN_STAGE_BYTES;   // bias, ln1 w/b, ln2 w/b as floats (5 x n_out)
    const int off_bar = off_par + 5 * n_out * 4;
    float* par = reinterpret_cast<float*>(smem + off_par);
    float *bias_s = par, *g1 = par + n_out, *b1 = par + 2 * n_out, *g2 = par + 3 * n_out, *b2 = par + 4 * n_out;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int g = tid >> 7, t = tid & 127;
    const uint32_t wbar = sbase + off_bar;
    // xbar0 + 8: second x buffer; mbar0 + 8: second accumulator
    const uint32_t xbar0 = wbar + 8 * (1 + 2 * g), mbar0 = wbar + 8 * (9 + 2 * g);

    if (tid == 0) {
        for (int i = 0; i < 17; ++i) mbar_init(wbar + 8 * i, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
    }
    for (int i = tid; i < n_out; i += 512) {
        bias_s[i] = a.bias ? __bfloat162float(a.bias[i]) : 0.f;
        g1[i] = a.ln1_w ? __bfloat162float(a.ln1_w[i]) : 1.f;
        b1[i] = a.ln1_b ? __bfloat162float(a.ln1_b[i]) : 0.f;
        g2[i] = a.ln2_w ? __bfloat162float(a.ln2_w[i]) : 1.f;
        b2[i] = a.ln2_b ? __bfloat162float(a.ln2_b[i]) : 0.f;
    }
    if (warp == 0) tmem_alloc(sbase + off_bar + 136, 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (tid == 0) {   // weights: once per CTA
        mbar_expect_tx(wbar, (uint32_t)(KB * w_block));
        for (int kb = 0; kb < KB; ++kb)
            for (int r = 0; r < n_out; r += a.w_box_rows)
                tma_load_2d(sbase + kb * w_block + r * SW, &map_w, kb * KCOLS, r, wbar);
    }
    // up to here only weights, biases and LayerNorm parameters were read: everything the kernel before
    // this one in the stream may have written is touched after this wait
    pdl_wait();
    bool ok = mbar_wait(wbar, 0, abort);

    // columns of tensor memory per group: n_out rounded up to 32, groups side by side
    const int tm_cols = (n_out + 31) / 32 * 32;
    const uint32_t tm_lane = (uint32_t)((warp & 3) * 32) << 16;
    // two accumulators per group where tensor memory has room (a.nacc == 2): the product of the next
    // tile is issued before this tile's epilogue starts, so no tile waits for its product
    const int nacc = a.nacc;
    const uint32_t tm_acc_step = (uint32_t)(a.groups * tm_cols);
    const uint32_t tm_acc0 = tmem_base + tm_lane + g * tm_cols;
    const uint32_t tm_acc_mma0 = tmem_base + g * tm_cols;
    const uint32_t xs0 = sbase + off_x + 2 * g * X_BYTES;   // two x buffers
    unsigned char* stage = smem + off_stage + g * LIN_STAGE_BYTES;
    unsigned char* my_row = stage + t * LIN_STAGE_ROW;
    // columns are handled in slabs of 64 (32 when n_out is 32 or 96 leaves a half slab)
    const int nslabs = (n_out + 63) / 64;
    // one MMA covers at most 256 output columns
    const int n_half = n_out > 256 ? n_out / 2 : n_out;
    const uint32_t idesc = umma_idesc_bf16(128, n_half);
    uint32_t xph[2] = {0, 0};
    const float inv_c = 1.f / (float)n_out;
    const int nchunks = n_out / 32;

    const int64_t ntiles = (a.n + 127) / 128;
    if (g < a.groups) {
        const int64_t tile_step = (int64_t)gridDim.x * a.groups;
        const int64_t tile0 = (int64_t)blockIdx.x * a.groups + g;
        auto load_x = [&](int64_t tile, int b) {
            mbar_expect_tx(xbar0 + 8 * b, X_BYTES);
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(xs0 + b * X_BYTES + kb * X_BLOCK, &map_x, kb * KCOLS, (int)(tile * 128), xbar0 + 8 * b);
        };
        // The residual rows are read with plain loads in the middle of the epilogue; asking for
        // them a tile ahead (L2 prefetch, no registers held) takes the DRAM latency out of the
        // tile's serial chain.
        auto prefetch_residual = [&](int64_t tile) {
            const int64_t r = tile * 128 + t;
            if (a.residual_mode && tile < ntiles && r < a.n) {
                const char* p = reinterpret_cast<const char*>(a.residual + r * n_out);
                for (int b = 0; b < n_out * 2; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + b));
            }
        };
        // t == 0 only: the product of the x tile in buffer xb into accumulator acc
        auto issue_mma = [&](int xb, int acc) {
            const uint32_t xs = xs0 + xb * X_BYTES;
            fence_after_sync();
            for (int h = 0; h < n_out; h += n_half) {
#pragma unroll
                for (int k = 0; k < K / 16; ++k) {
                    const int kb = (k * 16) / KCOLS, kk = (k * 16) % KCOLS;
                    const uint64_t da = umma_desc_kmajor(xs + kb * X_BLOCK + kk * 2, SW);
                    const uint64_t db = umma_desc_kmajor(sbase + kb * w_block + h * SW + kk * 2, SW);
                    umma_bf16(tm_acc_mma0 + acc * tm_acc_step + h, da, db, idesc, k > 0);
                }
            }
            umma_commit(mbar0 + 8 * acc);
        };
        // residual slab 0 of a tile into the staging tile, asynchronously (the staging tile is free
        // from the end of one tile to the residual pass of the next)
        auto fetch_residual = [&](int64_t row0) {
            if (!a.residual_mode) return;
            if (n_out >= 64) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 3), c = idx & 7;
                    const bool in = row0 + r < a.n;
                    cp_async16_zfill(smem_u32_generic(stage + r * LIN_STAGE_ROW + c * 16),
                                     a.residual + (in ? row0 + r : 0) * n_out + c * 8, in);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 2), c = idx & 3;
                    const bool in = row0 + r < a.n;
                    cp_async16_zfill(smem_u32_generic(stage + r * LIN_STAGE_ROW + c * 16),
                                     a.residual + (in ? row0 + r : 0) * n_out + c * 8, in);
                }
            }
            cp_async_commit();
        };
        if (t == 0 && tile0 < ntiles) {
            load_x(tile0, 0);
            if (nacc == 2) {
                ok &= mbar_wait(xbar0, xph[0], abort);
                xph[0] ^= 1;
                issue_mma(0, 0);
                if (tile0 + tile_step < ntiles) load_x(tile0 + tile_step, 1);
            }
        }
        int j = 0;
        for (int64_t tile = tile0; tile < ntiles; tile += tile_step, ++j) {
            const int64_t row0 = tile * 128;
            const int buf = j & 1, cur = nacc == 2 ? buf : 0;
            fetch_residual(row0);
            prefetch_residual(tile + tile_step);
            if (nacc == 2) {
                ok &= mbar_wait(mbar0 + 8 * cur, (j >> 1) & 1, abort);
                if (t == 0 && tile + tile_step < ntiles) {
                    // the next tile's product into the other accumulator (its epilogue ended with
                    // the barrier that closed the previous tile), then the x tile after that into
                    // the buffer this tile's product has finished with
                    ok &= mbar_wait(xbar0 + 8 * (buf ^ 1), xph[buf ^ 1], abort);
                    xph[buf ^ 1] ^= 1;
                    issue_mma(buf ^ 1, buf ^ 1);
                    if (tile + 2 * tile_step < ntiles) load_x(tile + 2 * tile_step, buf);
                }
            } else {
                ok &= mbar_wait(xbar0 + 8 * buf, xph[buf], abort);
                xph[buf] ^= 1;
                if (t == 0) {
                    // the other buffer was consumed by the previous tile's MMAs, which have completed:
                    // fetch the next tile into it while this tile is multiplied and written out
                    if (tile + tile_step < ntiles) load_x(tile + tile_step, buf ^ 1);
                    issue_mma(buf, 0);
                }
                ok &= mbar_wait(mbar0, j & 1, abort);
            }
            fence_after_sync();
            const uint32_t tm_acc = tm_acc0 + cur * tm_acc_step;
            if (!a.residual_mode) {
                // Plain mode: a warp packs `slw` columns of its 32 rows into its own staging tile (rows
                // slw * 2 bytes wide, swizzled like the tensor map so that the 16-byte stores of a warp
                // do not collide) and one lane hands the tile to a TMA store, which writes whole lines.
                const int slw = a.out_box, lane = t & 31;
                const uint32_t wtile = smem_u32_generic(stage) + (t >> 5) * 4096;
                const uint32_t my = wtile + lane * (slw * 2), swz = slw == 64 ? (lane & 7) : ((lane >> 1) & 3);
                for (int sl = 0; sl < n_out / slw; ++sl) {
                    // the copy of the slab before has finished reading the staging tile
                    if (lane == 0) bulk_wait_read<0>();
                    __syncwarp();
                    for (int c = 0; c < slw / 32; ++c) {
                        const int ch0 = sl * slw + c * 32;
                        float4 bb[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) bb[i] = *reinterpret_cast<const float4*>(bias_s + ch0 + i * 4);
                        uint32_t v[32];
                        tmem_ld32(tm_acc + ch0, v);
                        tmem_ld_wait();
                        tmem_ld_fence(v);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 b0 = bb[2 * q], b1 = bb[2 * q + 1];
                            const uint32_t* vv = v + q * 8;
                            const uint32_t o0 = pack_bf16(__uint_as_float(vv[0]) + b0.x, __uint_as_float(vv[1]) + b0.y);
                            const uint32_t o1 = pack_bf16(__uint_as_float(vv[2]) + b0.z, __uint_as_float(vv[3]) + b0.w);
                            const uint32_t o2 = pack_bf16(__uint_as_float(vv[4]) + b1.x, __uint_as_float(vv[5]) + b1.y);
                            const uint32_t o3 = pack_bf16(__uint_as_float(vv[6]) + b1.z, __uint_as_float(vv[7]) + b1.w);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my + (((c * 4 + q) ^ swz) << 4)),
                                         "r"(o0), "r"(o1), "r"(o2), "r"(o3));
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0 && row0 + (t & ~31) < a.n) {
                        tma_store_2d(&map_o, sl * slw, (int)row0 + (t & ~31), wtile);
                        bulk_commit();
                    }
                }
            } else {
                // The arithmetic below works on pairs of channels (fma.rn.f32x2 / add.rn.f32x2), reads the
                // per-channel parameters two pairs at a time and converts to bf16 once per rounding
                // (cvt.rn.bf16x2.f32; the rounded floats are the two halves of that word): the epilogue
                // is bound by instruction issue, not by memory.
                // ---- first LayerNorm (optional): statistics of y = round(acc + bias)
                float mean1 = 0.f, rstd1 = 1.f;
                if (a.ln1_w) {
                    // one pass with sums shifted by the row's first value (no cancellation)
                    float sh = 0.f;
                    uint64_t nsh2 = 0, s1 = 0, q1 = 0;
                    for (int c = 0; c < nchunks; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tm_acc + c * 32, v);
                        tmem_ld_wait();
                        if (c == 0) {
                            sh = lin_round(__uint_as_float(v[0]) + bias_s[0]);
                            nsh2 = pack2(-sh, -sh);
                        }
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(bias_s + c * 32 + i);
                            uint32_t pk;
                            const uint64_t d0 = add2(round2(add2(pack2u(v[i], v[i + 1]), bb.x), pk), nsh2);
                            const uint64_t d1 = add2(round2(add2(pack2u(v[i + 2], v[i + 3]), bb.y), pk), nsh2);
                            s1 = add2(s1, add2(d0, d1));
                            q1 = fma2(d0, d0, q1);
                            q1 = fma2(d1, d1, q1);
                        }
                    }
                    const float md1 = hsum2(s1) * inv_c;
                    mean1 = sh + md1;
                    rstd1 = rsqrtf(fmaxf(hsum2(q1) * inv_c - md1 * md1, 0.f) + a.eps1);
                }
                const uint64_t nmean1 = pack2(-mean1, -mean1), rs1 = pack2(rstd1, rstd1);
                // ---- s = residual + t, stored and parked in tensor memory; shifted sums for LN2
                float shift = 0.f;
                uint64_t nshift2 = 0, s2p = 0, q2p = 0;
                for (int sl = 0; sl < nslabs; ++sl) {
                    const int cw = min(64, n_out - sl * 64);
                    // residual slab: coalesced into the staging tile (slab 0 was asked for at the top)
                    if (sl == 0) {
                        cp_async_wait<0>();
                    } else if (cw == 64) {
                        global_to_stage(stage, a.residual, row0, a.n, n_out, sl * 64, t);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 2), c = idx & 3;
                            uint4 v = make_uint4(0, 0, 0, 0);
                            if (row0 + r < a.n)
                                v = *reinterpret_cast<const uint4*>(a.residual + (row0 + r) * n_out + sl * 64 + c * 8);
                            *reinterpret_cast<uint4*>(stage + r * LIN_STAGE_ROW + c * 16) = v;
                        }
                    }
                    __syncwarp();      // the staging rows of a warp are its own
                    for (int c = 0; c < cw / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tm_acc + sl * 64 + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 rr = *reinterpret_cast<const uint4*>(my_row + c * 64 + q * 16);
                            const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
                            uint32_t ow[4];
                            const int ch0 = sl * 64 + c * 32 + q * 8;
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(bias_s + ch0 + h * 4);
                                ulonglong2 gg = {0, 0}, hh = {0, 0};
                                if (a.ln1_w) {
                                    gg = *reinterpret_cast<const ulonglong2*>(g1 + ch0 + h * 4);
                                    hh = *reinterpret_cast<const ulonglong2*>(b1 + ch0 + h * 4);
                                }
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int i = q * 8 + h * 4 + e * 2;      // first of the two columns
                                    uint32_t pk;
                                    uint64_t y = round2(add2(pack2u(v[i], v[i + 1]), e ? bb.y : bb.x), pk);
                                    if (a.ln1_w)
                                        y = round2(fma2(fma2(add2(y, nmean1), rs1, 0ull), e ? gg.y : gg.x,
                                                        e ? hh.y : hh.x), pk);
                                    const uint64_t sv = round2(add2(unpack_bf16x2(rw[h * 2 + e]), y), pk);
                                    ow[h * 2 + e] = pk;
                                    if (sl == 0 && c == 0 && q == 0 && h == 0 && e == 0) {
                                        float lo, hi;
                                        unpack2(sv, lo, hi);
                                        shift = lo;
                                        nshift2 = pack2(-lo, -lo);
                                    }
                                    const uint64_t d = add2(sv, nshift2);
                                    s2p = add2(s2p, d);
                                    q2p = fma2(d, d, q2p);
                                    v[i] = (uint32_t)sv;
                                    v[i + 1] = (uint32_t)(sv >> 32);
                                }
                            }
                            *reinterpret_cast<uint4*>(my_row + c * 64 + q * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        }
                        tmem_st32(tm_acc + sl * 64 + c * 32, v);
                    }
                    __syncwarp();      // the staging rows of a warp are its own
                    if (a.sum_out) {
                        if (cw == 64) {
                            stage_to_global(stage, a.sum_out, row0, a.n, n_out, sl * 64, t);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 2), c = idx & 3;
                                if (row0 + r < a.n)
                                    *reinterpret_cast<uint4*>(a.sum_out + (row0 + r) * n_out + sl * 64 + c * 8) =
                                        *reinterpret_cast<const uint4*>(stage + r * LIN_STAGE_ROW + c * 16);
                            }
                        }
                    }
                    __syncwarp();      // the staging rows of a warp are its own
                }
                const float s2 = hsum2(s2p), q2 = hsum2(q2p);
                tmem_st_wait();
                const float md = s2 * inv_c;                      // mean - shift
                const float var = fmaxf(q2 * inv_c - md * md, 0.f);
                const float mean2 = shift + md, rstd2 = rsqrtf(var + a.eps2);
                const uint64_t nmean2 = pack2(-mean2, -mean2), rs2 = pack2(rstd2, rstd2);
                for (int sl = 0; sl < nslabs; ++sl) {
                    const int cw = min(64, n_out - sl * 64);
                    for (int c = 0; c < cw / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tm_acc + sl * 64 + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t ow[4];
                            const int ch0 = sl * 64 + c * 32 + q * 8;
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const ulonglong2 gg = *reinterpret_cast<const ulonglong2*>(g2 + ch0 + h * 4);
                                const ulonglong2 hh = *reinterpret_cast<const ulonglong2*>(b2 + ch0 + h * 4);
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int i = q * 8 + h * 4 + e * 2;
                                    const uint64_t f = fma2(fma2(add2(pack2u(v[i], v[i + 1]), nmean2), rs2, 0ull),
                                                            e ? gg.y : gg.x, e ? hh.y : hh.x);
                                    float lo, hi;
                                    unpack2(f, lo, hi);
                                    ow[h * 2 + e] = pack_bf16(lo, hi);
                                }
                            }
                            *reinterpret_cast<uint4*>(my_row + c * 64 + q * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        }
                    }
                    __syncwarp();      // the staging rows of a warp are its own
                    if (cw == 64) {
                        stage_to_global(stage, a.norm_out, row0, a.n, n_out, sl * 64, t);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int idx = i * 32 + (t & 31), r = (t & ~31) + (idx >> 2), c = idx & 3;
                            if (row0 + r < a.n)
                                *reinterpret_cast<uint4*>(a.norm_out + (row0 + r) * n_out + sl * 64 + c * 8) =
                                    *reinterpret_cast<const uint4*>(stage + r * LIN_STAGE_ROW + c * 16);
                        }
                    }
                    __syncwarp();      // the staging rows of a warp are its own
                }
            }
            fence_before_sync();
            named_barrier(1 + g, 128);
        }
    }
    // shared memory stays allocated until the last TMA stores have read it
    if ((tid & 31) == 0) bulk_wait_read<0>();
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && (*abort || !ok)) atomicOr(a.status, PTV3_STATUS_WAIT_LIMIT);
}

static bool linear_shape_ok(int k, int n_out, bool residual_mode)
{
    if (k != 32 && k != 64 && k != 128) return false;
    if (residual_mode) return n_out == k;
    return n_out % 32 == 0 && n_out >= 32 && n_out <= 384 && (n_out <= 256 || (n_out / 2) % 16 == 0);
}

static int launch_linear(const void* x, const void* w, LinearArgs a, int k, cudaStream_t stream)
{
    const int sw = k >= 64 ? 128 : 64, kb = k >= 64 ? k / 64 : 1, kcols = k >= 64 ? 64 : k;
    a.w_box_rows = a.n_out <= 256 ? a.n_out : a.n_out / 2;
    const int tm_cols = (a.n_out + 31) / 32 * 32;
    int groups = 512 / tm_cols;
    if (groups > 4) groups = 4;
    // ... and as many as fit in shared memory next to the resident weights
    while (groups > 1 && (size_t)kb * a.n_out * sw + (size_t)groups * (2 * kb * 128 * sw + LIN_STAGE_BYTES) +
                                 5 * (size_t)a.n_out * 4 + 160 + 1024 > 220 * 1024)
        --groups;
    a.groups = groups;
    a.nacc = 2 * groups * tm_cols <= 512 ? 2 : 1;
    CUtensorMap mx, mw, mo;
    int rc = make_tensor_map_bf16(&mx, x, (uint64_t)a.n, k, (uint64_t)k * 2, 128, kcols);
    if (rc) return rc;
    mo = mx;      // residual mode writes its outputs with plain stores
    if (!a.residual_mode) {
        a.out_box = a.n_out % 64 == 0 ? 64 : 32;
        rc = make_tensor_map_bf16(&mo, a.out, (uint64_t)a.n, (uint64_t)a.n_out, (uint64_t)a.n_out * 2, 32, a.out_box);
        if (rc) return rc;
    }
    rc = make_tensor_map_bf16(&mw, w, a.n_out, k, (uint64_t)k * 2, a.w_box_rows, kcols);
    if (rc) return rc;
    const size_t smem = (size_t)kb * a.n_out * sw + (size_t)groups * (2 * kb * 128 * sw + LIN_STAGE_BYTES) +
                        5 * (size_t)a.n_out * 4 + 160 + 1024;
    const size_t smem_req = smem < 120 * 1024 ? 120 * 1024 : smem;   // one CTA per SM (it takes all of tensor memory)
    const int64_t ntiles = (a.n + 127) / 128;
    int64_t grid = (ntiles + groups - 1) / groups;
    if (grid > 148) grid = 148;
#define LIN_LAUNCH(KK)                                                                                       \
    do {                                                                                                     \
        auto kern = linear_tc05_kernel<KK>;                                                                  \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req) !=        \
            cudaSuccess)                                                                                     \
            return check_launch("ptv3_linear_fwd: shared memory attribute");                                 \
        launch_dependent(kern, dim3((unsigned)grid), dim3(512), smem_req, stream, mx, mw, mo, a);                \
    } while (0)
    if (k == 32) LIN_LAUNCH(32);
    else if (k == 64) LIN_LAUNCH(64);
    else LIN_LAUNCH(128);
#undef LIN_LAUNCH
    count_launches(1);
    return check_launch("ptv3_linear_fwd");
}

}  // namespace ptv3

extern "C" int ptv3_linear_supported(int k, int n_out, int residual_mode, int dtype)
{
    return dtype == PTV3_DTYPE_BF16 && ptv3::linear_shape_ok(k, n_out, residual_mode != 0);
}

extern "C" int ptv3_linear_fwd(const void* x, const void* weight, const void* bias, void* out, int64_t n, int k,
                               int n_out, int dtype, uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_linear_fwd: bad n");
    PTV3_REQUIRE(ptv3_linear_supported(k, n_out, 0, dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_linear_fwd: supported: bf16, k in {32, 64, 128}, n_out a multiple of 32 up to 384");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(x && weight && out && status, PTV3_ERR_INVALID_ARGUMENT, "ptv3_linear_fwd: null pointer");
    PTV3_REQUIRE((((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_linear_fwd: tensors must be 16-byte aligned");
    LinearArgs a{};
    a.bias = (const __nv_bfloat16*)bias;
    a.out = (__nv_bfloat16*)out;
    a.n = n;
    a.n_out = n_out;
    a.residual_mode = 0;
    a.status = status;
    return launch_linear(x, weight, a, k, (cudaStream_t)stream);
}

extern "C" int ptv3_linear_ln_fwd(const void* x, const void* weight, const void* bias, const void* residual,
                                  const void* ln1_weight, const void* ln1_bias, float ln1_eps, void* sum_out,
                                  const void* ln2_weight, const void* ln2_bias, float ln2_eps, void* norm_out,
                                  int64_t n, int channels, int dtype, uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_linear_ln_fwd: bad n");
    PTV3_REQUIRE(ptv3_linear_supported(channels, channels, 1, dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_linear_ln_fwd: supported: bf16, channels in {32, 64, 128}");
    PTV3_REQUIRE((ln1_weight == nullptr) == (ln1_bias == nullptr), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_linear_ln_fwd: LayerNorm weight and bias go together");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(x && weight && residual && ln2_weight && ln2_bias && norm_out && status,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_linear_ln_fwd: null pointer");
    PTV3_REQUIRE((((uintptr_t)x | (uintptr_t)weight | (uintptr_t)residual | (uintptr_t)norm_out |
                   (uintptr_t)sum_out) & 15) == 0,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_linear_ln_fwd: tensors must be 16-byte aligned");
    LinearArgs a{};
    a.bias = (const __nv_bfloat16*)bias;
    a.residual = (const __nv_bfloat16*)residual;
    a.ln1_w = (const __nv_bfloat16*)ln1_weight;
    a.ln1_b = (const __nv_bfloat16*)ln1_bias;
    a.ln2_w = (const __nv_bfloat16*)ln2_weight;
    a.ln2_b = (const __nv_bfloat16*)ln2_bias;
    a.sum_out = (__nv_bfloat16*)sum_out;
    a.norm_out = (__nv_bfloat16*)norm_out;
    a.eps1 = ln1_eps;
    a.eps2 = ln2_eps;
    a.n = n;
    a.n_out = channels;
    a.residual_mode = 1;
    a.status = status;
    return launch_linear(x, weight, a, channels, (cudaStream_t)stream);
}
