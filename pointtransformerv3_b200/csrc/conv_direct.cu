// Submanifold convolution with few input channels and a large kernel (the 5x5x5
// stem, model.py:766-779) without a kernel map: the neighbour table of such a
// convolution (125 x N int32) is several times larger than its input and its
// output, so the voxel hash table is probed inside the convolution instead.
//
// The voxels are indexed in two levels: a hash table of 4 x 4 x 4 blocks whose
// values point at 64-entry cell tables (cell -> row).  A CTA owns 128 voxels:
// each voxel first looks up the (at most 8) blocks its neighbourhood touches,
// then the kernel offsets are walked 25 at a time; in each round the 256 threads
// read 25 x 128 neighbour rows from the cell tables and gather the features of
// the neighbours found into shared memory (all independent, latencies overlap);
// then thread (voxel, half) accumulates half of the output channels in fp32
// registers, reading the weights (staged once per CTA) as warp-wide broadcasts
// and skipping absent neighbours.
// Epilogue: optional bias, optional BatchNorm(eval) scale/shift + exact GELU
// (model.py:848,860 for the stem), rounding, one contiguous store per thread.
//
// bf16 features take the tensor-core form of the same kernel (conv_direct_mma_kernel):
// the staged neighbour rows of 16 offsets are the A operand (128 voxels x K = 16 x 8
// padded channels, zero rows where a neighbour is absent) of mma.sync against that
// round's slice of the weights; nothing is skipped because the products are cheap - the
// CUDA-core form spends most of its instructions unpacking bf16 weights for the FMAs.
#include "common.cuh"
#include "convert.cuh"
#include "kmap.cuh"
#include "mma_util.cuh"
#include "voxel_index.cuh"
#include "vec.cuh"

namespace ptv3 {

constexpr int CD_TM = 128;
constexpr int CD_THREADS = 256;
constexpr int CD_MAX_CIN = 8;

__device__ __forceinline__ float cd_gelu(float x)
{
    return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
}

constexpr int CD_CHUNK = 25;   // kernel offsets staged per round

// [cout][kvol][cin] -> [kvol][cin][cout], once per call (a few thousand elements)
template <typename T>
__global__ void conv_direct_transpose_kernel(const T* __restrict__ w, T* __restrict__ wt, int cout,
                                             int kvol, int cin)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= cout * kvol * cin) return;
    const int ci = idx % cin, rest = idx / cin;
    const int o = rest % kvol, co = rest / kvol;
    wt[((size_t)o * cin + ci) * cout + co] = w[idx];
}

// CO: output channels per thread (c_out = 2 * CO)
template <typename T, int CO>
__global__ void __launch_bounds__(CD_THREADS) conv_direct_kernel(
    const T* __restrict__ feat, const int32_t* __restrict__ indices, const T* __restrict__ weight,
    const T* __restrict__ bias, const float* __restrict__ bn_scale, const float* __restrict__ bn_shift,
    int apply_gelu, T* __restrict__ out, const int64_t* __restrict__ row_order, int64_t n, int cin,
    int ksize, const unsigned long long* __restrict__ keys, const uint32_t* __restrict__ vals,
    uint64_t cap_mask, const uint32_t* __restrict__ cells, uint32_t* __restrict__ status)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const int kvol = ksize * ksize * ksize;
    const int cout = 2 * CO;
    // staged neighbour features of one round: [CD_CHUNK][128][CD_MAX_CIN], zero where absent
    T* x_s = reinterpret_cast<T*>(smem);
    unsigned char* has_s = smem + (size_t)CD_CHUNK * CD_TM * CD_MAX_CIN * sizeof(T);   // [CD_CHUNK][128]
    T* w_s = reinterpret_cast<T*>(has_s + CD_CHUNK * CD_TM);                            // kvol x cin x cout
    __shared__ int4 coord_s[CD_TM];
    __shared__ uint32_t block_s[8][CD_TM];   // table id of the 2 x 2 x 2 blocks around each voxel
    __shared__ char4 delta_s[343];           // (dx, dy, dz) of every kernel offset

    const int tid = threadIdx.x;
    const int v = tid % CD_TM, half = tid / CD_TM;
    const int64_t i = (int64_t)blockIdx.x * CD_TM + v;
    const int64_t row = i < n ? (row_order ? row_order[i] : i) : -1;
    const int r = ksize / 2;
    const int4 c = row >= 0 ? reinterpret_cast<const int4*>(indices)[row] : make_int4(-1, 0, 0, 0);
    if (half == 0) coord_s[v] = c;
    for (int o = tid; o < kvol; o += CD_THREADS)
        delta_s[o] = make_char4((char)(o / (ksize * ksize) - r), (char)((o / ksize) % ksize - r),
                                (char)(o % ksize - r), 0);
    // weights, already transposed to [kvol][cin][cout]: straight 16-byte copy
    {
        const int nvec = kvol * cin * cout / Vec<T>::N;
        const typename Vec<T>::Raw* src = reinterpret_cast<const typename Vec<T>::Raw*>(weight);
        typename Vec<T>::Raw* dst = reinterpret_cast<typename Vec<T>::Raw*>(w_s);
        for (int idx = tid; idx < nvec; idx += CD_THREADS) dst[idx] = src[idx];
    }
    // the 8 candidate blocks of this voxel: 4 probes per thread
    bool overflow = false;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int bi = half * 4 + q;   // bit 2: x, bit 1: y, bit 0: z  (0 = block of coord - r)
        uint32_t id = VI_NO_ROW;
        if (c.x >= 0) {
            const int bx = ((c.y - r) >> 2) + ((bi >> 2) & 1);
            const int by = ((c.z - r) >> 2) + ((bi >> 1) & 1);
            const int bz = ((c.w - r) >> 2) + (bi & 1);
            uint64_t key;
            if (vi_block_key(c.x, bx, by, bz, key)) id = vi_block_lookup(keys, vals, cap_mask, key, &overflow);
        }
        block_s[bi][v] = id;
    }
    __syncthreads();

    float acc[CO];
#pragma unroll
    for (int k = 0; k < CO; ++k) acc[k] = 0.f;

    for (int o0 = 0; o0 < kvol; o0 += CD_CHUNK) {
        const int no = min(CD_CHUNK, kvol - o0);
        // neighbour row from the cell tables + feature gather; all independent
        for (int idx = tid; idx < no * CD_TM; idx += CD_THREADS) {
            const int ol = idx / CD_TM, vv = idx % CD_TM;
            const int4 cc = coord_s[vv];
            const char4 d = delta_s[o0 + ol];
            uint32_t j = VI_NO_ROW;
            if (cc.x >= 0) {
                const int x = cc.y + d.x, y = cc.z + d.y, z = cc.w + d.z;
                const int bi = (((x >> 2) - ((cc.y - r) >> 2)) << 2) | (((y >> 2) - ((cc.z - r) >> 2)) << 1) |
                               ((z >> 2) - ((cc.w - r) >> 2));
                const uint32_t id = block_s[bi][vv];
                if (id != VI_NO_ROW) j = cells[(size_t)id * 64 + ((x & 3) << 4 | (y & 3) << 2 | (z & 3))];
            }
            T* dst = x_s + ((size_t)ol * CD_TM + vv) * CD_MAX_CIN;
            has_s[ol * CD_TM + vv] = j != VI_NO_ROW;
            if (j != VI_NO_ROW) {
                const T* src = feat + (int64_t)j * cin;
#pragma unroll
                for (int ci = 0; ci < CD_MAX_CIN; ++ci) dst[ci] = ci < cin ? src[ci] : from_f<T>(0.f);
            }
        }
        __syncthreads();
        for (int ol = 0; ol < no; ++ol) {
            if (!has_s[ol * CD_TM + v]) continue;
            const T* xp = x_s + ((size_t)ol * CD_TM + v) * CD_MAX_CIN;
            float x[CD_MAX_CIN];
#pragma unroll
            for (int ci = 0; ci < CD_MAX_CIN; ci += Vec<T>::N)
                Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::Raw*>(xp + ci), x + ci);
            const T* w = w_s + (size_t)(o0 + ol) * cin * cout + half * CO;
#pragma unroll
            for (int ci = 0; ci < CD_MAX_CIN; ++ci) {
                if (ci < cin) {
                    // CO consecutive weights with 16-byte shared-memory loads (same address warp-wide)
#pragma unroll
                    for (int k = 0; k < CO; k += Vec<T>::N) {
                        float wv[Vec<T>::N];
                        Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::Raw*>(w + ci * cout + k), wv);
#pragma unroll
                        for (int q = 0; q < Vec<T>::N; ++q) acc[k + q] = fmaf(x[ci], wv[q], acc[k + q]);
                    }
                }
            }
        }
        __syncthreads();
    }
    if (overflow) atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
    if (row < 0) return;
    T* op = out + row * (int64_t)cout + half * CO;
#pragma unroll
    for (int k = 0; k < CO; ++k) {
        const int ch = half * CO + k;
        float y = acc[k];
        if (bias) y += to_f<T>(bias[ch]);
        if (bn_scale) {
            // the convolution output is rounded to the element type first, as a
            // separate normalisation module would see it
            y = to_f<T>(from_f<T>(y));
            y = fmaf(y, bn_scale[ch], bn_shift[ch]);
        }
        if (apply_gelu) {
            if (bn_scale) y = to_f<T>(from_f<T>(y));
            y = cd_gelu(y);
        }
        op[k] = from_f<T>(y);
    }
}

constexpr int CDM_CH = 16;   // kernel offsets per round of the tensor-core form (K = 128)

// [cout][kvol][cin] -> [kvol rounded up to CDM_CH][8][cout], zero padded
__global__ void conv_direct_transpose_pad_kernel(const __nv_bfloat16* __restrict__ w,
                                                 __nv_bfloat16* __restrict__ wt, int cout, int kvol, int cin,
                                                 int kvol_pad)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= kvol_pad * 8 * cout) return;
    const int co = idx % cout, ci = (idx / cout) % 8, o = idx / (8 * cout);
    wt[idx] = (o < kvol && ci < cin) ? w[((size_t)co * kvol + o) * cin + ci] : __float2bfloat16(0.f);
}

// NT: 8-wide output channel tiles (c_out = 8 NT, NT even)
template <int NT>
__global__ void __launch_bounds__(CD_THREADS) conv_direct_mma_kernel(
    const __nv_bfloat16* __restrict__ feat, const int32_t* __restrict__ indices,
    const __nv_bfloat16* __restrict__ wt, const __nv_bfloat16* __restrict__ bias,
    const float* __restrict__ bn_scale, const float* __restrict__ bn_shift, int apply_gelu,
    __nv_bfloat16* __restrict__ out, const int64_t* __restrict__ row_order, int64_t n, int cin, int ksize,
    const unsigned long long* __restrict__ keys, const uint32_t* __restrict__ vals, uint64_t cap_mask,
    const uint32_t* __restrict__ cells, uint32_t* __restrict__ status)
{
    constexpr int COUT = 8 * NT;
    constexpr int WROW = COUT * 2 + 16;   // weight row pitch: 16 bytes of padding keep ldmatrix conflict-free
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* x_s = smem;                                   // [CDM_CH][128] rows of 8 channels (16 B)
    unsigned char* w_s = smem + CDM_CH * CD_TM * 16;             // [CDM_CH * 8][COUT (+ padding)] of this round
    __shared__ int4 coord_s[CD_TM];
    __shared__ int row_s[CD_TM];
    __shared__ uint32_t block_s[8][CD_TM];
    __shared__ char4 delta_s[343];

    const int kvol = ksize * ksize * ksize;
    const int kvol_pad = (kvol + CDM_CH - 1) / CDM_CH * CDM_CH;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v = tid % CD_TM, half = tid / CD_TM;
    const int64_t i = (int64_t)blockIdx.x * CD_TM + v;
    const int64_t row = i < n ? (row_order ? row_order[i] : i) : -1;
    const int r = ksize / 2;
    const int4 c = row >= 0 ? reinterpret_cast<const int4*>(indices)[row] : make_int4(-1, 0, 0, 0);
    if (half == 0) {
        coord_s[v] = c;
        row_s[v] = (int)row;
    }
    for (int o = tid; o < kvol; o += CD_THREADS)
        delta_s[o] = make_char4((char)(o / (ksize * ksize) - r), (char)((o / ksize) % ksize - r),
                                (char)(o % ksize - r), 0);
    bool overflow = false;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int bi = half * 4 + q;   // bit 2: x, bit 1: y, bit 0: z  (0 = block of coord - r)
        uint32_t id = VI_NO_ROW;
        if (c.x >= 0) {
            const int bx = ((c.y - r) >> 2) + ((bi >> 2) & 1);
            const int by = ((c.z - r) >> 2) + ((bi >> 1) & 1);
            const int bz = ((c.w - r) >> 2) + (bi & 1);
            uint64_t key;
            if (vi_block_key(c.x, bx, by, bz, key)) id = vi_block_lookup(keys, vals, cap_mask, key, &overflow);
        }
        block_s[bi][v] = id;
    }
    __syncthreads();

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const uint32_t xs_base = smem_u32(x_s), ws_base = smem_u32(w_s);
    const bool words = (cin & 1) == 0;   // rows of an even channel count are 4-byte aligned

    for (int o0 = 0; o0 < kvol_pad; o0 += CDM_CH) {
        // this round's weights: CDM_CH * 8 rows of COUT
        for (int idx = tid; idx < CDM_CH * COUT; idx += CD_THREADS)
            cp_async16(ws_base + (idx / NT) * WROW + (idx % NT) * 16, wt + ((size_t)o0 * 8 * COUT + (size_t)idx * 8));
        cp_async_commit();
        // neighbour rows from the cell tables, then their features; all independent
        uint32_t j[CDM_CH * CD_TM / CD_THREADS];
#pragma unroll
        for (int k = 0; k < CDM_CH * CD_TM / CD_THREADS; ++k) {
            const int idx = tid + k * CD_THREADS;
            const int ol = idx / CD_TM, vv = idx % CD_TM;
            const int4 cc = coord_s[vv];
            j[k] = VI_NO_ROW;
            if (cc.x >= 0 && o0 + ol < kvol) {
                const char4 d = delta_s[o0 + ol];
                const int x = cc.y + d.x, y = cc.z + d.y, z = cc.w + d.z;
                const int bi = (((x >> 2) - ((cc.y - r) >> 2)) << 2) | (((y >> 2) - ((cc.z - r) >> 2)) << 1) |
                               ((z >> 2) - ((cc.w - r) >> 2));
                const uint32_t id = block_s[bi][vv];
                if (id != VI_NO_ROW) j[k] = cells[(size_t)id * 64 + ((x & 3) << 4 | (y & 3) << 2 | (z & 3))];
            }
        }
#pragma unroll
        for (int k = 0; k < CDM_CH * CD_TM / CD_THREADS; ++k) {
            const int idx = tid + k * CD_THREADS;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (j[k] != VI_NO_ROW) {
                const __nv_bfloat16* src = feat + (int64_t)j[k] * cin;
                if (words) {
                    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
                    val.x = s32[0];
                    if (cin > 2) val.y = s32[1];
                    if (cin > 4) val.z = s32[2];
                    if (cin > 6) val.w = s32[3];
                } else {
                    unsigned short e[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
#pragma unroll
                    for (int ci = 0; ci < 8; ++ci)
                        if (ci < cin) e[ci] = s16[ci];
                    val = make_uint4(e[0] | (uint32_t)e[1] << 16, e[2] | (uint32_t)e[3] << 16,
                                     e[4] | (uint32_t)e[5] << 16, e[6] | (uint32_t)e[7] << 16);
                }
            }
            *reinterpret_cast<uint4*>(x_s + (size_t)idx * 16) = val;
        }
        cp_async_wait<0>();
        __syncthreads();
        // out[16 voxels of this warp][COUT] += X[16][128] . W[128][COUT]
#pragma unroll
        for (int ks = 0; ks < CDM_CH / 2; ++ks) {
            uint32_t a[4];
            {
                const int mi = lane >> 3, rr = lane & 7;
                const int vv = 16 * warp + (mi & 1) * 8 + rr, ol = 2 * ks + (mi >> 1);
                ldmatrix_x4(a, xs_base + (ol * CD_TM + vv) * 16);
            }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                const int mi = lane >> 3, rr = lane & 7;
                const int kk = 16 * ks + (mi & 1) * 8 + rr, n0 = np * 16 + (mi >> 1) * 8;
                ldmatrix_x4_trans(b, ws_base + kk * WROW + n0 * 2);
                mma_bf16(acc[2 * np], a, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    if (overflow) atomicOr(status, PTV3_STATUS_PROBE_LIMIT);

    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        const int orow = row_s[16 * warp + g + 8 * hrow];
        if (orow < 0) continue;
        uint32_t* op = reinterpret_cast<uint32_t*>(out + (int64_t)orow * COUT);
#pragma unroll
        for (int jn = 0; jn < NT; ++jn) {
            float y[2] = {acc[jn][2 * hrow], acc[jn][2 * hrow + 1]};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int ch = 8 * jn + 2 * t + e;
                if (bias) y[e] += __bfloat162float(bias[ch]);
                if (bn_scale) {
                    // the convolution output is rounded to the element type first, as a
                    // separate normalisation module would see it
                    y[e] = __bfloat162float(__float2bfloat16(y[e]));
                    y[e] = fmaf(y[e], bn_scale[ch], bn_shift[ch]);
                }
                if (apply_gelu) {
                    if (bn_scale) y[e] = __bfloat162float(__float2bfloat16(y[e]));
                    y[e] = cd_gelu(y[e]);
                }
            }
            op[4 * jn + t] = pack_bf16(y[0], y[1]);
        }
    }
}

static int launch_conv_direct_mma(const void* feat, const int32_t* indices, const void* weight, const void* bias,
                                  const float* bn_scale, const float* bn_shift, int apply_gelu, void* out,
                                  const int64_t* row_order, int64_t n, int cin, int cout, int ksize,
                                  const unsigned long long* keys, const uint32_t* vals, uint64_t cap_mask,
                                  const uint32_t* cells, uint32_t* status, void* wt, cudaStream_t stream)
{
    const int kvol = ksize * ksize * ksize;
    const int kvol_pad = (kvol + CDM_CH - 1) / CDM_CH * CDM_CH;
    conv_direct_transpose_pad_kernel<<<(kvol_pad * 8 * cout + 255) / 256, 256, 0, stream>>>(
        (const __nv_bfloat16*)weight, (__nv_bfloat16*)wt, cout, kvol, cin, kvol_pad);
    const size_t smem = (size_t)CDM_CH * CD_TM * 16 + (size_t)CDM_CH * 8 * (cout * 2 + 16);
    const unsigned blocks = (unsigned)((n + CD_TM - 1) / CD_TM);
#define CDM_LAUNCH(NT)                                                                                      \
    do {                                                                                                    \
        auto kern = conv_direct_mma_kernel<NT>;                                                             \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=           \
            cudaSuccess)                                                                                    \
            return check_launch("ptv3_subm_conv_direct_fwd: shared memory attribute");                      \
        kern<<<blocks, CD_THREADS, smem, stream>>>(                                                          \
            (const __nv_bfloat16*)feat, indices, (const __nv_bfloat16*)wt, (const __nv_bfloat16*)bias,       \
            bn_scale, bn_shift, apply_gelu, (__nv_bfloat16*)out, row_order, n, cin, ksize, keys, vals,       \
            cap_mask, cells, status);                                                                       \
    } while (0)
    switch (cout) {
        case 16: CDM_LAUNCH(2); break;
        case 32: CDM_LAUNCH(4); break;
        case 48: CDM_LAUNCH(6); break;
        case 64: CDM_LAUNCH(8); break;
        default:
            set_error("ptv3_subm_conv_direct_fwd: c_out %d (supported: 16, 32, 48, 64)", cout);
            return PTV3_ERR_UNSUPPORTED;
    }
#undef CDM_LAUNCH
    count_launches(2);
    return check_launch("ptv3_subm_conv_direct_fwd");
}

template <typename T>
static int launch_conv_direct(const void* feat, const int32_t* indices, const void* weight, const void* bias,
                              const float* bn_scale, const float* bn_shift, int apply_gelu, void* out,
                              const int64_t* row_order, int64_t n, int cin, int cout, int ksize,
                              const unsigned long long* keys, const uint32_t* vals, uint64_t cap_mask,
                              const uint32_t* cells, uint32_t* status, void* wt, cudaStream_t stream)
{
    const int kvol = ksize * ksize * ksize;
    conv_direct_transpose_kernel<T><<<(cout * kvol * cin + 255) / 256, 256, 0, stream>>>(
        (const T*)weight, (T*)wt, cout, kvol, cin);
    weight = wt;
    const size_t smem = (size_t)CD_CHUNK * CD_TM * (CD_MAX_CIN * sizeof(T) + 1) +
                        (size_t)kvol * cin * cout * sizeof(T);
    const unsigned blocks = (unsigned)((n + CD_TM - 1) / CD_TM);
#define CD_LAUNCH(CO)                                                                                    \
    do {                                                                                                 \
        auto kern = conv_direct_kernel<T, CO>;                                                           \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=        \
            cudaSuccess)                                                                                 \
            return check_launch("ptv3_subm_conv_direct_fwd: shared memory attribute");                   \
        kern<<<blocks, CD_THREADS, smem, stream>>>((const T*)feat, indices, (const T*)weight,             \
                                                   (const T*)bias, bn_scale, bn_shift, apply_gelu,        \
                                                   (T*)out, row_order, n, cin, ksize, keys, vals,         \
                                                   cap_mask, cells, status);                              \
    } while (0)
    if (smem > 220 * 1024) {
        set_error("ptv3_subm_conv_direct_fwd: %zu bytes of shared memory needed", smem);
        return PTV3_ERR_UNSUPPORTED;
    }
    switch (cout) {
        case 16: CD_LAUNCH(8); break;
        case 32: CD_LAUNCH(16); break;
        case 48: CD_LAUNCH(24); break;
        case 64: CD_LAUNCH(32); break;
        default:
            set_error("ptv3_subm_conv_direct_fwd: c_out %d (supported: 16, 32, 48, 64)", cout);
            return PTV3_ERR_UNSUPPORTED;
    }
#undef CD_LAUNCH
    count_launches(2);
    return check_launch("ptv3_subm_conv_direct_fwd");
}

static size_t conv_direct_weight_bytes(int ksize) { return align_up((size_t)ksize * ksize * ksize * 8 * 64 * 4, 256); }
// hash table of blocks (sized for one block per voxel), block counter, one 64-entry table per block
static size_t conv_direct_index_bytes(int64_t n) { return voxel_index_bytes(n); }

}  // namespace ptv3

extern "C" size_t ptv3_subm_conv_direct_workspace_bytes(int64_t n, int ksize)
{
    return n > 0 ? ptv3::conv_direct_index_bytes(n) + ptv3::conv_direct_weight_bytes(ksize) : 0;
}

extern "C" int ptv3_subm_conv_direct_fwd(const void* feat, const int32_t* indices, const void* weight,
                                         const void* bias, const float* bn_scale, const float* bn_shift,
                                         int apply_gelu, void* out, const int64_t* row_order, int64_t n,
                                         int c_in, int c_out, int ksize, int dtype, uint32_t* status,
                                         void* workspace, size_t workspace_bytes, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_subm_conv_direct_fwd: bad n");
    PTV3_REQUIRE(c_in >= 1 && c_in <= CD_MAX_CIN, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_direct_fwd: c_in %d outside [1, %d]", c_in, CD_MAX_CIN);
    PTV3_REQUIRE(ksize == 1 || ksize == 3 || ksize == 5, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_direct_fwd: kernel size %d (supported: 1, 3, 5)", ksize);
    PTV3_REQUIRE(dtype == PTV3_DTYPE_F32 || dtype == PTV3_DTYPE_BF16, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_direct_fwd: dtype %d", dtype);
    PTV3_REQUIRE((bn_scale == nullptr) == (bn_shift == nullptr), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_direct_fwd: bn_scale and bn_shift go together");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(feat && indices && weight && out && status && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_direct_fwd: null pointer");
    PTV3_REQUIRE(((uintptr_t)indices & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_subm_conv_direct_fwd: indices must be 16-byte aligned");
    const size_t need = conv_direct_index_bytes(n) + conv_direct_weight_bytes(ksize);
    PTV3_REQUIRE(workspace_bytes >= need, PTV3_ERR_WORKSPACE,
                 "ptv3_subm_conv_direct_fwd: workspace %zu < %zu bytes", workspace_bytes, need);
    PTV3_REQUIRE(((size_t)ksize * ksize * ksize * c_in * c_out) % 8 == 0, PTV3_ERR_UNSUPPORTED,
                 "ptv3_subm_conv_direct_fwd: weight size must be a multiple of 8 elements");
    void* wt = static_cast<char*>(workspace) + conv_direct_index_bytes(n);
    cudaStream_t stream = (cudaStream_t)stream_;
    VoxelIndex vi;
    {
        const int rc = build_voxel_index(indices, n, workspace, status, stream, &vi);
        if (rc != PTV3_OK) return rc;
    }
    const unsigned long long* keys = vi.keys;
    const uint32_t* vals = vi.vals;
    const uint64_t cap_mask = vi.cap_mask;
    const uint32_t* cells = vi.cells;
    if (dtype == PTV3_DTYPE_F32)
        return launch_conv_direct<float>(feat, indices, weight, bias, bn_scale, bn_shift, apply_gelu, out,
                                         row_order, n, c_in, c_out, ksize, keys, vals, cap_mask, cells, status,
                                         wt, stream);
    return launch_conv_direct_mma(feat, indices, weight, bias, bn_scale, bn_shift, apply_gelu, out, row_order, n,
                                  c_in, c_out, ksize, keys, vals, cap_mask, cells, status, wt, stream);
}
