// Integer bookkeeping of the hierarchy: the patch padding plan of serialized
// attention and the cluster / pooled-order plan of serialized pooling.
//
// Replaces model.py:382-438 (get_padding_and_inverse) and the index part of
// model.py:639-695 (unique / sort / cumsum / argsort / scatter_ of
// SerializedPooling.forward).  Pooled orders need no sort: children of a parent
// cell are contiguous in every order, so the pooled order of row r is the
// cluster id sequence along the fine order of row r with repeats removed.
#include "common.cuh"
#include "scan.cuh"
#include "../../include/ptv3_b200.h"

namespace ptv3 {

// ----------------------------------------------------------------------------
// padding plan
// ----------------------------------------------------------------------------
constexpr int PAD_MAX_SCENES = 4096;

__global__ void __launch_bounds__(256) pad_plan_kernel(const int64_t* __restrict__ offset, int B,
                                                       int K, int64_t n, int64_t n_pad, int n_seq,
                                                       int64_t* __restrict__ pad,
                                                       int64_t* __restrict__ unpad,
                                                       int32_t* __restrict__ cu_seqlens,
                                                       uint32_t* __restrict__ status)
{
    extern __shared__ int64_t sm[];
    int64_t* off = sm;                  // B + 1, unpadded scene starts
    int64_t* off_pad = sm + (B + 1);    // B + 1, padded scene starts
    int64_t* seq0 = sm + 2 * (B + 1);   // B + 1, first sequence of each scene
    if (threadIdx.x == 0) {
        off[0] = 0;
        off_pad[0] = 0;
        seq0[0] = 0;
        for (int s = 0; s < B; ++s) {
            const int64_t end = offset[s];
            const int64_t c = end - off[s];
            const int64_t cp = c > K ? (c + K - 1) / K * K : c;   // model.py:394-404
            off[s + 1] = end;
            off_pad[s + 1] = off_pad[s] + cp;
            seq0[s + 1] = seq0[s] + (cp + K - 1) / K;
        }
        if (blockIdx.x == 0 && (off[B] != n || off_pad[B] != n_pad || seq0[B] != n_seq))
            atomicOr(status, PTV3_STATUS_BAD_INDEX);
    }
    __syncthreads();
    if (off[B] != n || off_pad[B] != n_pad || seq0[B] != n_seq) return;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < n_pad; p += stride) {
        int lo = 0, hi = B;  // last s with off_pad[s] <= p
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (off_pad[mid] <= p) lo = mid; else hi = mid;
        }
        // scenes without points have equal starts; the search lands on the last one
        const int s = lo;
        const int64_t j = p - off_pad[s];
        const int64_t c = off[s + 1] - off[s];
        // tail of the last patch re-uses the ranks one patch earlier (model.py:412-423)
        pad[p] = off[s] + (j < c ? j : j - K);
        if (j < c) unpad[off[s] + j] = p;                          // model.py:411
        if (j % K == 0) cu_seqlens[seq0[s] + j / K] = (int32_t)p;  // model.py:424-432
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) cu_seqlens[n_seq] = (int32_t)n_pad;
}

// ----------------------------------------------------------------------------
// pooling plan
// ----------------------------------------------------------------------------
struct RowPerm {
    int src[PTV3_MAX_ORDERS];
};

// flag: first element of a cluster along order row 0
struct ClusterFlag {
    const int64_t* code0;
    const int64_t* order0;
    int shift;
    __device__ bool operator()(int, int64_t j) const
    {
        if (j == 0) return true;
        return (code0[order0[j]] >> shift) != (code0[order0[j - 1]] >> shift);
    }
};

struct ClusterSink {
    const int64_t* code;    // k x n
    const int64_t* order0;
    const int32_t* grid;    // n x 3
    const int64_t* batch;
    int64_t n;
    int k, shift, pooling_depth;
    RowPerm perm;
    int64_t* cluster;       // n
    int64_t* idx_ptr;       // cap + 1
    int64_t* head;          // cap
    int64_t* pcode;         // k x m, packed: the row stride is the cluster count, read from `total`
    int32_t* pgrid;         // cap x 3
    int64_t* pbatch;        // cap
    const uint32_t* total;  // number of clusters (written by the scan of the tile sums)
    unsigned long long* scene_count;  // B
    __device__ void operator()(int, int64_t j, uint32_t pos, bool f) const
    {
        const int64_t p = order0[j];
        const int64_t cid = (int64_t)pos + (f ? 1 : 0) - 1;
        cluster[p] = cid;
        if (f) {
            idx_ptr[cid] = j;
            head[cid] = p;
            for (int r = 0; r < k; ++r)
                pcode[(int64_t)r * (int64_t)*total + cid] = code[(int64_t)perm.src[r] * n + p] >> shift;
            pgrid[3 * cid + 0] = grid[3 * p + 0] >> pooling_depth;
            pgrid[3 * cid + 1] = grid[3 * p + 1] >> pooling_depth;
            pgrid[3 * cid + 2] = grid[3 * p + 2] >> pooling_depth;
            const int64_t b = batch[p];
            pbatch[cid] = b;
            // one atomic per scene and warp instead of one per cluster: the lanes that reached
            // this point with the same scene elect a leader (clusters of a warp mostly share it)
            const unsigned peers = __match_any_sync(__activemask(), (unsigned long long)b);
            if ((int)(threadIdx.x & 31) == __ffs(peers) - 1)
                atomicAdd(&scene_count[b], (unsigned long long)__popc(peers));
        }
    }
};

// flag: cluster id changes along the fine order of (source) row r
struct OrderFlag {
    const int64_t* order;    // k x n
    const int64_t* cluster;  // n
    int64_t n;
    RowPerm perm;
    __device__ bool operator()(int r, int64_t j) const
    {
        if (j == 0) return true;
        const int64_t* o = order + (int64_t)perm.src[r] * n;
        return cluster[o[j]] != cluster[o[j - 1]];
    }
};

struct OrderSink {
    const int64_t* order;
    const int64_t* cluster;
    int64_t n;
    const uint32_t* total;   // number of clusters = row stride of the packed outputs
    RowPerm perm;
    int64_t* porder;    // k x m, packed
    int64_t* pinverse;  // k x m, packed
    __device__ void operator()(int r, int64_t j, uint32_t pos, bool f) const
    {
        if (!f) return;
        const int64_t c = cluster[order[(int64_t)perm.src[r] * n + j]];
        const int64_t m = (int64_t)*total;
        porder[(int64_t)r * m + pos] = c;
        pinverse[(int64_t)r * m + c] = pos;
    }
};

__global__ void pool_meta_kernel(const uint32_t* __restrict__ totals, int k, int64_t n, int B,
                                 const unsigned long long* __restrict__ scene_count,
                                 int64_t* __restrict__ idx_ptr, int64_t* __restrict__ meta,
                                 int64_t* __restrict__ meta_host, uint32_t* __restrict__ status)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int64_t m = totals[0];
        idx_ptr[m] = n;
        meta[0] = m;
        for (int r = 1; r <= k; ++r)
            if ((int64_t)totals[r] != m) atomicOr(status, PTV3_STATUS_BAD_INDEX);
        for (int b = 0; b < B; ++b) meta[1 + b] = (int64_t)scene_count[b];
        if (meta_host) {
            // the same numbers and the status word, stored straight into the caller's mapped host
            // memory: the host reads them after waiting for the stream, with no copy in between
            // (a copy would queue behind whatever else the copy engine is busy with)
            for (int b = 0; b <= B; ++b) meta_host[b] = meta[b];
            meta_host[1 + B] = (int64_t)*reinterpret_cast<volatile uint32_t*>(status);
            __threadfence_system();
            // "everything above has been stored": a host that zeroed this word before the call may
            // poll it instead of waiting for the stream
            *reinterpret_cast<volatile int64_t*>(&meta_host[2 + B]) = 1;
            __threadfence_system();
        }
    }
}

struct PoolWs {
    int ntiles;
    size_t bytes;
};
static PoolWs pool_ws(int k, int64_t n, int B)
{
    PoolWs w;
    w.ntiles = ceil_div(n, SC_TILE);
    w.bytes = align_up((size_t)(k + 1) * w.ntiles * sizeof(uint32_t), 256) +
              align_up((size_t)(k + 1) * sizeof(uint32_t), 256) +
              align_up((size_t)B * sizeof(unsigned long long), 256);
    return w;
}

// ----------------------------------------------------------------------------
// batch index of every point from the scene offsets, and the (batch, x, y, z) rows
// of the sparse tensor (model.py:35-40 and :150-152)
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) batch_indices_kernel(const int64_t* __restrict__ offset, int B,
                                                            const int32_t* __restrict__ grid_coord, int64_t n,
                                                            int64_t* __restrict__ batch,
                                                            int32_t* __restrict__ indices)
{
    extern __shared__ int64_t sm[];      // B scene ends
    for (int s = threadIdx.x; s < B; s += blockDim.x) sm[s] = offset[s];
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        int lo = 0, hi = B - 1;          // first scene whose end lies beyond i (the last one at worst)
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (sm[mid] > i) hi = mid; else lo = mid + 1;
        }
        if (batch) batch[i] = lo;
        if (indices)
            reinterpret_cast<int4*>(indices)[i] =
                make_int4(lo, grid_coord[3 * i], grid_coord[3 * i + 1], grid_coord[3 * i + 2]);
    }
}

}  // namespace ptv3

extern "C" int ptv3_batch_indices(const int64_t* offset, int n_scenes, const int32_t* grid_coord, int64_t n,
                                  int64_t* batch, int32_t* indices, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n_scenes >= 1 && n_scenes <= PAD_MAX_SCENES, PTV3_ERR_UNSUPPORTED,
                 "ptv3_batch_indices: %d scenes outside [1, %d]", n_scenes, PAD_MAX_SCENES);
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_batch_indices: n < 0");
    if (n == 0 || (!batch && !indices)) return PTV3_OK;
    PTV3_REQUIRE(offset && (!indices || grid_coord), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_batch_indices: null pointer");
    PTV3_REQUIRE(((uintptr_t)indices & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_batch_indices: indices must be 16-byte aligned");
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    batch_indices_kernel<<<(unsigned)blocks, 256, (size_t)n_scenes * sizeof(int64_t), (cudaStream_t)stream>>>(
        offset, n_scenes, grid_coord, n, batch, indices);
    count_launches(1);
    return check_launch("ptv3_batch_indices");
}

extern "C" int ptv3_pad_plan(const int64_t* offset, int n_scenes, int patch, int64_t n, int64_t n_pad,
                             int n_seq, int64_t* pad, int64_t* unpad, int32_t* cu_seqlens,
                             uint32_t* status, void* stream)
{
    using namespace ptv3;
    PTV3_REQUIRE(n_scenes >= 1 && n_scenes <= PAD_MAX_SCENES, PTV3_ERR_UNSUPPORTED,
                 "ptv3_pad_plan: %d scenes outside [1, %d]", n_scenes, PAD_MAX_SCENES);
    PTV3_REQUIRE(patch >= 1 && n >= 0 && n_pad >= n && n_seq >= 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_pad_plan: bad sizes");
    PTV3_REQUIRE(offset && cu_seqlens && status && (n_pad == 0 || (pad && unpad)),
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_pad_plan: null pointer");
    int64_t blocks = (n_pad + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    const size_t smem = 3 * (size_t)(n_scenes + 1) * sizeof(int64_t);
    pad_plan_kernel<<<(unsigned)blocks, 256, smem, (cudaStream_t)stream>>>(
        offset, n_scenes, patch, n, n_pad, n_seq, pad, unpad, cu_seqlens, status);
    count_launches(1);
    return check_launch("ptv3_pad_plan");
}

extern "C" size_t ptv3_pool_plan_workspace_bytes(int k, int64_t n, int n_scenes)
{
    if (k <= 0 || n <= 0 || n_scenes <= 0) return 0;
    return ptv3::pool_ws(k, n, n_scenes).bytes;
}

extern "C" int ptv3_pool_plan(const int64_t* code, const int64_t* order, const int32_t* grid_coord,
                              const int64_t* batch, int k, int64_t n, int n_scenes,
                              int pooling_depth, const int* row_perm, int64_t* cluster,
                              int64_t* idx_ptr, int64_t* head, int64_t* pooled_code,
                              int64_t* pooled_order, int64_t* pooled_inverse,
                              int32_t* pooled_grid_coord, int64_t* pooled_batch, int64_t* meta,
                              int64_t* meta_host, uint32_t* status, void* workspace,
                              size_t workspace_bytes, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(k >= 1 && k <= PTV3_MAX_ORDERS && n >= 1 && n_scenes >= 1,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_plan: bad k/n/n_scenes");
    PTV3_REQUIRE(pooling_depth >= 0 && pooling_depth <= 16, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_pool_plan: bad pooling_depth");
    PTV3_REQUIRE(n < (1ll << 31), PTV3_ERR_UNSUPPORTED, "ptv3_pool_plan: n too large");
    PTV3_REQUIRE(code && order && grid_coord && batch && cluster && idx_ptr && head && pooled_code &&
                     pooled_order && pooled_inverse && pooled_grid_coord && pooled_batch && meta &&
                     status && workspace,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_plan: null pointer");
    const PoolWs w = pool_ws(k, n, n_scenes);
    PTV3_REQUIRE(workspace_bytes >= w.bytes, PTV3_ERR_WORKSPACE,
                 "ptv3_pool_plan: workspace %zu < %zu bytes", workspace_bytes, w.bytes);
    cudaStream_t stream = (cudaStream_t)stream_;
    Carver cv(workspace);
    uint32_t* tile_sums = cv.take<uint32_t>((size_t)(k + 1) * w.ntiles);
    uint32_t* totals = cv.take<uint32_t>(k + 1);
    unsigned long long* scene_count = cv.take<unsigned long long>(n_scenes);
    cudaMemsetAsync(scene_count, 0, (size_t)n_scenes * sizeof(unsigned long long), stream);

    RowPerm perm;
    for (int r = 0; r < PTV3_MAX_ORDERS; ++r) perm.src[r] = r < k ? (row_perm ? row_perm[r] : r) : 0;
    for (int r = 0; r < k; ++r)
        PTV3_REQUIRE(perm.src[r] >= 0 && perm.src[r] < k, PTV3_ERR_INVALID_ARGUMENT,
                     "ptv3_pool_plan: row_perm[%d] = %d outside [0, %d)", r, perm.src[r], k);

    const int shift = 3 * pooling_depth;
    // clusters along row 0 of the caller's (already shuffled) rows
    ClusterFlag cf{code, order, shift};
    ClusterSink cs{code, order, grid_coord, batch, n, k, shift, pooling_depth, perm, cluster, idx_ptr,
                   head, pooled_code, pooled_grid_coord, pooled_batch, totals, scene_count};
    scan_tile_sums_kernel<<<dim3(w.ntiles, 1), SC_THREADS, 0, stream>>>(cf, n, w.ntiles, tile_sums);
    scan_sums_kernel<<<1, SC_THREADS, 0, stream>>>(tile_sums, w.ntiles, totals);
    scan_apply_kernel<<<dim3(w.ntiles, 1), SC_THREADS, 0, stream>>>(cf, cs, n, w.ntiles, tile_sums);
    // pooled orders of the k (permuted) rows
    uint32_t* ts2 = tile_sums + w.ntiles;
    OrderFlag of{order, cluster, n, perm};
    OrderSink os{order, cluster, n, totals, perm, pooled_order, pooled_inverse};
    scan_tile_sums_kernel<<<dim3(w.ntiles, k), SC_THREADS, 0, stream>>>(of, n, w.ntiles, ts2);
    scan_sums_kernel<<<k, SC_THREADS, 0, stream>>>(ts2, w.ntiles, totals + 1);
    scan_apply_kernel<<<dim3(w.ntiles, k), SC_THREADS, 0, stream>>>(of, os, n, w.ntiles, ts2);
    pool_meta_kernel<<<1, 32, 0, stream>>>(totals, k, n, n_scenes, scene_count, idx_ptr, meta, meta_host, status);
    count_launches(7);
    return check_launch("ptv3_pool_plan");
}
