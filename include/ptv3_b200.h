/*
 * C ABI of libptv3_b200: hand-written sm_100a kernels for the inference path of
 * Point Transformer V3 (serialization, patch attention, submanifold
 * convolution, pooling).  This is the boundary the Python host code binds with
 * ctypes; it is also what any other host language would bind.
 *
 * Conventions
 *   - every function returns 0 on success or a negative PTV3_ERR_* code;
 *     ptv3_last_error() returns a thread-local description of the last failure
 *   - all pointers are DEVICE pointers unless a parameter says "host"
 *   - the library never allocates or frees device memory: outputs and
 *     workspaces are passed in; *_workspace_bytes() gives the size to pass
 *   - `stream` is a cudaStream_t passed as void*; no call synchronises
 *   - index tensors exposed to callers are int64 (as the reference's are)
 *   - the kernels of the feature path (convolution, Linear / GEMM, LayerNorm,
 *     attention, MLP, pooling) are launched with the programmatic-serialization
 *     attribute: a kernel of this library may be brought up while the kernel
 *     before it in the stream is finishing, and waits (griddepcontrol.wait) before
 *     it reads or writes anything but its weights and parameters.  Stream order is
 *     unchanged for the caller: work queued before or after a call, this
 *     library's or not, sees the same results as with plain launches.  Weights,
 *     biases and normalisation parameters must not be written by the operation
 *     queued directly before a call that reads them
 *
 * "Replaces" lines cite the reference implementation by its path inside the
 * reference project.
 */
#ifndef PTV3_B200_H
#define PTV3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTV3_MAX_ORDERS 8

/* order ids, serialization/default.py:10 */
#define PTV3_ORDER_Z 0
#define PTV3_ORDER_Z_TRANS 1
#define PTV3_ORDER_HILBERT 2
#define PTV3_ORDER_HILBERT_TRANS 3

/* element types of feature tensors */
#define PTV3_DTYPE_F32 0
#define PTV3_DTYPE_BF16 1

/* status codes */
#define PTV3_OK 0
#define PTV3_ERR_INVALID_ARGUMENT (-1)
#define PTV3_ERR_UNSUPPORTED (-2)
#define PTV3_ERR_WORKSPACE (-3)
#define PTV3_ERR_CUDA (-4)
#define PTV3_ERR_DEVICE_STATUS (-5)

/* bits kernels OR into a caller-provided device status word instead of trapping */
#define PTV3_STATUS_BAD_INDEX 1u
#define PTV3_STATUS_PROBE_LIMIT 2u
#define PTV3_STATUS_WAIT_LIMIT 4u

const char* ptv3_last_error(void);
int ptv3_version(void);
/* kernels launched by this library in this process so far */
long long ptv3_launch_count(void);
/* clears a device status word in stream order (a memset, not a kernel) */
int ptv3_status_reset(uint32_t* status, void* stream);

/*
 * Space-filling-curve codes.
 * Replaces serialization/default.py:8-24 (encode), z_order.py:66-101 (xyz2key),
 * hilbert.py:91-198 (encode).
 *   grid_coord  n x 3 int32, row-major; only the low `depth` bits are used
 *   batch       n int64 scene ids, or NULL (no batch bits)
 *   orders      HOST array of n_orders order ids, one per output row
 *   codes       n_orders x n int64, row r = order orders[r];
 *               code = batch << 3*depth | curve(x, y, z)
 */
int ptv3_encode(const int32_t* grid_coord, const int64_t* batch, int64_t n, int depth,
                const int* orders, int n_orders, int64_t* codes, void* stream);

/*
 * Inverse of ptv3_encode for the orders PTV3_ORDER_Z and PTV3_ORDER_HILBERT.
 * Replaces serialization/default.py:27-38 (decode), z_order.py:104-126 (key2xyz),
 * hilbert.py:201-303 (decode).  (The reference's z-order wrapper, default.py:48-51,
 * fails on its own return value; this is what it is meant to return.)
 *   grid_coord  n x 3 int64; batch  n int64 (code >> 3*depth) or NULL
 */
int ptv3_decode(const int64_t* codes, int64_t n, int depth, int order, int64_t* grid_coord, int64_t* batch,
                void* stream);

/*
 * Stable argsort of every code row and its inverse permutation.
 * Replaces model.py:118-126 (torch.argsort + scatter_) and :667-674.
 *   codes     k x n int64, non-negative, nothing set above bit sig_bits-1
 *   order     k x n int64: codes[r][order[r][j]] is non-decreasing in j, ties
 *             by ascending index
 *   inverse   k x n int64: inverse[r][order[r][j]] = j
 *   status    one uint32 or NULL: the tiles of a pass wait for the tiles before them
 *             (bounded); a wait that ran out ORs PTV3_STATUS_WAIT_LIMIT into it and the
 *             outputs are then undefined
 * n is limited to 2^28 - 1 elements per row.
 */
size_t ptv3_argsort_workspace_bytes(int k, int64_t n, int sig_bits);
int ptv3_argsort_inverse(const int64_t* codes, int k, int64_t n, int sig_bits, int64_t* order,
                         int64_t* inverse, uint32_t* status, void* workspace, size_t workspace_bytes,
                         void* stream);

/*
 * The scene index of every point and the (batch, x, y, z) rows of the sparse tensor,
 * from the scene offsets.  Replaces offset2batch (model.py:35-40) and the concatenation
 * of Point.sparsify (model.py:150-152).
 *   offset      n_scenes int64 (device): cumulative point counts, offset[last] = n
 *   grid_coord  n x 3 int32 (needed only with `indices`)
 *   batch       n int64 out, or NULL
 *   indices     n x 4 int32 out (16-byte aligned), or NULL
 */
int ptv3_batch_indices(const int64_t* offset, int n_scenes, const int32_t* grid_coord, int64_t n,
                       int64_t* batch, int32_t* indices, void* stream);

/*
 * Patch padding plan of serialized attention.
 * Replaces model.py:382-438 (SerializedAttention.get_padding_and_inverse).
 * A scene with c > patch points is padded to a multiple of `patch`; the tail of
 * its last patch re-uses the ranks one patch earlier.
 *   offset      n_scenes int64, cumulative point counts
 *   n, n_pad, n_seq   totals the caller derived from the same offsets (checked
 *               on the device; a mismatch sets PTV3_STATUS_BAD_INDEX in *status
 *               and leaves the outputs unwritten)
 *   pad         n_pad int64: serialized rank feeding padded row p
 *   unpad       n int64: padded row owned by serialized rank j
 *   cu_seqlens  n_seq + 1 int32: first padded row of every patch, then n_pad
 *   status      one uint32, OR-ed with PTV3_STATUS_* bits (never cleared here)
 */
int ptv3_pad_plan(const int64_t* offset, int n_scenes, int patch, int64_t n, int64_t n_pad,
                  int n_seq, int64_t* pad, int64_t* unpad, int32_t* cu_seqlens, uint32_t* status,
                  void* stream);

/*
 * Patch attention core: out[p] = softmax(q k^T * scale) v within each patch.
 * Replaces model.py:452-484 (row gather qkv[order[pad]], non-flash attention
 * :458-474, gather feat[unpad[inverse]]); the two Linear layers stay outside.
 *   qkv         n x 3*channels, channel split (3, heads, head_dim) (model.py:461)
 *   order       n int64, ONE row of serialized_order
 *   pad, unpad, cu_seqlens   as written by ptv3_pad_plan
 *   out         n x channels, every row written exactly once
 *   max_seqlen  longest patch (rows); head_dim = channels / heads in {8,16,32,64}
 *   dtype       PTV3_DTYPE_*; algo 0 = automatic, 1 = CUDA-core path,
 *               2 = mma.sync tensor-core path (bf16, head_dim 16, max_seqlen
 *               <= 2048; what "automatic" takes when it applies), 3 = the same
 *               with the exponent arguments rounded to bf16 and two exps per
 *               instruction (measured no faster on B200: the exp unit's rate
 *               per element is the same; kept for comparison), 4 = tcgen05 /
 *               tensor-memory path (bf16, head_dim 16, max_seqlen <= 1024,
 *               needs `status`; measured 40 % slower than 2 on B200: at head
 *               dimension 16 the tensor pipe is bound by the number of tiny
 *               products, not by their arithmetic)
 *   status      one uint32 or NULL.  Every path ORs PTV3_STATUS_BAD_INDEX into it
 *               when cu_seqlens holds a patch longer than max_seqlen (that patch is
 *               skipped, its output rows stay unwritten; with NULL it is skipped
 *               silently); path 4 also ORs PTV3_STATUS_WAIT_LIMIT when one of its
 *               bounded waits ran out (the output is then undefined)
 */
int ptv3_attention_fwd(const void* qkv, const int64_t* order, const int64_t* pad,
                       const int64_t* unpad, const int32_t* cu_seqlens, void* out, int64_t n,
                       int n_seq, int max_seqlen, int channels, int heads, float scale, int dtype,
                       int algo, uint32_t* status, void* stream);

/*
 * ptv3_attention_fwd with the relative position bias of model.py:297-316, 372-380,
 * 468-469 added to the scaled scores (CUDA-core path, either dtype):
 *   bias(i, j, h) = sum over axes a of
 *                   rpe_table[clamp(g_i[a] - g_j[a], -pos_bnd, pos_bnd) + pos_bnd + a * (2 pos_bnd + 1)][h]
 *   grid_coord  n x 3 int32 (point-major, like qkv)
 *   rpe_table   3 * (2 pos_bnd + 1) x heads fp32; pos_bnd <= 64
 */
int ptv3_attention_rpe_fwd(const void* qkv, const int64_t* order, const int64_t* pad,
                           const int64_t* unpad, const int32_t* cu_seqlens, const int32_t* grid_coord,
                           const float* rpe_table, int pos_bnd, void* out, int64_t n, int n_seq,
                           int max_seqlen, int channels, int heads, float scale, int dtype, void* stream);

/*
 * Kernel map of a submanifold convolution.
 * Replaces spconv's indice-pair build behind model.py:546-552 and :767-774.
 *   indices     n x 4 int32 rows (batch, x, y, z), 16-byte aligned, each field
 *               in [0, 65535]
 *   nbr         ksize^3 x n int32, OFFSET-major: nbr[o][i] = row of the voxel at
 *               coordinate(i) + offset o, or -1; o = ((dx+r)*k + (dy+r))*k + (dz+r)
 *               with r = ksize/2.  Duplicate rows resolve to the lowest row.
 */
size_t ptv3_kmap_workspace_bytes(int64_t n);
int ptv3_kmap_build(const int32_t* indices, int64_t n, int ksize, int32_t* nbr, uint32_t* status,
                    void* workspace, size_t workspace_bytes, void* stream);
/*
 * The same table with its columns in the order the convolution walks its tiles:
 * column p describes voxel row_order[p] (nbr[o][p] = row of the voxel at
 * coordinate(row_order[p]) + offset o; the stored rows keep the natural numbering).
 * This is ptv3_kmap_build followed by a permutation of the columns, without the
 * second pass over the table.  row_order: n int64, a permutation (the serialized
 * order of model.py:118-126 in the backbone), or NULL for the natural order.
 */
int ptv3_kmap_build_ordered(const int32_t* indices, int64_t n, int ksize, const int64_t* row_order,
                            int32_t* nbr, uint32_t* status, void* workspace, size_t workspace_bytes,
                            void* stream);

/*
 * ptv3_kmap_build for callers that cannot hand over a workspace because they
 * cannot allocate device memory at the point of the call: a plugin running
 * inside a host framework that owns the whole device heap, or a latency-bound
 * service loop where cudaMalloc (a device-wide synchronisation) is forbidden
 * after start-up.  This entry point has no counterpart in the reference.
 * The hash table lives in a static device array of the library (1.5 MiB on
 * every GPU that loads it, until the process exits), so
 *   - n is limited to ptv3_kmap_static_max_voxels() (65536); larger inputs are
 *     rejected with PTV3_ERR_UNSUPPORTED and the caller should fall back to
 *     ptv3_kmap_build
 *   - nothing is allocated or freed, here or in any library it calls
 *   - the first call on each device resolves the array's device address and caches
 *     it for the life of the process (the cache is atomic: first calls from several
 *     host threads are safe); make that first call outside any stream capture, and
 *     do not call cudaDeviceReset() afterwards, which would leave the cached
 *     address pointing into a context that no longer exists
 *   - all calls on a device share the one table (it is re-initialised at the
 *     start of each call, in stream order): two calls whose kernels may overlap
 *     on the GPU (different streams or threads) race and must be serialised by
 *     the caller
 * Inputs, outputs and `status` are as for ptv3_kmap_build and are still
 * provided by the caller.
 */
int64_t ptv3_kmap_static_max_voxels(void);
int ptv3_kmap_build_static(const int32_t* indices, int64_t n, int ksize, int32_t* nbr,
                           uint32_t* status, void* stream);

/*
 * Submanifold convolution over a kernel map:
 *   out[i] = bias + sum_o weight[:, o, :] . feat[nbr[o][i]]
 * Replaces spconv.SubMConv3d.forward at model.py:546-552 and :767-774.
 *   weight      c_out x kernel_volume x c_in (the [C_out, k, k, k, C_in] layout)
 *   bias        c_out or NULL
 *   row_order   n int64 permutation of the voxels or NULL: the order in which
 *               voxels are grouped into tiles (a serialized order makes a tile
 *               spatially compact).  When given, column j of nbr must describe
 *               voxel row_order[j], i.e. nbr = kernel_map[:, row_order]; the
 *               result is the same as without it
 *   algo        0 = automatic, 1 = CUDA-core path, 2 = mma.sync tensor-core path,
 *               3 = tcgen05 path (bf16, at most 27 offsets, channels 32 -> 32 or
 *               multiples of 64; accumulates every offset of a tile in tensor memory
 *               in a fixed order, so the result is the same bit for bit on every run)
 *   status      one device word, zeroed by the caller; the tcgen05 path sets
 *               PTV3_STATUS_WAIT_LIMIT in it if a device wait runs out.  May be NULL,
 *               in which case the tcgen05 path is not used
 */
int ptv3_subm_conv_fwd(const void* feat, const int32_t* nbr, const void* weight, const void* bias,
                       void* out, const int64_t* row_order, int64_t n, int c_in, int c_out,
                       int kernel_volume, int dtype, int algo, uint32_t* status, void* stream);

/*
 * Pair-list form of the submanifold convolution, for levels with few voxels and
 * wide channels (the tensor-core path of ptv3_subm_conv_fwd multiplies a tile of
 * output voxels by every offset that any of them has; on coarse levels most of
 * those rows are zero).  ptv3_conv_pairs_build lists, offset by offset, the pairs
 * (nbr[o][j], j) with nbr[o][j] >= 0; ptv3_subm_conv_pairs_fwd multiplies 128
 * pairs of one offset at a time and accumulates with atomics in 64-bit fixed
 * point (32 fractional bits): integer sums do not depend on the order of the
 * additions, so the result is the same bit for bit on every run.
 * Replaces spconv's gather-GEMM-scatter behind model.py:546-552.
 *   nbr, row_order   as for ptv3_subm_conv_fwd (pair_out = row_order[j] when given)
 *   pair_in/out      kernel_volume * n int32 each (upper bound)
 *   off_start, tile_start   kernel_volume + 1 int32 each (device)
 *   workspace (conv) n x c_out 64-bit integers (8 bytes each)
 */
size_t ptv3_conv_pairs_workspace_bytes(int64_t n, int kernel_volume);
int ptv3_conv_pairs_build(const int32_t* nbr, const int64_t* row_order, int64_t n, int kernel_volume,
                          int32_t* pair_in, int32_t* pair_out, int32_t* off_start, int32_t* tile_start,
                          void* workspace, size_t workspace_bytes, void* stream);
int ptv3_subm_conv_pairs_fwd(const void* feat, const int32_t* pair_in, const int32_t* pair_out,
                             const int32_t* off_start, const int32_t* tile_start, const void* weight,
                             const void* bias, void* out, void* workspace, size_t workspace_bytes,
                             int64_t n, int c_in, int c_out, int kernel_volume, int dtype, void* stream);

/*
 * Submanifold convolution with few input channels and a large kernel, without a
 * kernel map: the voxel hash table is built in `workspace` and probed inside
 * the convolution.  Replaces the stem of model.py:766-779 (SubMConv3d 5x5x5,
 * bias=False) and, optionally, the BatchNorm1d(eval) + GELU that follow it
 * (model.py:776-779).
 *   indices     n x 4 int32 (batch, x, y, z) as for ptv3_kmap_build
 *   weight      c_out x ksize^3 x c_in; ksize in {1, 3, 5}; c_in <= 8; c_out in {16, 32, 48, 64}
 *   bias        c_out or NULL; bn_scale/bn_shift fp32 per channel or both NULL
 *   apply_gelu  non-zero: exact GELU after the (optional) normalisation
 *   row_order   optional voxel permutation used to group voxels into tiles
 */
size_t ptv3_subm_conv_direct_workspace_bytes(int64_t n, int ksize);
int ptv3_subm_conv_direct_fwd(const void* feat, const int32_t* indices, const void* weight,
                              const void* bias, const float* bn_scale, const float* bn_shift,
                              int apply_gelu, void* out, const int64_t* row_order, int64_t n, int c_in,
                              int c_out, int ksize, int dtype, uint32_t* status, void* workspace,
                              size_t workspace_bytes, void* stream);

/*
 * Cluster and order bookkeeping of serialized pooling.
 * Replaces the index part of model.py:639-695 (unique, sort, cumsum, head
 * gather, argsort + scatter_ of the pooled codes, row shuffle).
 *   code, order k x n int64 rows of the fine level, in its current row order
 *   row_perm    HOST array of k ints or NULL: pooled row r is built from fine
 *               row row_perm[r] (the reference's code[perm], model.py:676-680)
 *   cluster     n int64: rank of (code[0] >> 3*pooling_depth) among its unique
 *               values (= pooling_inverse)
 *   idx_ptr     n + 1 int64 (m + 1 used): run starts of the clusters in order[0]
 *   head        n int64 (m used): one member point of every cluster
 *   pooled_*    outputs sized for m = n; the k-row tensors (code, order, inverse)
 *               are written packed, k x m with row stride m, at the start of
 *               their k x n buffers, so that a view of the first k * m
 *               elements is the contiguous result
 *   meta        1 + n_scenes int64: m, then the number of clusters per scene
 *   meta_host   NULL, or 3 + n_scenes int64 of page-locked HOST memory that the
 *               device can address (cudaHostAlloc / a pinned torch tensor): the last
 *               kernel stores meta, then the status word, then the value 1 there, so
 *               the host can read them without a device-to-host copy, either after
 *               waiting for the stream or by zeroing the last word before the call
 *               and polling it
 */
size_t ptv3_pool_plan_workspace_bytes(int k, int64_t n, int n_scenes);
int ptv3_pool_plan(const int64_t* code, const int64_t* order, const int32_t* grid_coord,
                   const int64_t* batch, int k, int64_t n, int n_scenes, int pooling_depth,
                   const int* row_perm, int64_t* cluster, int64_t* idx_ptr, int64_t* head,
                   int64_t* pooled_code, int64_t* pooled_order, int64_t* pooled_inverse,
                   int32_t* pooled_grid_coord, int64_t* pooled_batch, int64_t* meta,
                   int64_t* meta_host, uint32_t* status, void* workspace, size_t workspace_bytes,
                   void* stream);

/*
 * Segment reduction over clusters (reduce: 0 max, 1 min, 2 sum, 3 mean, as
 * torch_scatter.segment_csr's `reduce`) fused with BatchNorm(eval) + GELU, and the mean
 * coordinate.  Replaces torch_scatter.segment_csr at model.py:684-689 and the
 * norm/act at model.py:707-710.
 *   x           (points) x channels, already projected (model.py:685)
 *   indices     points sorted by cluster (order[0] of the fine level)
 *   bn_scale/shift   per-channel fp32 (weight/sqrt(var+eps), bias-mean*scale),
 *               or both NULL for a plain max
 *   coord/coord_out  fp32 x 3, or NULL to skip the mean
 */
int ptv3_pool_fwd(const void* x, const float* coord, const int64_t* indices, const int64_t* idx_ptr,
                  int64_t m, int channels, const float* bn_scale, const float* bn_shift, void* out,
                  float* coord_out, int reduce, int dtype, void* stream);

/*
 * out[i] = GELU(BN(skip[i])) + GELU(BN(child[cluster[i]])); skip_act (optional)
 * receives the first term alone.  Replaces model.py:726-735,744-746 after the
 * two Linear layers.
 */
int ptv3_unpool_fwd(const void* skip, const void* child, const int64_t* cluster, int64_t n,
                    int channels, const float* skip_scale, const float* skip_shift,
                    const float* child_scale, const float* child_shift, void* out, void* skip_act,
                    int dtype, void* stream);

/*
 * Residual + LayerNorm glue between the GEMMs of a block, one pass over the rows:
 *     t   = ln1 given ? LayerNorm(x; ln1) : x
 *     sum = residual given ? residual + t : t      -> sum_out  (optional)
 *     y   = LayerNorm(sum; ln2)                    -> norm_out (with ln2 only)
 * Replaces the LayerNorm modules and residual additions of Block.forward
 * (model.py:553-554, 589-592, 594, 598-600, 602).  All tensors n x channels in
 * `dtype`; LayerNorm weights and biases have `dtype` too.  channels / (16 bytes
 * worth of elements) must be a power of two or three times one.
 */
int ptv3_add_layernorm_fwd(const void* x, const void* residual, const void* ln1_weight,
                           const void* ln1_bias, float ln1_eps, void* sum_out, const void* ln2_weight,
                           const void* ln2_bias, float ln2_eps, void* norm_out, int64_t n, int channels,
                           int dtype, void* stream);

/*
 * Fused MLP of a block: out = residual + fc2(GELU(fc1(x) + b1)) + b2, the hidden
 * activation kept on chip (tcgen05 tensor cores, TMEM accumulators, TMA loads).
 * Replaces MLP.forward and the residual addition, model.py:510-516, 601-602.
 *   x, residual, out   n x channels bf16 (out may alias residual)
 *   fc1_weight  hidden x channels, fc2_weight  channels x hidden (nn.Linear layout)
 * ptv3_mlp_supported() tells whether a shape is covered (bf16, channels 32 or 64,
 * hidden = 4 x channels); other shapes use separate GEMMs.
 * A wait that exceeds its bound sets PTV3_STATUS_WAIT_LIMIT in *status.
 */
int ptv3_mlp_supported(int channels, int hidden, int dtype);
int ptv3_mlp_fwd(const void* x, const void* fc1_weight, const void* fc1_bias, const void* fc2_weight,
                 const void* fc2_bias, const void* residual, void* out, int64_t n, int channels,
                 int hidden, int dtype, uint32_t* status, void* stream);

/*
 * Linear layers of a block on the tcgen05 tensor cores (bf16, input width k in
 * {32, 64, 128}), weight in nn.Linear layout (n_out x k).
 *   ptv3_linear_fwd      out = x W^T + b, n_out a multiple of 32 up to 384.
 *                        Replaces the qkv projection, model.py:456.
 *   ptv3_linear_ln_fwd   y = x W^T + b (square, channels = k);
 *                        t = LayerNorm(y; ln1) if ln1 given else y;
 *                        sum_out = residual + t;  norm_out = LayerNorm(sum_out; ln2).
 *                        Replaces cpe.1 + cpe.2 + shortcut + norm1 (model.py:553-554,
 *                        589-592) and attn.proj + shortcut + norm2 (model.py:487, 594,
 *                        598-600).  sum_out may be NULL; it may alias residual.
 * ptv3_linear_supported() tells whether a shape is covered; wider layers use
 * ptv3_gemm_fwd followed by ptv3_add_layernorm_fwd.
 */
int ptv3_linear_supported(int k, int n_out, int residual_mode, int dtype);
/*
 * Linear layer with streamed weights on the tcgen05 tensor cores, for the widths
 * ptv3_linear_fwd does not take (bf16, k a multiple of 64, n_out a multiple of 128):
 *   out = [residual +] act(x W^T + b),  act = exact GELU if `gelu` else identity
 * with the roundings of the unfused sequence (the GEMM result is rounded to bf16
 * before GELU / the residual sum, which is rounded again).
 * Replaces nn.Linear in the blocks of the 256- and 512-channel levels (model.py:456,
 * 487, 553), MLP.forward with its residual for 128 channels and more (model.py:510-516,
 * 601-602: fc1 with gelu = 1, fc2 with the residual), and the pooling / unpooling
 * projections (model.py:684, 726-735).
 *   x  n x k;  weight  n_out x k (nn.Linear layout);  bias  n_out or NULL;
 *   residual  n x n_out or NULL (may alias out);  all 16-byte aligned
 * A wait that exceeds its bound sets PTV3_STATUS_WAIT_LIMIT in *status.
 */
int ptv3_gemm_supported(int k, int n_out, int dtype);
int ptv3_gemm_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* out,
                  int64_t n, int k, int n_out, int gelu, int dtype, uint32_t* status, void* stream);
int ptv3_linear_fwd(const void* x, const void* weight, const void* bias, void* out, int64_t n, int k,
                    int n_out, int dtype, uint32_t* status, void* stream);
int ptv3_linear_ln_fwd(const void* x, const void* weight, const void* bias, const void* residual,
                       const void* ln1_weight, const void* ln1_bias, float ln1_eps, void* sum_out,
                       const void* ln2_weight, const void* ln2_bias, float ln2_eps, void* norm_out,
                       int64_t n, int channels, int dtype, uint32_t* status, void* stream);

/*
 * One transformer block in one call (model.py:519-606, Block.forward, inference,
 * pre-norm, bf16): xCPE convolution + Linear + LayerNorm, attention with its two
 * Linear layers, MLP, the three residual additions.  The same kernels as the
 * single-operator entry points, queued from C++ so that a block costs the host
 * one call; widths up to 128 use ptv3_linear_ln_fwd / ptv3_linear_fwd (and ptv3_mlp_fwd
 * up to 64), wider ones ptv3_gemm_fwd with ptv3_add_layernorm_fwd; ptv3_block_supported
 * tells whether every layer of a block has a kernel.  All pointers are device pointers
 * except the struct.
 */
typedef struct ptv3_block_args {
    int64_t n;                      /* voxels of the level */
    int channels, heads, hidden;    /* hidden = MLP width */
    int dtype;                      /* PTV3_DTYPE_BF16 */
    int n_seq, max_seqlen;          /* patches, longest patch (as for ptv3_attention_fwd) */
    int attention_algo;             /* algo of ptv3_attention_fwd, 0 = automatic */
    float scale;                    /* attention scale */
    float cpe_ln_eps, n1_eps, n2_eps;
    const void* conv_in;            /* n x C rows the convolution reads (the sparse tensor's features) */
    const void* feat;               /* n x C residual stream entering the block */
    void* out;                      /* n x C result */
    /* convolution geometry: the kernel map (nbr, optional row_order) or, when pair_in is
       given, the pair list of ptv3_conv_pairs_build */
    const int32_t* nbr;
    const int64_t* row_order;
    const int32_t *pair_in, *pair_out, *off_start, *tile_start;
    /* attention geometry, as for ptv3_attention_fwd */
    const int64_t *order, *pad, *unpad;
    const int32_t* cu_seqlens;
    /* parameters, in the layouts of the reference's state_dict */
    const void *conv_weight, *conv_bias;      /* cpe.0 */
    const void *cpe_w, *cpe_b;                /* cpe.1 */
    const void *cpe_ln_w, *cpe_ln_b;          /* cpe.2 */
    const void *n1_w, *n1_b;                  /* norm1.0 */
    const void *qkv_w, *qkv_b;                /* attn.qkv */
    const void *proj_w, *proj_b;              /* attn.proj */
    const void *n2_w, *n2_b;                  /* norm2.0 */
    const void *fc1_w, *fc1_b, *fc2_w, *fc2_b; /* mlp.0.fc1 / fc2 */
    uint32_t* status;               /* device status word, OR-ed with PTV3_STATUS_* bits */
    void* workspace;                /* ptv3_block_workspace_bytes(args) bytes, 256-byte aligned */
    size_t workspace_bytes;
} ptv3_block_args;

int ptv3_block_supported(int channels, int heads, int hidden, int dtype);
/* reads n, channels, hidden, dtype and pair_in (null or not) of the argument block */
size_t ptv3_block_workspace_bytes(const ptv3_block_args* args);
int ptv3_block_fwd(const ptv3_block_args* args, void* stream);

/*
 * Voxelisation front end (the step before the backbone).
 *
 * ptv3_grid_coord: grid_coord = trunc((coord - min over all n points) / grid_size),
 * the derivation of model.py:88-96 / 156-158 (batch-global minimum, fp32
 * arithmetic, truncation toward zero).
 *   coord       n x 3 float32       origin   3 float32 (out: the minimum)
 *   grid_coord  n x 3 int32 (out)
 *
 * ptv3_voxel_dedup: keeps the first point (lowest row) of every occupied voxel
 * of every scene; kept rows stay in input order.  The reference leaves this to
 * its data pipeline (grid sampling); its submanifold convolutions assume it.
 *   indices      n x 4 int32 rows (scene, x, y, z), 16-byte aligned; scenes contiguous
 *   offset       n_scenes int64 cumulative point counts (may be NULL with n_scenes 0)
 *   keep         n int64 (out): rows kept, ascending; the first *count are valid
 *   point2voxel  n int64 (out): position in `keep` of the point's voxel
 *   new_offset   n_scenes int64 (out, optional): cumulative kept counts
 *   count        1 int64 (out): number of voxels
 */
int ptv3_grid_coord(const float* coord, int64_t n, float grid_size, float* origin, int32_t* grid_coord,
                    void* stream);
size_t ptv3_voxel_dedup_workspace_bytes(int64_t n);
int ptv3_voxel_dedup(const int32_t* indices, int64_t n, const int64_t* offset, int n_scenes, int64_t* keep,
                     int64_t* point2voxel, int64_t* new_offset, int64_t* count, uint32_t* status,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * Segmentation head (the step after the backbone; the reference file ends with the
 * backbone, model.py:966-982, and the head is the segmentor's Linear on
 * dec_channels[0]): logits = feat W^T + b and/or the per-point arg max in one pass.
 *   feat     n x channels (16-byte aligned rows)     weight  classes x channels, bias classes or NULL
 *   logits   n x classes in the feature dtype, or NULL
 *   labels   n int64 arg max of the (rounded) logits, lowest index on ties, or NULL
 * classes <= 64; channels a multiple of 4 (fp32) / 8 (bf16), up to 512.
 */
int ptv3_seg_head_fwd(const void* feat, const void* weight, const void* bias, void* logits, int64_t* labels,
                      int64_t n, int channels, int classes, int dtype, void* stream);

/*
 * Stage transitions in one call each (bf16): the Linear projection(s) on the tensor-core
 * Linear kernels (ptv3_linear_fwd or ptv3_gemm_fwd, whichever takes the shape;
 * ptv3_pool_stage_supported tells whether one does), then the kernel of ptv3_pool_fwd /
 * ptv3_unpool_fwd with the same arguments.
 *   ptv3_pool_stage_fwd     SerializedPooling: proj + segment reduction + BN + GELU
 *                           (model.py:684-689, 707-710); x is n x c_in, out m x c_out
 *   ptv3_unpool_stage_fwd   SerializedUnpooling: proj and proj_skip + BN + GELU + gather-add
 *                           (model.py:726-735, 744-746); skip_feat n x c_skip, child_feat m x c_child
 * Weights in nn.Linear layout (c_out x c_in), biases required.  status: one uint32, OR-ed
 * with PTV3_STATUS_WAIT_LIMIT when a bounded wait of the Linear kernels ran out.
 */
int ptv3_pool_stage_supported(int c_in, int c_out, int dtype);
size_t ptv3_pool_stage_workspace_bytes(int64_t n, int c_out);
int ptv3_pool_stage_fwd(const void* x, const void* weight, const void* bias, const float* coord,
                        const int64_t* indices, const int64_t* idx_ptr, int64_t n, int64_t m, int c_in, int c_out,
                        const float* bn_scale, const float* bn_shift, void* out, float* coord_out, int reduce,
                        int dtype, uint32_t* status, void* workspace, size_t workspace_bytes, void* stream);
size_t ptv3_unpool_stage_workspace_bytes(int64_t n, int64_t m, int c_out);
int ptv3_unpool_stage_fwd(const void* skip_feat, const void* child_feat, const void* w_skip, const void* b_skip,
                          const void* w_child, const void* b_child, const int64_t* cluster, int64_t n, int64_t m,
                          int c_skip, int c_child, int c_out, const float* skip_scale, const float* skip_shift,
                          const float* child_scale, const float* child_shift, void* out, void* skip_act, int dtype,
                          uint32_t* status, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PTV3_B200_H */
