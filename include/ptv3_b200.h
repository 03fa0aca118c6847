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

const char* ptv3_last_error(void);
int ptv3_version(void);

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
 * Stable argsort of every code row and its inverse permutation.
 * Replaces model.py:118-126 (torch.argsort + scatter_) and :667-674.
 *   codes     k x n int64, non-negative, nothing set above bit sig_bits-1
 *   order     k x n int64: codes[r][order[r][j]] is non-decreasing in j, ties
 *             by ascending index
 *   inverse   k x n int64: inverse[r][order[r][j]] = j
 */
size_t ptv3_argsort_workspace_bytes(int k, int64_t n, int sig_bits);
int ptv3_argsort_inverse(const int64_t* codes, int k, int64_t n, int sig_bits, int64_t* order,
                         int64_t* inverse, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PTV3_B200_H */
