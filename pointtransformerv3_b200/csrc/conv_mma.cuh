// Launchers of the tensor-core submanifold convolution paths (conv_mma.cu, conv_tc05.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptv3 {

bool conv_mma_supported(int c_in, int c_out, int kernel_volume);
// row_order: optional permutation of the voxels (n int64); tile t then owns
// voxels row_order[128 t .. 128 t + 127] and column j of nbr describes voxel
// row_order[j].  NULL = natural order.
int launch_conv_mma(const void* feat, const int32_t* nbr, const void* weight, const void* bias,
                    void* out, const int64_t* row_order, int64_t n, int c_in, int c_out,
                    int kernel_volume, cudaStream_t stream);

// tcgen05 form (conv_tc05.cu): same operands, accumulator in tensor memory; `status` receives
// PTV3_STATUS_WAIT_LIMIT if a device wait runs out.
bool conv_tc05_supported(int c_in, int c_out, int kernel_volume);
int launch_conv_tc05(const void* feat, const int32_t* nbr, const void* weight, const void* bias, void* out,
                     const int64_t* row_order, int64_t n, int c_in, int c_out, int kernel_volume,
                     uint32_t* status, cudaStream_t stream);

// Pair-list form (coarse levels): pairs sorted by kernel offset, 128-pair tiles,
// atomic fixed-point accumulation into acc (n x c_out 64-bit integers of workspace), then
// bias + rounding into out.
bool conv_pairs_supported(int c_in, int c_out, int kernel_volume);
int launch_conv_pairs(const void* feat, const int32_t* pair_in, const int32_t* pair_out,
                      const int32_t* off_start, const int32_t* tile_start, int64_t max_tiles,
                      const void* weight, const void* bias, void* out, long long* acc, int64_t n, int c_in,
                      int c_out, int kernel_volume, cudaStream_t stream);

}  // namespace ptv3
