// Launchers of the tensor-core attention paths (attention_mma.cu: mma.sync,
// attention_tc05.cu: tcgen05 + tensor memory).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptv3 {

constexpr int ATTN_MMA_MAX_SEQLEN = 2048;   // keys+values of one head: 128 KiB of shared memory

bool attn_mma_supported(int channels, int heads, int max_seqlen);
int launch_attn_mma(const void* qkv, const int64_t* order, const int64_t* pad, const int64_t* unpad,
                    const int32_t* cu_seqlens, void* out, int n_seq, int max_seqlen, int channels,
                    int heads, float scale, bool packed_exp, uint32_t* status, cudaStream_t stream);

constexpr int ATTN_TC05_MAX_SEQLEN = 1024;  // keys + values of one head: 64 KiB of shared memory

bool attn_tc05_supported(int channels, int heads, int max_seqlen);
int launch_attn_tc05(const void* qkv, const int64_t* order, const int64_t* pad, const int64_t* unpad,
                     const int32_t* cu_seqlens, void* out, int n_seq, int max_seqlen, int channels,
                     int heads, float scale, uint32_t* status, cudaStream_t stream);

}  // namespace ptv3
