// Voxel hash table shared by the kernel-map builder and the kernels that probe
// it directly: open addressing with linear probing over 64-bit keys
// (batch << 48 | x << 32 | y << 16 | z) and 32-bit row values.
#pragma once
#include "common.cuh"

namespace ptv3 {

constexpr uint64_t KM_EMPTY = ~0ull;

__device__ __forceinline__ uint64_t km_mix(uint64_t h)
{
    h ^= h >> 33;
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
    h *= 0xc4ceb9fe1a85ec53ull;
    h ^= h >> 33;
    return h;
}

__device__ __forceinline__ bool km_key(int b, int x, int y, int z, uint64_t& key)
{
    if ((unsigned)b > 0xfffeu || (unsigned)x > 0xffffu || (unsigned)y > 0xffffu || (unsigned)z > 0xffffu)
        return false;
    key = ((uint64_t)b << 48) | ((uint64_t)x << 32) | ((uint64_t)y << 16) | (uint64_t)z;
    return true;
}

// row of the voxel with `key`, or -1; sets *overflow when the probe limit is hit
__device__ __forceinline__ int32_t km_lookup(const unsigned long long* __restrict__ keys,
                                             const uint32_t* __restrict__ vals, uint64_t cap_mask,
                                             uint64_t key, bool* overflow)
{
    uint64_t slot = km_mix(key) & cap_mask;
    for (uint64_t probe = 0; probe <= cap_mask; ++probe) {
        const unsigned long long kk = keys[slot];
        if (kk == key) return (int32_t)vals[slot];
        if (kk == KM_EMPTY) return -1;
        slot = (slot + 1) & cap_mask;
    }
    *overflow = true;
    return -1;
}

uint64_t km_capacity(int64_t n);
size_t km_table_bytes(int64_t n);
// fills the table in `workspace` (km_table_bytes(n) bytes) with the n voxels
int km_build_table(const int32_t* indices, int64_t n, void* workspace, uint32_t* status,
                   cudaStream_t stream, unsigned long long** keys_out, uint32_t** vals_out,
                   uint64_t* cap_mask_out);

}  // namespace ptv3
