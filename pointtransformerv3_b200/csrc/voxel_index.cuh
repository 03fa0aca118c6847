// Two-level voxel index: a hash table of 4 x 4 x 4 blocks whose values point at
// 64-entry cell tables (cell -> row of the voxel, VI_NO_ROW where empty).
// A (2r+1)^3 neighbourhood with r <= 2 touches at most 2 blocks per axis, so a voxel
// needs 8 hash probes instead of one per kernel offset; each offset then costs a
// few integer operations and one load from a 256-byte cell table.  Duplicate
// voxels resolve to the lowest row.
#pragma once
#include "common.cuh"
#include "kmap.cuh"

namespace ptv3 {

constexpr uint32_t VI_NO_ROW = 0xffffffffu;

__device__ __forceinline__ bool vi_block_key(int b, int bx, int by, int bz, uint64_t& key)
{
    if ((unsigned)b > 0xfffeu || (unsigned)bx > 0x3fffu || (unsigned)by > 0x3fffu || (unsigned)bz > 0x3fffu)
        return false;
    key = ((uint64_t)b << 48) | ((uint64_t)bx << 32) | ((uint64_t)by << 16) | (uint64_t)bz;
    return true;
}

__device__ __forceinline__ uint32_t vi_block_lookup(const unsigned long long* __restrict__ keys,
                                                    const uint32_t* __restrict__ vals, uint64_t cap_mask,
                                                    uint64_t key, bool* overflow)
{
    uint64_t slot = km_mix(key) & cap_mask;
    for (uint64_t probe = 0; probe <= cap_mask; ++probe) {
        const unsigned long long kk = keys[slot];
        if (kk == key) return vals[slot];
        if (kk == KM_EMPTY) return VI_NO_ROW;
        slot = (slot + 1) & cap_mask;
    }
    *overflow = true;
    return VI_NO_ROW;
}


struct VoxelIndex {
    const unsigned long long* keys;   // block hash table
    const uint32_t* vals;             // block -> cell table id
    uint64_t cap_mask;
    const uint32_t* cells;            // 64 rows per table
};

// cell of coordinate (x, y, z) inside its block
__device__ __forceinline__ int vi_cell(int x, int y, int z) { return (x & 3) << 4 | (y & 3) << 2 | (z & 3); }

size_t voxel_index_bytes(int64_t n);
// builds the index of n voxels (rows of (batch, x, y, z) int32) in `workspace`
int build_voxel_index(const int32_t* indices, int64_t n, void* workspace, uint32_t* status, cudaStream_t stream,
                      VoxelIndex* out);

}  // namespace ptv3
