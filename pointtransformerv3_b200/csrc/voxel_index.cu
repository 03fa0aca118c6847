#include "voxel_index.cuh"

namespace ptv3 {

// every voxel claims its block: the first claimant takes the next table and clears it
__global__ void __launch_bounds__(256) vi_block_insert_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                              unsigned long long* __restrict__ keys,
                                                              uint32_t* __restrict__ vals, uint64_t cap_mask,
                                                              uint32_t* __restrict__ counter,
                                                              uint32_t* __restrict__ cells,
                                                              uint32_t* __restrict__ status)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int4 v = reinterpret_cast<const int4*>(indices)[i];
    uint64_t key;
    if ((unsigned)v.y > 0xffffu || (unsigned)v.z > 0xffffu || (unsigned)v.w > 0xffffu ||
        !vi_block_key(v.x, v.y >> 2, v.z >> 2, v.w >> 2, key)) {
        atomicOr(status, PTV3_STATUS_BAD_INDEX);
        return;
    }
    uint64_t slot = km_mix(key) & cap_mask;
    for (uint64_t probe = 0; probe <= cap_mask; ++probe) {
        const unsigned long long prev = atomicCAS(&keys[slot], KM_EMPTY, key);
        if (prev == KM_EMPTY) {
            const uint32_t id = atomicAdd(counter, 1u);
            uint4* tab = reinterpret_cast<uint4*>(cells + (size_t)id * 64);
#pragma unroll
            for (int q = 0; q < 16; ++q) tab[q] = make_uint4(VI_NO_ROW, VI_NO_ROW, VI_NO_ROW, VI_NO_ROW);
            __threadfence();
            vals[slot] = id;
            return;
        }
        if (prev == key) return;
        slot = (slot + 1) & cap_mask;
    }
    atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
}

// second pass (all tables exist now): every voxel writes its row into its cell;
// duplicates resolve to the lowest row
__global__ void __launch_bounds__(256) vi_cell_fill_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                           const unsigned long long* __restrict__ keys,
                                                           const uint32_t* __restrict__ vals, uint64_t cap_mask,
                                                           uint32_t* __restrict__ cells,
                                                           uint32_t* __restrict__ status)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int4 v = reinterpret_cast<const int4*>(indices)[i];
    uint64_t key;
    if ((unsigned)v.y > 0xffffu || (unsigned)v.z > 0xffffu || (unsigned)v.w > 0xffffu ||
        !vi_block_key(v.x, v.y >> 2, v.z >> 2, v.w >> 2, key))
        return;
    bool overflow = false;
    const uint32_t id = vi_block_lookup(keys, vals, cap_mask, key, &overflow);
    if (id == VI_NO_ROW) {
        atomicOr(status, overflow ? PTV3_STATUS_PROBE_LIMIT : PTV3_STATUS_BAD_INDEX);
        return;
    }
    atomicMin(&cells[(size_t)id * 64 + ((v.y & 3) << 4 | (v.z & 3) << 2 | (v.w & 3))], (uint32_t)i);
}


// hash table of blocks (sized for one block per voxel), block counter, one 64-entry table per voxel at most
size_t voxel_index_bytes(int64_t n) { return km_table_bytes(n) + 256 + align_up((size_t)n * 256, 256); }

int build_voxel_index(const int32_t* indices, int64_t n, void* workspace, uint32_t* status, cudaStream_t stream,
                      VoxelIndex* out)
{
    const uint64_t cap = km_capacity(n);
    Carver cv(workspace);
    unsigned long long* keys = cv.take<unsigned long long>(cap);
    uint32_t* vals = cv.take<uint32_t>(cap);
    uint32_t* counter = cv.take<uint32_t>(64);
    uint32_t* cells = cv.take<uint32_t>((size_t)n * 64);
    cudaMemsetAsync(keys, 0xff, cap * sizeof(uint64_t), stream);
    cudaMemsetAsync(counter, 0, sizeof(uint32_t), stream);
    const unsigned vb = (unsigned)((n + 255) / 256);
    vi_block_insert_kernel<<<vb, 256, 0, stream>>>(indices, n, keys, vals, cap - 1, counter, cells, status);
    vi_cell_fill_kernel<<<vb, 256, 0, stream>>>(indices, n, keys, vals, cap - 1, cells, status);
    count_launches(2);
    out->keys = keys;
    out->vals = vals;
    out->cap_mask = cap - 1;
    out->cells = cells;
    return check_launch("voxel index");
}

}  // namespace ptv3
