// Voxelisation front end: the step right before the serialized backbone.
//
//   ptv3_grid_coord    grid_coord = trunc((coord - min over all points) / grid_size)
//                      as the reference derives it when only coordinates are given
//                      (model.py:88-96, 156-158): batch-global minimum, fp32
//                      subtraction and division, truncation toward zero.
//   ptv3_voxel_dedup   one point per occupied voxel of every scene: the first
//                      point (lowest row) of each (scene, x, y, z) is kept, kept
//                      rows stay in input order (so scenes stay contiguous), and
//                      every input point learns the kept row of its voxel.  The
//                      reference leaves this to its data pipeline (grid sampling);
//                      the backbone assumes at most one point per voxel for its
//                      submanifold convolutions.
//
// The voxel hash table is the one of the kernel-map builder (lowest row wins on
// insertion); positions come from the flag scan used by the pooling plan.
#include <algorithm>

#include "common.cuh"
#include "kmap.cuh"
#include "scan.cuh"

namespace ptv3 {

// ---- grid coordinates ---------------------------------------------------------
__device__ __forceinline__ void atomic_min_float(float* addr, float v)
{
    // non-negative floats order like signed ints, negative ones in reverse like unsigned ints
    if (v >= 0.f)
        atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
    else
        atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__global__ void vox_origin_init_kernel(float* origin)
{
    if (threadIdx.x < 3) origin[threadIdx.x] = __int_as_float(0x7f800000);   // +inf
}

__global__ void __launch_bounds__(256) vox_min_kernel(const float* __restrict__ coord, int64_t n,
                                                      float* __restrict__ origin)
{
    float m[3] = {__int_as_float(0x7f800000), __int_as_float(0x7f800000), __int_as_float(0x7f800000)};
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        m[0] = fminf(m[0], coord[3 * i + 0]);
        m[1] = fminf(m[1], coord[3 * i + 1]);
        m[2] = fminf(m[2], coord[3 * i + 2]);
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m[a] = fminf(m[a], __shfl_xor_sync(0xffffffffu, m[a], o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomic_min_float(origin + 0, m[0]);
        atomic_min_float(origin + 1, m[1]);
        atomic_min_float(origin + 2, m[2]);
    }
}

__global__ void __launch_bounds__(256) vox_grid_kernel(const float* __restrict__ coord, int64_t n3,
                                                       float grid_size, const float* __restrict__ origin,
                                                       int32_t* __restrict__ grid)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n3) return;
    // IEEE subtraction and division (the build enables fast-math approximations elsewhere)
    const float d = __fsub_rn(coord[i], origin[i % 3]);
    grid[i] = (int32_t)truncf(__fdiv_rn(d, grid_size));
}

// ---- one point per voxel ----------------------------------------------------------
__global__ void __launch_bounds__(256) vox_first_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                        const unsigned long long* __restrict__ keys,
                                                        const uint32_t* __restrict__ vals, uint64_t cap_mask,
                                                        uint32_t* __restrict__ first, uint32_t* __restrict__ status)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int4 v = reinterpret_cast<const int4*>(indices)[i];
    uint64_t key;
    uint32_t f = (uint32_t)i;   // a point outside the key range (reported through the status) keeps itself
    if (km_key(v.x, v.y, v.z, v.w, key)) {
        bool overflow = false;
        const int32_t r = km_lookup(keys, vals, cap_mask, key, &overflow);
        if (overflow) atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
        if (r >= 0) f = (uint32_t)r;
    }
    first[i] = f;
}

struct FirstFlag {
    const uint32_t* first;
    __device__ bool operator()(int, int64_t j) const { return first[j] == (uint32_t)j; }
};

struct KeepSink {
    int64_t* keep;
    uint32_t* rank;
    __device__ void operator()(int, int64_t j, uint32_t pos, bool f) const
    {
        if (f) {
            keep[pos] = j;
            rank[j] = pos;
        }
    }
};

__global__ void __launch_bounds__(256) vox_inverse_kernel(const uint32_t* __restrict__ first,
                                                          const uint32_t* __restrict__ rank, int64_t n,
                                                          const uint32_t* __restrict__ total,
                                                          const int64_t* __restrict__ offset, int n_scenes,
                                                          int64_t* __restrict__ point2voxel,
                                                          int64_t* __restrict__ new_offset,
                                                          int64_t* __restrict__ count)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < n) point2voxel[i] = rank[first[i]];
    if (i == 0) *count = *total;
    if (i < n_scenes && new_offset) {
        // the first point of a scene is the first point of its voxel, so its rank is the number
        // of voxels kept before the scene
        const int64_t end = offset[i];
        new_offset[i] = end < n ? (int64_t)rank[end] : (int64_t)*total;
    }
}

static size_t dedup_scratch_bytes(int64_t n)
{
    const int ntiles = ceil_div(n, SC_TILE);
    return align_up((size_t)n * 4, 256) * 2 + align_up((size_t)ntiles * 4, 256) + 256;
}

}  // namespace ptv3

using namespace ptv3;

extern "C" int ptv3_grid_coord(const float* coord, int64_t n, float grid_size, float* origin, int32_t* grid_coord,
                               void* stream_)
{
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_grid_coord: n < 0");
    PTV3_REQUIRE(grid_size > 0.f, PTV3_ERR_INVALID_ARGUMENT, "ptv3_grid_coord: grid_size must be positive");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(coord && origin && grid_coord, PTV3_ERR_INVALID_ARGUMENT, "ptv3_grid_coord: null pointer");
    cudaStream_t stream = (cudaStream_t)stream_;
    vox_origin_init_kernel<<<1, 32, 0, stream>>>(origin);
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 8);
    vox_min_kernel<<<blocks, 256, 0, stream>>>(coord, n, origin);
    vox_grid_kernel<<<(unsigned)((3 * n + 255) / 256), 256, 0, stream>>>(coord, 3 * n, grid_size, origin, grid_coord);
    count_launches(3);
    return check_launch("ptv3_grid_coord");
}

extern "C" size_t ptv3_voxel_dedup_workspace_bytes(int64_t n)
{
    if (n <= 0) return 0;
    return km_table_bytes(n) + dedup_scratch_bytes(n);
}

extern "C" int ptv3_voxel_dedup(const int32_t* indices, int64_t n, const int64_t* offset, int n_scenes,
                                int64_t* keep, int64_t* point2voxel, int64_t* new_offset, int64_t* count,
                                uint32_t* status, void* workspace, size_t workspace_bytes, void* stream_)
{
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_voxel_dedup: bad n");
    PTV3_REQUIRE(n_scenes >= 0 && (n_scenes == 0 || offset), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_voxel_dedup: offset missing");
    PTV3_REQUIRE(count != nullptr, PTV3_ERR_INVALID_ARGUMENT, "ptv3_voxel_dedup: null pointer");
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n == 0) {
        cudaMemsetAsync(count, 0, sizeof(int64_t), stream);
        if (new_offset && n_scenes > 0) cudaMemsetAsync(new_offset, 0, sizeof(int64_t) * n_scenes, stream);
        return check_launch("ptv3_voxel_dedup");
    }
    PTV3_REQUIRE(indices && keep && point2voxel && status && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_voxel_dedup: null pointer");
    PTV3_REQUIRE(((uintptr_t)indices & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_voxel_dedup: indices must be 16-byte aligned");
    PTV3_REQUIRE(n_scenes <= n, PTV3_ERR_INVALID_ARGUMENT, "ptv3_voxel_dedup: more scenes than points");
    const size_t need = ptv3_voxel_dedup_workspace_bytes(n);
    PTV3_REQUIRE(workspace_bytes >= need, PTV3_ERR_WORKSPACE, "ptv3_voxel_dedup: workspace %zu < %zu bytes",
                 workspace_bytes, need);
    unsigned long long* keys;
    uint32_t* vals;
    uint64_t cap_mask;
    int rc = km_build_table(indices, n, workspace, status, stream, &keys, &vals, &cap_mask);
    if (rc != PTV3_OK) return rc;
    Carver cv(static_cast<char*>(workspace) + km_table_bytes(n));
    const int ntiles = ceil_div(n, SC_TILE);
    uint32_t* first = cv.take<uint32_t>(n);
    uint32_t* rank = cv.take<uint32_t>(n);
    uint32_t* tile_sums = cv.take<uint32_t>(ntiles);
    uint32_t* total = cv.take<uint32_t>(1);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    vox_first_kernel<<<blocks, 256, 0, stream>>>(indices, n, keys, vals, cap_mask, first, status);
    const FirstFlag flag{first};
    scan_tile_sums_kernel<FirstFlag><<<dim3(ntiles, 1), SC_THREADS, 0, stream>>>(flag, n, ntiles, tile_sums);
    scan_sums_kernel<<<1, SC_THREADS, 0, stream>>>(tile_sums, ntiles, total);
    scan_apply_kernel<FirstFlag, KeepSink><<<dim3(ntiles, 1), SC_THREADS, 0, stream>>>(
        flag, KeepSink{keep, rank}, n, ntiles, tile_sums);
    vox_inverse_kernel<<<blocks, 256, 0, stream>>>(first, rank, n, total, offset, n_scenes, point2voxel, new_offset,
                                                   count);
    count_launches(5);
    return check_launch("ptv3_voxel_dedup");
}
