// Kernel map of a submanifold convolution: for every active voxel and every
// kernel offset, the row of the active voxel at (coordinate + offset), or -1.
// Built with an open-addressing hash table in a caller-provided workspace.
//
// Replaces the indice-pair construction spconv.SubMConv3d performs for the call
// sites model.py:546-552 (3x3x3, cached per indice_key) and model.py:767-774
// (5x5x5 stem).  The table is offset-major, nbr[o][i], so that a tile of
// consecutive voxels reads each offset's neighbour rows coalesced.
// Offset index o = ((dx+r)*k + (dy+r))*k + (dz+r), r = k/2.
#include <atomic>

#include "common.cuh"
#include "kmap.cuh"
#include "voxel_index.cuh"

namespace ptv3 {

__global__ void __launch_bounds__(256) km_insert_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                        unsigned long long* __restrict__ keys,
                                                        uint32_t* __restrict__ vals, uint64_t cap_mask,
                                                        uint32_t* __restrict__ status)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int4 v = reinterpret_cast<const int4*>(indices)[i];
    uint64_t key;
    if (!km_key(v.x, v.y, v.z, v.w, key)) {
        atomicOr(status, PTV3_STATUS_BAD_INDEX);
        return;
    }
    uint64_t slot = km_mix(key) & cap_mask;
    for (uint64_t probe = 0; probe <= cap_mask; ++probe) {
        const unsigned long long prev = atomicCAS(&keys[slot], KM_EMPTY, key);
        if (prev == KM_EMPTY || prev == key) {
            atomicMin(&vals[slot], (uint32_t)i);   // duplicates: lowest row wins
            return;
        }
        slot = (slot + 1) & cap_mask;
    }
    atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
}

__global__ void __launch_bounds__(256) km_probe_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                       int ksize,
                                                       const unsigned long long* __restrict__ keys,
                                                       const uint32_t* __restrict__ vals,
                                                       uint64_t cap_mask, int32_t* __restrict__ nbr,
                                                       const int64_t* __restrict__ row_order,
                                                       uint32_t* __restrict__ status)
{
    // the offset is the same for the whole CTA: one thread does the runtime divisions
    __shared__ int delta[3];
    if (threadIdx.x == 0) {
        const int o = blockIdx.y, r = ksize / 2;
        delta[0] = o / (ksize * ksize) - r;
        delta[1] = (o / ksize) % ksize - r;
        delta[2] = o % ksize - r;
    }
    __syncthreads();
    const int o = blockIdx.y;
    const int dx = delta[0], dy = delta[1], dz = delta[2];
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    // column i of the table describes voxel row_order[i] (voxel i without an order)
    const int4 v = reinterpret_cast<const int4*>(indices)[row_order ? row_order[i] : i];
    int32_t found = -1;
    uint64_t key;
    if (km_key(v.x, v.y + dx, v.z + dy, v.w + dz, key)) {
        uint64_t slot = km_mix(key) & cap_mask;
        uint64_t probe = 0;
        for (; probe <= cap_mask; ++probe) {
            const unsigned long long kk = keys[slot];
            if (kk == key) {
                found = (int32_t)vals[slot];
                break;
            }
            if (kk == KM_EMPTY) break;
            slot = (slot + 1) & cap_mask;
        }
        if (probe > cap_mask) atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
    }
    nbr[(int64_t)o * n + i] = found;
}

// Neighbour table from the two-level voxel index: one thread per voxel looks up the 8 blocks
// its neighbourhood touches, then every offset is one cell-table load (kernel sizes up to 5).
__global__ void __launch_bounds__(256) km_block_probe_kernel(const int32_t* __restrict__ indices, int64_t n,
                                                             int ksize, VoxelIndex vi,
                                                             int32_t* __restrict__ nbr,
                                                             const int64_t* __restrict__ row_order,
                                                             uint32_t* __restrict__ status)
{
    __shared__ uint32_t block_s[8][256];
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = ksize / 2;
    // column i of the table describes voxel row_order[i] (voxel i without an order)
    const int4 c = reinterpret_cast<const int4*>(indices)[row_order ? row_order[i] : i];
    bool overflow = false;
#pragma unroll
    for (int bi = 0; bi < 8; ++bi) {
        uint64_t key;
        uint32_t id = VI_NO_ROW;
        if (vi_block_key(c.x, ((c.y - r) >> 2) + ((bi >> 2) & 1), ((c.z - r) >> 2) + ((bi >> 1) & 1),
                         ((c.w - r) >> 2) + (bi & 1), key))
            id = vi_block_lookup(vi.keys, vi.vals, vi.cap_mask, key, &overflow);
        block_s[bi][threadIdx.x] = id;
    }
    if (overflow) atomicOr(status, PTV3_STATUS_PROBE_LIMIT);
    const int bx0 = (c.y - r) >> 2, by0 = (c.z - r) >> 2, bz0 = (c.w - r) >> 2;
    int o = 0;
    for (int dx = -r; dx <= r; ++dx)
        for (int dy = -r; dy <= r; ++dy)
            for (int dz = -r; dz <= r; ++dz, ++o) {
                const int x = c.y + dx, y = c.z + dy, z = c.w + dz;
                const int bi = (((x >> 2) - bx0) << 2) | (((y >> 2) - by0) << 1) | ((z >> 2) - bz0);
                const uint32_t id = block_s[bi][threadIdx.x];
                uint32_t j = VI_NO_ROW;
                if (id != VI_NO_ROW) j = vi.cells[(size_t)id * 64 + vi_cell(x, y, z)];
                nbr[(int64_t)o * n + i] = (int32_t)j;   // VI_NO_ROW is -1 as an int32
            }
}

uint64_t km_capacity(int64_t n)
{
    uint64_t c = 1024;
    while (c < (uint64_t)n * 2) c <<= 1;
    return c;
}

size_t km_table_bytes(int64_t n)
{
    const uint64_t cap = km_capacity(n);
    return align_up(cap * sizeof(uint64_t), 256) + align_up(cap * sizeof(uint32_t), 256);
}

int km_build_table(const int32_t* indices, int64_t n, void* workspace, uint32_t* status,
                   cudaStream_t stream, unsigned long long** keys_out, uint32_t** vals_out,
                   uint64_t* cap_mask_out)
{
    const uint64_t cap = km_capacity(n);
    Carver cv(workspace);
    unsigned long long* keys = cv.take<unsigned long long>(cap);
    uint32_t* vals = cv.take<uint32_t>(cap);
    cudaMemsetAsync(keys, 0xff, cap * sizeof(uint64_t), stream);
    cudaMemsetAsync(vals, 0xff, cap * sizeof(uint32_t), stream);
    km_insert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(indices, n, keys, vals, cap - 1,
                                                                      status);
    count_launches(1);
    *keys_out = keys;
    *vals_out = vals;
    *cap_mask_out = cap - 1;
    return check_launch("voxel hash table");
}

}  // namespace ptv3

extern "C" size_t ptv3_kmap_workspace_bytes(int64_t n)
{
    if (n <= 0) return 0;
    return ptv3::voxel_index_bytes(n);   // covers the plain hash table of the 7x7x7 path too
}

extern "C" int ptv3_kmap_build(const int32_t* indices, int64_t n, int ksize, int32_t* nbr,
                               uint32_t* status, void* workspace, size_t workspace_bytes,
                               void* stream_)
{
    return ptv3_kmap_build_ordered(indices, n, ksize, nullptr, nbr, status, workspace, workspace_bytes, stream_);
}

extern "C" int ptv3_kmap_build_ordered(const int32_t* indices, int64_t n, int ksize, const int64_t* row_order,
                                       int32_t* nbr, uint32_t* status, void* workspace, size_t workspace_bytes,
                                       void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0 && n < (1ll << 31), PTV3_ERR_INVALID_ARGUMENT, "ptv3_kmap_build: bad n");
    PTV3_REQUIRE(ksize == 1 || ksize == 3 || ksize == 5 || ksize == 7, PTV3_ERR_UNSUPPORTED,
                 "ptv3_kmap_build: kernel size %d (supported: 1, 3, 5, 7)", ksize);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(indices && nbr && status && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_kmap_build: null pointer");
    PTV3_REQUIRE(((uintptr_t)indices & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_kmap_build: indices must be 16-byte aligned");
    const size_t need = ptv3_kmap_workspace_bytes(n);
    PTV3_REQUIRE(workspace_bytes >= need, PTV3_ERR_WORKSPACE,
                 "ptv3_kmap_build: workspace %zu < %zu bytes", workspace_bytes, need);
    cudaStream_t stream = (cudaStream_t)stream_;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (ksize <= 5) {
        VoxelIndex vi;
        const int rc = build_voxel_index(indices, n, workspace, status, stream, &vi);
        if (rc != PTV3_OK) return rc;
        km_block_probe_kernel<<<blocks, 256, 0, stream>>>(indices, n, ksize, vi, nbr, row_order, status);
        count_launches(1);
        return check_launch("ptv3_kmap_build");
    }
    const uint64_t cap = km_capacity(n);
    Carver cv(workspace);
    unsigned long long* keys = cv.take<unsigned long long>(cap);
    uint32_t* vals = cv.take<uint32_t>(cap);
    if (cudaMemsetAsync(keys, 0xff, cap * sizeof(uint64_t), stream) != cudaSuccess ||
        cudaMemsetAsync(vals, 0xff, cap * sizeof(uint32_t), stream) != cudaSuccess)
        return check_launch("ptv3_kmap_build: table reset");
    km_insert_kernel<<<blocks, 256, 0, stream>>>(indices, n, keys, vals, cap - 1, status);
    km_probe_kernel<<<dim3(blocks, ksize * ksize * ksize), 256, 0, stream>>>(
        indices, n, ksize, keys, vals, cap - 1, nbr, row_order, status);
    count_launches(2);
    return check_launch("ptv3_kmap_build");
}

// ----------------------------------------------------------------------------
// Kernel map without any caller-provided or allocated scratch memory.
// ----------------------------------------------------------------------------
namespace ptv3 {

// Largest voxel count the static table serves, and the table itself: 131072
// slots of an 8-byte key plus a 4-byte row index (1.5 MiB per GPU that loads
// the library, held until the process exits).
constexpr int64_t KM_STATIC_MAX_VOXELS = 65536;
constexpr uint64_t KM_STATIC_SLOTS = 131072;
constexpr size_t KM_STATIC_KEY_BYTES = KM_STATIC_SLOTS * sizeof(uint64_t);
constexpr size_t KM_STATIC_BYTES = KM_STATIC_KEY_BYTES + KM_STATIC_SLOTS * sizeof(uint32_t);
static __device__ __align__(256) unsigned char g_kmap_static_scratch[KM_STATIC_BYTES];

constexpr int KM_MAX_DEVICES = 64;
// device address of the static table on each device, resolved on first use there; atomic, so
// that first calls from two host threads do not race (both would store the same address)
static std::atomic<void*> g_kmap_static_ptr[KM_MAX_DEVICES];

// In host code `g_kmap_static_scratch` is only a handle for the runtime, not an
// address a kernel could use, so the device address is looked up once per
// device (with that device current) and handed to the kernels as a pointer.
static int km_static_table(void** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= KM_MAX_DEVICES) {
        set_error("ptv3_kmap_build_static: cannot identify the current device (%s)",
                  e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
        return PTV3_ERR_CUDA;
    }
    void* cached = g_kmap_static_ptr[dev].load(std::memory_order_acquire);
    if (cached == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_kmap_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("ptv3_kmap_build_static: cudaGetSymbolAddress failed on device %d (%s)", dev,
                      cudaGetErrorString(e));
            return PTV3_ERR_CUDA;
        }
        g_kmap_static_ptr[dev].store(p, std::memory_order_release);
        cached = p;
    }
    *out = cached;
    return PTV3_OK;
}

}  // namespace ptv3

extern "C" int64_t ptv3_kmap_static_max_voxels(void) { return ptv3::KM_STATIC_MAX_VOXELS; }

extern "C" int ptv3_kmap_build_static(const int32_t* indices, int64_t n, int ksize, int32_t* nbr,
                                      uint32_t* status, void* stream_)
{
    using namespace ptv3;
    PTV3_REQUIRE(n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_kmap_build_static: bad n");
    PTV3_REQUIRE(n <= KM_STATIC_MAX_VOXELS, PTV3_ERR_UNSUPPORTED,
                 "ptv3_kmap_build_static: %lld voxels exceed the static table's limit of %lld; use "
                 "ptv3_kmap_build with a workspace",
                 (long long)n, (long long)KM_STATIC_MAX_VOXELS);
    PTV3_REQUIRE(ksize == 1 || ksize == 3 || ksize == 5 || ksize == 7, PTV3_ERR_UNSUPPORTED,
                 "ptv3_kmap_build_static: kernel size %d (supported: 1, 3, 5, 7)", ksize);
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(indices && nbr && status, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_kmap_build_static: null pointer");
    PTV3_REQUIRE(((uintptr_t)indices & 15) == 0, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_kmap_build_static: indices must be 16-byte aligned");
    void* table = nullptr;
    const int rc = km_static_table(&table);
    if (rc != PTV3_OK) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(table);
    uint32_t* vals = reinterpret_cast<uint32_t*>(static_cast<char*>(table) + KM_STATIC_KEY_BYTES);
    // the table still holds the previous call's entries: reset exactly the slots this call uses
    const uint64_t cap = km_capacity(n);   // <= KM_STATIC_SLOTS because n <= KM_STATIC_MAX_VOXELS
    if (cudaMemsetAsync(keys, 0xff, cap * sizeof(uint64_t), stream) != cudaSuccess ||
        cudaMemsetAsync(vals, 0xff, cap * sizeof(uint32_t), stream) != cudaSuccess)
        return check_launch("ptv3_kmap_build_static: table reset");
    const unsigned blocks = (unsigned)((n + 255) / 256);
    km_insert_kernel<<<blocks, 256, 0, stream>>>(indices, n, keys, vals, cap - 1, status);
    km_probe_kernel<<<dim3(blocks, ksize * ksize * ksize), 256, 0, stream>>>(
        indices, n, ksize, keys, vals, cap - 1, nbr, nullptr, status);
    count_launches(2);
    return check_launch("ptv3_kmap_build_static");
}
