#include "tc05.cuh"
#include "common.cuh"

namespace ptv3 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library does
// not link against libcuda.
static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return PTV3_ERR_CUDA;
    }
    const uint32_t span = box_cols * 2;
    if ((span != 64 && span != 128) || box_rows == 0 || box_rows > 256 || ((uintptr_t)base & 15) ||
        (pitch_bytes & 15)) {
        set_error("tensor map: unsupported box (%u x %u) or alignment", box_rows, box_cols);
        return PTV3_ERR_INVALID_ARGUMENT;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d)", (int)r);
        return PTV3_ERR_CUDA;
    }
    return PTV3_OK;
}

}  // namespace ptv3
