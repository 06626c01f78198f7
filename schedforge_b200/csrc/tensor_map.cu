// Host-side TMA descriptor (CUtensorMap) construction.  The driver function is fetched
// at run time with cudaGetDriverEntryPoint, so the library has no link-time dependency on
// libcuda and still loads on a machine without a GPU driver.
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace sfb {
namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(entry);
    });
    return fn;
}

}  // namespace

bool encode_tensor_map_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                               uint32_t box_rows, uint32_t box_cols) {
    EncodeTiled encode = encode_fn();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available"); return false; }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                              box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(2d) failed with CUresult " + std::to_string(static_cast<int>(r)));
        return false;
    }
    return true;
}

// Bytes, no swizzle: rows of `cols` bytes (a multiple of 16); the box lands row-major in shared memory.
bool encode_tensor_map_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                             uint32_t box_cols) {
    EncodeTiled encode = encode_fn();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available"); return false; }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(u8) failed with CUresult " + std::to_string(static_cast<int>(r)));
        return false;
    }
    return true;
}

bool encode_tensor_map_bf16_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1, uint64_t stride2, uint32_t box0, uint32_t box1, uint32_t box2) {
    EncodeTiled encode = encode_fn();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available"); return false; }
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
    const cuuint32_t box[3] = {box0, box1, box2};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                              box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(3d) failed with CUresult " + std::to_string(static_cast<int>(r)));
        return false;
    }
    return true;
}

}  // namespace sfb
