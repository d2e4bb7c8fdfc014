#pragma once
// Host-side construction of TMA descriptors (CUtensorMap).
// Counterpart of the `make_2d_tma_*_desc` helpers the reference's launch template calls
// (yan/jit_kernels/gemm.py:23-26) but never defines.
//
// cuTensorMapEncodeTiled is resolved at run time through cudaGetDriverEntryPoint, so the
// library does not link libcuda and still loads on a machine without a driver.

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace yan {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2D row-major byte matrix [rows, row_bytes-wide rows of `cols` one-byte elements], box = box_rows x 128 bytes,
// 128-byte swizzle, out-of-bounds elements read as zero.  `ok` is cleared on failure.
inline CUtensorMap make_2d_tma_desc_u8_sw128(const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                                             uint32_t box_rows, bool& ok) {
    CUtensorMap map{};
    EncodeTiledFn encode = get_encode_tiled();
    if (encode == nullptr) {
        ok = false;
        return map;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) ok = false;
    return map;
}

}  // namespace yan
