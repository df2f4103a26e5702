// Host-side construction of TMA tensor maps. The driver entry point is fetched at run time
// through the runtime API, so the library does not link against libcuda.
#pragma once
#include <cuda.h>  // CUtensorMap and its enums (types only)
#include <cuda_runtime.h>
#include <stdint.h>

namespace ako {
namespace tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// Byte matrix [rows, row_bytes] (row-major); box = 128 bytes x box_rows; 128-byte swizzle.
inline bool byte_matrix_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes,
                            uint32_t box_rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128u, box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 matrix [rows, cols] with a row stride in bytes; box = 64 columns (128 bytes) x box_rows;
// 128-byte swizzle: the K-major operand layout of tcgen05.mma.
inline bool bf16_matrix_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                            uint64_t row_stride_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {64u, box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Paged byte matrices: `pages` pages of `page_stride` bytes, each starting with [rows, 128] bytes;
// box = one page's 128 x rows block; 128-byte swizzle.
inline bool paged_byte_matrix_map(CUtensorMap* m, const void* base, uint64_t pages, uint64_t page_stride,
                                  uint32_t rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {128u, rows, pages};
  const cuuint64_t strides[2] = {128u, page_stride};
  const cuuint32_t box[3] = {128u, rows, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tma
}  // namespace ako
