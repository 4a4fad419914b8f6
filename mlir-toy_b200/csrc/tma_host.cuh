// Host-side construction of TMA tensor maps, without linking libcuda: cuTensorMapEncodeTiled is
// resolved through the CUDA runtime's driver entry-point query.
#pragma once

#include <cuda.h>

#include "nb200_common.cuh"

namespace nb200 {

using EncodeTiledFnT = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

inline EncodeTiledFnT tma_encode_fn() {
  static EncodeTiledFnT fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFnT>(p);
  }();
  return fn;
}

// Row-major [rows, cols] tensor of 16-bit elements; boxes of box_rows x 64 columns (128 bytes), 128-byte swizzle.
inline int tma_map_2d_sw128(CUtensorMap *tm, const void *ptr, long long rows, long long cols, int dtype, int box_rows,
                            const char *who) {
  EncodeTiledFnT enc = tma_encode_fn();
  NB200_REQUIRE(enc, NB200_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, dtype == NB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NB200_REQUIRE(r == CUDA_SUCCESS, NB200_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with code %d", who, (int)r);
  return NB200_OK;
}

// Row-major [rows, cols] fp32 tensor; boxes of box_rows x box_cols (box_cols * 4 bytes a multiple of 16), no swizzle.
inline int tma_map_2d_f32(CUtensorMap *tm, const void *ptr, long long rows, long long cols, int box_cols, int box_rows,
                          const char *who) {
  EncodeTiledFnT enc = tma_encode_fn();
  NB200_REQUIRE(enc, NB200_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NB200_REQUIRE(r == CUDA_SUCCESS, NB200_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with code %d", who, (int)r);
  return NB200_OK;
}

}  // namespace nb200
