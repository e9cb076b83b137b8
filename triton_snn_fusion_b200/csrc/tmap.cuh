// Host-side creation of tiled TMA tensor maps (128-byte swizzle, zero fill outside the tensor).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace snnb {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// dtype: SNNB_BF16 / SNNB_F16 / SNNB_U8 / SNNB_F32. swizzle_bytes: 128 (rows of 128 bytes), 64 (rows of 64 bytes)
// or 0 (no swizzle: the box lands in shared memory as a dense row-major array).
inline int encode_tmap(CUtensorMap *m, int dtype, int rank, const void *base, const cuuint64_t *dims, const cuuint64_t *strides,
           const cuuint32_t *box, int swizzle_bytes = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SNNB_ERR_CUDA, "conv_lif: cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SNNB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == SNNB_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : dtype == SNNB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, (cuuint32_t)rank, const_cast<void *>(base), dims, strides, box, ones,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE
                        : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SNNB_ERR_CUDA, "conv_lif: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SNNB_OK;
}

}  // namespace snnb
