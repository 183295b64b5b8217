// Host-side construction of TMA tensor maps without linking libcuda: the
// driver's encoder is looked up through the runtime at first use, so the
// library still loads (for symbol checks) on a machine that has no driver.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace h3s {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) ==
            cudaSuccess &&
        status == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// Rank-3 byte tensor (dim0 innermost, contiguous).  Out-of-bounds box
// elements read as zero.
inline int make_tensor_map_u8_3d(CUtensorMap *map, const void *base, uint64_t dim0, uint64_t dim1,
                                 uint64_t dim2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                                 uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle,
                                 const char *what) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(H3S_ECUDA, "%s: cuTensorMapEncodeTiled is unavailable", what);
  const cuuint64_t dims[3] = {dim0, dim1, dim2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides,
                         box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(H3S_ECUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, static_cast<int>(rc));
  return H3S_OK;
}

}  // namespace h3s
