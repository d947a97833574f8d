// cuTensorMapEncodeTiled without linking libcuda: the entry point comes from the runtime's driver-entry-point query.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace p0p {

typedef CUresult (*tmap_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline tmap_encode_fn tmap_encoder() {
  static tmap_encode_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess) fn = (tmap_encode_fn)f;
    (void)cudaGetLastError();
  }
  return fn;
}

// fp16 tensor [d2][d1][d0] (d0 innermost, contiguous; s1 / s2 = strides of d1 / d2 in elements), box 64 x box1 x 1 with the
// 128-byte swizzle; coordinates outside the tensor read as zero
inline bool make_map_3d(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box1) {
  tmap_encode_fn f = tmap_encoder();
  if (!f) return false;
  const cuuint64_t dims[3] = {d0, d1, d2}, strides[2] = {s1 * 2u, s2 * 2u};
  const cuuint32_t box[3] = {64u, box1, 1u}, el[3] = {1u, 1u, 1u};
  return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace p0p
