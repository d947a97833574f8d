// The tensor-core kernel for fp16 weights, one instantiation per fused epilogue (and the split-K second stage, which does not depend on the encoding).
#include "k_umma.cuh"

namespace p0p {

umma_kernel_fn umma_kernel_f16(uint32_t epi) {
  static const umma_kernel_fn table[7] = P0P_UMMA_ROW(P0P_ENC_F16, 1, true);
  return table[epi];
}

umma_finish_fn umma_finish_kernel(uint32_t epi) {
  static const umma_finish_fn table[7] = {k_umma_finish<P0P_EPI_F16>, k_umma_finish<P0P_EPI_F32>, k_umma_finish<P0P_EPI_RESADD>, k_umma_finish<P0P_EPI_SWIGLU>,
                                          k_umma_finish<P0P_EPI_HEADS>, k_umma_finish<P0P_EPI_BIAS>, k_umma_finish<P0P_EPI_ONORMGATE>};
  return table[epi];
}

}  // namespace p0p
