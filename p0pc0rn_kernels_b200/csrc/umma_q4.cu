// The tensor-core kernel for 4-bit (q4g32a.t64) weights, one instantiation per fused epilogue.
#include "k_umma.cuh"

namespace p0p {

umma_kernel_fn umma_kernel_q4(uint32_t epi) {
  static const umma_kernel_fn table[7] = P0P_UMMA_TABLE(P0P_ENC_Q4);
  return table[epi];
}

}  // namespace p0p
