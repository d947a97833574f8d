// The tensor-core kernel for 8-bit (q8g64s.t64) weights, one instantiation per fused epilogue.
#include "k_umma.cuh"

namespace p0p {

umma_kernel_fn umma_kernel_q8(uint32_t variant, uint32_t epi) {
  static const umma_kernel_fn table[4][7] = {P0P_UMMA_ROW(P0P_ENC_Q8, 1, true), P0P_UMMA_ROW(P0P_ENC_Q8, 2, true), P0P_UMMA_ROW(P0P_ENC_Q8, 2, false),
                                             P0P_UMMA_ROW(P0P_ENC_Q8, 4, false)};
  return table[variant][epi];
}

}  // namespace p0p
