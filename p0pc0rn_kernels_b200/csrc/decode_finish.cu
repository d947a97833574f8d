// Second stage of the decode-sized multiply (k_decode_finish of k_decode.cuh): one instantiation per (token columns, fused
// epilogue).
#include "k_decode.cuh"

namespace p0p {

typedef void (*decode_finish_fn)(const DecodeP);

#define P0P_FINISH_ROW(MP) {k_decode_finish<MP, P0P_EPI_F16>, k_decode_finish<MP, P0P_EPI_F32>, k_decode_finish<MP, P0P_EPI_RESADD>, k_decode_finish<MP, P0P_EPI_SWIGLU>, \
                            k_decode_finish<MP, P0P_EPI_HEADS>, k_decode_finish<MP, P0P_EPI_BIAS>, k_decode_finish<MP, P0P_EPI_ONORMGATE>}

decode_finish_fn decode_finish_kernel(uint32_t mp, uint32_t epi) {
  static const decode_finish_fn table[2][7] = {P0P_FINISH_ROW(8), P0P_FINISH_ROW(16)};
  return table[mp == 8u ? 0 : 1][epi];
}

}  // namespace p0p
