// The fused epilogues for kernels whose threads each own ONE output column of a 128-column block and carry
// TB tokens of it in registers (the split-K decode reduction and the tensor-core kernel, whose accumulator
// lanes are weight rows).  128 threads cooperate: the head epilogues reduce over the block's 128 columns.
// Arithmetic as in the reference shader, src/ops/gemm.js:191-254.
#pragma once
#include "common.cuh"

namespace p0p {

__device__ __forceinline__ void bar_sync_named(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// sh: shared scratch of at least TB * 132 floats, private to these 128 threads.  barid: a named barrier id
// private to them.  m0: first token row; rows m0 + j for j < TB with m0 + j < p.M are stored.
// nB: first column of the block (multiple of 128 for heads / onormgate).  c: this thread's column in the
// block (0..127).  acc[j]: fp32 accumulator of (row m0 + j, column nB + c).
template <int TB>
__device__ __forceinline__ void epilogue_cols(const KP& p, uint32_t m0, uint32_t nB, uint32_t c, float (&acc)[TB], float* sh, int barid) {
  const uint32_t col = nB + c, epi = p.epi, lane = c & 31u, wq = c >> 5;
  __half* Yh = reinterpret_cast<__half*>(p.Y); float* Yf = reinterpret_cast<float*>(p.Y);
  if (epi == P0P_EPI_HEADS || epi == P0P_EPI_ONORMGATE) {
    // ---- sum of squares over the 128 columns, per token
    float* part = sh;                 // [4][TB]
    float* xch = sh + 4 * TB;         // [TB][128] partner exchange for the (d, d+64) rotation
#pragma unroll
    for (int j = 0; j < TB; j++) {
      float s = acc[j] * acc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) part[wq * TB + j] = s;
    }
    bar_sync_named(barid, 128);
    const bool half_mode = epi == P0P_EPI_HEADS && (p.flags & P0P_F_ROPE_HALF);
    const uint32_t hd = nB / 128u, sec = epi == P0P_EPI_ONORMGATE ? 0u : (hd < p.Hq ? 0u : hd < p.Hq + p.Hkv ? 1u : 2u);
    const float nw = (epi == P0P_EPI_ONORMGATE || sec < 2u) ? __ldg(p.EV + p.evOff + (sec == 1u ? 128u : 0u) + c) : 1.0f;
    float v[TB];
#pragma unroll
    for (int j = 0; j < TB; j++) {
      const float ss = part[j] + part[TB + j] + part[2 * TB + j] + part[3 * TB + j];
      const float inv = rsqrtf(ss / 128.0f + p.eps);
      v[j] = (epi == P0P_EPI_ONORMGATE || sec < 2u) ? acc[j] * inv * nw : acc[j];
    }
    if (epi == P0P_EPI_ONORMGATE) {
#pragma unroll
      for (int j = 0; j < TB; j++) {
        const uint32_t m = m0 + j;
        if (m < p.M) {
          const float g = __half2float(p.GT[(size_t)m * p.Ltot + p.ny0 + col]);
          Yh[(size_t)m * p.ldy + p.ny0 + col] = __float2half_rn(v[j] / (1.0f + expf(-g)));
        }
      }
      bar_sync_named(barid, 128);     // `part` is free again
      return;
    }
    if (sec < 2u && half_mode) {
#pragma unroll
      for (int j = 0; j < TB; j++) xch[j * 128 + c] = v[j];
      bar_sync_named(barid, 128);
    }
#pragma unroll
    for (int j = 0; j < TB; j++) {
      const uint32_t m = m0 + j;
      const size_t row = (size_t)p.rowOff + min(m, p.M - 1u);
      float o = v[j];
      if (sec < 2u) {
        if (half_mode) {          // pairs (d, d+64), angle index d & 63
          const float other = xch[j * 128 + (c ^ 64u)];
          const uint32_t d = c & 63u;
          const float cs = __ldg(p.RP + row * 128u + 2u * d), sn = __ldg(p.RP + row * 128u + 2u * d + 1u);
          o = c < 64u ? v[j] * cs - other * sn : v[j] * cs + other * sn;
        } else {                  // interleaved pairs (2p, 2p+1)
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          const uint32_t pr = c >> 1;
          const float cs = __ldg(p.RP + row * 128u + 2u * pr), sn = __ldg(p.RP + row * 128u + 2u * pr + 1u);
          o = (c & 1u) ? other * sn + v[j] * cs : v[j] * cs - other * sn;
        }
      }
      if (m < p.M) Yh[((size_t)hd * p.Ltot + row) * 128u + c] = __float2half_rn(o);
    }
    bar_sync_named(barid, 128);       // scratch is free again
    return;
  }
  if (epi == P0P_EPI_SWIGLU) {
    // even lanes hold 'gate', odd lanes 'up' of output column o.  The pair splits the tokens: the even lane
    // finishes tokens j = 0, 2, .., the odd lane j = 1, 3, .., each getting the other half of its pair by one shuffle.
    const uint32_t o = col >> 1, odd = c & 1u;
    float gB = 0.0f, uB = 0.0f;
    if ((p.flags & P0P_F_BIAS) && col < p.N) { gB = __ldg(p.BV + p.bvOff + o); uB = __ldg(p.BV + p.bvOff + p.bvUp + o); }
#pragma unroll
    for (int j = 0; j < TB; j += 2) {
      const float other = __shfl_xor_sync(0xffffffffu, odd ? acc[j] : acc[j + 1], 1);
      const float g = (odd ? other : acc[j]) + gB, u = (odd ? acc[j + 1] : other) + uB;
      const uint32_t m = m0 + j + odd;
      if (m < p.M && col < p.N) {
        const float a = (p.flags & P0P_F_GELU) ? gelu_tanh(g) : __fdividef(g, 1.0f + __expf(-g));     // hardware exp / reciprocal: a few ulp, far inside the fp16 rounding
        Yh[(size_t)m * p.ldy + p.ny0 + o] = __float2half_rn(a * u);
      }
    }
    return;
  }
  if ((col & ~3u) >= p.N) return;                                   // stores go in groups of four columns (:196)
  float gate = 1.0f, bias = 0.0f;
  if (epi == P0P_EPI_RESADD) {
    if (p.flags & P0P_F_GATE) gate = __ldg(p.EV + p.evOff + col);
    if (p.flags & P0P_F_BIAS) bias = __ldg(p.BV + p.bvOff + col);
  } else if (epi == P0P_EPI_BIAS) bias = __ldg(p.EV + p.evOff + col);
  // read-modify-write epilogues fetch all TB old values first (TB loads in flight), then add and store
  float old[TB];
  const bool rmw32 = epi == P0P_EPI_RESADD && !(p.flags & P0P_F_STORE), rmw16 = epi == P0P_EPI_BIAS && (p.flags & P0P_F_RES);
#pragma unroll
  for (int j = 0; j < TB; j++) {
    const uint32_t m = m0 + j;
    const size_t yi = (size_t)min(m, p.M - 1u) * p.ldy + p.ny0 + col;
    old[j] = rmw32 ? __ldcg(Yf + yi) : rmw16 ? __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(Yh) + yi))) : 0.0f;
  }
#pragma unroll
  for (int j = 0; j < TB; j++) {
    const uint32_t m = m0 + j;
    if (m >= p.M) continue;
    const size_t yi = (size_t)m * p.ldy + p.ny0 + col;
    const float a = acc[j];
    if (epi == P0P_EPI_F16) Yh[yi] = __float2half_rn(a);
    else if (epi == P0P_EPI_F32) Yf[yi] = a;
    else if (epi == P0P_EPI_RESADD) Yf[yi] = old[j] + gate * (a + bias);
    else Yh[yi] = __float2half_rn(a + bias + old[j]);
  }
}

}  // namespace p0p
