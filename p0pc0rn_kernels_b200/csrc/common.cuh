// Shared device/host declarations of the gemm kernels: the parameter block every kernel takes (the
// reference shader's uniform struct P, src/ops/gemm.js:39-41, with the bindings resolved to pointers), and
// the weight decoders of docs/FORMAT.md.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/p0p.h"

namespace p0p {

struct KP {
  uint32_t M, N, K, ldx, kx0, wR0, wR1, wG, wk0, ldy, ny0;
  uint32_t rowOff, Ltot, Hq, Hkv;
  float eps;
  uint32_t pvOff, pvStride, evOff, statOff;
  uint32_t Hi, Wi, Ci, Ho, Wo, stride, padT, padL, ks, Nw, bvOff, bvUp;
  uint32_t enc, xmode, epi, flags;
  uint32_t vecx;     // X rows may be read with 16-byte loads (base, ld and k0 aligned)
  uint32_t vecw;     // f16 weight rows may be read with 16-byte loads
  const void* X;     // fp16 or fp32, at x.off
  const uint8_t* W;  // encoded weights, at w.off
  void* Y;           // fp16 or fp32, at y.off
  const float* ST; const float* PV; const float* EV; const float* BV; const float* RP; const __half* GT;
  uint32_t nyp;      // peer copies of Y: every store to Y is repeated at the same offset of YP[0..nyp)
  void* YP[7];
};

// ---- activations ------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + __expf(-z)); }
__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh(float g) {   // src/ops/gemm.js:208
  float t = 0.7978845608f * (g + 0.044715f * g * g * g);
  t = fminf(fmaxf(t, -15.0f), 15.0f);
  return g * 0.5f * (1.0f + tanhf(t));
}
// the same function through 0.5 (1 + tanh t) = 1 / (1 + e^-2t), with the hardware exponential and reciprocal
__device__ __forceinline__ float gelu_tanh_fast(float g) {
  float t = 0.7978845608f * (g + 0.044715f * g * g * g);
  t = fminf(fmaxf(t, -15.0f), 15.0f);
  return __fdividef(g, 1.0f + __expf(-2.0f * t));
}

// ---- weight decoding, one value (docs/FORMAT.md; index arithmetic of src/ops/gemm.js:143-171) ---------
// fp32 multiply-add then one rounding to fp16: q*s is exact in fp32, so this is f16(f32(q*s + min)).
__device__ __forceinline__ __half deq_q4(uint32_t q, float s, float mn) { return __float2half_rn(fmaf((float)q, s, mn)); }
__device__ __forceinline__ __half deq_q8(int q, float s) { return __float2half_rn((float)q * s); }

__device__ __forceinline__ uint32_t ldg32(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }

// value of weight row r, absolute column k, as the fp16 tile value
__device__ __forceinline__ __half wvalue(const KP& p, uint32_t r, uint32_t k) {
  if (p.enc == P0P_ENC_Q4) {
    const uint8_t* rec = p.W + ((size_t)(r >> 6) * p.wG + (k >> 5)) * 1280u;
    uint32_t rr = r & 63u, kk = k & 31u;
    uint32_t q = (ldg32(rec + rr * 16u + (kk >> 3) * 4u) >> (4u * (kk & 7u))) & 15u;
    uint32_t sm = ldg32(rec + 1024u + rr * 4u);
    return deq_q4(q, __half2float(__ushort_as_half((unsigned short)(sm & 0xffffu))), __half2float(__ushort_as_half((unsigned short)(sm >> 16))));
  } else if (p.enc == P0P_ENC_Q8) {
    const uint8_t* rec = p.W + ((size_t)(r >> 6) * p.wG + (k >> 6)) * 4224u;
    uint32_t rr = r & 63u, kk = k & 63u;
    int q = (int)(signed char)__ldg(rec + rr * 64u + kk);
    unsigned short hs = __ldg(reinterpret_cast<const unsigned short*>(rec + 4096u + rr * 2u));
    return deq_q8(q, __half2float(__ushort_as_half(hs)));
  } else {
    return __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p.W) + (size_t)r * p.wG + k));
  }
}

// ---- packed conversions used by the tensor-core kernels -------------------------------------------------
// Eight 4-bit codes of one u32 (nibble i = column 8w+i) -> four half2 in natural column order, each value
// f16(q*s + mn) with a single rounding (HFMA2 on exact small integers).  Exact when q*s+mn fits fp32 (see
// q4_pair_exact); the caller falls back to deq_q4 otherwise.
__device__ __forceinline__ void q4_word_to_half2x4(uint32_t w, __half2 s2, __half2 mn2, __half2 out[4]) {
  // byte b of w = (q[2b+1] << 4) | q[2b].  prmt builds {0x64, byte, 0x64, byte}; masking leaves
  // lo = 0x6400 | q[2b] (= 1024 + q) and hi = 0x6400 | q[2b+1] << 4 (= 1024 + 16 q).
  const __half2 mul = __halves2half2(__ushort_as_half(0x3c00), __ushort_as_half(0x2c00));   // (1, 1/16)
  const __half2 sub = __halves2half2(__ushort_as_half(0xe400), __ushort_as_half(0xd400));   // (-1024, -64)
#pragma unroll
  for (int b = 0; b < 4; b++) {
    uint32_t t = __byte_perm(w, 0x64646464u, 0x4040 | (b << 8) | b) ;   // bytes: [b, 0x64, b, 0x64] low->high
    t &= 0x64f0640fu;
    __half2 q = __hfma2(*reinterpret_cast<__half2*>(&t), mul, sub);      // exact integers 0..15
    out[b] = __hfma2(q, s2, mn2);
  }
}
// Four int8 codes of one u32 (byte i = column 4w+i) -> two half2 in natural order, each f16(q*s).
__device__ __forceinline__ void q8_word_to_half2x2(uint32_t w, __half2 s2, __half2 out[2]) {
  uint32_t u = w ^ 0x80808080u;                       // q + 128 in 0..255
  const __half2 off = __half2half2(__ushort_as_half(0xe480));   // -1152 = -(1024 + 128)
  uint32_t a = __byte_perm(u, 0x64646464u, 0x4140);   // [b0, 0x64, b1, 0x64]
  uint32_t b = __byte_perm(u, 0x64646464u, 0x4342);   // [b2, 0x64, b3, 0x64]
  out[0] = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&a), off), s2);
  out[1] = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&b), off), s2);
}
// true when f16(q*s+mn) by one HFMA equals f16(f32(q*s+mn)) for every code q: the exact sum needs at most 24
// significant bits: with e_s, e_m the fp16 exponents, q*s spans bits e_s-10 .. e_s+4 and mn spans e_m-10 .. e_m,
// so e_m <= e_s + 12 and e_s <= e_m + 9 keep the sum inside 24 bits (mn == 0 is always exact).
__device__ __forceinline__ bool q4_pair_exact(uint32_t sm) {
  uint32_t es = (sm >> 10) & 31u, em = (sm >> 26) & 31u, mm = (sm >> 16) & 0x7fffu;
  if (mm == 0u) return true;
  if (es == 0u) es = 1u;        // subnormal scale: lowest bit sits at 2^-24 either way
  if (em == 0u) em = 1u;
  return em <= es + 12u && es <= em + 9u;
}

}  // namespace p0p
