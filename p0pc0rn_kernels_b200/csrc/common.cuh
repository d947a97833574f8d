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
// The conversion of a weight block is bound by instruction count (its integer and fp16 instructions issue at half rate), so
// each tile value costs as few instructions as exactness allows.  The trick: a code is placed in the mantissa of an fp16
// SUBNORMAL (no exponent offset to subtract afterwards) and the scale is pre-multiplied by the matching power of two, so that
// ONE fused multiply-add per value pair yields q*s + mn with the exact product and a single rounding.
//
// q4.  Eight codes of one u32 (nibble i = column 8w+i) -> four half2 in natural column order.  With w4 = w << 4, byte b of w4
// holds q[2b] in bits 4..7 and byte b of w holds q[2b+1] there; prmt pairs the two bytes and a mask leaves the halves
// q[2b] * 2^-20 and q[2b+1] * 2^-20 (subnormals).  s20 = s * 2^20 must be finite: q4_row_fast().
__device__ __forceinline__ void q4_word_to_half2x4(uint32_t w, __half2 s20, __half2 mn2, __half2 out[4]) {
  const uint32_t w4 = w << 4;
#pragma unroll
  for (int b = 0; b < 4; b++) {
    uint32_t t = __byte_perm(w4, w, b | (b << 4) | ((4 + b) << 8) | ((4 + b) << 12)) & 0x00f000f0u;
    out[b] = __hfma2(*reinterpret_cast<__half2*>(&t), s20, mn2);
  }
}
// s * 2^20 as two exact multiplications by 2^10 (2^20 itself is not an fp16 number)
__device__ __forceinline__ __half2 q4_scale20(__half2 s2) {
  const __half2 k = __half2half2(__ushort_as_half(0x6400));      // 1024
  return __hmul2(__hmul2(s2, k), k);
}
// true when the packed path gives f16(f32(q*s+mn)) for every code q of a (scale, min) pair:
//  * s * 2^20 is finite (fp16 exponent field of s at most 10, i.e. s < 2^-4);
//  * q*s+mn needs at most 24 significant bits, so that rounding it to fp32 first changes nothing: with e_s, e_m the fp16
//    exponents, q*s spans bits e_s-10 .. e_s+4 and mn spans e_m-10 .. e_m, so e_m <= e_s + 12 and e_s <= e_m + 9 keep the sum
//    inside 24 bits (mn == 0 is always exact).
__device__ __forceinline__ bool q4_row_fast(uint32_t sm) {
  uint32_t es = (sm >> 10) & 31u, em = (sm >> 26) & 31u, mm = (sm >> 16) & 0x7fffu;
  if (es > 10u) return false;
  if (mm == 0u) return true;
  if (es == 0u) es = 1u;        // subnormal scale: lowest bit sits at 2^-24 either way
  if (em == 0u) em = 1u;
  return em <= es + 12u && es <= em + 9u;
}
// one row of a q4 record (32 k: four code words, sm = scale | min << 16) -> 16 half2, every value f16(f32(q*s+mn)).  The
// packed path serves almost every row; a lane whose (scale, min) pair fails the test redoes its row in fp32 (a divergent
// branch that is almost never taken; the warp is converged again on return).
__device__ __forceinline__ void q4_row32(const uint32_t (&w)[4], uint32_t sm, __half2 (&v)[16]) {
  const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)(sm & 0xffffu))), m2 = __half2half2(__ushort_as_half((unsigned short)(sm >> 16)));
  const __half2 s20 = q4_scale20(s2);
#pragma unroll
  for (int i = 0; i < 4; i++) q4_word_to_half2x4(w[i], s20, m2, v + 4 * i);
  if (!q4_row_fast(sm)) {
    const float sc = __half2float(__ushort_as_half((unsigned short)(sm & 0xffffu))), mn = __half2float(__ushort_as_half((unsigned short)(sm >> 16)));
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __halves2half2(deq_q4((w[i >> 2] >> (8 * (i & 3))) & 15u, sc, mn), deq_q4((w[i >> 2] >> (8 * (i & 3) + 4)) & 15u, sc, mn));
  }
  __syncwarp();
}

// q8.  Four int8 codes of one u32 (byte i = column 4w+i) -> two half2 in natural order, each f16(q*s).  u = q + 128 is placed
// as a subnormal u * 2^-24 (prmt with a zero register), s24 = s * 2^24, and the fused multiply-add adds -128*s: the result
// (u - 128) * s = q * s is exact before its single rounding.  s24 must be finite: q8_row_fast().
__device__ __forceinline__ void q8_word_to_half2x2(uint32_t w, __half2 s24, __half2 off, __half2 out[2]) {
  const uint32_t u = w ^ 0x80808080u;                       // q + 128 in 0..255
  uint32_t a = __byte_perm(u, 0u, 0x4140);                  // [b0, 0, b1, 0]
  uint32_t b = __byte_perm(u, 0u, 0x4342);                  // [b2, 0, b3, 0]
  out[0] = __hfma2(*reinterpret_cast<__half2*>(&a), s24, off);
  out[1] = __hfma2(*reinterpret_cast<__half2*>(&b), s24, off);
}
// the same for any scale: (u + 1024 as the pattern 0x6400 | u) - 1152 = q, then one multiplication
__device__ __forceinline__ void q8_word_to_half2x2_any(uint32_t w, __half2 s2, __half2 out[2]) {
  uint32_t u = w ^ 0x80808080u;
  const __half2 off = __half2half2(__ushort_as_half(0xe480));   // -1152 = -(1024 + 128)
  uint32_t a = __byte_perm(u, 0x64646464u, 0x4140);   // [b0, 0x64, b1, 0x64]
  uint32_t b = __byte_perm(u, 0x64646464u, 0x4342);   // [b2, 0x64, b3, 0x64]
  out[0] = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&a), off), s2);
  out[1] = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&b), off), s2);
}
__device__ __forceinline__ bool q8_row_fast(uint32_t s_bits) { return ((s_bits >> 10) & 31u) <= 6u; }      // s < 2^-8: s * 2^24 is finite
// NW code words of one row (4 codes each; a row of a q8 record is 16 words) -> 2 * NW half2, every value f16(q*s)
template <int NW>
__device__ __forceinline__ void q8_row(const uint32_t (&w)[NW], uint32_t s_bits, __half2 (&v)[2 * NW]) {
  const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)s_bits));
  if (__all_sync(0xffffffffu, q8_row_fast(s_bits))) {           // scales of one tensor are of one magnitude: the vote is all but always true
    const __half2 k = __half2half2(__ushort_as_half(0x6c00));   // 4096: s * 2^24 as two exact multiplications by 2^12
    const __half2 s24 = __hmul2(__hmul2(s2, k), k), off = __hmul2(s2, __half2half2(__ushort_as_half(0xd800)));      // -128 * s
#pragma unroll
    for (int i = 0; i < NW; i++) q8_word_to_half2x2(w[i], s24, off, v + 2 * i);
  } else {
#pragma unroll
    for (int i = 0; i < NW; i++) q8_word_to_half2x2_any(w[i], s2, v + 2 * i);
  }
}

}  // namespace p0p
