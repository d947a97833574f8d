// Host-side helpers of the C ABI: fp16 conversion, the q4/q8 weight encoders of docs/FORMAT.md, the
// convolution-weight reordering and the N-shard byte ranges.  CPU code, no device work.
// Behaviour follows src/core/gpu.js:275-299 and src/convert/encode.js:56-122 of the reference: fp32 maths,
// scales/minimums rounded to fp16, codes rounded half to even.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/p0p.h"

namespace {

inline uint32_t fbits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bitsf(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// round-to-nearest-even float -> half via the "magic add" for subnormals and an integer round for normals
inline uint16_t f2h_rne(float f) {
  uint32_t u = fbits(f), sign = (u >> 16) & 0x8000u;
  u &= 0x7fffffffu;
  if (u >= 0x47800000u) return (uint16_t)(sign | (u > 0x7f800000u ? 0x7e00u : 0x7c00u));   // >= 65536, inf, NaN
  if (u < 0x38800000u) {                                                                   // below 2^-14: subnormal half or zero
    const uint32_t magic = 126u << 23;                                                     // 0.5f: the float adder rounds at the half's ulp
    return (uint16_t)(sign | (fbits(bitsf(u) + bitsf(magic)) - magic));
  }
  uint32_t odd = (u >> 13) & 1u;
  u += 0xc8000fffu;                                                                        // rebias exponent, add rounding bias - 1
  u += odd;
  return (uint16_t)(sign | (u >> 13));
}
inline float h2f_exact(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, em = h & 0x7fffu;
  if (em >= 0x7c00u) return bitsf(sign | 0x7f800000u | ((em & 0x3ffu) << 13));
  if (em < 0x0400u) {                                                                      // subnormal: value = em * 2^-24
    float v = (float)em * 5.9604644775390625e-8f;
    return sign ? -v : v;
  }
  return bitsf(sign | ((em << 13) + 0x38000000u));
}
inline float round_h(float x) { return h2f_exact(f2h_rne(x)); }

template <class F>
void parallel_for(uint32_t n, F fn) {
  unsigned hw = std::thread::hardware_concurrency(); if (!hw) hw = 1;
  unsigned nt = std::min<unsigned>(hw, n);
  if (nt <= 1) { for (uint32_t i = 0; i < n; i++) fn(i); return; }
  std::vector<std::thread> th;
  for (unsigned t = 0; t < nt; t++) th.emplace_back([=] { for (uint32_t i = t; i < n; i += nt) fn(i); });
  for (auto& x : th) x.join();
}

}  // namespace

extern "C" {

uint16_t p0p_f2h(float v) { return f2h_rne(v); }
float p0p_h2f(uint16_t h) { return h2f_exact(h); }
void p0p_to_f16(const float* s, uint16_t* d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = f2h_rne(s[i]); }
void p0p_from_f16(const uint16_t* s, float* d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = h2f_exact(s[i]); }

int p0p_pack_q4(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq) {
  if (rows % 64u || K % 32u) return -1;   // 'q4g32a.t64 needs rows % 64 == 0 and K % 32 == 0'
  const uint32_t G = K / 32u;
  parallel_for(rows / 64u, [=](uint32_t t) {
    for (uint32_t g = 0; g < G; g++) {
      uint8_t* rec = out + ((size_t)t * G + g) * 1280u;
      for (uint32_t r = 0; r < 64u; r++) {
        const size_t base = ((size_t)t * 64u + r) * K + (size_t)g * 32u;
        const float* v = W + base;
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < 32; i++) { if (v[i] < lo) lo = v[i]; if (v[i] > hi) hi = v[i]; }
        const float mn = round_h(lo);
        float s = round_h((hi - mn) / 15.0f);
        if (s == 0.0f) s = 1.0f;
        uint8_t* codes = rec + r * 16u;
        for (int j = 0; j < 16; j++) {
          int q[2];
          for (int e = 0; e < 2; e++) {
            float c = std::nearbyintf((v[2 * j + e] - mn) / s);      // default rounding mode: half to even
            q[e] = c < 0.0f ? 0 : c > 15.0f ? 15 : (int)c;
            if (deq) deq[base + 2 * j + e] = std::fmaf((float)q[e], s, mn);   // q*s is exact, one rounding
          }
          codes[j] = (uint8_t)(q[0] | (q[1] << 4));
        }
        const uint32_t word = (uint32_t)f2h_rne(s) | ((uint32_t)f2h_rne(mn) << 16);
        std::memcpy(rec + 1024u + r * 4u, &word, 4);
      }
    }
  });
  return 0;
}

int p0p_pack_q8(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq) {
  if (rows % 64u || K % 64u) return -1;   // 'q8g64s.t64 needs rows % 64 == 0 and K % 64 == 0'
  const uint32_t G = K / 64u;
  parallel_for(rows / 64u, [=](uint32_t t) {
    for (uint32_t g = 0; g < G; g++) {
      uint8_t* rec = out + ((size_t)t * G + g) * 4224u;
      for (uint32_t r = 0; r < 64u; r++) {
        const size_t base = ((size_t)t * 64u + r) * K + (size_t)g * 64u;
        const float* v = W + base;
        float am = 0.0f;
        for (int i = 0; i < 64; i++) am = std::max(am, std::fabs(v[i]));
        float s = round_h(am / 127.0f);
        if (s == 0.0f) s = 1.0f;
        for (int i = 0; i < 64; i++) {
          float c = std::nearbyintf(v[i] / s);
          int q = c < -128.0f ? -128 : c > 127.0f ? 127 : (int)c;
          rec[r * 64u + i] = (uint8_t)(q & 255);
          if (deq) deq[base + i] = (float)q * s;
        }
        const uint16_t hs = f2h_rne(s);
        std::memcpy(rec + 4096u + r * 2u, &hs, 2);
      }
    }
  });
  return 0;
}

void p0p_reorder_conv_rows(const float* W, float* out, uint32_t rows, uint32_t I, uint32_t taps) {
  const size_t K = (size_t)I * taps;
  for (uint32_t r = 0; r < rows; r++) {
    const float* src = W + r * K; float* dst = out + r * K;
    for (uint32_t t = 0; t < taps; t++) for (uint32_t i = 0; i < I; i++) dst[(size_t)t * I + i] = src[(size_t)i * taps + t];
  }
}

uint64_t p0p_encoded_bytes(uint32_t enc, uint64_t rows, uint64_t cols) {
  switch (enc) {
    case P0P_ENC_Q4: return rows / 64u * (cols / 32u) * 1280u;
    case P0P_ENC_Q8: return rows / 64u * (cols / 64u) * 4224u;
    case P0P_ENC_F16: return rows * cols * 2u;
    default: return rows * cols * 4u;
  }
}

int p0p_shard_rows(uint32_t enc, uint64_t rows, uint64_t cols, uint32_t rank, uint32_t world,
                   uint64_t* row0, uint64_t* nrows, uint64_t* byte_off, uint64_t* bytes) {
  if (!world || rank >= world) return -1;
  const uint64_t gran = (enc == P0P_ENC_Q4 || enc == P0P_ENC_Q8) ? 64u : 1u;
  if (rows % (gran * world)) return -2;
  const uint64_t per = rows / world, r0 = per * rank;
  if (row0) *row0 = r0;
  if (nrows) *nrows = per;
  if (byte_off) *byte_off = p0p_encoded_bytes(enc, r0, cols);
  if (bytes) *bytes = p0p_encoded_bytes(enc, per, cols);
  return 0;
}

}  // extern "C"
