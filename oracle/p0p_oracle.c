/*
 * CPU oracle for the p0pc0rn-kernels `gemm` path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's CPU-side algorithm for the gemm path
 * (fp16 helpers, the seeded generators of its test-suite, the q4/q8/f16 weight encoders, the two CPU
 * reference multiplications of its tests) plus a restatement, on the CPU, of the arithmetic the
 * reference's generated shader performs for every prologue and epilogue.  It is never shipped and never
 * linked into the product library: only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg load it, and only as the checker.
 *
 * Pinning status: the reference stores no golden vectors for this path (its tests are generated from
 * seeds at run time) and no JavaScript engine exists in the build image, so the reference itself cannot
 * be executed.  The restatement is pinned on the known-answer constants the reference does hold (dtype
 * decodes, format sizes/offsets, the README quick-start value); everything else is "parity unpinned" in
 * the strict sense and anchored by restating the reference's seeded test cases one for one.
 *
 * Each function cites the reference file:line it follows (paths inside the reference project).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off, no fast-math: float arithmetic must round once
 * per operation exactly as Math.fround does in the reference's JavaScript).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * fp16 helpers — src/core/gpu.js:275-299
 * ---------------------------------------------------------------------------------------------- */

/* f2h: float32 -> binary16 bits, round to nearest even, subnormals kept, overflow -> inf,
 * NaN -> sign|0x7e00 (src/core/gpu.js:276-291). */
API uint16_t orc_f2h(float v) {
  uint32_t x; memcpy(&x, &v, 4);
  uint32_t sign = (x >> 16) & 0x8000u, e = (x >> 23) & 0xffu, m = x & 0x7fffffu;
  if (e == 0xff) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0u));
  int ne = (int)e - 112;
  if (ne >= 0x1f) return (uint16_t)(sign | 0x7c00u);
  if (ne <= 0) {
    if (ne < -10) return (uint16_t)sign;
    m |= 0x800000u;
    int sh = 14 - ne;
    uint32_t hm = m >> sh, rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (hm & 1u))) hm++;
    return (uint16_t)(sign | hm);
  }
  uint32_t r = sign | ((uint32_t)ne << 10) | (m >> 13), rem2 = m & 0x1fffu;
  if (rem2 > 0x1000u || (rem2 == 0x1000u && (r & 1u))) r++;
  return (uint16_t)r;
}

/* h2f: binary16 bits -> float32 (src/core/gpu.js:292-297). */
API float orc_h2f(uint16_t h) {
  double s = (h & 0x8000u) ? -1.0 : 1.0;
  uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) return (float)(s * (double)m * 5.960464477539063e-8);
  if (e == 31) return m ? NAN : (float)(s * INFINITY);
  return (float)(s * (1.0 + (double)m / 1024.0) * ldexp(1.0, (int)e - 15));
}

static inline float rf16(float x) { return orc_h2f(orc_f2h(x)); }   /* test/kernels.test.js:14 */

API void orc_to_f16(const float* src, uint16_t* dst, size_t n) {     /* src/core/gpu.js:298 */
  for (size_t i = 0; i < n; i++) dst[i] = orc_f2h(src[i]);
}
API void orc_from_f16(const uint16_t* src, float* dst, size_t n) {   /* src/core/gpu.js:299 */
  for (size_t i = 0; i < n; i++) dst[i] = orc_h2f(src[i]);
}
API void orc_round_f16(const float* src, float* dst, size_t n) {     /* test/kernels.test.js:15 */
  for (size_t i = 0; i < n; i++) dst[i] = rf16(src[i]);
}

/* bf16 round-to-nearest-even as the converter test writes it (test/kernels.test.js:196) and the decode
 * (src/convert/encode.js:49). */
API void orc_to_bf16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; i++) { uint32_t u; memcpy(&u, &src[i], 4); dst[i] = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16); }
}
API void orc_from_bf16(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; i++) { uint32_t u = (uint32_t)src[i] << 16; memcpy(&dst[i], &u, 4); }
}
/* fp8 decode tables (src/convert/encode.js:32-41). */
API float orc_f8(int e4m3, uint8_t i) {
  double s = (i & 0x80) ? -1.0 : 1.0;
  int e = e4m3 ? (i >> 3) & 15 : (i >> 2) & 31, m = e4m3 ? i & 7 : i & 3, mb = e4m3 ? 3 : 2, bias = e4m3 ? 7 : 15;
  if (e4m3 && e == 15 && m == 7) return NAN;
  if (!e4m3 && e == 31) return m ? NAN : (float)(s * INFINITY);
  return (float)(s * (e == 0 ? ((double)m / (1 << mb)) * ldexp(1.0, 1 - bias) : (1.0 + (double)m / (1 << mb)) * ldexp(1.0, e - bias)));
}

/* ------------------------------------------------------------------------------------------------
 * Seeded generators — test/kernels.test.js:12-13
 * ---------------------------------------------------------------------------------------------- */

/* xorshift32 whose middle shift is an ARITHMETIC shift of the int32 view (test/kernels.test.js:12). */
static inline double rng_next(uint32_t* s) {
  uint32_t x = *s;
  x ^= x << 13;
  x ^= (uint32_t)((int32_t)x >> 17);
  x ^= x << 5;
  *s = x;
  return (double)x / 4294967296.0;
}
/* Box–Muller on pairs, double maths, float store (test/kernels.test.js:13). */
API void orc_randn(float* o, size_t n, uint32_t seed, double scale) {
  uint32_t s = seed ? seed : 1u;
  for (size_t i = 0; i < n; i += 2) {
    double u = rng_next(&s); if (u < 1e-9) u = 1e-9;
    double v = rng_next(&s), m = sqrt(-2.0 * log(u)) * scale;
    o[i] = (float)(m * cos(2.0 * M_PI * v));
    if (i + 1 < n) o[i + 1] = (float)(m * sin(2.0 * M_PI * v));
  }
}
/* the raw uniform stream, for known-answer checks of the generator itself */
API void orc_rng_u32(uint32_t* o, size_t n, uint32_t seed) {
  uint32_t s = seed ? seed : 1u;
  for (size_t i = 0; i < n; i++) { rng_next(&s); o[i] = s; }
}

/* ------------------------------------------------------------------------------------------------
 * Weight encoders — src/convert/encode.js:56-95, docs/FORMAT.md:7-45
 * ---------------------------------------------------------------------------------------------- */

/* q4g32a.t64: 1280-byte records of (64 rows x 32 k) (src/convert/encode.js:56-74).  deq may be NULL. */
API int orc_pack_q4(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq) {
  if (rows % 64 || K % 32) return -1;
  uint32_t NT = rows / 64, G = K / 32;
  for (uint32_t t = 0; t < NT; t++) for (uint32_t g = 0; g < G; g++) {
    size_t rec = ((size_t)t * G + g) * 1280;
    for (uint32_t r = 0; r < 64; r++) {
      size_t n = (size_t)t * 64 + r, base = n * K + (size_t)g * 32;
      float mnv = INFINITY, mxv = -INFINITY;
      for (int i = 0; i < 32; i++) { float v = W[base + i]; if (v < mnv) mnv = v; if (v > mxv) mxv = v; }
      float mn = rf16(mnv);
      float s = rf16((float)((float)(mxv - mn) / 15.0f)); if (s == 0.0f) s = 1.0f;
      for (int j = 0; j < 16; j++) {
        float a0 = rintf((float)((float)(W[base + 2 * j] - mn) / s)), a1 = rintf((float)((float)(W[base + 2 * j + 1] - mn) / s));
        int q0 = a0 < 0 ? 0 : a0 > 15 ? 15 : (int)a0, q1 = a1 < 0 ? 0 : a1 > 15 ? 15 : (int)a1;
        out[rec + r * 16 + j] = (uint8_t)(q0 | (q1 << 4));
        if (deq) { deq[base + 2 * j] = (float)((double)q0 * (double)s + (double)mn); deq[base + 2 * j + 1] = (float)((double)q1 * (double)s + (double)mn); }
      }
      uint32_t word = (uint32_t)orc_f2h(s) | ((uint32_t)orc_f2h(mn) << 16);
      memcpy(out + rec + 1024 + r * 4, &word, 4);
    }
  }
  return 0;
}

/* q8g64s.t64: 4224-byte records of (64 rows x 64 k) (src/convert/encode.js:76-90). */
API int orc_pack_q8(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq) {
  if (rows % 64 || K % 64) return -1;
  uint32_t NT = rows / 64, G = K / 64;
  for (uint32_t t = 0; t < NT; t++) for (uint32_t g = 0; g < G; g++) {
    size_t rec = ((size_t)t * G + g) * 4224;
    for (uint32_t r = 0; r < 64; r++) {
      size_t n = (size_t)t * 64 + r, base = n * K + (size_t)g * 64;
      float am = 0.0f;
      for (int i = 0; i < 64; i++) { float a = fabsf(W[base + i]); if (a > am) am = a; }
      float s = rf16((float)(am / 127.0f)); if (s == 0.0f) s = 1.0f;
      for (int i = 0; i < 64; i++) {
        float a = rintf((float)(W[base + i] / s));
        int q = a < -128 ? -128 : a > 127 ? 127 : (int)a;
        out[rec + r * 64 + i] = (uint8_t)(q & 255);
        if (deq) deq[base + i] = (float)((double)q * (double)s);
      }
      uint16_t hs = orc_f2h(s);
      memcpy(out + rec + 4096 + r * 2, &hs, 2);
    }
  }
  return 0;
}

/* conv weight rows OIHW / OITHW (I*taps) -> (taps*I) (src/convert/encode.js:118-122). */
API void orc_reorder_conv_rows(const float* W, float* out, uint32_t rows, uint32_t I, uint32_t taps) {
  size_t K = (size_t)I * taps;
  for (uint32_t r = 0; r < rows; r++) for (uint32_t i = 0; i < I; i++) for (uint32_t t = 0; t < taps; t++)
    out[r * K + (size_t)t * I + i] = W[r * K + (size_t)i * taps + t];
}

/* ------------------------------------------------------------------------------------------------
 * Weight decode exactly as the shader indexes the bytes — src/ops/gemm.js:143-171
 * Returns the fp16 BITS of the tile value (what lands in workgroup memory) and optionally the fp32 value
 * before the fp16 rounding.
 * ---------------------------------------------------------------------------------------------- */
static inline uint32_t ld32(const uint8_t* p, size_t word) { uint32_t v; memcpy(&v, p + word * 4, 4); return v; }

/* enc: 0 q4, 1 q8, 2 f16.  r = weight row, k = absolute weight column (wk0 + k0 + ...), wG as in
 * src/ops/gemm.js:284 (K/32, K/64, or the row stride in halves). */
static inline uint16_t wdecode(int enc, const uint8_t* W, uint32_t r, uint32_t k, uint32_t wG, float* f32out) {
  if (enc == 0) {   /* src/ops/gemm.js:144-152 */
    size_t rec = ((size_t)(r >> 6) * wG + (k / 32u)) * 320u; uint32_t rr = r & 63u, kk = k & 31u;
    uint32_t q = (ld32(W, rec + rr * 4u + (kk >> 3)) >> (4u * (kk & 7u))) & 15u;
    uint32_t sm = ld32(W, rec + 256u + rr);
    float sc = orc_h2f((uint16_t)(sm & 0xffffu)), mn = orc_h2f((uint16_t)(sm >> 16));
    float v = (float)q * sc + mn;             /* q*sc is exact in fp32, so fused or not is the same */
    if (f32out) *f32out = v;
    return orc_f2h(v);
  } else if (enc == 1) {   /* src/ops/gemm.js:155-163 */
    size_t rec = ((size_t)(r >> 6) * wG + (k / 64u)) * 1056u; uint32_t rr = r & 63u, kk = k & 63u;
    uint32_t word = ld32(W, rec + rr * 16u + (kk >> 2));
    int32_t q = (int32_t)(word << (24u - 8u * (kk & 3u))) >> 24;
    uint32_t s2 = ld32(W, rec + 1024u + (rr >> 1));
    float sc = orc_h2f((uint16_t)((rr & 1u) ? (s2 >> 16) : (s2 & 0xffffu)));
    float v = (float)q * sc;
    if (f32out) *f32out = v;
    return orc_f2h(v);
  } else {   /* src/ops/gemm.js:165-170 */
    uint16_t h; memcpy(&h, W + ((size_t)r * wG + k) * 2, 2);
    if (f32out) *f32out = orc_h2f(h);
    return h;
  }
}

/* Dequantise rows [r0, r0+nr) x columns [0, K) of an encoded tensor: fp16 bits and/or fp32 values. */
API void orc_dequant(int enc, const uint8_t* W, uint32_t r0, uint32_t nr, uint32_t K, uint32_t ld, uint16_t* h16, float* f32) {
  uint32_t wG = enc == 0 ? K / 32 : enc == 1 ? K / 64 : (ld ? ld : K);
  for (uint32_t r = 0; r < nr; r++) for (uint32_t k = 0; k < K; k++) {
    float v; uint16_t h = wdecode(enc, W, r0 + r, k, wG, &v);
    if (h16) h16[(size_t)r * K + k] = h;
    if (f32) f32[(size_t)r * K + k] = v;
  }
}

/* ------------------------------------------------------------------------------------------------
 * The reference test-suite's CPU multiplications — test/kernels.test.js:29, 52-65, 16-21
 * ---------------------------------------------------------------------------------------------- */

/* cpuAttn (test/kernels.test.js:32-48): Q [Hq][Lq][D], K / V [Hkv][Lk][D] -> O [Lq][Hq*D] (token-major).  Scores are
 * accumulated in double and stored to a float array (the reference's Float32Array s), the maximum is tracked in double,
 * exp(s - mx) is stored as float, the sum and the PV products run in double, O is stored as float.  cap > 0: soft cap. */
API void orc_cpu_attn(const float* Q, const float* Kt, const float* V, float* O, uint32_t Hq, uint32_t Hkv, uint32_t Lq, uint32_t Lk, uint32_t D,
                      uint32_t mode, uint32_t nvalid, double scale, double cap, int threads) {
  const uint32_t grp = Hq / Hkv;
  (void)threads;
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
  for (uint32_t h = 0; h < Hq; h++)
    for (uint32_t i = 0; i < Lq; i++) {
      const uint32_t kh = h / grp;
      float* s = (float*)malloc((size_t)Lk * sizeof(float));
      double mx = -INFINITY;
      for (uint32_t j = 0; j < Lk; j++) {
        const uint32_t lim = i < nvalid - 1u ? i : nvalid - 1u;
        const int vis = mode == 1u ? j <= lim : mode == 2u ? j < nvalid : 1;
        if (!vis) { s[j] = -INFINITY; continue; }
        double a = 0.0;
        for (uint32_t d = 0; d < D; d++) a += (double)Q[((size_t)h * Lq + i) * D + d] * (double)Kt[((size_t)kh * Lk + j) * D + d];
        a *= scale;
        if (cap > 0.0) a = cap * tanh(a / cap);
        s[j] = (float)a;
        if (a > mx) mx = a;
      }
      double sum = 0.0;
      for (uint32_t j = 0; j < Lk; j++) { s[j] = isinf(s[j]) && s[j] < 0 ? 0.0f : (float)exp((double)s[j] - mx); sum += (double)s[j]; }
      for (uint32_t d = 0; d < D; d++) {
        double a = 0.0;
        for (uint32_t j = 0; j < Lk; j++) a += (double)s[j] * (double)V[((size_t)kh * Lk + j) * D + d];
        O[(size_t)i * Hq * D + (size_t)h * D + d] = (float)(a / sum);
      }
      free(s);
    }
}

/* cpuGemm: float64 accumulate, float32 store (test/kernels.test.js:29).  threads<=1: the single-threaded
 * loop of the reference; otherwise OpenMP over rows. */
API void orc_cpu_gemm(const float* X, const float* W, float* Y, uint32_t M, uint32_t N, uint32_t K, int threads) {
  (void)threads;
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
  for (uint32_t m = 0; m < M; m++) for (uint32_t n = 0; n < N; n++) {
    double a = 0; const float* x = X + (size_t)m * K; const float* w = W + (size_t)n * K;
    for (uint32_t k = 0; k < K; k++) a += (double)x[k] * (double)w[k];
    Y[(size_t)m * N + n] = (float)a;
  }
}

/* cpuConv3: THWC clip, 3x3x3, stride 1, time edge frames repeat, zeros in space (test/kernels.test.js:52-65). */
API void orc_cpu_conv3(const float* X, const float* Wt, float* Y, uint32_t T, uint32_t H, uint32_t Wd, uint32_t C, uint32_t N, int threads) {
  (void)threads;
  size_t K = 27 * (size_t)C;
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
  for (uint32_t t = 0; t < T; t++) for (uint32_t y = 0; y < H; y++) for (uint32_t x = 0; x < Wd; x++) for (uint32_t n = 0; n < N; n++) {
    double a = 0;
    for (int kt = 0; kt < 3; kt++) for (int ky = 0; ky < 3; ky++) for (int kx = 0; kx < 3; kx++) {
      int it = (int)t + kt - 1; if (it < 0) it = 0; if (it > (int)T - 1) it = (int)T - 1;
      int iy = (int)y + ky - 1, ix = (int)x + kx - 1;
      if (iy < 0 || ix < 0 || iy >= (int)H || ix >= (int)Wd) continue;
      size_t xo = (((size_t)it * H + iy) * Wd + ix) * C, wo = n * K + (size_t)(kt * 9 + ky * 3 + kx) * C;
      for (uint32_t c = 0; c < C; c++) a += (double)X[xo + c] * (double)Wt[wo + c];
    }
    Y[(((size_t)t * H + y) * Wd + x) * N + n] = (float)a;
  }
}

/* compare: cosine similarity and max abs error, double sums (test/kernels.test.js:16-21). out[0]=cos, out[1]=maxErr */
API void orc_compare(const float* got, const float* want, size_t n, double* out) {
  double dot = 0, ga = 0, wa = 0, me = 0;
  for (size_t i = 0; i < n; i++) {
    double g = got[i], w = want[i]; dot += g * w; ga += g * g; wa += w * w;
    double e = fabs(g - w);
    if (!(e <= me)) me = isfinite(e) ? (e > me ? e : me) : INFINITY;
  }
  double d = ga * wa; if (d < 1e-30) d = 1e-30;
  double c = dot / sqrt(d);
  out[0] = isfinite(c) ? c : 0; out[1] = me;
}

/* ------------------------------------------------------------------------------------------------
 * Full restatement of the shader arithmetic of gemm — src/ops/gemm.js:60-101 (prologues, weight rows),
 * :143-172 (dequantisation), :191-254 (epilogues), with the uniform fields of :39-41 / :317-322.
 *
 * Products use the fp16-rounded activation X' and the fp16-rounded tile value (as the shader does); the
 * sum over k is kept in float64 (as the reference's CPU references do) and rounded to fp32 once, which
 * stands in for the shader's fp32 accumulator.  Epilogue maths is fp32.
 * ---------------------------------------------------------------------------------------------- */
enum { ORC_X_F16 = 0, ORC_X_LNMOD = 1, ORC_X_RMS = 2, ORC_X_CONV = 3, ORC_X_CONV3 = 4 };
enum { ORC_EPI_F16 = 0, ORC_EPI_F32 = 1, ORC_EPI_RESADD = 2, ORC_EPI_SWIGLU = 3, ORC_EPI_HEADS = 4, ORC_EPI_BIAS = 5, ORC_EPI_ONORMGATE = 6 };
enum { ORC_F_GATE = 1, ORC_F_RES = 2, ORC_F_STORE = 4, ORC_F_GN = 8, ORC_F_UP2 = 16, ORC_F_PN = 32, ORC_F_BIAS = 64, ORC_F_GELU = 128, ORC_F_ROPE_HALF = 256 };

typedef struct {
  uint32_t enc, xmode, epi, flags;
  uint32_t M, N, K, ldx, kx0, wR0, wR1, wG, wk0, ldy, ny0;
  uint32_t rowOff, Ltot, Hq, Hkv; float eps;
  uint32_t pvOff, pvStride, evOff, statOff;
  uint32_t Hi, Wi, Ci, Ho, Wo, stride, padT, padL, ks, Nw, bvOff, bvUp;
  const void* X;        /* fp16 (modes f16/conv/conv3) or fp32 (lnmod/rms); already offset by x.off bytes */
  const uint8_t* W;     /* encoded weights, already offset by w.off bytes */
  void* Y;              /* fp16 or fp32 (epi f32/resadd); already offset by y.off bytes */
  const float* ST; const float* PV; const float* EV; const float* BV; const float* RP; const uint16_t* GT;
  int threads;
} orc_gemm_args;

static inline int iclamp(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }
static inline float siluf(float z) { return z / (1.0f + expf(-z)); }

/* X'[row, k] rounded to fp16 then widened — the value xload() returns (src/ops/gemm.js:60-95). */
static float xprime(const orc_gemm_args* a, uint32_t row, uint32_t k) {
  const uint16_t* Xh = (const uint16_t*)a->X; const float* Xf = (const float*)a->X;
  switch (a->xmode) {
    case ORC_X_F16: return orc_h2f(Xh[(size_t)row * a->ldx + a->kx0 + k]);                     /* :62 */
    case ORC_X_LNMOD: {                                                                         /* :64-66 */
      float xv = Xf[(size_t)row * a->ldx + a->kx0 + k]; size_t sr = ((size_t)a->statOff + row) * 2; uint32_t kk = a->kx0 + k;
      float v = (xv - a->ST[sr]) * a->ST[sr + 1] * (1.0f + a->PV[a->pvOff + kk]) + a->PV[a->pvOff + a->pvStride + kk];
      return rf16(v);
    }
    case ORC_X_RMS: {                                                                           /* :64-67 */
      float xv = Xf[(size_t)row * a->ldx + a->kx0 + k]; size_t sr = ((size_t)a->statOff + row) * 2; uint32_t kk = a->kx0 + k;
      return rf16(xv * a->ST[sr + 1] * a->PV[a->pvOff + kk]);
    }
    case ORC_X_CONV3: {                                                                         /* :69-80 */
      uint32_t HW = a->Ho * a->Wo, ot = row / HW, rem = row % HW, oy = rem / a->Wo, ox = rem % a->Wo;
      uint32_t tap = k / a->Ci, c = k % a->Ci, kt = tap / 9, ky = (tap / 3) % 3, kx = tap % 3;
      uint32_t itg = (uint32_t)iclamp((int)(ot + a->padT + kt) - 1, 0, (int)a->stride - 1);
      uint32_t it = a->ks > 1 ? itg % a->ks : itg - a->padL;
      int iy = (int)(oy + ky) - 1, ix = (int)(ox + kx) - 1;
      int ok = iy >= 0 && ix >= 0 && iy < (int)a->Hi && ix < (int)a->Wi;
      size_t vox = ((size_t)it * a->Hi + (uint32_t)iclamp(iy, 0, (int)a->Hi - 1)) * a->Wi + (uint32_t)iclamp(ix, 0, (int)a->Wi - 1);
      float xv = orc_h2f(Xh[vox * a->Ci + c]);
      if (a->flags & ORC_F_PN) { float z = xv * a->ST[vox]; return ok ? rf16(siluf(z)) : 0.0f; }
      return ok ? xv : 0.0f;
    }
    default: {                                                                                  /* conv, :82-91 */
      uint32_t oy = row / a->Wo, ox = row % a->Wo, tap = k / a->Ci, c = k % a->Ci;
      int iy = (int)(oy * a->stride + tap / a->ks) - (int)a->padT, ix = (int)(ox * a->stride + tap % a->ks) - (int)a->padL;
      int up = (a->flags & ORC_F_UP2) ? 1 : 0;
      int HH = (int)(up ? a->Hi * 2 : a->Hi), WW = (int)(up ? a->Wi * 2 : a->Wi);
      int ok = iy >= 0 && ix >= 0 && iy < HH && ix < WW;
      uint32_t sy = (uint32_t)(iy > 0 ? iy : 0) >> up, sx = (uint32_t)(ix > 0 ? ix : 0) >> up;
      if (sy > a->Hi - 1) sy = a->Hi - 1;
      if (sx > a->Wi - 1) sx = a->Wi - 1;
      float xv = orc_h2f(Xh[((size_t)sy * a->Wi + sx) * a->Ci + c]);
      if (a->flags & ORC_F_GN) { float z = xv * a->PV[a->pvOff + c] + a->PV[a->pvOff + a->pvStride + c]; return ok ? rf16(siluf(z)) : 0.0f; }
      return ok ? xv : 0.0f;
    }
  }
}

/* weight row feeding output/ws column `col` (absolute, = nB + cc) (src/ops/gemm.js:98-101) */
static inline uint32_t wrow(const orc_gemm_args* a, uint32_t col) {
  if (a->epi == ORC_EPI_SWIGLU) return ((col & 1u) == 0u ? a->wR0 : a->wR1) + (col >> 1);
  uint32_t r = a->wR0 + col; return r < a->Nw - 1 ? r : a->Nw - 1;
}

static inline float geluf(float g) {   /* src/ops/gemm.js:208 */
  float t = 0.7978845608f * (g + 0.044715f * g * g * g); if (t < -15.0f) t = -15.0f; if (t > 15.0f) t = 15.0f;
  return g * 0.5f * (1.0f + tanhf(t));
}

/* the epilogue of one output row m over the 128-column block starting at nB (or the narrower tail) */
static int epilogue_block(const orc_gemm_args* a, uint32_t m, uint32_t nB, uint32_t nb, const float* acc) {
  uint16_t* Yh = (uint16_t*)a->Y; float* Yf = (float*)a->Y;
  switch (a->epi) {
    case ORC_EPI_F16: for (uint32_t j = 0; j < nb; j++) Yh[(size_t)m * a->ldy + a->ny0 + nB + j] = orc_f2h(acc[j]); return 0;     /* :194-196 */
    case ORC_EPI_F32: for (uint32_t j = 0; j < nb; j++) Yf[(size_t)m * a->ldy + a->ny0 + nB + j] = acc[j]; return 0;
    case ORC_EPI_RESADD:                                                                                                        /* :197-203 */
      for (uint32_t j = 0; j < nb; j++) {
        uint32_t n = nB + j;
        float g = (a->flags & ORC_F_GATE) ? a->EV[a->evOff + n] : 1.0f, c = (a->flags & ORC_F_BIAS) ? a->BV[a->bvOff + n] : 0.0f;
        size_t i = (size_t)m * a->ldy + a->ny0 + n; float v = g * (acc[j] + c);
        Yf[i] = (a->flags & ORC_F_STORE) ? v : Yf[i] + v;
      }
      return 0;
    case ORC_EPI_SWIGLU:                                                                                                        /* :204-210 */
      for (uint32_t j = 0; j + 1 < nb; j += 2) {
        uint32_t o = (nB + j) / 2;
        float gB = (a->flags & ORC_F_BIAS) ? a->BV[a->bvOff + o] : 0.0f, uB = (a->flags & ORC_F_BIAS) ? a->BV[a->bvOff + a->bvUp + o] : 0.0f;
        float g = acc[j] + gB, u = acc[j + 1] + uB;
        float act = (a->flags & ORC_F_GELU) ? geluf(g) : siluf(g);
        Yh[(size_t)m * a->ldy + a->ny0 + o] = orc_f2h(act * u);
      }
      return 0;
    case ORC_EPI_BIAS:                                                                                                          /* :211-215 */
      for (uint32_t j = 0; j < nb; j++) {
        uint32_t n = nB + j; size_t i = (size_t)m * a->ldy + a->ny0 + n; float v = acc[j] + a->EV[a->evOff + n];
        if (a->flags & ORC_F_RES) v += orc_h2f(Yh[i]);
        Yh[i] = orc_f2h(v);
      }
      return 0;
    case ORC_EPI_ONORMGATE: {                                                                                                   /* :227-232 */
      double ss = 0; for (int d = 0; d < 128; d++) ss += (double)acc[d] * (double)acc[d];
      float inv = 1.0f / sqrtf((float)ss / 128.0f + a->eps);
      for (int d = 0; d < 128; d++) {
        float g = orc_h2f(a->GT[(size_t)m * a->Ltot + a->ny0 + nB + d]);
        Yh[(size_t)m * a->ldy + a->ny0 + nB + d] = orc_f2h(acc[d] * inv * a->EV[a->evOff + d] / (1.0f + expf(-g)));
      }
      return 0;
    }
    case ORC_EPI_HEADS: {                                                                                                       /* :216-226, 234-252 */
      uint32_t hd = nB / 128, sec = hd < a->Hq ? 0u : hd < a->Hq + a->Hkv ? 1u : 2u; size_t row = (size_t)a->rowOff + m;
      float v[128]; for (int d = 0; d < 128; d++) v[d] = acc[d];
      if (sec < 2) {
        double ss = 0; for (int d = 0; d < 128; d++) ss += (double)v[d] * (double)v[d];
        float inv = 1.0f / sqrtf((float)ss / 128.0f + a->eps); const float* nw = a->EV + a->evOff + (sec == 0 ? 0 : 128);
        for (int d = 0; d < 128; d++) v[d] = v[d] * inv * nw[d];
        if (a->flags & ORC_F_ROPE_HALF) {         /* pairs (d, d+64), angle index d (:241-244) */
          for (int d = 0; d < 64; d++) {
            float cs = a->RP[row * 128 + 2 * d], sn = a->RP[row * 128 + 2 * d + 1];
            float lo = v[d] * cs - v[d + 64] * sn, hi = v[d + 64] * cs + v[d] * sn; v[d] = lo; v[d + 64] = hi;
          }
        } else {                                  /* interleaved pairs (2p, 2p+1) (:245-249) */
          for (int p = 0; p < 64; p++) {
            float cs = a->RP[row * 128 + 2 * p], sn = a->RP[row * 128 + 2 * p + 1];
            float x0 = v[2 * p], x1 = v[2 * p + 1]; v[2 * p] = x0 * cs - x1 * sn; v[2 * p + 1] = x0 * sn + x1 * cs;
          }
        }
      }
      for (int d = 0; d < 128; d++) Yh[((size_t)hd * a->Ltot + row) * 128 + d] = orc_f2h(v[d]);
      return 0;
    }
    default: return -3;
  }
}

API int orc_gemm(const orc_gemm_args* a) {
  const uint32_t M = a->M, N = a->N, K = a->K;
  if (K % 32) return -1;
  const int red128 = a->epi == ORC_EPI_HEADS || a->epi == ORC_EPI_ONORMGATE;
  /* the shader works on column tiles; columns up to the tile edge exist (clamped weight rows) but only the
   * guarded ones are stored.  Whole 128-wide blocks for the head epilogues, else groups of 4 columns (the
   * store granularity of :196). */
  const uint32_t Ncols = red128 ? ((N + 127u) / 128u) * 128u : ((N + 3u) / 4u) * 4u;
  const int nthr = a->threads > 0 ? a->threads : 1; (void)nthr;
  float* Xp = (float*)malloc(sizeof(float) * (size_t)M * K);
  if (!Xp) return -2;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(nthr)
#endif
  for (uint32_t m = 0; m < M; m++) for (uint32_t k = 0; k < K; k++) Xp[(size_t)m * K + k] = xprime(a, m, k);
  int rc = 0;
  const uint32_t nblocks = (Ncols + 127u) / 128u;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthr)
#endif
  for (uint32_t b = 0; b < nblocks; b++) {
    uint32_t nB = b * 128u, nb = Ncols - nB < 128u ? Ncols - nB : 128u;
    float* Wd = (float*)malloc(sizeof(float) * (size_t)nb * K);
    if (!Wd) { rc = -2; continue; }
    for (uint32_t j = 0; j < nb; j++) { uint32_t r = wrow(a, nB + j); for (uint32_t k = 0; k < K; k++) Wd[(size_t)j * K + k] = orc_h2f(wdecode((int)a->enc, a->W, r, a->wk0 + k, a->wG, NULL)); }
    for (uint32_t m = 0; m < M; m++) {
      float acc[128]; const float* x = Xp + (size_t)m * K;
      for (uint32_t j = 0; j < nb; j++) { double s = 0; const float* w = Wd + (size_t)j * K; for (uint32_t k = 0; k < K; k++) s += (double)x[k] * (double)w[k]; acc[j] = (float)s; }
      int e = epilogue_block(a, m, nB, nb, acc); if (e) rc = e;
    }
    free(Wd);
  }
  free(Xp);
  return rc;
}

/* Row statistics the fused norm prologues consume: ST[(off+r)*2] = (mean, rstd); mode 0 LayerNorm, 1 RMS
 * (src/ops/misc.js:16-44).  Sums in double; the reference kernel sums fp32 in a tree. */
API void orc_rowstats(const float* X, uint32_t rows, uint32_t cols, uint32_t ld, int rms, float eps, float* ST) {
  for (uint32_t r = 0; r < rows; r++) {
    const float* x = X + (size_t)r * ld; double mean = 0;
    if (!rms) { double s = 0; for (uint32_t i = 0; i < cols; i++) s += x[i]; mean = (double)(float)(s / cols); }
    double q = 0; for (uint32_t i = 0; i < cols; i++) { double d = (double)(float)(x[i] - (float)mean); q += d * d; }
    float var = (float)(q / cols);
    ST[2 * (size_t)r] = (float)mean; ST[2 * (size_t)r + 1] = 1.0f / sqrtf(var + eps);
  }
}

/* pixstats (src/ops/video.js:301-318): R[ro + v] = 1 / sqrt(sum_c x[v][c]^2 / C + eps), x fp16 [V][C]; the shader sums
 * vec4 dot products in fp32, the sum is kept in float64 here and rounded once. */
API void orc_pixstats(const uint16_t* X, uint32_t V, uint32_t C, float eps, float* R) {
  for (uint32_t v = 0; v < V; v++) {
    double s = 0;
    for (uint32_t c = 0; c < C; c++) { double x = orc_h2f(X[(size_t)v * C + c]); s += x * x; }
    R[v] = 1.0f / sqrtf((float)(s / C) + eps);
  }
}

/* gnPartial (src/ops/misc.js:50-73): per 64-pixel chunk and group (32 groups of C / 32 channels) the count, the mean and
 * M2 = sum (x - mean)^2 by an exact two-pass over the chunk; PT[(wgOff + wg) * 32 + g] = (n, mean, M2, 0).  Sums in float64,
 * the mean rounded to fp32 before the second pass as in the shader. */
API void orc_gn_partial(const uint16_t* X, uint32_t pix, uint32_t C, uint32_t wgOff, float* PT) {
  const uint32_t nwg = (pix + 63u) / 64u, cpg = C / 32u;
  for (uint32_t wg = 0; wg < nwg; wg++) {
    const uint32_t px0 = wg * 64u, npx = pix - px0 < 64u ? pix - px0 : 64u;
    const float cnt = (float)(npx * cpg);
    for (uint32_t g = 0; g < 32u; g++) {
      double s = 0;
      for (uint32_t p = 0; p < npx; p++) for (uint32_t j = 0; j < cpg; j++) s += orc_h2f(X[((size_t)px0 + p) * C + g * cpg + j]);
      const float mean = (float)(s / (cnt > 1.0f ? cnt : 1.0f));
      double m2 = 0;
      for (uint32_t p = 0; p < npx; p++) for (uint32_t j = 0; j < cpg; j++) { double d = (double)(float)(orc_h2f(X[((size_t)px0 + p) * C + g * cpg + j]) - mean); m2 += d * d; }
      float* o = PT + (((size_t)wgOff + wg) * 32u + g) * 4u;
      o[0] = cnt; o[1] = mean; o[2] = (float)m2; o[3] = 0.0f;
    }
  }
}

/* gnFinalize (src/ops/misc.js:75-104): Chan's merge of the partial rows in row order (fp32, as the shader), then
 * a[c] = gamma[c] * rstd, b[c] = beta[c] - mean * a[c]; AB = a[C] then b[C]. */
API void orc_gn_finalize(const float* PT, uint32_t nwg, uint32_t C, float eps, const float* gamma, const float* beta, float* AB) {
  const uint32_t cpg = C / 32u;
  for (uint32_t g = 0; g < 32u; g++) {
    float n = 0, mean = 0, m2 = 0;
    for (uint32_t w = 0; w < nwg; w++) {
      const float* q = PT + ((size_t)w * 32u + g) * 4u;
      if (q[0] > 0.0f) { float nn = n + q[0], d = q[1] - mean; mean = mean + d * (q[0] / nn); m2 = m2 + q[2] + d * d * (n * q[0] / nn); n = nn; }
    }
    const float rs = 1.0f / sqrtf(m2 / (n > 1.0f ? n : 1.0f) + eps);
    for (uint32_t c = g * cpg; c < (g + 1u) * cpg; c++) { const float a = gamma[c] * rs; AB[c] = a; AB[C + c] = beta[c] - mean * a; }
  }
}

API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
