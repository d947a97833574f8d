// The general kernel: every prologue, every epilogue, every encoding, any alignment.  A CUDA-core tile
// kernel (64 x 128 outputs per block, 32-k steps through shared memory, fp32 accumulation of products of
// fp16-rounded operands) that serves the configurations the tensor-core kernels do not take and is the
// in-library cross-check for them.  Arithmetic follows the reference shader: src/ops/gemm.js:60-101
// (prologues, weight rows), :143-172 (tile values), :191-254 (epilogues).
#pragma once
#include "common.cuh"

namespace p0p {

constexpr int G_BM = 64, G_BN = 128, G_BK = 32, G_THREADS = 256;
constexpr int G_XS_LD = G_BM + 8, G_WS_LD = G_BN + 8;   // halves; padding keeps 16-byte row alignment

// One prologue-applied activation, fp16-rounded: the value xload() yields (src/ops/gemm.js:60-95).
template <int XMODE>
__device__ __forceinline__ __half xvalue(const KP& p, uint32_t row, uint32_t k) {
  if (XMODE == P0P_X_F16) {
    return __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p.X) + (size_t)row * p.ldx + p.kx0 + k));
  } else if (XMODE == P0P_X_LNMOD || XMODE == P0P_X_RMS) {
    float xv = __ldg(reinterpret_cast<const float*>(p.X) + (size_t)row * p.ldx + p.kx0 + k);
    size_t sr = ((size_t)p.statOff + row) * 2u; uint32_t kk = p.kx0 + k;
    if (XMODE == P0P_X_LNMOD)
      return __float2half_rn((xv - __ldg(p.ST + sr)) * __ldg(p.ST + sr + 1) * (1.0f + __ldg(p.PV + p.pvOff + kk)) + __ldg(p.PV + p.pvOff + p.pvStride + kk));
    return __float2half_rn(xv * __ldg(p.ST + sr + 1) * __ldg(p.PV + p.pvOff + kk));
  } else if (XMODE == P0P_X_CONV3) {
    uint32_t HW = p.Ho * p.Wo, ot = row / HW, rem = row % HW, oy = rem / p.Wo, ox = rem % p.Wo;
    uint32_t tap = k / p.Ci, c = k % p.Ci, kt = tap / 9u, ky = (tap / 3u) % 3u, kx = tap % 3u;
    int itg = min(max((int)(ot + p.padT + kt) - 1, 0), (int)p.stride - 1);
    uint32_t it = p.ks > 1u ? (uint32_t)itg % p.ks : (uint32_t)itg - p.padL;
    int iy = (int)(oy + ky) - 1, ix = (int)(ox + kx) - 1;
    bool ok = iy >= 0 && ix >= 0 && iy < (int)p.Hi && ix < (int)p.Wi;
    size_t vox = ((size_t)it * p.Hi + (uint32_t)min(max(iy, 0), (int)p.Hi - 1)) * p.Wi + (uint32_t)min(max(ix, 0), (int)p.Wi - 1);
    __half xv = __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p.X) + vox * p.Ci + c));
    if (p.flags & P0P_F_PN) { float z = __half2float(xv) * __ldg(p.ST + vox); return ok ? __float2half_rn(silu_exact(z)) : __ushort_as_half(0); }
    return ok ? xv : __ushort_as_half(0);
  } else {   // conv
    uint32_t oy = row / p.Wo, ox = row % p.Wo, tap = k / p.Ci, c = k % p.Ci;
    int iy = (int)(oy * p.stride + tap / p.ks) - (int)p.padT, ix = (int)(ox * p.stride + tap % p.ks) - (int)p.padL;
    const int up = (p.flags & P0P_F_UP2) ? 1 : 0;
    int HH = (int)(p.Hi << up), WW = (int)(p.Wi << up);
    bool ok = iy >= 0 && ix >= 0 && iy < HH && ix < WW;
    uint32_t sy = min((uint32_t)max(iy, 0) >> up, p.Hi - 1u), sx = min((uint32_t)max(ix, 0) >> up, p.Wi - 1u);
    __half xv = __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p.X) + ((size_t)sy * p.Wi + sx) * p.Ci + c));
    if (p.flags & P0P_F_GN) { float z = __half2float(xv) * __ldg(p.PV + p.pvOff + c) + __ldg(p.PV + p.pvOff + p.pvStride + c); return ok ? __float2half_rn(silu_exact(z)) : __ushort_as_half(0); }
    return ok ? xv : __ushort_as_half(0);
  }
}

// weight row behind tile column `col` (absolute) — wrow(), src/ops/gemm.js:98-101
__device__ __forceinline__ uint32_t wrow_of(const KP& p, uint32_t col) {
  if (p.epi == P0P_EPI_SWIGLU) return min(((col & 1u) ? p.wR1 : p.wR0) + (col >> 1), p.Nw - 1u);   // clamp added: tail columns of a partial tile
  return min(p.wR0 + col, p.Nw - 1u);
}

template <int XMODE>
__global__ void __launch_bounds__(G_THREADS) k_gemm_generic(const KP p) {
  __shared__ __align__(16) __half xs[G_BK * G_XS_LD];   // [k][m]
  __shared__ __align__(16) __half ws[G_BK * G_WS_LD];   // [k][n]
  const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
  const uint32_t mB = blockIdx.y * G_BM, nB = blockIdx.x * G_BN;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

  // loaders: X — row tid/4, 8 consecutive k from (tid%4)*8; W — column tid/2, 16 consecutive k from (tid%2)*16
  const uint32_t xr = tid >> 2, xk = (tid & 3u) * 8u;
  const uint32_t xrow = min(mB + xr, p.M - 1u);                  // rows clamped like the shader (:136-137)
  const uint32_t wc = tid >> 1, wk = (tid & 1u) * 16u;
  const uint32_t wr = wrow_of(p, nB + wc);

  for (uint32_t k0 = 0; k0 < p.K; k0 += G_BK) {
    // ---- X tile
    {
      __half v[8];
      if (XMODE == P0P_X_F16 && p.vecx) {
        uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.X) + (size_t)xrow * p.ldx + p.kx0 + k0 + xk));
        *reinterpret_cast<uint4*>(v) = q;
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = xvalue<XMODE>(p, xrow, k0 + xk + i);
      }
#pragma unroll
      for (int i = 0; i < 8; i++) xs[(xk + i) * G_XS_LD + xr] = v[i];
    }
    // ---- W tile (tile values rounded to fp16)
    {
      const uint32_t ka = p.wk0 + k0 + wk;
      __half v[16];
      if (p.enc == P0P_ENC_Q4) {
        const uint8_t* rec = p.W + ((size_t)(wr >> 6) * p.wG + (ka >> 5)) * 1280u; const uint32_t rr = wr & 63u;
        uint32_t w0 = ldg32(rec + rr * 16u + ((ka & 31u) >> 3) * 4u), w1 = ldg32(rec + rr * 16u + ((ka & 31u) >> 3) * 4u + 4u);
        uint32_t sm = ldg32(rec + 1024u + rr * 4u);
        float s = __half2float(__ushort_as_half((unsigned short)(sm & 0xffffu))), mn = __half2float(__ushort_as_half((unsigned short)(sm >> 16)));
#pragma unroll
        for (int i = 0; i < 8; i++) { v[i] = deq_q4((w0 >> (4 * i)) & 15u, s, mn); v[8 + i] = deq_q4((w1 >> (4 * i)) & 15u, s, mn); }
      } else if (p.enc == P0P_ENC_Q8) {
        const uint8_t* rec = p.W + ((size_t)(wr >> 6) * p.wG + (ka >> 6)) * 4224u; const uint32_t rr = wr & 63u;
        const uint8_t* cp = rec + rr * 64u + (ka & 63u);
        float s = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(rec + 4096u + rr * 2u))));
#pragma unroll
        for (int w = 0; w < 4; w++) {
          uint32_t q = ldg32(cp + 4 * w);
#pragma unroll
          for (int i = 0; i < 4; i++) v[4 * w + i] = deq_q8(((int)(q << (24 - 8 * i))) >> 24, s);
        }
      } else {
        const unsigned short* rp = reinterpret_cast<const unsigned short*>(p.W) + (size_t)wr * p.wG + ka;
        if (p.vecw) {
          *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(rp));
          *reinterpret_cast<uint4*>(v + 8) = __ldg(reinterpret_cast<const uint4*>(rp) + 1);
        } else {
#pragma unroll
          for (int i = 0; i < 16; i++) v[i] = __ushort_as_half(__ldg(rp + i));
        }
      }
#pragma unroll
      for (int i = 0; i < 16; i++) ws[(wk + i) * G_WS_LD + wc] = v[i];
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < G_BK; k++) {
      const uint2 xq = *reinterpret_cast<const uint2*>(&xs[k * G_XS_LD + ty * 4]);
      const uint4 wq = *reinterpret_cast<const uint4*>(&ws[k * G_WS_LD + tx * 8]);
      const __half2* xh = reinterpret_cast<const __half2*>(&xq); const __half2* wh = reinterpret_cast<const __half2*>(&wq);
      float xf[4], wf[8];
#pragma unroll
      for (int i = 0; i < 2; i++) { float2 f = __half22float2(xh[i]); xf[2 * i] = f.x; xf[2 * i + 1] = f.y; }
#pragma unroll
      for (int i = 0; i < 4; i++) { float2 f = __half22float2(wh[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(xf[i], wf[j], acc[i][j]);
    }
    __syncthreads();
  }

  // ---- epilogues (src/ops/gemm.js:191-254).  This thread: rows mB+ty*4+i, columns nB+tx*8+j.
  const uint32_t c0 = nB + tx * 8u;
  __half* Yh = reinterpret_cast<__half*>(p.Y); float* Yf = reinterpret_cast<float*>(p.Y);
  const uint32_t epi = p.epi;
  if (epi == P0P_EPI_HEADS || epi == P0P_EPI_ONORMGATE) {
    // sum of squares over the 128 columns of the head: 16 consecutive lanes hold one row
    float ss[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; j++) s = fmaf(acc[i][j], acc[i][j], s);
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      ss[i] = s;
    }
    if (epi == P0P_EPI_ONORMGATE) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t m = mB + ty * 4u + i; if (m >= p.M) continue;
        const float inv = rsqrtf(ss[i] / 128.0f + p.eps);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float g = __half2float(p.GT[(size_t)m * p.Ltot + p.ny0 + c0 + j]);
          Yh[(size_t)m * p.ldy + p.ny0 + c0 + j] = __float2half_rn(acc[i][j] * inv * __ldg(p.EV + p.evOff + tx * 8u + j) / (1.0f + expf(-g)));
        }
      }
      return;
    }
    const uint32_t hd = nB / 128u, sec = hd < p.Hq ? 0u : hd < p.Hq + p.Hkv ? 1u : 2u;
    const float* nw = p.EV + p.evOff + (sec == 0u ? 0u : 128u);
    const bool half_mode = (p.flags & P0P_F_ROPE_HALF) != 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t m = mB + ty * 4u + i;
      const size_t row = (size_t)p.rowOff + min(m, p.M - 1u);
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = acc[i][j];
      if (sec < 2u) {
        const float inv = rsqrtf(ss[i] / 128.0f + p.eps);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = v[j] * inv * __ldg(nw + tx * 8u + j);
        if (half_mode) {   // pairs (d, d+64): partner columns sit 8 lanes away
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 8);
            const uint32_t d = (tx * 8u + j) & 63u;
            const float cs = __ldg(p.RP + row * 128u + 2u * d), sn = __ldg(p.RP + row * 128u + 2u * d + 1u);
            v[j] = tx < 8u ? v[j] * cs - other * sn : v[j] * cs + other * sn;
          }
        } else {           // interleaved pairs (2p, 2p+1)
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const uint32_t pr = (tx * 8u + j) >> 1;
            const float cs = __ldg(p.RP + row * 128u + 2u * pr), sn = __ldg(p.RP + row * 128u + 2u * pr + 1u);
            const float x0 = v[j], x1 = v[j + 1];
            v[j] = x0 * cs - x1 * sn; v[j + 1] = x0 * sn + x1 * cs;
          }
        }
      }
      if (m < p.M) {
        __half2 o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) o[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4*>(Yh + ((size_t)hd * p.Ltot + row) * 128u + tx * 8u) = *reinterpret_cast<uint4*>(o);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t m = mB + ty * 4u + i; if (m >= p.M) continue;
    if (epi == P0P_EPI_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const uint32_t col = c0 + j; if (col >= p.N) continue;
        const uint32_t o = col >> 1;
        float g = acc[i][j], u = acc[i][j + 1];
        if (p.flags & P0P_F_BIAS) { g += __ldg(p.BV + p.bvOff + o); u += __ldg(p.BV + p.bvOff + p.bvUp + o); }
        const float a = (p.flags & P0P_F_GELU) ? gelu_tanh(g) : silu_exact(g);
        Yh[(size_t)m * p.ldy + p.ny0 + o] = __float2half_rn(a * u);
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint32_t col = c0 + j;
      if ((col & ~3u) >= p.N) continue;                 // stores go in groups of four columns (:196)
      const size_t yi = (size_t)m * p.ldy + p.ny0 + col;
      const float a = acc[i][j];
      if (epi == P0P_EPI_F16) Yh[yi] = __float2half_rn(a);
      else if (epi == P0P_EPI_F32) Yf[yi] = a;
      else if (epi == P0P_EPI_RESADD) {
        const float g = (p.flags & P0P_F_GATE) ? __ldg(p.EV + p.evOff + col) : 1.0f;
        const float c = (p.flags & P0P_F_BIAS) ? __ldg(p.BV + p.bvOff + col) : 0.0f;
        const float v = g * (a + c);
        Yf[yi] = (p.flags & P0P_F_STORE) ? v : Yf[yi] + v;
      } else {   // bias
        float v = a + __ldg(p.EV + p.evOff + col);
        if (p.flags & P0P_F_RES) v += __half2float(Yh[yi]);
        Yh[yi] = __float2half_rn(v);
      }
    }
  }
}

inline cudaError_t launch_generic(const KP& p, cudaStream_t st) {
  dim3 grid((p.N + G_BN - 1) / G_BN, (p.M + G_BM - 1) / G_BM);
  switch (p.xmode) {
    case P0P_X_F16: k_gemm_generic<P0P_X_F16><<<grid, G_THREADS, 0, st>>>(p); break;
    case P0P_X_LNMOD: k_gemm_generic<P0P_X_LNMOD><<<grid, G_THREADS, 0, st>>>(p); break;
    case P0P_X_RMS: k_gemm_generic<P0P_X_RMS><<<grid, G_THREADS, 0, st>>>(p); break;
    case P0P_X_CONV: k_gemm_generic<P0P_X_CONV><<<grid, G_THREADS, 0, st>>>(p); break;
    default: k_gemm_generic<P0P_X_CONV3><<<grid, G_THREADS, 0, st>>>(p); break;
  }
  return cudaGetLastError();
}

}  // namespace p0p
