// Small kernels beside the multiply: the dequantisation dump used to pin tile values bit for bit, and the
// row statistics (mean, rstd) the fused norm prologues read (src/ops/misc.js:16-44).
#pragma once
#include "common.cuh"

namespace p0p {

// One thread per (row, 32-column group): writes f16 tile values row-major [nr][cols].
// path 0: fp32 fma + one rounding per value.  path 1: the packed half2 conversion of the tensor-core kernels
// (q4_row32 / q8_row of common.cuh, with their exactness tests and fallbacks).
__global__ void k_dequant(uint32_t enc, const uint8_t* __restrict__ W, uint32_t wG, uint32_t cols, uint32_t r0, uint32_t nr, uint32_t path, __half* __restrict__ out) {
  const uint32_t groups = cols / 32u;
  const size_t n = (size_t)nr * groups, idx0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx0 < n;
  const size_t idx = live ? idx0 : n - 1u;        // surplus threads repeat the last item (the conversions are whole-warp operations) and store nothing
  const uint32_t lr = (uint32_t)(idx / groups), g = (uint32_t)(idx % groups), r = r0 + lr, rr = r & 63u;
  __half2 v[16];
  if (enc == P0P_ENC_Q4) {
    const uint8_t* rec = W + ((size_t)(r >> 6) * wG + g) * 1280u;
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(rec + rr * 16u));
    const uint32_t sm = ldg32(rec + 1024u + rr * 4u);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    if (path == 1u) q4_row32(w, sm, v);
    else {
      const float s = __half2float(__ushort_as_half((unsigned short)(sm & 0xffffu))), mn = __half2float(__ushort_as_half((unsigned short)(sm >> 16)));
#pragma unroll
      for (int i = 0; i < 16; i++) v[i] = __halves2half2(deq_q4((w[i >> 2] >> (8 * (i & 3))) & 15u, s, mn), deq_q4((w[i >> 2] >> (8 * (i & 3) + 4)) & 15u, s, mn));
    }
  } else if (enc == P0P_ENC_Q8) {
    const uint8_t* rec = W + ((size_t)(r >> 6) * wG + (g >> 1)) * 4224u;
    const uint4* cp = reinterpret_cast<const uint4*>(rec + rr * 64u + (g & 1u) * 32u);
    const uint4 qa = __ldg(cp), qb = __ldg(cp + 1);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const unsigned short hsb = __ldg(reinterpret_cast<const unsigned short*>(rec + 4096u + rr * 2u));
    if (path == 1u) q8_row<8>(w, hsb, v);
    else {
      const float s = __half2float(__ushort_as_half(hsb));
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const uint32_t x = w[i >> 1] >> (16 * (i & 1));
        v[i] = __halves2half2(deq_q8((int)(signed char)(x & 255u), s), deq_q8((int)(signed char)((x >> 8) & 255u), s));
      }
    }
  } else {
    const unsigned short* rp = reinterpret_cast<const unsigned short*>(W) + (size_t)r * wG + g * 32u;
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __halves2half2(__ushort_as_half(__ldg(rp + 2 * i)), __ushort_as_half(__ldg(rp + 2 * i + 1)));
  }
  if (!live) return;
  __half2* o = reinterpret_cast<__half2*>(out + (size_t)lr * cols + g * 32u);
#pragma unroll
  for (int i = 0; i < 16; i++) o[i] = v[i];
}

inline cudaError_t launch_dequant(uint32_t enc, const uint8_t* W, uint32_t wG, uint32_t cols, uint32_t r0, uint32_t nr, uint32_t path, __half* out, cudaStream_t st) {
  const size_t n = (size_t)nr * (cols / 32u);
  k_dequant<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(enc, W, wG, cols, r0, nr, path, out);
  return cudaGetLastError();
}

// ST[r*2] = (mean, rstd): mode 0 LayerNorm (mean removed), 1 RMS (mean = 0).  One block per row, fp32 sums,
// two passes like the reference kernel (mean first, then squared deviations).
__global__ void __launch_bounds__(256) k_rowstats(const float* __restrict__ X, uint32_t ld, uint32_t c0, uint32_t cols, uint32_t mode, float eps, float* __restrict__ ST) {
  __shared__ float red[8];
  const uint32_t row = blockIdx.x, t = threadIdx.x;
  const float* x = X + (size_t)row * ld + c0;
  auto block_sum = [&](float v) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((t & 31u) == 0) red[t >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) s += red[i];
    return s;
  };
  float mean = 0.0f;
  if (mode == 0u) { float s = 0.0f; for (uint32_t i = t; i < cols; i += 256u) s += x[i]; mean = block_sum(s) / (float)cols; }
  float q = 0.0f;
  for (uint32_t i = t; i < cols; i += 256u) { const float d = x[i] - mean; q = fmaf(d, d, q); }
  const float var = block_sum(q) / (float)cols;
  if (t == 0) { ST[(size_t)row * 2u] = mean; ST[(size_t)row * 2u + 1u] = rsqrtf(var + eps); }
}

inline cudaError_t launch_rowstats(const float* X, uint32_t ld, uint32_t c0, uint32_t rows, uint32_t cols, uint32_t mode, float eps, float* ST, cudaStream_t st) {
  k_rowstats<<<rows, 256, 0, st>>>(X, ld, c0, cols, mode, eps, ST);
  return cudaGetLastError();
}

}  // namespace p0p
