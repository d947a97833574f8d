// Producers of the statistics the fused prologues of gemm read: per-voxel PixelNorm factors for conv3's `pn` (pixstats,
// src/ops/video.js:301-318) and the GroupNorm scale / offset per channel for conv's `gn` (gnPartial + gnFinalize,
// src/ops/misc.js:50-120).  Bandwidth kernels: the tensor is read once (twice inside a 64-pixel chunk for the exact
// two-pass variance, the second time from L1 / L2).
#include "common.cuh"
#include "ctx.h"

using namespace p0p;

namespace {

// ---- pixstats: R[ro + v] = rsqrt(sum_c x[v][c]^2 / C + eps), x fp16 [V][C].  L lanes share a voxel (16-byte loads).
__global__ void __launch_bounds__(256) k_pixstats(const __half* __restrict__ X, uint32_t V, uint32_t C, uint32_t L, float eps, float* __restrict__ R, uint32_t vec) {
  const uint32_t gt = blockIdx.x * blockDim.x + threadIdx.x, sub = gt % L;
  const uint32_t v = gt / L;
  float s = 0.0f;
  if (v < V) {
    const __half* x = X + (size_t)v * C;
    if (vec) {
      for (uint32_t c = sub * 8u; c < C; c += L * 8u) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + c));
        const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h[i]); s = fmaf(f.x, f.x, s); s = fmaf(f.y, f.y, s); }
      }
    } else {
      for (uint32_t c = sub; c < C; c += L) { const float f = __half2float(x[c]); s = fmaf(f, f, s); }
    }
  }
  for (uint32_t o = L >> 1; o > 0u; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);      // L is a power of two <= 32: partners stay inside the voxel's lanes
  if (v < V && sub == 0u) R[v] = rsqrtf(s / (float)C + eps);
}

// ---- GroupNorm partial statistics: one block per 64 pixels of an HWC fp16 tensor [pix][C], 32 groups of C / 32 channels.
// PT[(wgOff + block) * 32 + g] = (count, mean, M2, 0) of the block's own chunk, by an exact two-pass (src/ops/misc.js:50-73).
// C is a power of two (32..512), so a thread's eight consecutive elements are the same eight channels in every round of 2048
// elements: per-thread channel sums -> per-channel sums over the threads that share channels -> per-group sums, all in a
// fixed order (deterministic).
__global__ void __launch_bounds__(256) k_gn_partial(const __half* __restrict__ X, uint32_t pix, uint32_t C, uint32_t wgOff, float4* __restrict__ PT) {
  __shared__ float part[256][9];      // per thread, per element of its 8 (padded against bank conflicts)
  __shared__ float chs[512];          // per channel
  __shared__ float mg[32];            // group means
  const uint32_t t = threadIdx.x, wg = blockIdx.x, px0 = wg * 64u, npx = min(64u, pix - min(px0, pix));
  const uint32_t n = npx * C, cpg = C / 32u, c0 = (t * 8u) % C, reps = 2048u / C, per = C / 8u;
  const __half* x = X + (size_t)px0 * C;
  const float cnt = (float)(npx * cpg);
  float acc[8];
  auto reduce_groups = [&](float* out32) {      // acc[] of all threads -> out32[g]; ends with a barrier
#pragma unroll
    for (int j = 0; j < 8; j++) part[t][j] = acc[j];
    __syncthreads();
    for (uint32_t c = t; c < C; c += 256u) { float s = 0.0f; for (uint32_t r = 0; r < reps; r++) s += part[c / 8u + r * per][c % 8u]; chs[c] = s; }
    __syncthreads();
    if (t < 32u) { float s = 0.0f; for (uint32_t j = 0; j < cpg; j++) s += chs[t * cpg + j]; out32[t] = s; }
    __syncthreads();
  };
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.0f;
  for (uint32_t e = t * 8u; e < n; e += 2048u) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + e));
    const __half* h = reinterpret_cast<const __half*>(&q);
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] += __half2float(h[j]);
  }
  reduce_groups(mg);
  if (t < 32u) mg[t] = mg[t] / fmaxf(cnt, 1.0f);
  __syncthreads();
  float mean[8];
#pragma unroll
  for (int j = 0; j < 8; j++) { mean[j] = mg[(c0 + j) / cpg]; acc[j] = 0.0f; }
  for (uint32_t e = t * 8u; e < n; e += 2048u) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + e));
    const __half* h = reinterpret_cast<const __half*>(&q);
#pragma unroll
    for (int j = 0; j < 8; j++) { const float d = __half2float(h[j]) - mean[j]; acc[j] = fmaf(d, d, acc[j]); }
  }
  __shared__ float m2[32];
  reduce_groups(m2);
  if (t < 32u) PT[((size_t)wgOff + wg) * 32u + t] = make_float4(cnt, mg[t], m2[t], 0.0f);
}

// ---- merge of the partial rows with Chan's parallel formula (src/ops/misc.js:75-104) -> per channel a = gamma * rstd,
// b = beta - mean * a.  Block = 32 groups x 32 lanes: a lane merges every 32nd row in order, then the 32 lane results
// merge pairwise (the formula is symmetric).
struct Chan { float n, mean, m2; };
__device__ __forceinline__ Chan chan_merge(Chan a, Chan b) {
  if (!(b.n > 0.0f)) return a;
  if (!(a.n > 0.0f)) return b;
  const float nn = a.n + b.n, d = b.mean - a.mean;
  Chan r; r.n = nn; r.mean = a.mean + d * (b.n / nn); r.m2 = a.m2 + b.m2 + d * d * (a.n * b.n / nn);
  return r;
}
__global__ void __launch_bounds__(1024) k_gn_finalize(const float4* __restrict__ PT, uint32_t nwg, uint32_t C, float eps, const float* __restrict__ GB, uint32_t gOff, uint32_t bOff,
                                                      float* __restrict__ AB) {
  const uint32_t g = threadIdx.x >> 5, l = threadIdx.x & 31u;
  Chan s{0.0f, 0.0f, 0.0f};
  for (uint32_t w = l; w < nwg; w += 32u) { const float4 q = __ldg(PT + (size_t)w * 32u + g); s = chan_merge(s, Chan{q.x, q.y, q.z}); }
  for (uint32_t o = 1; o < 32u; o <<= 1) {
    Chan b; b.n = __shfl_xor_sync(0xffffffffu, s.n, o); b.mean = __shfl_xor_sync(0xffffffffu, s.mean, o); b.m2 = __shfl_xor_sync(0xffffffffu, s.m2, o);
    s = (l & o) ? chan_merge(b, s) : chan_merge(s, b);      // both partners merge (lower, upper): the same value on both
  }
  const float rs = rsqrtf(s.m2 / fmaxf(s.n, 1.0f) + eps);
  const uint32_t cpg = C / 32u;
  for (uint32_t j = l; j < cpg; j += 32u) {
    const uint32_t c = g * cpg + j;
    const float a = __ldg(GB + gOff + c) * rs;
    AB[c] = a; AB[C + c] = __ldg(GB + bOff + c) - s.mean * a;
  }
}

inline bool live(const p0p_ctx* c, const p0p_buf* b) { return b && c->bufs.count(const_cast<p0p_buf*>(b)); }

}  // namespace

extern "C" int p0p_pixstats(p0p_ctx* c, const p0p_buf* x, uint64_t x_off, uint32_t V, uint32_t C, float eps, p0p_buf* r, uint32_t ro) {
  P0P_ALIVE(c);
  if (!live(c, x) || !live(c, r)) return fail(c, -4, "pixstats: missing binding");
  if (!V || !C) return 0;
  if (C % 4u) return fail(c, -5, "pixstats: C must be a multiple of 4");                  // the reference reads vec4<f16>
  if (x_off & 7u) return fail(c, -5, "pixstats: x.off must be a multiple of 8 bytes");
  const uint64_t xb = (uint64_t)V * C * 2ull, rb = ((uint64_t)ro + V) * 4ull;
  if (x_off > x->size || xb > x->size - x_off || rb > r->size) return fail(c, -7, "pixstats: a range is outside its buffer");
  DeviceGuard g(c->device);
  const __half* X = reinterpret_cast<const __half*>((const char*)x->ptr + x_off);
  const uint32_t vec = (C % 8u == 0u && ((uintptr_t)X & 15u) == 0u) ? 1u : 0u;
  uint32_t L = 1u; while (L < 32u && L * (vec ? 8u : 1u) < C) L <<= 1;                     // lanes per voxel: enough for one load each, at most a warp
  const uint64_t threads = (uint64_t)V * L;
  k_pixstats<<<(unsigned)((threads + 255u) / 256u), 256, 0, c->stream>>>(X, V, C, L, eps != 0.0f ? eps : 1e-8f, (float*)r->ptr + ro, vec);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "pixstats launch");
  c->launches += 1;
  return 0;
}

extern "C" int p0p_gn_partial(p0p_ctx* c, const p0p_buf* x, uint64_t x_off, uint32_t pix, uint32_t C, p0p_buf* part, uint32_t wgOff, uint32_t* nwg_out) {
  P0P_ALIVE(c);
  const uint32_t nwg = (pix + 63u) / 64u;
  if (nwg_out) *nwg_out = nwg;
  if (!live(c, x) || !live(c, part)) return fail(c, -4, "gnPartial: missing binding");
  if (!pix) return 0;
  if (C < 32u || C > 512u || (C & (C - 1u))) return fail(c, -5, "gnPartial: C must be a power of two from 32 to 512");      // src/ops/misc.js:110
  if (x_off & 15u) return fail(c, -5, "gnPartial: x.off must be a multiple of 16 bytes");
  const uint64_t xb = (uint64_t)pix * C * 2ull, pb = ((uint64_t)wgOff + nwg) * 512ull;
  if (x_off > x->size || xb > x->size - x_off || pb > part->size) return fail(c, -7, "gnPartial: a range is outside its buffer");
  DeviceGuard g(c->device);
  k_gn_partial<<<nwg, 256, 0, c->stream>>>(reinterpret_cast<const __half*>((const char*)x->ptr + x_off), pix, C, wgOff, (float4*)part->ptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "gnPartial launch");
  c->launches += 1;
  return 0;
}

extern "C" int p0p_gn_finalize(p0p_ctx* c, const p0p_buf* part, uint32_t nwg, uint32_t C, float eps, const p0p_buf* gb, uint32_t g_off, uint32_t b_off,
                               p0p_buf* ab, uint32_t ab_off) {
  P0P_ALIVE(c);
  if (!live(c, part) || !live(c, gb) || !live(c, ab)) return fail(c, -4, "gnFinalize: missing binding");
  if (C < 32u || C > 512u || (C & (C - 1u))) return fail(c, -5, "gnFinalize: C must be a power of two from 32 to 512");
  if ((uint64_t)nwg * 512ull > part->size || ((uint64_t)std::max(g_off, b_off) + C) * 4ull > gb->size || ((uint64_t)ab_off + 2ull * C) * 4ull > ab->size)
    return fail(c, -7, "gnFinalize: a range is outside its buffer");
  DeviceGuard g(c->device);
  k_gn_finalize<<<1, 1024, 0, c->stream>>>((const float4*)part->ptr, nwg, C, eps != 0.0f ? eps : 1e-6f, (const float*)gb->ptr, g_off, b_off, (float*)ab->ptr + ab_off);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "gnFinalize launch");
  c->launches += 1;
  return 0;
}
