// Flash attention, head_dim 128 (src/ops/attention.js): Q [Hq][Lq][128] f16, K / V [Hkv][Lk][128] f16 (head-major, as the
// GEMM's 'heads' epilogue writes them), O [Lq][ldo] f16 token-major at column h * 128.  fp32 scores, online-softmax
// statistics and accumulators; the Lq x Lk score matrix never leaves the block.
//   mask 0 = none; 1 = causal + valid length (key j visible to query i iff j <= min(i, nvalid - 1)); 2 = valid length (j < nvalid)
//   GQA: query head h reads kv head h / (Hq / Hkv)                                            (attention.js:8-10, 64, 93-99)
// One block = 64 queries of one head, 4 warps x 16 queries; key tiles of 64 through shared memory; QK^T and PV on the
// tensor cores (mma.sync m16n8k16; V fragments by ldmatrix.trans).  The step after the 'heads' projection, not part of the
// gemm path itself: a first, correct kernel, not yet a tcgen05 one.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace p0p {

struct AttnP {
  const __half* Q; const __half* K; const __half* V; __half* O;
  uint32_t Lq, Lk, ldo, Hq, Hkv, mode, nvalid;
  float scale_log2;      // scale * log2(e): the softmax runs on exp2
};

constexpr int AT_BQ = 64, AT_BK = 64, AT_LD = 136;                       // 136 halves per row: fragment loads and ldmatrix rows hit distinct banks
constexpr int AT_TILE = AT_BK * AT_LD;                                   // halves of one K or V tile
constexpr int AT_SMEM = 4 * AT_TILE * 2;                                 // two stages of (K, V); the Q tile borrows the first before the key loop

__device__ __forceinline__ void at_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void at_cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void at_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void at_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) { __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h); }

__global__ void __launch_bounds__(128) k_attn128(const AttnP p) {
  extern __shared__ __align__(16) unsigned char at_smem[];
  __half* Qs = reinterpret_cast<__half*>(at_smem); __half* KV = Qs;                            // KV: [stage][K | V][64][AT_LD]; Q lives there until its fragments are in registers
  const uint32_t tid = threadIdx.x, w = tid >> 5, lane = tid & 31u, g = lane >> 2, t4 = lane & 3u;
  const uint32_t h = blockIdx.y, hk = h / (p.Hq / p.Hkv), q0 = blockIdx.x * AT_BQ;
  const __half* Qg = p.Q + (size_t)h * p.Lq * 128u; const __half* Kg = p.K + (size_t)hk * p.Lk * 128u; const __half* Vg = p.V + (size_t)hk * p.Lk * 128u;
  // ---- Q tile (rows past Lq repeat the last row; their results are not stored)
  for (uint32_t i = tid; i < AT_BQ * 16u; i += 128u) {
    const uint32_t r = i >> 4, c = i & 15u, row = min(q0 + r, p.Lq - 1u);
    *reinterpret_cast<uint4*>(Qs + r * AT_LD + c * 8u) = __ldg(reinterpret_cast<const uint4*>(Qg + (size_t)row * 128u + c * 8u));
  }
  __syncthreads();
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ks++) {
    const __half* b = Qs + (w * 16u + g) * AT_LD + ks * 16 + 2u * t4;
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(b); qa[ks][1] = *reinterpret_cast<const uint32_t*>(b + 8 * AT_LD);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(b + 8); qa[ks][3] = *reinterpret_cast<const uint32_t*>(b + 8 * AT_LD + 8);
  }
  uint32_t kEnd = p.Lk;                                                                       // attention.js:64
  if (p.mode == 1u) kEnd = min(p.Lk, min(q0 + (uint32_t)AT_BQ - 1u, p.nvalid - 1u) + 1u);
  if (p.mode == 2u) kEnd = min(p.Lk, p.nvalid);
  float o[16][4];
#pragma unroll
  for (int d = 0; d < 16; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.0f, 0.0f};
  const uint32_t i0 = q0 + w * 16u + g, i1 = i0 + 8u;                                         // this thread's two query rows
  // K / V tiles arrive by cp.async, one tile ahead of the arithmetic (rows past Lk repeat the last row; they are masked)
  auto fetch = [&](uint32_t k0, uint32_t stage) {
    const uint32_t kdst = (uint32_t)__cvta_generic_to_shared(KV + stage * 2 * AT_TILE), vdst = kdst + AT_TILE * 2u;
    for (uint32_t i = tid; i < AT_BK * 16u; i += 128u) {
      const uint32_t r = i >> 4, c = i & 15u, row = min(k0 + r, p.Lk - 1u), off = (r * AT_LD + c * 8u) * 2u;
      at_cp16(kdst + off, Kg + (size_t)row * 128u + c * 8u);
      at_cp16(vdst + off, Vg + (size_t)row * 128u + c * 8u);
    }
    at_cp_commit();
  };
  __syncthreads();                   // every warp has its Q fragments: the tile's space is free
  fetch(0u, 0u);
  uint32_t stage = 0;
  for (uint32_t k0 = 0; k0 < kEnd; k0 += AT_BK, stage ^= 1u) {
    if (k0 + AT_BK < kEnd) { fetch(k0 + AT_BK, stage ^ 1u); at_cp_wait<1>(); } else at_cp_wait<0>();
    __syncthreads();
    const __half* Ks = KV + stage * 2 * AT_TILE; const __half* Vs = Ks + AT_TILE;
    // ---- scores of 16 queries x 64 keys
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
    // four 8 x 8 blocks of K per ldmatrix: (keys nb*8.., dims ks*16 + {0, 8, 16, 24}) = the B fragments of two 16-dim steps.
    // The key blocks are the inner loop: consecutive multiplies go to different accumulators.
    const uint32_t krow = (uint32_t)__cvta_generic_to_shared(Ks + (lane & 7u) * AT_LD + (lane >> 3) * 8u);
#pragma unroll
    for (int ks = 0; ks < 8; ks += 2) {
#pragma unroll
      for (int nb = 0; nb < 8; nb++) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(krow + (uint32_t)(nb * 8 * AT_LD * 2 + ks * 32)));
        at_mma(s[nb], qa[ks], b0, b1);
        at_mma(s[nb], qa[ks + 1], b2, b3);
      }
    }
    // ---- scale, mask, running maximum
    float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
    for (int nb = 0; nb < 8; nb++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint32_t j = k0 + nb * 8 + 2u * t4 + (e & 1), i = (e & 2) ? i1 : i0;
        const bool vis = j < p.Lk && (p.mode == 1u ? j <= min(i, p.nvalid - 1u) : p.mode == 2u ? j < p.nvalid : true);
        s[nb][e] = vis ? s[nb][e] * p.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
      }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1)); mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float alpha[2], mb[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mb[r] = mx[r] == -INFINITY ? 0.0f : mx[r];                   // nothing visible yet: keep the exponents finite
      alpha[r] = exp2f(mrow[r] - mb[r]);                           // exp2(-inf) = 0 on the first visible tile
      mrow[r] = mx[r]; lrow[r] *= alpha[r];
    }
#pragma unroll
    for (int d = 0; d < 16; d++) { o[d][0] *= alpha[0]; o[d][1] *= alpha[0]; o[d][2] *= alpha[1]; o[d][3] *= alpha[1]; }
#pragma unroll
    for (int nb = 0; nb < 8; nb++)
#pragma unroll
      for (int e = 0; e < 4; e++) { s[nb][e] = exp2f(s[nb][e] - mb[e >> 1]); lrow[e >> 1] += s[nb][e]; }
    // ---- O += P V: the score fragments of two key blocks are the A fragment of 16 keys
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
      const uint32_t pa[4] = {at_pack(s[2 * kk][0], s[2 * kk][1]), at_pack(s[2 * kk][2], s[2 * kk][3]), at_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]), at_pack(s[2 * kk + 1][2], s[2 * kk + 1][3])};
      const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + (lane & 15u)) * AT_LD);
#pragma unroll
      for (int d = 0; d < 16; d++) {
        uint32_t b0, b1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(vrow + d * 16u));
        at_mma(o[d], pa, b0, b1);
      }
    }
    __syncthreads();                 // everyone is done with this stage before the fetch of the tile after next overwrites it
  }
  // ---- normalise and store (token-major, head h at column h * 128)
#pragma unroll
  for (int r = 0; r < 2; r++) { lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1); lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2); }
  const float inv0 = 1.0f / lrow[0], inv1 = 1.0f / lrow[1];
#pragma unroll
  for (int d = 0; d < 16; d++) {
    if (i0 < p.Lq) *reinterpret_cast<uint32_t*>(p.O + (size_t)i0 * p.ldo + h * 128u + d * 8 + 2u * t4) = at_pack(o[d][0] * inv0, o[d][1] * inv0);
    if (i1 < p.Lq) *reinterpret_cast<uint32_t*>(p.O + (size_t)i1 * p.ldo + h * 128u + d * 8 + 2u * t4) = at_pack(o[d][2] * inv1, o[d][3] * inv1);
  }
}

}  // namespace p0p
