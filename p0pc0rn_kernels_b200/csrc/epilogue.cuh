// The fused epilogues for kernels whose threads each own ONE output column of a 128-column block and carry
// TB tokens of it in registers (the split-K decode reduction and the tensor-core kernel, whose accumulator
// lanes are weight rows).  128 threads cooperate: the head epilogues reduce over the block's 128 columns.
// Arithmetic as in the reference shader, src/ops/gemm.js:191-254.
#pragma once
#include "common.cuh"

namespace p0p {

__device__ __forceinline__ void bar_sync_named(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// ---- stores.  Every result goes to Y and, at the same offset, to the peer copies of Y (other GPUs' buffers: the
// all-gather of an N-sharded output fused into the store; nyp is 0 on one GPU and the loops vanish).
__device__ __forceinline__ void put_h(const KP& p, size_t i, __half v) {
  reinterpret_cast<__half*>(p.Y)[i] = v;
  for (uint32_t q = 0; q < p.nyp; q++) reinterpret_cast<__half*>(p.YP[q])[i] = v;
}
__device__ __forceinline__ void put_f(const KP& p, size_t i, float v) {
  reinterpret_cast<float*>(p.Y)[i] = v;
  for (uint32_t q = 0; q < p.nyp; q++) reinterpret_cast<float*>(p.YP[q])[i] = v;
}
__device__ __forceinline__ void put_h8(const KP& p, size_t i, uint4 v) {        // 8 halves, i a multiple of 8
  *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.Y) + i) = v;
  for (uint32_t q = 0; q < p.nyp; q++) *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.YP[q]) + i) = v;
}
__device__ __forceinline__ void put_f4(const KP& p, size_t i, float4 v) {       // 4 floats, i a multiple of 4
  *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.Y) + i) = v;
  for (uint32_t q = 0; q < p.nyp; q++) *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.YP[q]) + i) = v;
}

// ---- row-wise stores.  A thread owns a column, so its own stores are 2 or 4 bytes wide and a warp's store covers 64
// or 128 bytes of a row.  With `vec` the TB x 128 results of a pass go through shared memory instead and leave as
// 16-byte stores along the rows: an eighth of the store instructions.  The staging area is double-buffered by the
// pass's parity, which leaves one barrier per pass.
//
// Whether the output rows allow it (16-byte aligned pieces of 8 halves / 4 floats, no ragged edge inside a piece).
__device__ __forceinline__ bool epilogue_vec_ok(const KP& p) {
  const bool a16 = ((uintptr_t)p.Y & 15u) == 0u;
  switch (p.epi) {
    case P0P_EPI_HEADS: return a16;
    case P0P_EPI_F16: return a16 && p.ldy % 8u == 0u && p.ny0 % 8u == 0u && p.N % 8u == 0u;
    case P0P_EPI_BIAS: return a16 && !(p.flags & P0P_F_RES) && p.ldy % 8u == 0u && p.ny0 % 8u == 0u && p.N % 8u == 0u;
    case P0P_EPI_SWIGLU: return a16 && p.ldy % 8u == 0u && p.ny0 % 8u == 0u && p.N % 16u == 0u;
    case P0P_EPI_F32: case P0P_EPI_RESADD: return a16 && p.ldy % 4u == 0u && p.ny0 % 4u == 0u && p.N % 4u == 0u;
    default: return false;
  }
}
// fp16 results st[TB][W] (W = 128, or 64 for the gate|up epilogue) -> rows of Y.  ybase: element index of (row m0, first
// column of the block); valid: columns of the block that exist (a multiple of 8).
template <int TB, int W>
__device__ __forceinline__ void rows_out_f16(const KP& p, const __half* st, uint32_t t, uint32_t m0, size_t ybase, size_t row_stride, uint32_t valid) {
  constexpr int CPR = W / 8;                      // 16-byte pieces per row
#pragma unroll
  for (int i = 0; i < TB * CPR / 128; i++) {
    const uint32_t idx = (uint32_t)i * 128u + t, row = idx / CPR, ch = idx % CPR;
    if (m0 + row < p.M && ch * 8u < valid) put_h8(p, ybase + (size_t)row * row_stride + ch * 8u, *reinterpret_cast<const uint4*>(st + row * W + ch * 8u));
  }
}

// gate|up tokens of one pass: see the swiglu branch of epilogue_cols
template <int TB, bool GELU>
__device__ __forceinline__ void swiglu_tokens(const KP& p, uint32_t m0, uint32_t col, uint32_t c, const float (&acc)[TB], float gB, float uB, float* sh, bool vec, uint32_t par) {
  const uint32_t o = col >> 1, odd = c & 1u;
  // branch-free arithmetic first (a branch per token would end the scheduler's view at every token and serialise
  // the eight exp / reciprocal chains), then the stores
  __half out[TB / 2];
#pragma unroll
  for (int j = 0; j < TB; j += 2) {
    const float other = __shfl_xor_sync(0xffffffffu, odd ? acc[j] : acc[j + 1], 1);
    const float g = (odd ? other : acc[j]) + gB, u = (odd ? acc[j + 1] : other) + uB;
    const float a = GELU ? gelu_tanh_fast(g) : __fdividef(g, 1.0f + __expf(-g));       // hardware exp / reciprocal: a few ulp, far inside the fp16 rounding
    out[j / 2] = __float2half_rn(a * u);
  }
  if (vec) {
    __half* st = reinterpret_cast<__half*>(sh) + (par * TB + odd) * 64 + (c >> 1);
#pragma unroll
    for (int j = 0; j < TB; j += 2) st[j * 64] = out[j / 2];
  } else if (col < p.N) {
#pragma unroll
    for (int j = 0; j < TB; j += 2)
      if (m0 + j + odd < p.M) put_h(p, (size_t)(m0 + j + odd) * p.ldy + p.ny0 + o, out[j / 2]);
  }
}

// sh: shared scratch private to these 128 threads: TB * 132 floats, or 2 * TB * 132 floats with `vec`.  barid: a named
// barrier id private to them.  m0: first token row; rows m0 + j for j < TB with m0 + j < p.M are stored.
// nB: first column of the block (multiple of 128 for heads / onormgate).  c: this thread's column in the
// block (0..127).  acc[j]: fp32 accumulator of (row m0 + j, column nB + c).  vec: row-wise 16-byte stores (needs
// epilogue_vec_ok, TB == 16); par: parity of the pass (alternates between consecutive calls).
// EPI_T: the epilogue kind as a compile-time constant (P0P_EPI_*), or -1 to read it from p.epi.  A kernel that is
// instantiated per kind carries only that kind's code: with all seven kinds inlined a kernel grows by ~400 KB.
template <int TB, int EPI_T = -1>
__device__ __forceinline__ void epilogue_cols(const KP& p, uint32_t m0, uint32_t nB, uint32_t c, float (&acc)[TB], float* sh, int barid, bool vec = false, uint32_t par = 0) {
  const uint32_t col = nB + c, epi = EPI_T >= 0 ? (uint32_t)EPI_T : p.epi, lane = c & 31u, wq = c >> 5;
  __half* Yh = reinterpret_cast<__half*>(p.Y); float* Yf = reinterpret_cast<float*>(p.Y);
  if (epi == P0P_EPI_HEADS || epi == P0P_EPI_ONORMGATE) {
    float* part = sh;                 // [4][TB] sums of squares per warp
    float* xch = sh + 4 * TB;         // [TB][128] partner exchange for the (d, d+64) rotation
    const bool half_mode = epi == P0P_EPI_HEADS && (p.flags & P0P_F_ROPE_HALF);
    const uint32_t hd = nB / 128u, sec = epi == P0P_EPI_ONORMGATE ? 0u : (hd < p.Hq ? 0u : hd < p.Hq + p.Hkv ? 1u : 2u);
    float v[TB];
    // the rotation table is fetched first: its L2 latency then hides behind the norm's reduction instead of following it
    float cs[TB], sn[TB];
    if (epi == P0P_EPI_HEADS && sec < 2u) {
      const uint32_t ang = half_mode ? (c & 63u) : (c >> 1);
#pragma unroll
      for (int j = 0; j < TB; j++) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(p.RP + ((size_t)p.rowOff + min(m0 + j, p.M - 1u)) * 128u) + ang);
        cs[j] = t.x; sn[j] = t.y;
      }
    }
    if (sec < 2u) {                   // Q, K (and onormgate): RMS norm over the block's 128 columns; V heads pass through
      // ---- sum of squares over the 128 columns, per token
      if (TB == 16) {
        // transposing reduction: at each step a lane hands half of its tokens to its partner and keeps the other half, so 16
        // shuffles (instead of 80) leave every lane pair with one token's sum over the warp's 32 columns
        float s[16];
#pragma unroll
        for (int j = 0; j < 16; j++) s[j] = acc[j % TB] * acc[j % TB];
#pragma unroll
        for (int w = 8; w >= 1; w >>= 1) {                       // w tokens kept per lane after the step with partner lane ^ (2 w)
          const bool up = (lane & (2u * w)) != 0u;
#pragma unroll
          for (int i = 0; i < w; i++) {
            const float send = up ? s[i] : s[i + w], keep = up ? s[i + w] : s[i];
            s[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2 * w);
          }
        }
        s[0] += __shfl_xor_sync(0xffffffffu, s[0], 1);
        const uint32_t t = ((lane >> 4) & 1u) * 8u + ((lane >> 3) & 1u) * 4u + ((lane >> 2) & 1u) * 2u + ((lane >> 1) & 1u);
        if (!(lane & 1u)) part[wq * TB + t] = s[0];
      } else {
#pragma unroll
        for (int j = 0; j < TB; j++) {
          float s = acc[j] * acc[j];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          if (lane == 0) part[wq * TB + j] = s;
        }
      }
      bar_sync_named(barid, 128);
      const float nw = __ldg(p.EV + p.evOff + (sec == 1u ? 128u : 0u) + c);
      if (TB % 4 == 0) {
#pragma unroll
        for (int j = 0; j < TB; j += 4) {
          const float4 a0 = *reinterpret_cast<const float4*>(part + j), a1 = *reinterpret_cast<const float4*>(part + TB + j);
          const float4 a2 = *reinterpret_cast<const float4*>(part + 2 * TB + j), a3 = *reinterpret_cast<const float4*>(part + 3 * TB + j);
          v[j] = acc[j] * rsqrtf((a0.x + a1.x + a2.x + a3.x) / 128.0f + p.eps) * nw;
          v[j + 1] = acc[j + 1] * rsqrtf((a0.y + a1.y + a2.y + a3.y) / 128.0f + p.eps) * nw;
          v[j + 2] = acc[j + 2] * rsqrtf((a0.z + a1.z + a2.z + a3.z) / 128.0f + p.eps) * nw;
          v[j + 3] = acc[j + 3] * rsqrtf((a0.w + a1.w + a2.w + a3.w) / 128.0f + p.eps) * nw;
        }
      } else {
#pragma unroll
        for (int j = 0; j < TB; j++) v[j] = acc[j] * rsqrtf((part[j] + part[TB + j] + part[2 * TB + j] + part[3 * TB + j]) / 128.0f + p.eps) * nw;
      }
    } else {
#pragma unroll
      for (int j = 0; j < TB; j++) v[j] = acc[j];
    }
    if (epi == P0P_EPI_ONORMGATE) {
#pragma unroll
      for (int j = 0; j < TB; j++) {
        const uint32_t m = m0 + j;
        if (m < p.M) {
          const float g = __half2float(p.GT[(size_t)m * p.Ltot + p.ny0 + col]);
          put_h(p, (size_t)m * p.ldy + p.ny0 + col, __float2half_rn(v[j] / (1.0f + expf(-g))));
        }
      }
      bar_sync_named(barid, 128);     // `part` is free again
      return;
    }
    // the section and rotation mode are uniform over the block: chosen outside the token loops, which stay branch-free
    // (all of a pass's cos / sin loads in flight together)
    if (sec < 2u) {
      float other[TB];
      if (half_mode) {            // pairs (d, d+64), angle index d & 63
#pragma unroll
        for (int j = 0; j < TB; j++) xch[j * 128 + c] = v[j];
        bar_sync_named(barid, 128);
#pragma unroll
        for (int j = 0; j < TB; j++) other[j] = xch[j * 128 + (c ^ 64u)];
#pragma unroll
        for (int j = 0; j < TB; j++) v[j] = c < 64u ? v[j] * cs[j] - other[j] * sn[j] : v[j] * cs[j] + other[j] * sn[j];
      } else {                    // interleaved pairs (2p, 2p+1)
#pragma unroll
        for (int j = 0; j < TB; j++) other[j] = __shfl_xor_sync(0xffffffffu, v[j], 1);
#pragma unroll
        for (int j = 0; j < TB; j++) v[j] = (c & 1u) ? other[j] * sn[j] + v[j] * cs[j] : v[j] * cs[j] - other[j] * sn[j];
      }
    }
    if (vec) {
      __half* st = reinterpret_cast<__half*>(sh + TB * 132) + par * TB * 128 + c;
#pragma unroll
      for (int j = 0; j < TB; j++) st[j * 128] = __float2half_rn(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < TB; j++)
        if (m0 + j < p.M) put_h(p, ((size_t)hd * p.Ltot + p.rowOff + m0 + j) * 128u + c, __float2half_rn(v[j]));
    }
    bar_sync_named(barid, 128);       // results staged / scratch is free again
    if (vec) rows_out_f16<TB, 128>(p, reinterpret_cast<const __half*>(sh + TB * 132) + par * TB * 128, c, m0, ((size_t)hd * p.Ltot + p.rowOff + m0) * 128u, 128u, 128u);
    return;
  }
  if (epi == P0P_EPI_SWIGLU) {
    // even lanes hold 'gate', odd lanes 'up' of output column o.  The pair splits the tokens: the even lane
    // finishes tokens j = 0, 2, .., the odd lane j = 1, 3, .., each getting the other half of its pair by one shuffle.
    const uint32_t o = col >> 1;
    float gB = 0.0f, uB = 0.0f;
    if ((p.flags & P0P_F_BIAS) && col < p.N) { gB = __ldg(p.BV + p.bvOff + o); uB = __ldg(p.BV + p.bvOff + p.bvUp + o); }
    // the activation is chosen outside the token loop: inside it the compiler evaluates both branches per element
    if (p.flags & P0P_F_GELU) swiglu_tokens<TB, true>(p, m0, col, c, acc, gB, uB, sh, vec, par);
    else swiglu_tokens<TB, false>(p, m0, col, c, acc, gB, uB, sh, vec, par);
    if (vec) {
      bar_sync_named(barid, 128);
      rows_out_f16<TB, 64>(p, reinterpret_cast<const __half*>(sh) + par * TB * 64, c, m0, (size_t)m0 * p.ldy + p.ny0 + (nB >> 1), p.ldy, nB < p.N ? min(64u, (p.N - nB) >> 1) : 0u);
    }
    return;
  }
  if (vec) {
    const uint32_t valid = nB < p.N ? min(128u, p.N - nB) : 0u;
    if (epi == P0P_EPI_F16 || epi == P0P_EPI_BIAS) {
      const float bias = (epi == P0P_EPI_BIAS && col < p.N) ? __ldg(p.EV + p.evOff + col) : 0.0f;
      __half* st = reinterpret_cast<__half*>(sh) + par * TB * 128;
#pragma unroll
      for (int j = 0; j < TB; j++) st[j * 128 + c] = __float2half_rn(acc[j] + bias);
      bar_sync_named(barid, 128);
      rows_out_f16<TB, 128>(p, st, c, m0, (size_t)m0 * p.ldy + p.ny0 + nB, p.ldy, valid);
    } else {                                                        // f32 / resadd: fp32 rows, four columns per piece
      float* st = sh + par * TB * 132;
#pragma unroll
      for (int j = 0; j < TB; j++) st[j * 132 + c] = acc[j];
      bar_sync_named(barid, 128);
      const uint32_t ch = c & 31u, c4 = nB + ch * 4u;
      const bool live = ch * 4u < valid, rmw = epi == P0P_EPI_RESADD && !(p.flags & P0P_F_STORE);
      float g4[4] = {1.0f, 1.0f, 1.0f, 1.0f}, b4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (epi == P0P_EPI_RESADD && live) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          if (p.flags & P0P_F_GATE) g4[q] = __ldg(p.EV + p.evOff + c4 + q);
          if (p.flags & P0P_F_BIAS) b4[q] = __ldg(p.BV + p.bvOff + c4 + q);
        }
      }
      float4 old[TB / 4];
#pragma unroll
      for (int i = 0; i < TB / 4; i++) {
        const uint32_t row = (uint32_t)i * 4u + (c >> 5);
        old[i] = (rmw && live && m0 + row < p.M) ? __ldcg(reinterpret_cast<const float4*>(Yf + (size_t)(m0 + row) * p.ldy + p.ny0 + c4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int i = 0; i < TB / 4; i++) {
        const uint32_t row = (uint32_t)i * 4u + (c >> 5);
        if (!live || m0 + row >= p.M) continue;
        const float4 a = *reinterpret_cast<const float4*>(st + row * 132 + ch * 4u);
        float4 o;
        if (epi == P0P_EPI_F32) o = a;
        else { o.x = old[i].x + g4[0] * (a.x + b4[0]); o.y = old[i].y + g4[1] * (a.y + b4[1]); o.z = old[i].z + g4[2] * (a.z + b4[2]); o.w = old[i].w + g4[3] * (a.w + b4[3]); }
        put_f4(p, (size_t)(m0 + row) * p.ldy + p.ny0 + c4, o);
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
    if (epi == P0P_EPI_F16) put_h(p, yi, __float2half_rn(a));
    else if (epi == P0P_EPI_F32) put_f(p, yi, a);
    else if (epi == P0P_EPI_RESADD) put_f(p, yi, old[j] + gate * (a + bias));
    else put_h(p, yi, __float2half_rn(a + bias + old[j]));
  }
}

}  // namespace p0p
