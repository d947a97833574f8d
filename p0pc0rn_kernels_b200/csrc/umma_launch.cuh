// Host side of the tensor-core kernel (k_umma.cuh): which configurations it takes, the tile / split-K plan of a call, the
// tensor maps, the launch; and the two one-pass prologue kernels that prepare its token operand.
#pragma once
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "k_umma.cuh"
#include "tmap.h"

namespace p0p {

// ---- fused-norm prologue as one pass: X fp32 [M][ldx] -> X' fp16 [M][K] (src/ops/gemm.js:63-67)
__global__ void k_prologue_f16(const KP p, __half* __restrict__ out) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4u;
  if (i >= (size_t)p.M * p.K) return;
  const uint32_t m = (uint32_t)(i / p.K), k = (uint32_t)(i % p.K);
  const float4 x = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.X) + (size_t)m * p.ldx + p.kx0 + k));
  const size_t sr = ((size_t)p.statOff + m) * 2u;
  const float mean = __ldg(p.ST + sr), rstd = __ldg(p.ST + sr + 1);
  const float* pv = p.PV + p.pvOff + p.kx0 + k;
  const float xv[4] = {x.x, x.y, x.z, x.w};
  __half o[4];
#pragma unroll
  for (int j = 0; j < 4; j++)
    o[j] = __float2half_rn(p.xmode == P0P_X_LNMOD ? (xv[j] - mean) * rstd * (1.0f + __ldg(pv + j)) + __ldg(pv + p.pvStride + j) : xv[j] * rstd * __ldg(pv + j));
  *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<const uint2*>(o);
}

// ---- fused GroupNorm-apply + SiLU of the 2-D convolution as one pass over the image: X fp16 [Hi*Wi][Ci] ->
// X' = f16(silu(a[c] * x + b[c])) (src/ops/gemm.js:88-90).  The zero padding of the convolution is applied after it (the
// tensor map's out-of-range fill), as the reference does.
__global__ void k_prologue_gn(const KP p, __half* __restrict__ out) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8u, n = (size_t)p.Hi * p.Wi * p.Ci;
  if (i >= n) return;
  const uint32_t c = (uint32_t)(i % p.Ci);
  const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.X) + i));
  const __half* h = reinterpret_cast<const __half*>(&q);
  __half o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) o[j] = __float2half_rn(silu_exact(__half2float(h[j]) * __ldg(p.PV + p.pvOff + c + j) + __ldg(p.PV + p.pvOff + p.pvStride + c + j)));
  *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(o);
}

// ---- host side ------------------------------------------------------------------------------------------
// [rows][ld] fp16, box 64 (k) x box_rows, 128-byte swizzle, rows past the end read as zero
inline bool make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems, uint32_t box_rows) {
  tmap_encode_fn f = tmap_encoder();
  if (!f) return false;
  const cuuint64_t dims[2] = {cols, rows}, strides[1] = {ld_elems * 2u};
  const cuuint32_t box[2] = {64u, box_rows}, el[2] = {1u, 1u};
  return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Image / clip [frames][Hi][Wi][Ci] fp16: a box brings 64 channels x Wo columns x box_rows image rows of one frame, walking
// the image with element stride `step` along x and y (the 2-D convolution's stride; 1 for conv3).  In the map's terms the
// box spans (n - 1) * step + 1 positions, of which every step-th is copied.
inline bool make_map_clip(CUtensorMap* m, const void* base, uint32_t Ci, uint32_t Wi, uint32_t Hi, uint32_t frames, uint32_t Wo, uint32_t box_rows, uint32_t step = 1u) {
  tmap_encode_fn f = tmap_encoder();
  if (!f) return false;
  const cuuint64_t dims[4] = {Ci, Wi, Hi, frames}, strides[3] = {(cuuint64_t)Ci * 2u, (cuuint64_t)Wi * Ci * 2u, (cuuint64_t)Hi * Wi * Ci * 2u};
  const cuuint32_t box[4] = {64u, (Wo - 1u) * step + 1u, (box_rows - 1u) * step + 1u, 1u}, el[4] = {1u, step, step, 1u};
  return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Convolution token tile: R whole output rows of a frame.  R depends on the image only, never on M: a clip run whole, in chunks
// or from a ring must take the same tiles (the results are required to be bit-identical).  0 = no tile shape fits.
inline uint32_t conv_tile_rows(const KP& p, bool atm) {
  const uint32_t step = p.xmode == P0P_X_CONV ? p.stride : 1u;
  if (p.Wo > 256u || p.Wo % 8u || (p.Wo - 1u) * step + 1u > 256u) return 0u;
  // Quantised weights (operand in tensor memory): the fewest rows that give a tile of at least 128 tokens (small tiles
  // spread better over the SMs, a chunk of a few frames has few tiles, and two accumulators share the k loop).  fp16
  // weights (both operands through shared memory, whose bandwidth bounds the k-step): the largest tile that fits.
  uint32_t best = 0u;
  for (uint32_t R = 1u; R <= p.Ho && R * p.Wo <= (atm ? 384u : 256u); R++) {
    const uint32_t bt = R * p.Wo;
    if (p.Ho % R || bt < 16u || (R - 1u) * step + 1u > 256u) continue;
    if (bt <= 256u ? bt % 16u != 0u : (R % 2u != 0u || bt % 32u != 0u)) continue;
    best = R;
    if (atm && bt >= 128u) break;
  }
  return best;
}

inline bool umma_supported(const p0p_ctx*, const KP& p) {
  if (!tmap_encoder()) return false;
  if (p.K % 64u) return false;
  if (p.xmode == P0P_X_CONV || p.xmode == P0P_X_CONV3) {
    // one 64-k step inside one tap, whole tiles of whole image rows.  conv3: plain fp16 clip (no fused PixelNorm).
    // conv: any kernel size / stride / padding; the fused GroupNorm becomes a pre-pass; the fused 2x upsample is not taken.
    if (p.Ci % 64u || ((uintptr_t)p.X & 15u)) return false;
    if (p.xmode == P0P_X_CONV3 ? (p.flags & P0P_F_PN) != 0u : (p.flags & P0P_F_UP2) != 0u) return false;
    if (p.xmode == P0P_X_CONV && (p.stride > 8u || ((p.flags & P0P_F_GN) && (p.Ci % 8u)))) return false;
    const uint32_t R = conv_tile_rows(p, p.enc != P0P_ENC_F16);
    if (!R || p.M % (R * p.Wo)) return false;
  }
  if (p.xmode == P0P_X_F16 && !p.vecx) return false;
  if ((p.xmode == P0P_X_RMS || p.xmode == P0P_X_LNMOD) && (((uintptr_t)p.X & 15u) || p.ldx % 4u || p.kx0 % 4u)) return false;
  if ((uintptr_t)p.W & 15u) return false;
  if (p.epi == P0P_EPI_HEADS && ((uintptr_t)p.RP & 7u)) return false;      // the epilogue reads (cos, sin) as one 8-byte load
  if (p.enc == P0P_ENC_F16) {
    if (!p.vecw || p.epi == P0P_EPI_SWIGLU) return false;
  } else {
    if (p.wR0 % 64u) return false;
    if (p.epi == P0P_EPI_SWIGLU && (p.wR1 % 64u)) return false;
    if (p.enc == P0P_ENC_Q8 && (p.wk0 % 64u)) return false;
  }
  return true;
}

inline int launch_umma(p0p_ctx* c, const KP& p0) {
  KP p = p0;
  UmmaP u{};
  const uint32_t sms = (uint32_t)c->prop.multiProcessorCount;
  const bool is_conv = p.xmode == P0P_X_CONV || p.xmode == P0P_X_CONV3;
  // ---- the fused norm prologues become one pass into an fp16 scratch copy of the tokens (of the image, for the 2-D
  // convolution's GroupNorm)
  const void* xbase = nullptr; uint64_t xld = 0, pro_bytes = 0;
  const bool pre = p.xmode == P0P_X_RMS || p.xmode == P0P_X_LNMOD, pre_gn = p.xmode == P0P_X_CONV && (p.flags & P0P_F_GN);
  if (pre) { pro_bytes = ((uint64_t)p.M * p.K * 2u + 255u) & ~255ull; xld = p.K; }      // (launched below, once the scratch is sized)
  else if (pre_gn) pro_bytes = ((uint64_t)p.Hi * p.Wi * p.Ci * 2u + 255u) & ~255ull;
  else if (is_conv) { xbase = p.X; xld = 0; }
  else { xbase = reinterpret_cast<const __half*>(p.X) + p.kx0; xld = p.ldx; }
  // ---- tile shape.  fp16 weights: both operands in shared memory, up to 256 tokens, two accumulators.  Quantised
  // weights (operand in tensor memory): up to 192 tokens with two accumulators, or up to 384 with one; the cheapest
  // total by the cost model below wins.
  const bool atm = p.enc != P0P_ENC_F16;
  const uint32_t ncols = (p.epi == P0P_EPI_SWIGLU || p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? p.N : ((p.N + 3u) & ~3u);
  u.n_tiles = (ncols + 127u) / 128u;
  const uint32_t bt_max = atm ? 384u : 256u, KSn = p.K / 64u;
  uint32_t BT;
  if (is_conv) { u.cvR = conv_tile_rows(p, atm); BT = u.cvR * p.Wo; }
  else if (p.M <= 256u) BT = std::max(16u, (p.M + 15u) & ~15u);
  else {
    double best = 1e300; BT = 0;
    for (uint32_t cand = bt_max; cand >= 128u; cand -= 16u) {
      if (cand > 256u && cand % 32u) continue;
      const uint64_t t = (uint64_t)u.n_tiles * ((p.M + cand - 1u) / cand);
      // measured: a k-step costs ~750 cycles up to 256 tokens (four dependent multiplies, or the dequantisation) and
      // ~2.5 cycles per token beyond; a single-accumulator tile exposes its epilogue, whose cost per token depends on the kind
      const uint64_t kstep = std::max<uint64_t>(5u * cand / 2u, atm ? 750u : 720u);
      const uint64_t epi_tok = (p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? 150u : p.epi == P0P_EPI_SWIGLU ? 30u : 24u;
      // (with two accumulators the epilogue hides behind the next tile's k loop unless it is the longer of the two; it runs
      // about half as fast there, sharing the issue slots with the dequantisation)
      const uint64_t per_tile = (atm && cand > 128u) ? (uint64_t)KSn * kstep + epi_tok * cand : std::max<uint64_t>((uint64_t)KSn * kstep, 2u * epi_tok * cand);
      // Rounds of tiles over the SMs.  Fewer tiles than SMs: split-K (below) spreads their k loops over all SMs, so what counts
      // is the total work, not one round of it.  A last round that is not full is split as well, at some cost.
      const double whole = (double)(t / sms), frac = (double)(t % sms) / (double)sms;
      const double rounds = t < sms ? frac : whole + (frac > 0.0 ? std::min(1.0, frac + 0.1) : 0.0);
      if (rounds * (double)per_tile < best) { best = rounds * (double)per_tile; BT = cand; }
    }
  }
  // ---- tensor memory (512 columns).  fp16 weights: two accumulator buffers of 256 columns.  Quantised weights: the accumulators
  // first, the dequantised operand's stages in all the columns behind them.  Two accumulator buffers (the next tile's multiplies
  // overlap the epilogue) for tiles up to 128 tokens, one beyond.  Every hand-over between the roles is a round trip of several
  // hundred cycles, so the number of operand stages in flight, not the conversion or the multiplies, is what bounds narrow and
  // medium tiles: they get every column the accumulators leave.  (Consecutive multiplies into one accumulator issue back to back
  // at the tensor pipe's rate, so a tile has ONE accumulator: KSPLIT stays 1.)
  u.BT = BT; u.KSPLIT = 1u;
  u.NACC = atm ? (BT <= 128u ? 2u : 1u) : (BT > 256u ? 1u : 2u);
  u.m_tiles = (p.M + BT - 1u) / BT;
  // ---- split-K: when the tiles leave SMs idle (few output columns) or the last round is nearly empty, each tile's k loop
  // is cut into S units whose fp32 partial sums a second kernel adds.  Never for conv3 (S would depend on M, and chunked
  // and whole-clip calls must add in the same order).
  const uint32_t tiles_all = u.n_tiles * u.m_tiles;
  u.S = 1u; u.ks_per = KSn; u.T0 = tiles_all;
  if (p.xmode != P0P_X_CONV3) {
    const uint64_t tiles = tiles_all;
    const uint64_t kstep = std::max<uint64_t>(5u * BT / 2u, 750u), epi = 24u * BT;
    const uint64_t whole = KSn * kstep + (u.NACC == 1u ? epi : 0u);                  // one unsplit tile
    uint64_t best = ((tiles + sms - 1) / sms) * whole;
    // (a) every tile split (few tiles)
    for (uint32_t S = 2u; S <= 16u; S++) {
      const uint32_t per = (KSn + S - 1u) / S;
      if (per < 8u || (uint64_t)(S - 1u) * per >= KSn) continue;                     // every unit gets k-steps, at least 8 each
      const uint64_t cost = ((tiles * S + sms - 1) / sms) * (per * kstep + epi + 3000u) + 6000u + (uint64_t)S * BT * 40u;   // + pipeline fill per unit; second kernel: launch, partials written and read
      if (cost * 20u < best * 19u) { best = cost; u.S = S; u.ks_per = per; u.T0 = 0u; }
    }
    // (b) only the tiles of the last round split over the SMs that round would leave idle
    const uint64_t t0 = (tiles / sms) * sms, tail = tiles - t0;
    if (t0 && tail) {
      for (uint32_t S = 2u; S <= 16u; S++) {
        const uint32_t per = (KSn + S - 1u) / S;
        if (per < 4u || (uint64_t)(S - 1u) * per >= KSn) continue;
        const uint64_t cost = (t0 / sms) * whole + ((tail * S + sms - 1) / sms) * (per * kstep + epi + 3000u) + 6000u;
        if (cost * 20u < best * 19u) { best = cost; u.S = S; u.ks_per = per; u.T0 = (uint32_t)t0; }
      }
    }
  }
  // pipeline step: 128 k for quantised weights up to 256 tokens (the hand-over costs dominate there), 64 k otherwise (wide tiles
  // are bound by the multiplies and their stages are large; fp16 weights are bound by shared memory).  Depends on the tile only.
  u.KW = (atm && BT <= 256u) ? 2u : 1u;
  // ... except where every tile above 128 tokens is split along K (few output columns): the units are short, and with 64-k steps
  // four stages fit where two of 128 k do, so a unit's fill and drain are half as long (measured: the LLM block's down GEMM at
  // 512 tokens 68.7 -> 64.2 us; unsplit tiles of that width lose 4 % that way)
  if (atm && BT > 128u && BT <= 256u && u.S > 1u && u.T0 == 0u && u.ks_per >= 48u) u.KW = 1u;      // (long units only: 4096 x 4096 at 600 tokens lost 5 %)
  // 256 k for quantised weights on tiles up to 128 tokens: there each role's loop, not its work, is what a step costs (a record
  // stage is then one such step: 8 KB per 64-row tile of 4-bit weights, 17 KB of 8-bit ones).  Three operand stages of 128 columns
  // must fit behind the accumulators: one accumulator buffer above 64 tokens.  Not for units of few k-steps (split-K of a small
  // weight): two or three such steps would be all fill and drain.
  // (8-bit weights up to 96 tokens: beyond, their 34-KB record stages and the 64-KB token stages leave two of each)
  if (atm && BT <= (p.enc == P0P_ENC_Q4 ? 128u : 96u) && u.ks_per >= 32u) { u.KW = 4u; if (BT > 64u) u.NACC = 1u; }
#ifdef P0P_KNOBS      // (tuning experiments only: a library built with -DP0P_KNOBS lets environment variables override the plan)
  if (const char* e = getenv("P0P_NACC")) u.NACC = (uint32_t)atoi(e);
  if (const char* e = getenv("P0P_KW")) u.KW = (uint32_t)atoi(e);
#endif
  u.acc_stride = atm ? BT : 256u;
  u.a_col0 = atm ? ((u.NACC * BT + 31u) & ~31u) : 512u;
  // Token-ring stages: what shared memory allows for wide tiles; more for narrow ones, whose loads would otherwise be exposed.
  // fp16 weights have no operand ring of their own: the weight tile travels with the tokens (lock step, shared barriers).
  if (!atm) { u.NS = BT > 192u ? 3u : 4u; u.NA = u.NS; u.LOCK = 1u; }
  else {
    u.NA = std::min<uint32_t>(U_NA_MAX, (512u - u.a_col0) / (32u * u.KW));
    // (shared memory: up to 144 KB of token stages, less where three record stages would not fit beside them)
    const uint32_t xstage = u.KW * BT * 128u;
    const uint32_t qst = p.enc == P0P_ENC_Q4 ? UQ<P0P_ENC_Q4>::STAGE : (u.KW == 4u ? UQ<P0P_ENC_Q8, 4>::STAGE : UQ<P0P_ENC_Q8>::STAGE);
    const uint32_t xroom = std::min<uint32_t>(144u * 1024u, 227u * 1024u - 20u * 1024u - 3u * qst);
    u.NS = std::max(2u, std::min<uint32_t>(U_NX_MAX, xroom / xstage));
    u.LOCK = 0u;
    // Tiles above 128 tokens are bound by the multiplies, and there every instruction the issuing warp runs between two
    // multiplies shows: the two rings advance in lock step on shared barriers (one wait, one commit per step).
    if (u.KW == 1u || BT > 128u) { u.NS = std::min(u.NS, u.NA); u.NA = u.NS; u.LOCK = 1u; }
  }
#ifdef P0P_KNOBS
  if (const char* e = getenv("P0P_NS")) u.NS = (uint32_t)atoi(e);
  if (const char* e = getenv("P0P_NA")) u.NA = (uint32_t)atoi(e);
  if (const char* e = getenv("P0P_LOCK")) u.LOCK = (uint32_t)atoi(e);
  if (u.LOCK) u.NA = u.NS = std::min(u.NS, u.NA);
#endif
  // record stages: as many as fit beside the operand stages, up to about 100 KB in flight
  const size_t qstage = p.enc == P0P_ENC_Q4 ? UQ<P0P_ENC_Q4>::STAGE : p.enc == P0P_ENC_Q8 ? (u.KW == 4u ? UQ<P0P_ENC_Q8, 4>::STAGE : UQ<P0P_ENC_Q8>::STAGE) : 0;
  const size_t fixed = 1024 + (atm ? 0 : (size_t)u.NS * U_A_BYTES) + (size_t)u.NS * u.KW * BT * 128u + (size_t)U_EPI_BYTES + 1024u;
  size_t q_cap = 100 * 1024;
#ifdef P0P_KNOBS
  if (const char* e = getenv("P0P_QCAP")) q_cap = (size_t)atoi(e) * 1024;
#endif
  u.NQ = qstage ? (uint32_t)std::min<size_t>(std::min<size_t>(U_NQ_MAX, (q_cap + qstage - 1) / qstage), (227 * 1024 - fixed) / qstage) : 0u;
  if (qstage && u.NQ < 2u) return fail(c, -12, "gemm: no room for the record stages of this tile shape");
  const uint64_t sk_bytes = u.S > 1u ? (uint64_t)u.S * (tiles_all - u.T0) * BT * 128u * 4u : 0u;
  if (pro_bytes + sk_bytes) {
    if (int r = ensure_scratch(c, pro_bytes + sk_bytes + 256)) return r;
  }
  if (pre) {
    const size_t n4 = (size_t)p.M * p.K / 4u;
    k_prologue_f16<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(p, reinterpret_cast<__half*>(c->scratch));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(c, e, "prologue launch");
    c->launches += 1;
    xbase = c->scratch;
  } else if (pre_gn) {
    const size_t n8 = (size_t)p.Hi * p.Wi * p.Ci / 8u;
    k_prologue_gn<<<(unsigned)((n8 + 255) / 256), 256, 0, c->stream>>>(p, reinterpret_cast<__half*>(c->scratch));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(c, e, "GroupNorm prologue launch");
    c->launches += 1;
    xbase = c->scratch;
  }
  u.sk_part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(c->scratch) + pro_bytes);
  {   // a wave of `sms` tiles reads G token tiles and sms / G weight tiles: least bytes at G = sqrt(sms * weight tile / token tile)
    const double wt = 128.0 * (p.enc == P0P_ENC_Q4 ? 0.625 : p.enc == P0P_ENC_Q8 ? 1.03125 : 2.0), xt = 2.0 * BT;
    const double g = std::sqrt((double)sms * wt / xt);
    u.G = (uint32_t)std::min<double>(std::max(1.0, std::floor(g + 0.5)), (double)u.m_tiles);
  }
  u.p = p; u.status = c->dev_status;
  CUtensorMap mx, mw;
  if (p.xmode == P0P_X_CONV3) {
    const uint32_t frames = p.ks > 1u ? p.ks : p.stride - p.padL;
    if (!make_map_clip(&mx, xbase, p.Ci, p.Wi, p.Hi, frames, p.Wo, BT > 256u ? u.cvR / 2u : u.cvR)) return fail(c, -12, "gemm: the clip tensor map could not be encoded");
  } else if (p.xmode == P0P_X_CONV) {
    if (!make_map_clip(&mx, xbase, p.Ci, p.Wi, p.Hi, 1u, p.Wo, BT > 256u ? u.cvR / 2u : u.cvR, p.stride)) return fail(c, -12, "gemm: the image tensor map could not be encoded");
  } else if (!make_map(&mx, xbase, p.K, p.M, xld, BT > 256u ? BT / 2u : BT)) return fail(c, -12, "gemm: the token tensor map could not be encoded");
  if (p.enc == P0P_ENC_F16) {
    if (!make_map(&mw, reinterpret_cast<const __half*>(p.W) + p.wk0, p.K, p.Nw, p.wG, 128u)) return fail(c, -12, "gemm: the weight tensor map could not be encoded");
  } else mw = mx;
  const size_t qbytes = u.NQ * qstage;
  // at least 120 KB: one block per SM, so that a block never waits for another's tensor memory
  const size_t smem = std::max<size_t>(120 * 1024, 1024 + (atm ? 0 : (size_t)u.NS * U_A_BYTES) + (size_t)u.NS * u.KW * BT * 128u + qbytes + (size_t)U_EPI_BYTES + 1024u);
  const int grid = (int)std::min<uint64_t>((uint64_t)u.T0 + (uint64_t)(tiles_all - u.T0) * u.S, sms);
  const int smem_max = 227 * 1024;          // the most dynamic shared memory a block may opt into on sm_100
  if (smem > (size_t)smem_max) return fail(c, -12, "gemm: tile configuration needs %zu bytes of shared memory", smem);
  const uint32_t variant = u.KW == 1u ? 0u : u.KW == 4u ? 3u : u.LOCK ? 1u : 2u;
  const umma_kernel_fn kern = p.enc == P0P_ENC_Q4 ? umma_kernel_q4(variant, p.epi) : p.enc == P0P_ENC_Q8 ? umma_kernel_q8(variant, p.epi) : umma_kernel_f16(p.epi);
  // the shared-memory ceiling is an attribute of (kernel, device): raised once for each pair
  static DeviceOnce once[3][4][7];
  cudaError_t e = cudaSuccess;
  if (once[p.enc][variant][p.epi].run(c->device, [&] { e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max); return (int)e; }))
    return cuda_fail(c, e != cudaSuccess ? e : cudaErrorInvalidDevice, "tensor-core kernel attribute");
  const uint32_t plan[8] = {u.BT, u.KW, u.LOCK, u.NS, u.NA, u.NACC, u.S, u.T0};
  std::copy(plan, plan + 8, c->last_plan);
  void* args[3] = {&u, &mx, &mw};
  if ((e = cudaLaunchKernel(reinterpret_cast<const void*>(kern), dim3(grid), dim3(U_THREADS), args, smem, c->stream)) != cudaSuccess) return cuda_fail(c, e, "tensor-core kernel launch");
  c->launches += 1;
  if (u.S > 1u) {
    void* fargs[1] = {&u};
    if ((e = cudaLaunchKernel(reinterpret_cast<const void*>(umma_finish_kernel(p.epi)), dim3(tiles_all - u.T0, (BT + U_EPI_TB - 1u) / U_EPI_TB), dim3(128), fargs, 0, c->stream)) != cudaSuccess)
      return cuda_fail(c, e, "split-K second stage launch");
    c->launches += 1;
  }
  return 0;
}

}  // namespace p0p
