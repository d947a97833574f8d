// The tensor-core kernel: tcgen05.mma with fp32 accumulators in tensor memory (TMEM).  Serves 9 tokens and more, every
// weight encoding, the plain / RMSNorm / LayerNorm+modulation prologues and the 3x3x3 conv3 mode, every epilogue.
//
// Orientation.  The 128 lanes of an accumulator are 128 weight rows (= output columns n) and its columns
// are tokens:  D[n, m] = sum_k W[n, k] * X'[m, k].  Weights are the A operand (UMMA M = 128), tokens the B
// operand (UMMA N = tokens), K-major fp16 tiles of 64 k.  A small M therefore costs a narrow instruction instead
// of a mostly empty 128-row tile, and every epilogue thread owns one output column, which is what the fused
// epilogues need (epilogue.cuh).
//
// Pipeline of one block (persistent over work units, one block per SM), by warp:
//   warp 0          producer   TMA tensor-map loads of the token tile (2-D map of the tokens, or 4-D boxes of the conv3
//                              clip) and of fp16 weight tiles, mbarrier-tracked
//   warp 1          MMA        the whole warp walks the loop, one elected lane issues 4 x tcgen05.mma (k = 16 each, x 2
//                              for tiles wider than 256 tokens) per step and commits to the stage's "free" barrier; after
//                              the unit's last step it commits to the accumulator's "full" barrier
//   warps 2..5      epilogue   tcgen05.ld of 16 tokens at a time, fused epilogue (or the raw partial sums of a split-K
//                              unit), row-wise 16-byte stores
//   warps 6..       dequant    U_NG groups of four warps take the k-steps in turn: codes -> fp16 tile values f16(q*s+mn) /
//                              f16(q*s), bit-exact (packed HFMA2 path with a per-warp exactness test and an fp32 fallback),
//                              written straight into tensor memory (tcgen05.st): the multiply takes A from there
//   last warp       records    bulk copies of the quantised records (two 64-row record tiles x up to 256 k per copy pair)
// Tensor memory: 384 accumulator columns + four 32-column operand stages (quantised weights), or 512 accumulator columns
// (fp16 weights, both operands in shared memory).  The accumulator columns hold two tiles of up to 192 tokens (the next
// tile's multiply overlaps the epilogue), or one tile of up to 384, or 2 / 4 accumulators of one narrow tile that take the
// 16-k multiplies in turn (see launch_umma for why).  gate|up (swiglu) tiles interleave gate and up rows in the A tile, so
// that (gate, up) of one output sit in adjacent lanes.  RMSNorm / LayerNorm+modulation prologues are applied by a one-pass
// kernel into an fp16 scratch copy of the tokens (the same token tile would otherwise be re-normalised by every column
// tile).  Few output columns: the k loop is split into units whose partial sums k_umma_finish adds (split-K).
// Every mbarrier wait is bounded (sync.cuh); on a time-out the block reports a code and winds down.
#pragma once
#include <cuda.h>

#include <cmath>

#include "common.cuh"
#include "ctx.h"
#include "epilogue.cuh"
#include "sync.cuh"
#include "umma.cuh"

namespace p0p {

constexpr int U_NG = 2;                  // dequantisation groups of four warps that take the k-steps in turn
constexpr int U_THREADS = (6 + 4 * U_NG + 1) * 32;
constexpr int U_NQ_MAX = 8;              // most stages of quantised records
constexpr int U_A_BYTES = 128 * 128;     // one weight operand stage: 128 rows x 64 fp16
constexpr int U_EPI_TB = 16;             // tokens per epilogue pass
constexpr int U_TMEM_COLS = 512;
constexpr int U_EPI_BYTES = 2 * U_EPI_TB * 132 * 4;   // epilogue scratch: two staging areas for the row-wise stores

struct UmmaP {
  KP p;
  uint32_t BT;          // tokens per tile: a multiple of 16 up to 256 (one UMMA of N = BT), or of 32 up to 384 (two of N = BT / 2)
  uint32_t NACC;        // accumulators: 2 (the next tile's multiply overlaps the epilogue) or 1 (wide tiles: tensor memory holds one)
  uint32_t KSPLIT;      // accumulators per tile that take the 16-k multiplies in turn (1, 2 or 4), summed by the epilogue
  uint32_t NS;          // operand stages (3 or 4)
  uint32_t NQ;          // stages of quantised records (each KSUP k-steps long)
  uint32_t n_tiles, m_tiles;
  uint32_t G;           // token tiles per group of the tile order (tile_coords)
  uint32_t cvR;         // conv3: image rows per token tile (tile = cvR x Wo output positions of one frame)
  uint32_t T0, S, ks_per;   // split-K: the first T0 tiles (in tile order) are whole units; each of the rest is S units of ks_per
                            // k-steps whose fp32 partial sums go to sk_part.  T0 = all tiles: no split; T0 = 0: every tile split;
                            // in between: only the tiles of the last, nearly empty round are split over the idle SMs
  float* sk_part;           // [S][tiles - T0][BT][128] partial sums (k_umma_finish adds them and applies the epilogue)
  int* status;
};

// A stage of quantised records covers KSUP k-steps (64 k each) of both 64-row record tiles of the block's 128 rows:
// two bulk copies of KSUP * RB bytes (the records of one row tile are consecutive along K), 64 bytes apart in
// shared memory so that the two tiles fall into different banks.  Large copies matter: the copy engine's request
// rate, not its byte rate, bounds many small copies.
template <int ENC> struct UQ { static constexpr uint32_t REC = 0, REC_K = 64, RB = 0, KSUP = 1, STAGE = 0; };
template <> struct UQ<P0P_ENC_Q4> { static constexpr uint32_t REC = 1280, REC_K = 32, RB = 2560, KSUP = 4, STAGE = 2 * 4 * 2560 + 128; };
template <> struct UQ<P0P_ENC_Q8> { static constexpr uint32_t REC = 4224, REC_K = 64, RB = 4224, KSUP = 2, STAGE = 2 * 2 * 4224 + 128; };

__device__ __forceinline__ void sts128(uint32_t a, uint4 v) { asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }
__device__ __forceinline__ uint4 u_lds128(uint32_t a) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ uint32_t u_lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ uint16_t u_lds16(uint32_t a) { uint16_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a) : "memory"); return v; }

// Tile order.  The blocks that run together should re-read as little as possible: a group of G token tiles is walked
// column tile by column tile (the G blocks of one column tile share its weights), group after group.  G = m_tiles is
// column-major order (weights stream once, every token tile is re-read per column tile: right when the tokens fit
// the L2), G = 1 the opposite; launch_umma picks G from the two tile sizes.
__device__ __forceinline__ void tile_coords(const UmmaP& u, uint32_t tile, uint32_t& nt, uint32_t& mt) {
  const uint32_t per = u.G * u.n_tiles, g = tile / per, local = tile - g * per, gsz = min(u.G, u.m_tiles - g * u.G);
  nt = local / gsz; mt = g * u.G + (local - nt * gsz);
}

// work unit -> tile and k range
struct UnitOf { uint32_t tile, sp, kb, ke; bool split; };
__device__ __forceinline__ UnitOf unit_of(const UmmaP& u, uint32_t unit, uint32_t tiles, uint32_t KS) {
  UnitOf r;
  if (unit < u.T0) { r.tile = unit; r.sp = 0u; r.kb = 0u; r.ke = KS; r.split = false; }
  else {
    const uint32_t tail = tiles - u.T0, v = unit - u.T0;
    r.sp = v / tail; r.tile = u.T0 + (v - r.sp * tail); r.kb = r.sp * u.ks_per; r.ke = min(KS, r.kb + u.ks_per); r.split = true;
  }
  return r;
}

// ring position that wraps without division
struct Ring {
  uint32_t s = 0, ph = 0, n;
  __device__ __forceinline__ explicit Ring(uint32_t n_) : n(n_) {}
  __device__ __forceinline__ void next() { if (++s == n) { s = 0; ph ^= 1u; } }
};

// ATM: the dequantised weight operand lives in tensor memory (written with tcgen05.st) instead of shared memory.
// Shared-memory bandwidth is what bounds the kernel otherwise: per 64-k step a 128 x 64 fp16 tile would be
// written once and read once there, on top of the token tile and the records.  Tensor memory then holds 384
// accumulator columns and four 32-column operand stages (384 + 4 x 32 = 512).  The accumulator columns are two
// tiles of up to 192 tokens (the next tile's multiply overlaps the epilogue) or ONE tile of up to 384 tokens: the
// dequantisation of a weight block costs the same whatever the tile's width, so a wide tile halves that cost per
// token, which is worth more than the overlap whenever M gives the wide tile enough tokens.
constexpr uint32_t U_ACC_STRIDE_ATM = 192, U_A_COL0_ATM = 384;
template <int ENC, bool ATM>
__global__ void __launch_bounds__(U_THREADS, 1) k_gemm_umma(const UmmaP u, const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW) {
  extern __shared__ unsigned char smem_raw[];
  const KP& p = u.p;
  const uint32_t BT = u.BT, NS = u.NS, NQ = u.NQ;
  const uint32_t HB = BT > 256u ? BT / 2u : BT, NH = BT > 256u ? 2u : 1u;          // tokens per UMMA / TMA box, and how many of them make a tile
  const bool two_acc = u.NACC == 2u;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;                     // operand tiles need 1024-byte alignment
  unsigned char* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_st = base, x_st = a_st + (ATM ? 0u : NS * U_A_BYTES), q_st = x_st + NS * BT * 128u;
  const uint32_t acc_stride = ATM ? U_ACC_STRIDE_ATM : 256u;
  const uint32_t epi_sh = q_st + (ENC == P0P_ENC_F16 ? 0u : NQ * UQ<ENC>::STAGE);
  const uint32_t bars = epi_sh + (uint32_t)U_EPI_BYTES;
  float* epi_ptr = reinterpret_cast<float*>(gbase + (epi_sh - base));
  // barrier slots (8 bytes each): operands of a stage ready / stage free / record stage ready / record stage free / accumulator ready / free
  const uint32_t full = bars, empty = full + 8u * 4u, wq_full = empty + 8u * 4u, wq_empty = wq_full + 8u * U_NQ_MAX;
  const uint32_t acc_full = wq_empty + 8u * U_NQ_MAX, acc_empty = acc_full + 16u, tmem_slot = acc_empty + 16u;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  if (tid == 0) {
    for (uint32_t s = 0; s < 4u; s++) {
      mbar_init(full + 8u * s, ENC == P0P_ENC_F16 ? 1u : 5u);     // the producer's expect_tx arrival (+ the four warps of a dequant group)
      mbar_init(empty + 8u * s, 1u);
    }
    for (uint32_t s = 0; s < (uint32_t)U_NQ_MAX; s++) { mbar_init(wq_full + 8u * s, 1u); mbar_init(wq_empty + 8u * s, 4u * U_NG); }
    for (uint32_t b = 0; b < 2u; b++) { mbar_init(acc_full + 8u * b, 1u); mbar_init(acc_empty + 8u * b, 4u); }
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, U_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot - base));

  const uint32_t tiles = u.n_tiles * u.m_tiles, KS = p.K / 64u, units = u.T0 + (tiles - u.T0) * u.S;
  const bool swiglu = p.epi == P0P_EPI_SWIGLU;

  if (warp == 0) {
    // ================================================================= producer of the token tiles (and fp16 weight tiles)
    if (lane == 0) {
      Ring r(NS);
      bool ok = true;
      for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t tile = un.tile, kb = un.kb, ke = un.ke;
        uint32_t nt, mt; tile_coords(u, tile, nt, mt);
        for (uint32_t ks = kb; ks < ke; ks++, r.next()) {
          if (!mbar_wait(empty + 8u * r.s, r.ph ^ 1u, u.status, 201, 200u)) { ok = false; break; }
          mbar_expect_tx(full + 8u * r.s, BT * 128u + (ENC == P0P_ENC_F16 ? U_A_BYTES : 0u));
          if (p.xmode == P0P_X_CONV3) {
            // implicit GEMM (src/ops/gemm.js:68-80): the 64 k of this step are channels c0.. of ONE tap (kt, ky, kx); the tile's
            // tokens are cvR whole rows of one output frame, so their inputs are a box of the clip shifted by the tap, and
            // what falls outside the image reads as zero.  Frame index: clamp to the clip, then ring slot or chunk offset.
            const uint32_t tpf = p.Ho / u.cvR, ot = mt / tpf, oy0 = (mt - ot * tpf) * u.cvR;
            const uint32_t kg = ks * 64u, tap = kg / p.Ci, c0 = kg - tap * p.Ci, kt = tap / 9u, ky = (tap / 3u) % 3u, kx = tap % 3u;
            const int itg = min(max((int)(ot + p.padT + kt) - 1, 0), (int)p.stride - 1);
            const int it = p.ks > 1u ? itg % (int)p.ks : itg - (int)p.padL;
            const uint32_t rb = u.cvR / NH;
            for (uint32_t h = 0; h < NH; h++)
              tma_load_4d(x_st + r.s * BT * 128u + h * HB * 128u, &mapX, (int)c0, (int)kx - 1, (int)(oy0 + h * rb + ky) - 1, it, full + 8u * r.s);
          } else
            for (uint32_t h = 0; h < NH; h++) tma_load_2d(x_st + r.s * BT * 128u + h * HB * 128u, &mapX, (int)(ks * 64u), (int)(mt * BT + h * HB), full + 8u * r.s);
          if (ENC == P0P_ENC_F16) tma_load_2d(a_st + r.s * U_A_BYTES, &mapW, (int)(ks * 64u), (int)(p.wR0 + nt * 128u), full + 8u * r.s);
        }
      }
    }
  } else if (warp == 6u + 4u * U_NG) {
    // ================================================================= producer of the quantised records: runs ahead of
    // everything else by NQ stages (its only wait is for a free record stage)
    if (ENC != P0P_ENC_F16 && lane == 0) {
      Ring q(NQ);
      bool ok = true;
      const uint32_t last = (p.Nw >> 6) - 1u;                  // record tiles past the weight's end do not exist: their columns are never stored
      for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t tile = un.tile, kb = un.kb, ke = un.ke;
        uint32_t nt, mt; tile_coords(u, tile, nt, mt);
        uint32_t trow[2];
        if (swiglu) { trow[0] = min((p.wR0 + nt * 64u) >> 6, last); trow[1] = min((p.wR1 + nt * 64u) >> 6, last); }
        else { trow[0] = min((p.wR0 + nt * 128u) >> 6, last); trow[1] = min(trow[0] + 1u, last); }
        const unsigned char* src0 = p.W + ((size_t)trow[0] * p.wG + p.wk0 / UQ<ENC>::REC_K) * UQ<ENC>::REC;
        const unsigned char* src1 = p.W + ((size_t)trow[1] * p.wG + p.wk0 / UQ<ENC>::REC_K) * UQ<ENC>::REC;
        for (uint32_t ks = kb; ks < ke; ks += UQ<ENC>::KSUP, q.next()) {
          const uint32_t bytes = min(UQ<ENC>::KSUP, ke - ks) * UQ<ENC>::RB;
          if (!mbar_wait(wq_empty + 8u * q.s, q.ph ^ 1u, u.status, 202, 500u)) { ok = false; break; }
          mbar_expect_tx(wq_full + 8u * q.s, 2u * bytes);
          bulk_g2s(q_st + q.s * UQ<ENC>::STAGE, src0 + (size_t)ks * UQ<ENC>::RB, bytes, wq_full + 8u * q.s);
          bulk_g2s(q_st + q.s * UQ<ENC>::STAGE + UQ<ENC>::KSUP * UQ<ENC>::RB + 64u, src1 + (size_t)ks * UQ<ENC>::RB, bytes, wq_full + 8u * q.s);
        }
      }
    }
  } else if (warp == 1) {
    // ================================================================= MMA issuer.  The WHOLE warp walks the loop and one
    // elected lane issues: in warp-uniform control flow the descriptors live in uniform registers, which is what the
    // instruction takes; inside a one-lane branch every operand of every tcgen05.mma is first moved there, which
    // costs more than the multiply itself.
    const uint32_t idesc = umma_idesc_f16(128u, HB);
    Ring r(NS);
    uint32_t tl = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x, tl++) {
      const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t kb = un.kb, ke = un.ke;
      const uint32_t buf = two_acc ? tl & 1u : 0u, par = two_acc ? (tl >> 1) & 1u : tl & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + 8u * buf, par ^ 1u, u.status, 203, 100u))) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * acc_stride;
      for (uint32_t ks = kb; ks < ke; ks++, r.next()) {
        if (!__all_sync(0xffffffffu, mbar_wait(full + 8u * r.s, r.ph, u.status, 204))) { ok = false; break; }
        tc_fence_after();
        const uint64_t bd = umma_desc_sw128(x_st + r.s * BT * 128u);
        const uint32_t at = tmem_base + U_A_COL0_ATM + r.s * 32u;
        const uint64_t ad = umma_desc_sw128(a_st + r.s * U_A_BYTES);
        const uint32_t first = ks - kb;                             // 0 on the unit's first k-step: the first multiply overwrites
        if (elect_one()) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4u; kk++) {                      // per 16 k: 8 tensor-memory columns / +32 bytes
            // consecutive multiplies into ONE accumulator start ~180 cycles apart whatever their width; into different
            // accumulators ~35.  Narrow tiles therefore rotate over KSPLIT accumulators (wide ones over their two halves).
            const uint32_t dk = d_tmem + (kk & (u.KSPLIT - 1u)) * BT, accum = first | (kk >= u.KSPLIT ? 1u : 0u);
            if (ATM) {
              umma_f16_ts(dk, at + 8u * kk, bd + 2u * kk, idesc, accum);
              if (NH == 2u) umma_f16_ts(dk + HB, at + 8u * kk, bd + ((HB * 128u) >> 4) + 2u * kk, idesc, accum);
            } else {
              umma_f16_ss(dk, ad + 2u * kk, bd + 2u * kk, idesc, accum);
              if (NH == 2u) umma_f16_ss(dk + HB, ad + 2u * kk, bd + ((HB * 128u) >> 4) + 2u * kk, idesc, accum);
            }
          }
          umma_commit(empty + 8u * r.s);
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(acc_full + 8u * buf);
      __syncwarp();
    }
  } else if (warp < 6) {
    // ================================================================= epilogue (TMEM lanes 32*(warp%4) .. +31)
    const uint32_t q = warp & 3u, c = q * 32u + lane;
    uint32_t tl = 0, pass = 0;
    bool ok = true;
    const bool vec = epilogue_vec_ok(p);
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x, tl++) {
      const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t tile = un.tile, sp = un.sp;
      uint32_t nt, mt; tile_coords(u, tile, nt, mt);
      const uint32_t buf = two_acc ? tl & 1u : 0u, par = two_acc ? (tl >> 1) & 1u : tl & 1u;
      if (ok && !mbar_wait(acc_full + 8u * buf, par, u.status, 206, 1000u)) ok = false;
      tc_fence_after();
      const uint32_t m0 = mt * BT, nchunks = min(BT, p.M - m0 + (U_EPI_TB - 1u)) / U_EPI_TB;
      const uint32_t t0 = tmem_base + ((q * 32u) << 16) + buf * acc_stride;
      uint32_t r[16];
      tmem_ld16(t0, r);                                      // (tensor memory stays allocated after a time-out: the load is safe, its result unused)
      for (uint32_t ch = 0; ch < nchunks; ch++, pass++) {   // uniform over the four warps: the epilogue's named barrier needs all 128 threads
        float acc[U_EPI_TB];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < U_EPI_TB; j++) acc[j] = ok ? __uint_as_float(r[j]) : 0.0f;
        for (uint32_t a = 1; a < u.KSPLIT; a++) {            // the tile's other accumulators (narrow tiles only: few passes)
          tmem_ld16(t0 + a * BT + ch * U_EPI_TB, r); tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < U_EPI_TB; j++) acc[j] += ok ? __uint_as_float(r[j]) : 0.0f;
        }
        if (ch + 1u < nchunks) tmem_ld16(t0 + (ch + 1u) * U_EPI_TB, r);      // the next pass's accumulators load behind this pass's work
        if (un.split) {
          // split-K: this unit's partial sums, fp32, to its own slab; a warp's store covers 128 bytes of a row
          float* dst = u.sk_part + (((size_t)sp * (tiles - u.T0) + (tile - u.T0)) * BT + ch * U_EPI_TB) * 128u + c;
#pragma unroll
          for (int j = 0; j < U_EPI_TB; j++) dst[(size_t)j * 128u] = acc[j];
        } else epilogue_cols<U_EPI_TB>(p, m0 + ch * U_EPI_TB, nt * 128u, c, acc, epi_ptr, 2, vec, pass & 1u);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8u * buf);
    }
  } else if (ENC != P0P_ENC_F16 && warp < 6u + 4u * U_NG) {
    // ================================================================= dequantisation: codes -> swizzled fp16 operand rows.
    // The groups of four warps take the k-steps in turn; a thread converts one whole operand row (64 k) of a step.
    const uint32_t dw = warp - 6u, grp = dw >> 2, r = (warp & 3u) * 32u + lane;      // a warp reaches the tensor-memory lanes 32 * (warp % 4) .. + 31
    const uint32_t tsel = swiglu ? (r & 1u) : (r >> 6), rr = swiglu ? (r >> 1) : (r & 63u);
    const uint32_t rsw = r & 7u;
    const uint32_t rec_row = tsel * (UQ<ENC>::KSUP * UQ<ENC>::RB + 64u) + (ENC == P0P_ENC_Q4 ? rr * 16u : rr * 64u);
    const uint32_t rec_sm = tsel * (UQ<ENC>::KSUP * UQ<ENC>::RB + 64u) + (ENC == P0P_ENC_Q4 ? 1024u + rr * 4u : 4096u + rr * 2u);
    Ring ar(NS), qr(NQ);
    uint32_t sub = 0, turn = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t kb = un.kb, ke = un.ke;
      for (uint32_t ks = kb; ks < ke; ks++) {
        const bool last_sub = sub == UQ<ENC>::KSUP - 1u || ks == ke - 1u;
        if (turn == grp) {
          // the record stage is awaited at this group's first use of it only (its first U_NG k-steps: the groups take turns)
          if ((sub < (uint32_t)U_NG && !mbar_wait(wq_full + 8u * qr.s, qr.ph, u.status, 207)) || !mbar_wait(empty + 8u * ar.s, ar.ph ^ 1u, u.status, 208)) { ok = false; break; }
          const uint32_t rec = q_st + qr.s * UQ<ENC>::STAGE + sub * UQ<ENC>::RB;
          const uint32_t dst = a_st + ar.s * U_A_BYTES + r * 128u;
          if (ENC == P0P_ENC_Q4) {
            // both 32-k halves of the row are fetched first and share ONE exactness vote: a vote and a branch per half
            // would expose the shared-memory latency twice and end the scheduler's view between the halves
            const uint4 c0 = u_lds128(rec + rec_row), c1 = u_lds128(rec + rec_row + 1280u);
            const uint32_t sm0 = u_lds32(rec + rec_sm), sm1 = u_lds32(rec + rec_sm + 1280u);
            const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            __half2 v[32];
            if (__all_sync(0xffffffffu, q4_pair_exact(sm0) && q4_pair_exact(sm1))) {
              const __half2 s20 = __half2half2(__ushort_as_half((unsigned short)(sm0 & 0xffffu))), m20 = __half2half2(__ushort_as_half((unsigned short)(sm0 >> 16)));
              const __half2 s21 = __half2half2(__ushort_as_half((unsigned short)(sm1 & 0xffffu))), m21 = __half2half2(__ushort_as_half((unsigned short)(sm1 >> 16)));
#pragma unroll
              for (int i = 0; i < 4; i++) q4_word_to_half2x4(w[i], s20, m20, v + 4 * i);
#pragma unroll
              for (int i = 4; i < 8; i++) q4_word_to_half2x4(w[i], s21, m21, v + 4 * i);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++) {
                const uint32_t sm = i < 16 ? sm0 : sm1;
                const float sc = __half2float(__ushort_as_half((unsigned short)(sm & 0xffffu))), mn = __half2float(__ushort_as_half((unsigned short)(sm >> 16)));
                v[i] = __halves2half2(deq_q4((w[i >> 2] >> (8 * (i & 3))) & 15u, sc, mn), deq_q4((w[i >> 2] >> (8 * (i & 3) + 4)) & 15u, sc, mn));
              }
            }
            if (ATM) {
              const uint32_t ta = tmem_base + (((warp & 3u) * 32u) << 16) + U_A_COL0_ATM + ar.s * 32u;
              tmem_st16(ta, *reinterpret_cast<const uint32_t(*)[16]>(v));
              tmem_st16(ta + 16u, *reinterpret_cast<const uint32_t(*)[16]>(v + 16));
            } else {
#pragma unroll
              for (uint32_t j = 0; j < 8u; j++) sts128(dst + ((j ^ rsw) << 4), reinterpret_cast<const uint4*>(v)[j]);
            }
          } else {
            const __half2 s2 = __half2half2(__ushort_as_half(u_lds16(rec + rec_sm)));
            // shared-memory operand: each row pair starts at another 16-byte chunk (no bank conflicts).  Tensor-memory
            // operand: the store's column must be the same in every lane, so all lanes walk the chunks in order.
            const uint32_t rot = ATM ? 0u : (rr >> 1) & 3u;
#pragma unroll
            for (uint32_t jj = 0; jj < 4u; jj++) {
              const uint32_t j = (jj + rot) & 3u;                    // 16 codes = two output chunks
              const uint4 cq = u_lds128(rec + rec_row + j * 16u);
              const uint32_t w[4] = {cq.x, cq.y, cq.z, cq.w};
              __half2 v[8];
#pragma unroll
              for (int i = 0; i < 4; i++) q8_word_to_half2x2(w[i], s2, v + 2 * i);
              if (ATM) {
                uint32_t t8[8];
#pragma unroll
                for (int i = 0; i < 8; i++) t8[i] = *reinterpret_cast<const uint32_t*>(&v[i]);
                tmem_st8(tmem_base + (((warp & 3u) * 32u) << 16) + U_A_COL0_ATM + ar.s * 32u + j * 8u, t8);
              } else {
                sts128(dst + (((2u * j) ^ rsw) << 4), reinterpret_cast<const uint4*>(v)[0]);
                sts128(dst + (((2u * j + 1u) ^ rsw) << 4), reinterpret_cast<const uint4*>(v)[1]);
              }
            }
          }
          if (ATM) { tmem_st_wait(); tc_fence_before(); }           // tensor-memory stores done and ordered before the MMA warp's read
          else fence_proxy_async();                                   // generic-proxy stores -> visible to the tensor core's async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(full + 8u * ar.s);
        }
        // every warp walks every k-step, so it releases each record stage exactly once, after its own last use of it
        if (last_sub) { __syncwarp(); if (lane == 0) mbar_arrive(wq_empty + 8u * qr.s); qr.next(); sub = 0; } else sub++;
        ar.next(); if (++turn == (uint32_t)U_NG) turn = 0u;
      }
    }
  }
  // ---- wind down: every role is past its last use of tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, U_TMEM_COLS); }
}

// ---- split-K second stage: the S partial sums of 16 tokens x 128 columns of a split tile are added in split order
// (deterministic) and the fused epilogue runs on the sum.  grid = (split tiles, 16-token groups of a tile), 128 threads.
__global__ void __launch_bounds__(128) k_umma_finish(const UmmaP u) {
  __shared__ __align__(16) float sh[2 * U_EPI_TB * 132];
  const KP& p = u.p;
  const uint32_t tiles = u.n_tiles * u.m_tiles, tail = tiles - u.T0, t = blockIdx.x, c = threadIdx.x;
  uint32_t nt, mt; tile_coords(u, u.T0 + t, nt, mt);
  const uint32_t r0 = blockIdx.y * U_EPI_TB, m0 = mt * u.BT + r0;
  if (m0 >= p.M) return;
  float acc[U_EPI_TB];
#pragma unroll
  for (int j = 0; j < U_EPI_TB; j++) acc[j] = 0.0f;
  for (uint32_t sp = 0; sp < u.S; sp++) {
    const float* src = u.sk_part + (((size_t)sp * tail + t) * u.BT + r0) * 128u + c;
    float v[U_EPI_TB];
#pragma unroll
    for (int j = 0; j < U_EPI_TB; j++) v[j] = __ldcg(src + (size_t)j * 128u);      // rows up to the tile's padding exist
#pragma unroll
    for (int j = 0; j < U_EPI_TB; j++) acc[j] += v[j];
  }
  epilogue_cols<U_EPI_TB>(p, m0, nt * 128u, c, acc, sh, 1, epilogue_vec_ok(p), 0u);
}

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

// ---- host side ------------------------------------------------------------------------------------------
typedef CUresult (*tmap_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline tmap_encode_fn tmap_encoder() {
  static tmap_encode_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess) fn = (tmap_encode_fn)f;
    (void)cudaGetLastError();
  }
  return fn;
}
// [rows][ld] fp16, box 64 (k) x box_rows, 128-byte swizzle, rows past the end read as zero
inline bool make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems, uint32_t box_rows) {
  tmap_encode_fn f = tmap_encoder();
  if (!f) return false;
  const cuuint64_t dims[2] = {cols, rows}, strides[1] = {ld_elems * 2u};
  const cuuint32_t box[2] = {64u, box_rows}, el[2] = {1u, 1u};
  return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// conv3 clip [frames][Hi][Wi][Ci] fp16: box = 64 channels x Wo columns x box_rows image rows of one frame
inline bool make_map_clip(CUtensorMap* m, const void* base, uint32_t Ci, uint32_t Wi, uint32_t Hi, uint32_t frames, uint32_t Wo, uint32_t box_rows) {
  tmap_encode_fn f = tmap_encoder();
  if (!f) return false;
  const cuuint64_t dims[4] = {Ci, Wi, Hi, frames}, strides[3] = {(cuuint64_t)Ci * 2u, (cuuint64_t)Wi * Ci * 2u, (cuuint64_t)Hi * Wi * Ci * 2u};
  const cuuint32_t box[4] = {64u, Wo, box_rows, 1u}, el[4] = {1u, 1u, 1u, 1u};
  return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// conv3 token tile: R whole output rows of a frame.  R depends on the image only, never on M: a clip run whole, in chunks
// or from a ring must take the same tiles (the results are required to be bit-identical).  0 = no tile shape fits.
inline uint32_t conv3_tile_rows(const KP& p, bool atm) {
  if (p.Wo > 256u || p.Wo % 8u) return 0u;
  // Quantised weights (operand in tensor memory): the fewest rows that give a tile of at least 128 tokens (small tiles
  // spread better over the SMs, a chunk of a few frames has few tiles, and two accumulators share the k loop).  fp16
  // weights (both operands through shared memory, whose bandwidth bounds the k-step): the largest tile that fits.
  uint32_t best = 0u;
  for (uint32_t R = 1u; R <= p.Ho && R * p.Wo <= 384u; R++) {
    const uint32_t bt = R * p.Wo;
    if (p.Ho % R || bt < 16u) continue;
    if (bt <= 256u ? bt % 16u != 0u : (R % 2u != 0u || bt % 32u != 0u)) continue;
    best = R;
    if (atm && bt >= 128u) break;
  }
  return best;
}

inline bool umma_supported(const p0p_ctx*, const KP& p) {
  if (!tmap_encoder()) return false;
  if (p.K % 64u) return false;
  if (p.xmode == P0P_X_CONV) return false;
  if (p.xmode == P0P_X_CONV3) {
    // one 64-k step inside one tap, plain fp16 clip (no fused PixelNorm), whole tiles of whole image rows
    if (p.Ci % 64u || (p.flags & P0P_F_PN) || ((uintptr_t)p.X & 15u)) return false;
    const uint32_t R = conv3_tile_rows(p, p.enc != P0P_ENC_F16);
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
  // ---- the fused norm prologue becomes one pass into an fp16 scratch copy of the tokens
  const void* xbase = nullptr; uint64_t xld = 0, pro_bytes = 0;
  const bool pre = p.xmode == P0P_X_RMS || p.xmode == P0P_X_LNMOD;
  if (pre) { pro_bytes = ((uint64_t)p.M * p.K * 2u + 255u) & ~255ull; xld = p.K; }      // (launched below, once the scratch is sized)
  else if (p.xmode == P0P_X_CONV3) { xbase = p.X; xld = 0; }
  else { xbase = reinterpret_cast<const __half*>(p.X) + p.kx0; xld = p.ldx; }
  // ---- tile shape.  fp16 weights: both operands in shared memory, up to 256 tokens, two accumulators.  Quantised
  // weights (operand in tensor memory): up to 192 tokens with two accumulators, or up to 384 with one; the cheapest
  // total by the cost model below wins.
  const bool atm = p.enc != P0P_ENC_F16;
  const uint32_t ncols = (p.epi == P0P_EPI_SWIGLU || p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? p.N : ((p.N + 3u) & ~3u);
  u.n_tiles = (ncols + 127u) / 128u;
  const uint32_t bt_max = atm ? 384u : 256u, KSn = p.K / 64u;
  uint32_t BT;
  if (p.xmode == P0P_X_CONV3) { u.cvR = conv3_tile_rows(p, atm); BT = u.cvR * p.Wo; }
  else if (p.M <= 256u) BT = std::max(16u, (p.M + 15u) & ~15u);
  else {
    uint64_t best = ~0ull; BT = 0;
    for (uint32_t cand = bt_max; cand >= 128u; cand -= 16u) {
      if (cand > 256u && cand % 32u) continue;
      const uint64_t t = (uint64_t)u.n_tiles * ((p.M + cand - 1u) / cand), rounds = (t + sms - 1) / sms;
      // measured: a k-step costs ~750 cycles up to 256 tokens (four dependent multiplies, or the dequantisation) and
      // ~2.5 cycles per token beyond; a single-accumulator tile exposes its epilogue, whose cost per token depends on the kind
      const uint64_t kstep = std::max<uint64_t>(5u * cand / 2u, atm ? 750u : 720u);
      const uint64_t epi_tok = (p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? 150u : p.epi == P0P_EPI_SWIGLU ? 30u : 24u;
      // (with two accumulators the epilogue hides behind the next tile's k loop unless it is the longer of the two; it runs
      // about half as fast there, sharing the issue slots with the dequantisation)
      const uint64_t per_tile = (atm && cand > 192u) ? (uint64_t)KSn * kstep + epi_tok * cand : std::max<uint64_t>((uint64_t)KSn * kstep, 2u * epi_tok * cand);
      if (rounds * per_tile < best) { best = rounds * per_tile; BT = cand; }
    }
  }
  u.BT = BT; u.NACC = (BT > (atm ? 192u : 256u)) ? 1u : 2u;
  // accumulators per tile: as many as the accumulator columns hold (192 per buffer with the operand in tensor memory, 256
  // without).  96 < BT <= 192 gives up the second buffer for a second accumulator when the k loop is long enough to pay
  // for the exposed epilogue.
  const uint32_t acc_cols = atm ? 192u : 256u;
  u.KSPLIT = BT * 4u <= acc_cols ? 4u : BT * 2u <= acc_cols ? 2u : 1u;
  if (atm && u.KSPLIT == 1u && BT <= acc_cols && KSn >= 24u) { u.KSPLIT = 2u; u.NACC = 1u; }      // (depends on K and the tile only: conv3 chunks and the whole clip agree)
  u.NS = (BT > 256u || (!atm && BT > 192u)) ? 3u : 4u;
  // record stages: as many as fit beside the operand stages, up to about 100 KB in flight
  const size_t qstage = p.enc == P0P_ENC_Q4 ? UQ<P0P_ENC_Q4>::STAGE : p.enc == P0P_ENC_Q8 ? UQ<P0P_ENC_Q8>::STAGE : 0;
  const size_t fixed = 1024 + (atm ? 0 : (size_t)u.NS * U_A_BYTES) + (size_t)u.NS * BT * 128u + (size_t)U_EPI_BYTES + 512u;
  u.NQ = qstage ? (uint32_t)std::min<size_t>(std::min<size_t>(U_NQ_MAX, (100 * 1024 + qstage - 1) / qstage), (227 * 1024 - fixed) / qstage) : 0u;
  if (qstage && u.NQ < 2u) return fail(c, -12, "gemm: no room for the record stages of this tile shape");
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
  } else if (!make_map(&mx, xbase, p.K, p.M, xld, BT > 256u ? BT / 2u : BT)) return fail(c, -12, "gemm: the token tensor map could not be encoded");
  if (p.enc == P0P_ENC_F16) {
    if (!make_map(&mw, reinterpret_cast<const __half*>(p.W) + p.wk0, p.K, p.Nw, p.wG, 128u)) return fail(c, -12, "gemm: the weight tensor map could not be encoded");
  } else mw = mx;
  const size_t qbytes = p.enc == P0P_ENC_Q4 ? u.NQ * UQ<P0P_ENC_Q4>::STAGE : p.enc == P0P_ENC_Q8 ? u.NQ * UQ<P0P_ENC_Q8>::STAGE : 0;
  // at least 120 KB: one block per SM, so that a block never waits for another's tensor memory
  const size_t smem = std::max<size_t>(120 * 1024, 1024 + (atm ? 0 : (size_t)u.NS * U_A_BYTES) + (size_t)u.NS * BT * 128u + qbytes + (size_t)U_EPI_BYTES + 512u);
  const int grid = (int)std::min<uint64_t>((uint64_t)u.T0 + (uint64_t)(tiles_all - u.T0) * u.S, sms);
  const int smem_max = 227 * 1024;          // the most dynamic shared memory a block may opt into on sm_100
  if (smem > (size_t)smem_max) return fail(c, -12, "gemm: tile configuration needs %zu bytes of shared memory", smem);
  static bool ready = false;
  cudaError_t e = cudaSuccess;
  if (!ready) {
    if ((e = cudaFuncSetAttribute(k_gemm_umma<P0P_ENC_Q4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(k_gemm_umma<P0P_ENC_Q8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(k_gemm_umma<P0P_ENC_Q4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(k_gemm_umma<P0P_ENC_Q8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(k_gemm_umma<P0P_ENC_F16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max)) != cudaSuccess)
      return cuda_fail(c, e, "tensor-core kernel attribute");
    ready = true;
  }
  if (p.enc == P0P_ENC_Q4) { if (atm) k_gemm_umma<P0P_ENC_Q4, true><<<grid, U_THREADS, smem, c->stream>>>(u, mx, mw); else k_gemm_umma<P0P_ENC_Q4, false><<<grid, U_THREADS, smem, c->stream>>>(u, mx, mw); }
  else if (p.enc == P0P_ENC_Q8) { if (atm) k_gemm_umma<P0P_ENC_Q8, true><<<grid, U_THREADS, smem, c->stream>>>(u, mx, mw); else k_gemm_umma<P0P_ENC_Q8, false><<<grid, U_THREADS, smem, c->stream>>>(u, mx, mw); }
  else k_gemm_umma<P0P_ENC_F16, false><<<grid, U_THREADS, smem, c->stream>>>(u, mx, mw);
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(c, e, "tensor-core kernel launch");
  c->launches += 1;
  if (u.S > 1u) {
    k_umma_finish<<<dim3(tiles_all - u.T0, (BT + U_EPI_TB - 1u) / U_EPI_TB), 128, 0, c->stream>>>(u);
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(c, e, "split-K second stage launch");
    c->launches += 1;
  }
  return 0;
}

}  // namespace p0p
