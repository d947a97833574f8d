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
//   warps 6..13     dequant    two groups of four warps; a thread converts whole operand rows of 64 k (warp % 4 picks the 32 rows
//                              a warp may reach in tensor memory, warp / 4 the group): codes -> fp16 tile
//                              values f16(q*s+mn) / f16(q*s), bit-exact (packed HFMA2 path; a row whose scale / minimum fail the
//                              exactness test is redone in fp32 by its own lane), written straight into tensor memory
//                              (tcgen05.st): the multiply takes A from there
//   last warp       records    bulk copies of the quantised records (two 64-row record tiles x up to 256 k per copy pair)
// Tensor memory (512 columns): the accumulators first - two buffers for tiles up to 128 tokens (the next tile's multiplies
// overlap the epilogue), one beyond - then the dequantised operand's stages in every column behind them (quantised weights),
// or two accumulator buffers of 256 columns (fp16 weights, both operands in shared memory).  A tile has ONE accumulator:
// consecutive multiplies into the same accumulator issue back to back at the tensor pipe's rate (measured: 8.7 cycles each
// at 16 tokens, 114 at 256, whether they alternate between accumulators or not).  gate|up (swiglu) tiles interleave gate and
// up rows in the A tile, so
// that (gate, up) of one output sit in adjacent lanes.  RMSNorm / LayerNorm+modulation prologues are applied by a one-pass
// kernel into an fp16 scratch copy of the tokens (the same token tile would otherwise be re-normalised by every column
// tile).  Few output columns: the k loop is split into units whose partial sums k_umma_finish adds (split-K).
// Every mbarrier wait is bounded (sync.cuh); on a time-out the block reports a code and winds down.
#pragma once
#include <cuda.h>

#include <cmath>

#include "common.cuh"
#include "ctx.h"
#include "device_once.h"
#include "epilogue.cuh"
#include "sync.cuh"
#include "umma.cuh"

namespace p0p {

constexpr int U_THREADS = (6 + 8 + 1) * 32;   // producer, MMA, 4 epilogue, 8 dequantisation, record producer
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
  uint32_t NS;          // stages of the token ring (2 .. 8)
  uint32_t KW;          // k-steps of 64 k per pipeline step (1, 2 or 4)
  uint32_t NA;          // stages of the dequantised operand in tensor memory (a_col0 + NA * KW * 32 <= 512, NA <= 8); fp16 weights: = NS
  uint32_t acc_stride;  // tensor-memory columns from one accumulator buffer to the next
  uint32_t a_col0;      // first tensor-memory column of the operand stages (quantised weights): the accumulators end there
  uint32_t LOCK;        // 1: the token ring and the operand ring advance together and share their barriers (NA == NS)
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
// (KW: the pipeline step of the kernel variant; a record stage holds at least one whole step.)
template <int ENC, int KW = 1> struct UQ { static constexpr uint32_t REC = 0, REC_K = 64, RB = 0, KSUP = 1, STAGE = 0; };
template <int KW> struct UQ<P0P_ENC_Q4, KW> { static constexpr uint32_t REC = 1280, REC_K = 32, RB = 2560, KSUP = 4, STAGE = 2 * KSUP * RB + 128; };
template <int KW> struct UQ<P0P_ENC_Q8, KW> { static constexpr uint32_t REC = 4224, REC_K = 64, RB = 4224, KSUP = KW > 2 ? KW : 2, STAGE = 2 * KSUP * RB + 128; };

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

// Quantised weights: the dequantised operand lives in tensor memory (written with tcgen05.st) instead of shared memory.
// Shared-memory bandwidth is what bounds the kernel otherwise: per 64-k step a 128 x 64 fp16 tile would be
// written once and read once there, on top of the token tile and the records.  The dequantisation of a weight block costs
// the same whatever the tile's width, so a wide tile (up to 384 tokens as two multiplies of 192) halves that cost per token.
// fp16 weights: both operands in shared memory (TMA), 512 accumulator columns.
//
// EPI: the fused epilogue, a compile-time constant.  One instantiation per (encoding, epilogue): a kernel that carries
// all seven epilogues is ~470 KB of code, most of it never run by a given launch.
constexpr uint32_t U_NA_MAX = 8;         // most operand stages in tensor memory
constexpr uint32_t U_DEQ_WARPS = 8;      // two groups of four
constexpr uint32_t U_NX_MAX = 8;         // most stages of the token ring
// Pipeline steps.  One step covers KW k-steps of 64 k (KW = 1, 2 or 4, chosen per launch): every hand-over between the roles - a
// barrier wait, a fence, a commit, a trip round a warp's loop - costs a few hundred cycles of single-warp latency, which for
// narrow and medium tiles is more than the multiplies of 64 k take, so those tiles move 128 k per hand-over.
// Three producers feed the multiply, each through a ring of stages with a "ready" and a "free" mbarrier per stage:
//   X  token tiles (and fp16 weight tiles), NS stages of shared memory of KW sub-tiles each, filled by TMA;
//   Q  quantised records, NQ stages of shared memory, filled by bulk copies (KSUP k-steps each, a multiple of KW);
//   A  dequantised weight operand: NA stages of KW 32-column sub-stages of tensor memory (NA * KW <= 4), filled by the
//      dequantisation warps.
// Wide tiles are bound by the multiplies, and there every instruction the issuing warp runs between two multiplies shows in the
// total: X and A then advance in lock step (NA = NS) and SHARE their barriers - one wait and one commit per step.  Narrow tiles
// are bound by the hand-overs instead; their token tiles are small, so the X ring gets its own barriers and more stages than
// tensor memory has operand stages (the load of a tile is only issued once its stage is free, and with few stages that round
// trip would be exposed).
// Dequantisation: two groups of four warps; a thread converts one whole operand row (64 k) per k-step.  The groups take the steps
// in turn (each step's one or two k-steps by one group), except in the lock-step 128-k variant, whose two operand stages
// leave no room for that: there group g converts sub-step g of every step, both side by side.  The warps that wait are
// parked by the hardware (mbar_try), not spinning beside the ones that work.
// KW and LOCK are compile-time (four variants exist: (1, lock), (2, lock), (2, separate), (4, separate; 4-bit weights)): the issuing warp's loop is the
// critical path of wide tiles and must not carry run-time choices.
template <int ENC, int EPI, int KW_, bool LOCK_>
__global__ void __launch_bounds__(U_THREADS, 1) k_gemm_umma(const UmmaP u, const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW) {
  extern __shared__ unsigned char smem_raw[];
  constexpr bool ATM = ENC != P0P_ENC_F16;
  constexpr uint32_t KW = KW_;
  using Q = UQ<ENC, KW_>;
  constexpr bool lock = LOCK_;
  const KP& p = u.p;
  const uint32_t BT = u.BT, NS = u.NS, NQ = u.NQ;
  const uint32_t HB = BT > 256u ? BT / 2u : BT, NH = BT > 256u ? 2u : 1u;          // tokens per UMMA / TMA box, and how many of them make a tile
  const bool two_acc = u.NACC == 2u;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;                     // operand tiles need 1024-byte alignment
  unsigned char* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t XT = BT * 128u, XS = KW * XT;                                     // bytes of a token sub-tile (64 k) and of a stage
  const uint32_t a_st = base, x_st = a_st + (ATM ? 0u : NS * U_A_BYTES), q_st = x_st + NS * XS;
  const uint32_t acc_stride = u.acc_stride;
  const uint32_t epi_sh = q_st + (ENC == P0P_ENC_F16 ? 0u : NQ * Q::STAGE);
  const uint32_t bars = epi_sh + (uint32_t)U_EPI_BYTES;
  float* epi_ptr = reinterpret_cast<float*>(gbase + (epi_sh - base));
  // barrier slots (8 bytes each)
  const uint32_t xfull = bars, xempty = xfull + 8u * U_NX_MAX, afull = xempty + 8u * U_NX_MAX, aempty = afull + 8u * U_NA_MAX;
  const uint32_t wq_full = aempty + 8u * U_NA_MAX, wq_empty = wq_full + 8u * U_NQ_MAX;
  const uint32_t acc_full = wq_empty + 8u * U_NQ_MAX, acc_empty = acc_full + 16u, tmem_slot = acc_empty + 16u;
  const uint32_t NA = u.NA;                                                       // operand stage of step g: g % NA, its parity: (g / NA) & 1
  const uint32_t pfull = lock ? afull : xfull, pempty = lock ? aempty : xempty;   // the barriers the token producer works with

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  if (tid == 0) {
    for (uint32_t s = 0; s < U_NX_MAX; s++) { mbar_init(xfull + 8u * s, 1u); mbar_init(xempty + 8u * s, 1u); }      // the producer's expect_tx arrival / the multiplies' commit
    for (uint32_t s = 0; s < U_NA_MAX; s++) { mbar_init(afull + 8u * s, (ATM ? (KW == 2u && lock ? 8u : 4u) : 0u) + (lock ? 1u : 0u)); mbar_init(aempty + 8u * s, 1u); }       // the dequantisation warps of a step (+ the token producer) / the commit
    for (uint32_t s = 0; s < (uint32_t)U_NQ_MAX; s++) { mbar_init(wq_full + 8u * s, 1u); mbar_init(wq_empty + 8u * s, U_DEQ_WARPS); }
    for (uint32_t b = 0; b < 2u; b++) { mbar_init(acc_full + 8u * b, 1u); mbar_init(acc_empty + 8u * b, 4u); }
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, U_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot - base));

  const uint32_t tiles = u.n_tiles * u.m_tiles, KS = p.K / 64u, units = u.T0 + (tiles - u.T0) * u.S;
  constexpr bool swiglu = EPI == P0P_EPI_SWIGLU;

  if (warp == 0) {
    // ================================================================= producer of the token tiles (and fp16 weight tiles)
    if (lane == 0) {
      Ring r(NS);
      bool ok = true;
      const uint32_t nap = BT <= 64u ? 32u : 200u;                     // narrow tiles turn over quickly: poll their stages often
      for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t tile = un.tile, kb = un.kb, ke = un.ke;
        uint32_t nt, mt; tile_coords(u, tile, nt, mt);
        for (uint32_t k0 = kb; k0 < ke; k0 += KW, r.next()) {
          const uint32_t cnt = min(KW, ke - k0);
          if (!mbar_wait(pempty + 8u * r.s, r.ph ^ 1u, u.status, 201, nap)) { ok = false; break; }
          mbar_expect_tx(pfull + 8u * r.s, cnt * (XT + (ENC == P0P_ENC_F16 ? U_A_BYTES : 0u)));
          for (uint32_t j = 0; j < cnt; j++) {
            const uint32_t ks = k0 + j, dst = x_st + r.s * XS + j * XT;
            if (p.xmode == P0P_X_CONV3) {
              // implicit GEMM (src/ops/gemm.js:68-80): the 64 k of this k-step are channels c0.. of ONE tap (kt, ky, kx); the tile's
              // tokens are cvR whole rows of one output frame, so their inputs are a box of the clip shifted by the tap, and
              // what falls outside the image reads as zero.  Frame index: clamp to the clip, then ring slot or chunk offset.
              const uint32_t tpf = p.Ho / u.cvR, ot = mt / tpf, oy0 = (mt - ot * tpf) * u.cvR;
              const uint32_t kg = ks * 64u, tap = kg / p.Ci, c0 = kg - tap * p.Ci, kt = tap / 9u, ky = (tap / 3u) % 3u, kx = tap % 3u;
              const int itg = min(max((int)(ot + p.padT + kt) - 1, 0), (int)p.stride - 1);
              const int it = p.ks > 1u ? itg % (int)p.ks : itg - (int)p.padL;
              const uint32_t rb = u.cvR / NH;
              for (uint32_t h = 0; h < NH; h++)
                tma_load_4d(dst + h * HB * 128u, &mapX, (int)c0, (int)kx - 1, (int)(oy0 + h * rb + ky) - 1, it, pfull + 8u * r.s);
            } else if (p.xmode == P0P_X_CONV) {
              // 2-D implicit GEMM (src/ops/gemm.js:81-91): the tile's tokens are cvR whole output rows; the 64 k of this k-step are
              // channels c0.. of one tap (ky, kx) = (tap / ks, tap % ks).  The tensor map's element strides walk the input by the
              // convolution's stride, so output (oy, ox) reads input (oy * stride + ky - padT, ox * stride + kx - padL): the box
              // starts at the first output row / column's input position and what falls outside the image reads as zero.
              const uint32_t oy0 = mt * u.cvR;
              const uint32_t kg = ks * 64u, tap = kg / p.Ci, c0 = kg - tap * p.Ci, ky = tap / p.ks, kx = tap - ky * p.ks;
              const uint32_t rb = u.cvR / NH;
              for (uint32_t h = 0; h < NH; h++)
                tma_load_4d(dst + h * HB * 128u, &mapX, (int)c0, (int)kx - (int)p.padL, (int)((oy0 + h * rb) * p.stride + ky) - (int)p.padT, 0, pfull + 8u * r.s);
            } else
              for (uint32_t h = 0; h < NH; h++) tma_load_2d(dst + h * HB * 128u, &mapX, (int)(ks * 64u), (int)(mt * BT + h * HB), pfull + 8u * r.s);
            if (ENC == P0P_ENC_F16) tma_load_2d(a_st + (r.s * KW + j) * U_A_BYTES, &mapW, (int)(ks * 64u), (int)(p.wR0 + nt * 128u), pfull + 8u * r.s);
          }
        }
      }
    }
  } else if (warp == 6u + U_DEQ_WARPS) {
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
        const unsigned char* src0 = p.W + ((size_t)trow[0] * p.wG + p.wk0 / Q::REC_K) * Q::REC;
        const unsigned char* src1 = p.W + ((size_t)trow[1] * p.wG + p.wk0 / Q::REC_K) * Q::REC;
        for (uint32_t ks = kb; ks < ke; ks += Q::KSUP, q.next()) {
          const uint32_t bytes = min(Q::KSUP, ke - ks) * Q::RB;
          if (!mbar_wait(wq_empty + 8u * q.s, q.ph ^ 1u, u.status, 202, 200u)) { ok = false; break; }
          mbar_expect_tx(wq_full + 8u * q.s, 2u * bytes);
          bulk_g2s(q_st + q.s * Q::STAGE, src0 + (size_t)ks * Q::RB, bytes, wq_full + 8u * q.s);
          bulk_g2s(q_st + q.s * Q::STAGE + Q::KSUP * Q::RB + 64u, src1 + (size_t)ks * Q::RB, bytes, wq_full + 8u * q.s);
        }
      }
    }
  } else if (warp == 1) {
    // ================================================================= MMA issuer.  The WHOLE warp walks the loop and one
    // elected lane issues: in warp-uniform control flow the descriptors live in uniform registers, which is what the
    // instruction takes; inside a one-lane branch every operand of every tcgen05.mma is first moved there, which
    // costs more than the multiply itself.
    const uint32_t idesc = umma_idesc_f16(128u, HB);
    Ring r(NS), ar(NA);
    uint32_t tl = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x, tl++) {
      const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t kb = un.kb, ke = un.ke;
      const uint32_t buf = two_acc ? tl & 1u : 0u, par = two_acc ? (tl >> 1) & 1u : tl & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + 8u * buf, par ^ 1u, u.status, 203, 100u))) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * acc_stride;
      for (uint32_t k0 = kb; k0 < ke; k0 += KW, r.next(), ar.next()) {
        const uint32_t as = ar.s, cnt = min(KW, ke - k0);
        bool rdy = lock || mbar_wait(xfull + 8u * r.s, r.ph, u.status, 204);
        if (ATM || lock) rdy = rdy && mbar_wait(afull + 8u * as, ar.ph, u.status, 205);
        if (!__all_sync(0xffffffffu, rdy)) { ok = false; break; }
        tc_fence_after();
        // (operands computed in warp-uniform control flow: they stay in uniform registers, which is what the instruction takes)
        uint64_t bd[KW], ad[KW]; uint32_t at[KW];
#pragma unroll
        for (uint32_t j = 0; j < KW; j++) {
          bd[j] = umma_desc_sw128(x_st + r.s * XS + j * XT);
          at[j] = tmem_base + u.a_col0 + (as * KW + j) * 32u;
          ad[j] = umma_desc_sw128(a_st + (r.s * KW + j) * U_A_BYTES);
        }
        const uint32_t first = k0 - kb;                             // 0 on the unit's first k-step: the first multiply overwrites
        if (elect_one()) {
#pragma unroll
          for (uint32_t j = 0; j < KW; j++) {
            if (j < cnt) {
#pragma unroll
              for (uint32_t kk = 0; kk < 4u; kk++) {                  // per 16 k: 8 tensor-memory columns / +32 bytes
                // consecutive multiplies into ONE accumulator start ~180 cycles apart whatever their width; into different
                // accumulators ~35.  Narrow tiles therefore rotate over KSPLIT accumulators (wide ones over their two halves).
                const uint32_t dk = d_tmem + (kk & (u.KSPLIT - 1u)) * BT, accum = first | j | (kk >= u.KSPLIT ? 1u : 0u);
                if (ATM) {
                  umma_f16_ts(dk, at[j] + 8u * kk, bd[j] + 2u * kk, idesc, accum);
                  if (NH == 2u) umma_f16_ts(dk + HB, at[j] + 8u * kk, bd[j] + ((HB * 128u) >> 4) + 2u * kk, idesc, accum);
                } else {
                  umma_f16_ss(dk, ad[j] + 2u * kk, bd[j] + 2u * kk, idesc, accum);
                  if (NH == 2u) umma_f16_ss(dk + HB, ad[j] + 2u * kk, bd[j] + ((HB * 128u) >> 4) + 2u * kk, idesc, accum);
                }
              }
            }
          }
          if (!lock) umma_commit(xempty + 8u * r.s);
          if (ATM || lock) umma_commit(aempty + 8u * as);
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
        else {                                                   // the tile's last values are in registers: the accumulator is free for
          tc_fence_before();                                     // the next tile's multiplies while this pass still computes and stores
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty + 8u * buf);
        }
        if (un.split) {
          // split-K: this unit's partial sums, fp32, to its own slab; a warp's store covers 128 bytes of a row
          float* dst = u.sk_part + (((size_t)sp * (tiles - u.T0) + (tile - u.T0)) * BT + ch * U_EPI_TB) * 128u + c;
#pragma unroll
          for (int j = 0; j < U_EPI_TB; j++) dst[(size_t)j * 128u] = acc[j];
        } else epilogue_cols<U_EPI_TB, EPI>(p, m0 + ch * U_EPI_TB, nt * 128u, c, acc, epi_ptr, 2, vec, pass & 1u);
      }
      if (nchunks == 0u) {                                       // (cannot happen: a tile has tokens; kept so that the barrier's count never slips)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8u * buf);
      }
    }
  } else if (ENC != P0P_ENC_F16 && warp < 6u + U_DEQ_WARPS) {
    // ================================================================= dequantisation: codes -> fp16 operand rows in tensor
    // memory.  A warp reaches the tensor-memory lanes 32 * (warp % 4) .. + 31, which fixes its 32 weight rows; a thread
    // converts one whole operand row (64 k) of a k-step.  The loop runs over record stages (KSUP k-steps, i.e. KSUP / KW pipeline
    // steps); inside a stage a group visits its own k-steps: those of its parity in the running count of steps (KW = 1), or
    // sub-step `grp` of every step (KW = 2; a step whose second sub-step does not exist still gets group 1's arrival).
    const uint32_t r = (warp & 3u) * 32u + lane, grp = (warp - 6u) >> 2;
    const uint32_t tsel = swiglu ? (r & 1u) : (r >> 6), rr = swiglu ? (r >> 1) : (r & 63u);
    const uint32_t tile_off = tsel * (Q::KSUP * Q::RB + 64u);
    const uint32_t rec_row = tile_off + (ENC == P0P_ENC_Q4 ? rr * 16u : rr * 64u);
    const uint32_t rec_sm = tile_off + (ENC == P0P_ENC_Q4 ? 1024u + rr * 4u : 4096u + rr * 2u);
    const uint32_t ta0 = tmem_base + (((warp & 3u) * 32u) << 16) + u.a_col0;
    // How the two groups share the steps.  Steps of 64 k, and steps of 128 k with rings of their own (narrow tiles): the groups
    // take whole steps in turn, so a warp pays its trip round this loop - a few hundred cycles of serial latency whatever the work -
    // once per step it converts, and with three or more operand stages neither group waits for the multiplies of its own last
    // step.  Steps of 128 k in lock step (two stages only): group g converts sub-step g of every step, both side by side.
    constexpr bool ALT = KW == 1u || !lock;
    const uint32_t stride = ALT ? 2u : 1u;
    uint32_t as = ALT ? grp : 0u, aph = 0u;
    Ring qr(NQ);
    uint32_t gpar = 0;                                             // parity of the count of steps before this record stage (ALT)
    bool ok = true;
    // one operand row of k-step jj of the record stage -> 32 columns of tensor memory at ta
    auto convert = [&](uint32_t jj, uint32_t ta) {
      const uint32_t rec = q_st + qr.s * Q::STAGE + jj * Q::RB;
      if (ENC == P0P_ENC_Q4) {
        // both 32-k halves of the row are fetched first, so that the second half's loads are in flight while the first converts
        const uint4 c0 = u_lds128(rec + rec_row), c1 = u_lds128(rec + rec_row + 1280u);
        const uint32_t sm0 = u_lds32(rec + rec_sm), sm1 = u_lds32(rec + rec_sm + 1280u);
        const uint32_t w0[4] = {c0.x, c0.y, c0.z, c0.w}, w1[4] = {c1.x, c1.y, c1.z, c1.w};
        __half2 v[16];
        q4_row32(w0, sm0, v);
        tmem_st16(ta, *reinterpret_cast<const uint32_t(*)[16]>(v));
        q4_row32(w1, sm1, v);
        tmem_st16(ta + 16u, *reinterpret_cast<const uint32_t(*)[16]>(v));
      } else {
        const uint32_t sb = u_lds16(rec + rec_sm);
#pragma unroll
        for (uint32_t h = 0; h < 2u; h++) {
          const uint4 c0 = u_lds128(rec + rec_row + h * 32u), c1 = u_lds128(rec + rec_row + h * 32u + 16u);
          const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          __half2 v[16];
          q8_row<8>(w, sb, v);
          tmem_st16(ta + h * 16u, *reinterpret_cast<const uint32_t(*)[16]>(v));
        }
      }
    };
    for (uint32_t unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      const UnitOf un = unit_of(u, unit, tiles, KS); const uint32_t n = un.ke - un.kb;
      for (uint32_t j0 = 0; j0 < n && ok; j0 += Q::KSUP, qr.next()) {
        const uint32_t cnt = min(Q::KSUP, n - j0);
        bool fresh = true;                                         // the record stage is awaited at this group's first k-step in it
        if (ALT) {
          // the stage's steps (KW k-steps each, the last may be short); this group's are those of its parity in the running count
          const uint32_t nst = (cnt + KW - 1u) / KW;
          for (uint32_t st = grp ^ gpar; st < nst; st += 2u) {
            if ((fresh && !mbar_wait(wq_full + 8u * qr.s, qr.ph, u.status, 207)) || !mbar_wait(aempty + 8u * as, aph ^ 1u, u.status, 208)) { ok = false; break; }
            fresh = false;
#pragma unroll
            for (uint32_t sub = 0; sub < KW; sub++)
              if (st * KW + sub < cnt) convert(st * KW + sub, ta0 + (as * KW + sub) * 32u);
            tmem_st_wait(); tc_fence_before();                      // tensor-memory stores done and ordered before the MMA warp's read
            __syncwarp();
            if (lane == 0) mbar_arrive(afull + 8u * as);
            as += stride; if (as >= NA) { as -= NA; aph ^= 1u; }
          }
          gpar ^= nst & 1u;
        } else {
          // k-step jj of the record stage is this group's when jj % 2 == grp (sub-step grp of a step).  An odd tail: group 1 passes
          // the missing sub-step once, only to arrive (after the same wait for the free stage as any arrival).
          const uint32_t jend = cnt + (grp & cnt & 1u);
          for (uint32_t jj = grp; jj < jend; jj += 2u) {
            const bool have = jj < cnt;
            if ((have && fresh && !mbar_wait(wq_full + 8u * qr.s, qr.ph, u.status, 207)) || !mbar_wait(aempty + 8u * as, aph ^ 1u, u.status, 208)) { ok = false; break; }
            if (have) {
              fresh = false;
              convert(jj, ta0 + (as * KW + grp) * 32u);
              tmem_st_wait(); tc_fence_before();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(afull + 8u * as);
            as += stride; if (as >= NA) { as -= NA; aph ^= 1u; }
          }
        }
        // Every warp releases every record stage once, after its last k-step there.  A group with no k-step of its own in the
        // stage still waits for the stage to be filled first: its release must not land in the barrier phase of the stage's
        // previous contents.
        if (ok && fresh && !mbar_wait(wq_full + 8u * qr.s, qr.ph, u.status, 209)) { ok = false; break; }
        __syncwarp();
        if (lane == 0) mbar_arrive(wq_empty + 8u * qr.s);
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
template <int EPI>
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
  epilogue_cols<U_EPI_TB, EPI>(p, m0, nt * 128u, c, acc, sh, 1, epilogue_vec_ok(p), 0u);
}

// ---- the instantiations live in three translation units (umma_q4.cu, umma_q8.cu, umma_f16.cu); these tables find them.
// variant: 0 = (KW 1, lock step), 1 = (KW 2, lock step), 2 = (KW 2, separate token ring); fp16 weights have variant 0 only.
typedef void (*umma_kernel_fn)(const UmmaP, const CUtensorMap, const CUtensorMap);
typedef void (*umma_finish_fn)(const UmmaP);
umma_kernel_fn umma_kernel_q4(uint32_t variant, uint32_t epi);
umma_kernel_fn umma_kernel_q8(uint32_t variant, uint32_t epi);
umma_kernel_fn umma_kernel_f16(uint32_t epi);
umma_finish_fn umma_finish_kernel(uint32_t epi);
#define P0P_UMMA_ROW(ENC, KW, LOCK) {k_gemm_umma<ENC, P0P_EPI_F16, KW, LOCK>, k_gemm_umma<ENC, P0P_EPI_F32, KW, LOCK>, k_gemm_umma<ENC, P0P_EPI_RESADD, KW, LOCK>, \
                                     k_gemm_umma<ENC, P0P_EPI_SWIGLU, KW, LOCK>, k_gemm_umma<ENC, P0P_EPI_HEADS, KW, LOCK>, k_gemm_umma<ENC, P0P_EPI_BIAS, KW, LOCK>, \
                                     k_gemm_umma<ENC, P0P_EPI_ONORMGATE, KW, LOCK>}

}  // namespace p0p
