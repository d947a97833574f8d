// Decode-sized multiply (up to 16 tokens, the library's own choice up to 8; q4 / q8 weights): the call is bound by
// streaming the weights out of HBM once, so the kernel is built around that stream.
//
//   stage 1  k_decode_stream   The weight is cut into (64-row tile) x (k-block) units, a unit into stages of 256 k; the
//            stages, in unit order, are dealt out evenly to a grid of about three blocks per SM: every block gets the
//            same number of stages (+-1), so a block's range may begin and end inside a unit, and a unit may be shared
//            by two blocks (never three: a range is at least a unit long).  Handing out whole units instead left the
//            LLM block's shapes (896 units on 444 blocks) with a few blocks that had 3 units against 2.
//            In each block one producer lane moves whole records from global to
//            shared memory with bulk asynchronous copies (cp.async.bulk, mbarrier-tracked, a ring of stages);
//            eight consumer warps: four row groups of 16 rows, two warps each that split a stage's records.
//            Codes go to the tensor cores WITHOUT being dequantised.  A 4-bit code q is left where it sits and read as
//            an fp16 SUBNORMAL: masked to bits 0..3 of a half it is q * 2^-24, masked to bits 4..7 it is 16 q * 2^-24
//            (its token is staged pre-divided by 16), one AND per code pair and no offset to correct for.  An 8-bit
//            code becomes the pattern 0x6400|(q+128) (= 1152 + q).  mma.sync.m16n8k16 (weights = A, tokens = B, fp32
//            accumulate) sums code * x over one group; the group's scale and minimum are applied to the fp32 sum:
//            q4:  y += (s * 2^24) * acc + mn * Sx;   q8:  y += s * (acc - 1152 * Sx),
//            where Sx (the sum of the group's tokens) depends only on the tokens and is tabulated once per k-block
//            (q8: as the accumulator's starting value).  The tokens are staged in shared memory in the operand order
//            of the instruction, with the fused prologue (plain fp16 / RMSNorm / LayerNorm+modulation)
//            applied on the way in.  The 64 x M partial sums of each unit, or of each part of a shared unit, go to a
//            scratch buffer: part 0 = the part that starts at the unit's first stage, part 1 = the rest.
//   stage 2  k_decode_finish   sums the partials in a fixed order (k-block by k-block, part 0 then part 1; which units have
//            a part 1 follows from the same arithmetic that dealt out the stages: deterministic, no atomics, nothing to
//            clear) and applies the fused epilogue.
// Both kernels are launched as programmatic dependents: stage 2 is resident before stage 1 ends, and the next call's
// stage 1 streams its first weights while this call's stage 2 still runs; each waits (griddepcontrol.wait) before it
// touches what the kernel before it writes.
//
// Every wait on an mbarrier is bounded; on a time-out the block records a code in the context's status word
// and leaves.
#pragma once
#include "common.cuh"
#include "ctx.h"
#include "epilogue.cuh"
#include "sync.cuh"

namespace p0p {

constexpr int D_CONSUMERS = 256;            // 8 warps: 4 row groups of 16 rows x 2 warps that split each stage's records
constexpr int D_THREADS = D_CONSUMERS + 32; // + the producer warp
constexpr int D_STAGES = 5;
constexpr int D_STAGE_K = 256;              // k per stage: 8 q4 records (10240 B) or 4 q8 records (16896 B): one bulk copy each
constexpr int D_STAGE_BYTES_Q4 = 10240, D_STAGE_BYTES_Q8 = 16896;
constexpr int D_MAX_KC = 2048;              // largest k-block
constexpr int D_SMEM_MAX = 144 * 1024;      // dynamic shared memory ceiling of the stream kernel

struct DecodeP {
  KP p;
  uint32_t Mp;        // token columns fed to the tensor core: 8 or 16
  uint32_t tiles;     // 64-row tiles the call touches (swiglu: gate tiles then up tiles)
  uint32_t th;        // swiglu: tiles per half; else = tiles
  uint32_t KC, S;     // k-block length (multiple of 128) and count
  uint32_t units;     // tiles * S
  uint32_t nslots;    // tiles * 64
  uint32_t T, G;      // stages of the whole call (tiles * K / 256) and blocks of the stream kernel: block b takes stages [b*T/G, (b+1)*T/G)
  uint32_t whole;     // 1: the ranges are rounded to whole units instead (many units per block: the even split gains nothing there
                      // and costs a partial unit per block)
  float* scratch;     // [S][2 parts][M][nslots] fp32
  int* status;
  uint32_t vec32;     // fp32 tokens and the prologue vector may be read with 16-byte loads
};

// weight tile index (64 rows) of unit-local tile t
__device__ __forceinline__ uint32_t d_tile_row0(const DecodeP& d, uint32_t t) {
  if (d.p.epi == P0P_EPI_SWIGLU) return t < d.th ? d.p.wR0 + t * 64u : d.p.wR1 + (t - d.th) * 64u;
  return d.p.wR0 + t * 64u;
}

// Stage i of the call, in unit order (k-block by k-block, tile by tile, then along k): which unit, and where in it.
struct DSeg { uint32_t kb, t, st, spk; };       // k-block, tile, stage within the unit, stages of this k-block's units
__device__ __forceinline__ DSeg d_seg(const DecodeP& d, uint32_t i) {
  const uint32_t spk = d.KC / (uint32_t)D_STAGE_K, per_kb = d.tiles * spk;
  DSeg g;
  g.kb = min(i / per_kb, d.S - 1u);
  const uint32_t rem = i - g.kb * per_kb;
  g.spk = min(d.KC, d.p.K - g.kb * d.KC) / (uint32_t)D_STAGE_K;               // the last k-block may be shorter
  g.t = rem / g.spk; g.st = rem - g.t * g.spk;
  return g;
}
// (T * G stays below 2^32: the plan sees to it, so that these divisions are 32-bit ones — the second stage does two per k-block)
__device__ __forceinline__ uint32_t d_range(const DecodeP& d, uint32_t b) {
  return d.whole ? ((b * d.units) / d.G) * (d.KC / (uint32_t)D_STAGE_K) : (b * d.T) / d.G;
}
// does a block boundary fall strictly inside the unit that spans stages [u0, u0 + n)?  (then the unit has a part 1)
__device__ __forceinline__ bool d_unit_split(const DecodeP& d, uint32_t u0, uint32_t n) {
  if (d.whole) return false;
  const uint32_t b = ((u0 + 1u) * d.G + d.T - 1u) / d.T;                         // the first boundary above u0
  return b < d.G && d_range(d, b) < u0 + n;
}

// ---- token staging: one thread per (token, 8 consecutive k): 16-byte loads, the fused prologue, 16 bytes of operand.
// The 4 (q4: groups of 32 k) or 8 (q8: groups of 64 k) neighbouring lanes of a scale group add up the group's token sum:
//   cts[gi][token pair] = float2(Sx_a, Sx_b)                     q4: the plain sums (they carry the group minimum)
//   ctc[gi][token pair] = float4(-C_a, -C_b, -C_a, -C_b)          q8: C = 1152 * Sx, the accumulator fragment (rows g / g+8 x
//                                                                tokens a, b) the multiply starts from
// klen is a multiple of 256, so a warp's 32 items are consecutive chunks of ONE token and the lane groups line up.
template <int ENC, int XMODE, int MP>
__device__ __forceinline__ void d_stage_tokens(const DecodeP& d, uint32_t kb0, uint32_t klen, unsigned char* xs, float* ctc, float* cts, uint32_t tok_stride, uint32_t tid) {
  const KP& p = d.p;
  constexpr uint32_t GL = ENC == P0P_ENC_Q4 ? 4u : 8u;            // lanes per scale group
  const uint32_t chunks = klen / 8u, lane = tid & 31u;
  for (uint32_t it = tid; it < p.M * chunks; it += D_CONSUMERS) {
    const uint32_t m = it / chunks, c8 = it - m * chunks, k0 = kb0 + c8 * 8u;
    float v[8];
    if (XMODE == P0P_X_F16) {
      const __half* src = reinterpret_cast<const __half*>(p.X) + (size_t)m * p.ldx + p.kx0 + k0;
      if (p.vecx) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(src));
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __half2float(src[i]);
      }
    } else {
      // (the host admits this kernel only when x rows and the vector are 16-byte aligned: see decode_supported)
      const float* src = reinterpret_cast<const float*>(p.X) + (size_t)m * p.ldx + p.kx0 + k0;
      const size_t sr = ((size_t)p.statOff + m) * 2u;
      const float mean = __ldg(p.ST + sr), rstd = __ldg(p.ST + sr + 1);
      const float* pv = p.PV + p.pvOff + p.kx0 + k0;
      float xv[8], g1[8], g2[8];
      if (d.vec32) {
        *reinterpret_cast<float4*>(xv) = __ldg(reinterpret_cast<const float4*>(src)); *reinterpret_cast<float4*>(xv + 4) = __ldg(reinterpret_cast<const float4*>(src) + 1);
        *reinterpret_cast<float4*>(g1) = __ldg(reinterpret_cast<const float4*>(pv)); *reinterpret_cast<float4*>(g1 + 4) = __ldg(reinterpret_cast<const float4*>(pv) + 1);
        if (XMODE == P0P_X_LNMOD) { *reinterpret_cast<float4*>(g2) = __ldg(reinterpret_cast<const float4*>(pv + p.pvStride)); *reinterpret_cast<float4*>(g2 + 4) = __ldg(reinterpret_cast<const float4*>(pv + p.pvStride) + 1); }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) { xv[i] = __ldg(src + i); g1[i] = __ldg(pv + i); if (XMODE == P0P_X_LNMOD) g2[i] = __ldg(pv + p.pvStride + i); }
      }
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float t = XMODE == P0P_X_LNMOD ? (xv[i] - mean) * rstd * (1.0f + g1[i]) + g2[i] : xv[i] * rstd * g1[i];
        v[i] = __half2float(__float2half_rn(t));            // the prologue's result is an fp16 value (src/ops/gemm.js:66-67)
      }
    }
    float sx = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    __half2 o[4];
    if (ENC == P0P_ENC_Q4) {
      // per 8 columns: [k0, k4, k1/16, k5/16, k2, k6, k3/16, k7/16]  (odd nibbles carry 16*q, so their token is pre-divided)
      o[0] = __floats2half2_rn(v[0], v[4]);
      o[1] = __floats2half2_rn(v[1] * 0.0625f, v[5] * 0.0625f);
      o[2] = __floats2half2_rn(v[2], v[6]);
      o[3] = __floats2half2_rn(v[3] * 0.0625f, v[7] * 0.0625f);
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) o[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(xs + (size_t)m * tok_stride + (size_t)c8 * 16u) = *reinterpret_cast<const uint4*>(o);
    // the group's sum: its GL lanes are neighbours (a whole warp always runs this loop body together: M * chunks is a multiple of 32)
#pragma unroll
    for (uint32_t o2 = 1; o2 < GL; o2 <<= 1) sx += __shfl_xor_sync(0xffffffffu, sx, o2);
    if ((lane & (GL - 1u)) == 0u) {
      const uint32_t gi = c8 / GL;
      if (ENC == P0P_ENC_Q4) cts[((size_t)gi * (MP / 2) + (m >> 1)) * 2u + (m & 1u)] = sx;
      else { float* c = ctc + ((size_t)gi * (MP / 2) + (m >> 1)) * 4u + (m & 1u); c[0] = -1152.0f * sx; c[2] = -1152.0f * sx; }
    }
  }
}

// Loads through 32-bit shared-window addresses: address arithmetic stays in 32 bits and folds into immediates.
// They are plain (non-volatile) asm so that the compiler may overlap the records of a stage; `anchor` ties their
// addresses to a point after the stage's mbarrier wait, so none of them can move above it.
__device__ __forceinline__ uint32_t anchor(uint32_t a) { uint32_t v; asm volatile("mov.u32 %0, %1;" : "=r"(v) : "r"(a) : "memory"); return v; }
// The byte offset is a template argument so that it becomes the instruction's immediate (an asm operand in a
// register would cost one address add per load).
template <uint32_t O> __device__ __forceinline__ uint32_t lds32(uint32_t a) { uint32_t v; asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(O)); return v; }
template <uint32_t O> __device__ __forceinline__ uint16_t lds16(uint32_t a) { uint16_t v; asm("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(a), "n"(O)); return v; }
template <uint32_t O> __device__ __forceinline__ uint4 lds128(uint32_t a) { uint4 v; asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(O)); return v; }
template <uint32_t O> __device__ __forceinline__ float2 lds64f(uint32_t a) { float2 v; asm("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(a), "n"(O)); return v; }
template <uint32_t O> __device__ __forceinline__ float4 lds128f(uint32_t a) { float4 v; asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a), "n"(O)); return v; }
// the token operand of lanes whose token column does not exist is zero: the load is predicated off for them
template <uint32_t O> __device__ __forceinline__ uint4 lds128_if(uint32_t a, uint32_t on) {
  uint4 v;
  asm("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\tmov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}"
      : "=&r"(v.x), "=&r"(v.y), "=&r"(v.z), "=&r"(v.w) : "r"(a), "r"(on), "n"(O));
  return v;
}

// (a & mask) | magic in ONE instruction (left to the compiler this becomes two)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(magic));
  return d;
}

// D = A * B + C with C given separately (the correction terms ride in on C)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, const float (&c)[4]) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// per-lane constants of the consumer loop
struct DLane { uint32_t MLO, MHI, MAGIC; uint32_t on0, on1; bool one; };

// one q4 record (64 rows x 32 k) of this warp's share of a stage: R is its index in the share.  ta: sums of s * acc (to be
// scaled by 2^24), tb: sums of mn * Sx.
template <int MP, uint32_t R>
__device__ __forceinline__ void d_rec_q4(float (&ta)[MP / 8][4], float (&tb)[MP / 8][4], uint32_t ca, uint32_t sa, uint32_t xk0, uint32_t xk1, uint32_t sk, const DLane& L) {
  const uint32_t wl = lds32<R * 1280u>(ca), wh = lds32<R * 1280u + 128u>(ca);
  const uint32_t sml = lds32<R * 1280u>(sa), smh = lds32<R * 1280u + 32u>(sa);
  // nibble pairs as fp16 subnormals: (k0,k4) (k1,k5) of the low byte pair, then (k2,k6) (k3,k7)
  const uint32_t wl8 = wl >> 8, wh8 = wh >> 8;
  const uint32_t l0 = wl & L.MLO, h0 = wl & L.MHI, l1 = wl8 & L.MLO, h1 = wl8 & L.MHI;
  const uint32_t L0 = wh & L.MLO, H0 = wh & L.MHI, L1 = wh8 & L.MLO, H1 = wh8 & L.MHI;
  const float2 fl = __half22float2(*reinterpret_cast<const __half2*>(&sml)), fh = __half22float2(*reinterpret_cast<const __half2*>(&smh));   // (scale, min)
  const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int h = 0; h < MP / 8; h++) {
    const uint4 b = h == 0 ? lds128<R * 64u>(xk0) : lds128<R * 64u>(xk1);                     // token columns past M read the row of zeros
    const float2 sx = h == 0 ? lds64f<R * (MP / 2) * 8u>(sk) : lds64f<(R * (MP / 2) + 4u) * 8u>(sk);
    float acc[4], acc2[4];
    mma_16816(acc, l0, L0, h0, H0, b.x, b.y, zero);
    mma_16816(acc2, l1, L1, h1, H1, b.z, b.w, acc);
    ta[h][0] = fmaf(fl.x, acc2[0], ta[h][0]); tb[h][0] = fmaf(fl.y, sx.x, tb[h][0]);
    ta[h][2] = fmaf(fh.x, acc2[2], ta[h][2]); tb[h][2] = fmaf(fh.y, sx.x, tb[h][2]);
    if (!L.one) {
      ta[h][1] = fmaf(fl.x, acc2[1], ta[h][1]); tb[h][1] = fmaf(fl.y, sx.y, tb[h][1]);
      ta[h][3] = fmaf(fh.x, acc2[3], ta[h][3]); tb[h][3] = fmaf(fh.y, sx.y, tb[h][3]);
    }
  }
}
// one q8 record (64 rows x 64 k)
template <int MP, uint32_t R>
__device__ __forceinline__ void d_rec_q8(float (&tot)[MP / 8][4], uint32_t ca, uint32_t sa, uint32_t xk0, uint32_t xk1, uint32_t ck, const DLane& L) {
  const uint4 ql = lds128<R * 4224u>(ca), qh = lds128<R * 4224u + 512u>(ca);
  const float sl = __half2float(__ushort_as_half(lds16<R * 4224u>(sa))), sh = __half2float(__ushort_as_half(lds16<R * 4224u + 16u>(sa)));
  const uint32_t wl[4] = {ql.x ^ 0x80808080u, ql.y ^ 0x80808080u, ql.z ^ 0x80808080u, ql.w ^ 0x80808080u};
  const uint32_t wh[4] = {qh.x ^ 0x80808080u, qh.y ^ 0x80808080u, qh.z ^ 0x80808080u, qh.w ^ 0x80808080u};
#pragma unroll
  for (int h = 0; h < MP / 8; h++) {
    // this lane's 16 columns of the record: 16*t4 .. 16*t4+15, natural order, 32 bytes
    const uint4 b0 = h == 0 ? lds128_if<R * 128u>(xk0, L.on0) : lds128_if<R * 128u>(xk1, L.on1);
    const uint4 b1 = h == 0 ? lds128_if<R * 128u + 16u>(xk0, L.on0) : lds128_if<R * 128u + 16u>(xk1, L.on1);
    const uint32_t bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const float4 c = h == 0 ? lds128f<R * (MP / 2) * 16u>(ck) : lds128f<(R * (MP / 2) + 4u) * 16u>(ck);      // the accumulator starts at -C
    float acc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float nx[4];
      mma_16816(nx, __byte_perm(wl[j], 0x64646464u, 0x4140), __byte_perm(wh[j], 0x64646464u, 0x4140),
                __byte_perm(wl[j], 0x64646464u, 0x4342), __byte_perm(wh[j], 0x64646464u, 0x4342), bb[2 * j], bb[2 * j + 1], acc);
#pragma unroll
      for (int i = 0; i < 4; i++) acc[i] = nx[i];
    }
    tot[h][0] = fmaf(sl, acc[0], tot[h][0]);
    tot[h][1] = fmaf(sl, acc[1], tot[h][1]);
    tot[h][2] = fmaf(sh, acc[2], tot[h][2]);
    tot[h][3] = fmaf(sh, acc[3], tot[h][3]);
  }
}

template <int ENC, int XMODE, int MP>
__global__ void __launch_bounds__(D_THREADS) k_decode_stream(const DecodeP d) {
  extern __shared__ __align__(128) unsigned char smem[];
  const KP& p = d.p;
  constexpr uint32_t TOK_PAD = ENC == P0P_ENC_Q4 ? 64u : 16u;           // keeps the operand loads free of bank conflicts
  constexpr uint32_t GS = ENC == P0P_ENC_Q4 ? 32u : 64u;
  const uint32_t tok_stride = d.KC * 2u + TOK_PAD;
  // layout: stages | token tile (M rows + one row of zeros) | C fragments | Sx pairs | pair-combine buffer | barriers
  unsigned char* stages = smem;
  constexpr uint32_t D_STAGE_BYTES = ENC == P0P_ENC_Q4 ? D_STAGE_BYTES_Q4 : D_STAGE_BYTES_Q8;
  unsigned char* xs = stages + D_STAGES * D_STAGE_BYTES;
  float* ctc = reinterpret_cast<float*>(xs + (((p.M + 1u) * tok_stride + 127u) & ~127u));       // [group][pair] float4 (-Ca, -Cb, -Ca, -Cb)
  float* cts = ctc + (d.KC / GS) * (MP / 2) * 4u;                                              // [group][pair] float2 (Sx_a, Sx_b)   (q4 only)
  float* comb = cts + (ENC == P0P_ENC_Q4 ? (d.KC / GS) * (MP / 2) * 2u : 0u);                  // [4 row groups][32 lanes][MP/2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(comb + 4u * 32u * (MP / 2));
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + D_STAGES);

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  if (tid == 0) {
    for (int s = 0; s < D_STAGES; s++) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, D_CONSUMERS / 32); }
    fence_mbar_init();
  }
  // the row of zeros that token columns past M read
  for (uint32_t i = tid; i < tok_stride / 16u; i += D_THREADS) reinterpret_cast<uint4*>(xs + (size_t)p.M * tok_stride)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  grid_launch_dependents();                 // the second stage may be brought onto the SMs now; it waits for this grid to finish

  const uint32_t i0 = d_range(d, blockIdx.x), i1 = d_range(d, blockIdx.x + 1u);      // this block's stages
  constexpr uint32_t REC = ENC == P0P_ENC_Q4 ? 1280u : 4224u, REC_K = ENC == P0P_ENC_Q4 ? 32u : 64u;
  constexpr uint32_t STAGE_TX = (D_STAGE_K / REC_K) * REC;              // a k-block is a whole number of stages (K % 128 == 0)
  constexpr uint32_t RPW = (D_STAGE_K / REC_K) / 2u;                    // records of a stage per consumer warp (two warps share 16 rows)

  if (warp == D_CONSUMERS / 32) {
    // ------------------------------------------------------------------ producer: one lane streams the records
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      for (uint32_t i = i0; i < i1;) {
        const DSeg sg = d_seg(d, i);
        const uint32_t n = min(i1 - i, sg.spk - sg.st);                           // stages of this unit in the block's range
        const uint32_t r0 = d_tile_row0(d, sg.t);
        const unsigned char* src = p.W + ((size_t)(r0 >> 6) * p.wG + (p.wk0 + sg.kb * d.KC + sg.st * D_STAGE_K) / REC_K) * REC;
        for (uint32_t q = 0; q < n; q++, src += STAGE_TX) {
          if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, d.status, 101, 200u)) return;
          mbar_expect_tx(full0 + 8u * s, STAGE_TX);
          bulk_g2s(smem_u32(stages + s * D_STAGE_BYTES), src, STAGE_TX, full0 + 8u * s);
          if (++s == D_STAGES) { s = 0; ph ^= 1u; }
        }
        i += n;
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers: warp = (half, row group)
  const uint32_t g = lane >> 2, t4 = lane & 3u, rg = warp & 3u, half = warp >> 2;
  const uint32_t rlo = rg * 16u + g;                                     // this lane's rows: rlo and rlo + 8
  // shared-window addresses that stay fixed for the whole kernel (this warp's first record of a stage included)
  const uint32_t code0 = smem_u32(stages) + half * RPW * REC + (ENC == P0P_ENC_Q4 ? rlo * 16u + t4 * 4u : rlo * 64u + t4 * 16u);
  const uint32_t sm0 = smem_u32(stages) + half * RPW * REC + (ENC == P0P_ENC_Q4 ? 1024u + rlo * 4u : 4096u + rlo * 2u);
  // token columns past M read the row of zeros
  const uint32_t xrow0 = smem_u32(xs) + min(g, p.M) * tok_stride + half * RPW * REC_K * 2u + (ENC == P0P_ENC_Q4 ? t4 * 16u : t4 * 32u);
  const uint32_t xrow1 = smem_u32(xs) + min(g + 8u, p.M) * tok_stride + half * RPW * REC_K * 2u + (ENC == P0P_ENC_Q4 ? t4 * 16u : t4 * 32u);
  // this lane's token pair (2 t4, 2 t4 + 1); + 4 pairs for tokens 8..15.  With a single token every lane reads pair 0
  // (one address per warp instead of four)
  const uint32_t tp = p.M == 1u ? 0u : t4;
  const uint32_t ctc_l = smem_u32(ctc) + (half * RPW * (MP / 2) + tp) * 16u;
  const uint32_t cts_l = smem_u32(cts) + (half * RPW * (MP / 2) + tp) * 8u;
  float* comb_l = comb + (rg * 32u + lane) * (MP / 2);
  DLane L;
  L.MLO = 0x000f000fu; L.MHI = 0x00f000f0u; L.MAGIC = 0x64006400u;      // (masks live in registers: as immediates each AND would cost a constant load)
  L.on0 = g < p.M ? 1u : 0u; L.on1 = g + 8u < p.M ? 1u : 0u;            // does this lane's token column exist?
  L.one = p.M == 1u;                                                     // a single token: only the accumulators of token 0 are kept up
  uint32_t s = 0, ph = 0, cur_kb = 0xffffffffu;
  bool ok = true;
  // The weights stream from the start (the producer above never waits for another kernel).  Tokens, statistics and the scratch
  // buffer may still be in use by the kernel before this one in the stream: the consumers wait for it here.
  grid_dependency_wait();
  // `ok` turns false when a bounded wait ran out: the warp then skips all work but still meets the others at
  // the named barriers below, so nobody is left waiting for it.
  for (uint32_t si = i0; si < i1;) {
    const DSeg sg = d_seg(d, si);
    const uint32_t nst = min(i1 - si, sg.spk - sg.st);
    si += nst;
    const uint32_t kb = sg.kb, t = sg.t;
    const uint32_t k_beg = kb * d.KC, klen = sg.spk * D_STAGE_K, kfrom = sg.st * D_STAGE_K, kto = kfrom + nst * D_STAGE_K;
    const uint32_t part = sg.st ? 1u : 0u;
    if (kb != cur_kb) {                       // a new k-block: restage the tokens (all consumers are past the old ones)
      bar_sync_named(1, D_CONSUMERS);
      if (ok) d_stage_tokens<ENC, XMODE, MP>(d, k_beg, klen, xs, ctc, cts, tok_stride, tid);
      bar_sync_named(1, D_CONSUMERS);
      cur_kb = kb;
    }
    float tot[MP / 8][4], tmn[MP / 8][4];            // q4: tot = sums of s * acc (still to be scaled by 2^24), tmn = sums of mn * Sx
#pragma unroll
    for (int h = 0; h < MP / 8; h++)
#pragma unroll
      for (int i = 0; i < 4; i++) { tot[h][i] = 0.0f; tmn[h][i] = 0.0f; }

    for (uint32_t k = kfrom; ok && k < kto; k += D_STAGE_K) {
      if (!mbar_wait(full0 + 8u * s, ph, d.status, 102)) { ok = false; break; }
      const uint32_t so = anchor(s * D_STAGE_BYTES), ko = anchor(k);
      const uint32_t ca = code0 + so, sa = sm0 + so;
      const uint32_t xk0 = xrow0 + ko * 2u, xk1 = xrow1 + ko * 2u;
      if (ENC == P0P_ENC_Q4) {
        const uint32_t sk = cts_l + (ko / GS) * (MP / 2) * 8u;
        static_assert(D_STAGE_K == 256, "four q4 records / two q8 records per consumer warp and stage");
        d_rec_q4<MP, 0>(tot, tmn, ca, sa, xk0, xk1, sk, L);
        d_rec_q4<MP, 1>(tot, tmn, ca, sa, xk0, xk1, sk, L);
        d_rec_q4<MP, 2>(tot, tmn, ca, sa, xk0, xk1, sk, L);
        d_rec_q4<MP, 3>(tot, tmn, ca, sa, xk0, xk1, sk, L);
      } else {
        const uint32_t ck = ctc_l + (ko / GS) * (MP / 2) * 16u;
        d_rec_q8<MP, 0>(tot, ca, sa, xk0, xk1, ck, L);
        d_rec_q8<MP, 1>(tot, ca, sa, xk0, xk1, ck, L);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8u * s);
      if (++s == D_STAGES) { s = 0; ph ^= 1u; }
    }
    // ---- the two warps of a row group add up (through shared memory), then this unit's partial sums go to
    // scratch[kb][part][token][slot].  Both named barriers are met in drain mode too.
    if (ENC == P0P_ENC_Q4) {
#pragma unroll
      for (int h = 0; h < MP / 8; h++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[h][i] = fmaf(tot[h][i], 16777216.0f, tmn[h][i]);      // the codes entered as q * 2^-24
    }
    if (half == 1u) {
#pragma unroll
      for (int h = 0; h < MP / 8; h++) *reinterpret_cast<float4*>(comb_l + 4 * h) = make_float4(tot[h][0], tot[h][1], tot[h][2], tot[h][3]);
    }
    bar_sync_named(2 + rg, 64);
    if (half == 0u && ok) {
#pragma unroll
      for (int h = 0; h < MP / 8; h++) {
        const float4 o = *reinterpret_cast<const float4*>(comb_l + 4 * h);
        const float v[4] = {tot[h][0] + o.x, tot[h][1] + o.y, tot[h][2] + o.z, tot[h][3] + o.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const uint32_t tok = 2u * t4 + (i & 1) + 8u * h, row = (i & 2) ? rlo + 8u : rlo;
          if (tok < p.M) d.scratch[((size_t)(kb * 2u + part) * p.M + tok) * d.nslots + t * 64u + row] = v[i];
        }
      }
    }
    bar_sync_named(2 + rg, 64);
  }
}

// ---- stage 2: fixed-order sum over the k-blocks, then the fused epilogue (a compile-time constant: one instantiation per
// kind keeps this latency-bound kernel small).  One block per 128 output columns.
template <int MP, int EPI>
__global__ void __launch_bounds__(128) k_decode_finish(const DecodeP d) {
  __shared__ __align__(16) float sh[MP * 132];
  const KP& p = d.p;
  const uint32_t c = threadIdx.x, nB = blockIdx.x * 128u, col = nB + c;
  uint32_t slot;
  if (EPI == P0P_EPI_SWIGLU) slot = ((col & 1u) ? d.th * 64u : 0u) + (col >> 1);
  else slot = col;
  slot = min(slot, d.nslots - 1u);
  grid_dependency_wait();                       // the partial sums come from the stream kernel this launch may overlap with
  // the partials of one output are read in batches of eight independent loads (a unit's part 1 only where the unit was
  // shared by two blocks), then added in k-block order
  const uint32_t tile = slot >> 6, spk = d.KC / (uint32_t)D_STAGE_K;
  float acc[MP];
#pragma unroll
  for (int j = 0; j < MP; j++) acc[j] = 0.0f;
  for (uint32_t kb0 = 0; kb0 < d.S; kb0 += 8u) {
    uint32_t two = 0u;                                            // bit i: k-block kb0 + i has a part 1 for this column's tile
#pragma unroll
    for (uint32_t i = 0; i < 8u; i++) {
      const uint32_t kb = min(kb0 + i, d.S - 1u), n = min(d.KC, p.K - kb * d.KC) / (uint32_t)D_STAGE_K;
      if (kb0 + i < d.S && d_unit_split(d, kb * d.tiles * spk + tile * n, n)) two |= 1u << i;
    }
#pragma unroll
    for (int j = 0; j < MP; j++) {
      if ((uint32_t)j < p.M) {
        float v[8], w[8];
#pragma unroll
        for (uint32_t i = 0; i < 8u; i++) {
          const float* src = d.scratch + ((size_t)((kb0 + i) * 2u) * p.M + j) * d.nslots + slot;
          v[i] = kb0 + i < d.S ? __ldcg(src) : 0.0f;
          w[i] = (two >> i) & 1u ? __ldcg(src + (size_t)p.M * d.nslots) : 0.0f;
        }
#pragma unroll
        for (uint32_t i = 0; i < 8u; i++) { acc[j] += v[i]; acc[j] += w[i]; }
      }
    }
  }
  grid_launch_dependents();
  epilogue_cols<MP, EPI>(p, 0u, nB, c, acc, sh, 1);
}

// ---- host side (decode.cu): which calls the kernel pair takes, the plan of a call, the launches
bool decode_supported(const KP& p);
// fills tiles / k-blocks / scratch need of a call; `sms` and `smem_per_sm` describe the device.  Returns the bytes of split-K scratch.
struct DecodeLaunch { int grid; size_t smem; uint32_t fin_blocks; };
uint64_t plan_decode(DecodeP& d, DecodeLaunch& L, int sms, size_t smem_per_sm);
// both kernels of a planned call on `st` (d.scratch and d.status set by the caller); device = the current device's ordinal
cudaError_t launch_decode_pair(const DecodeP& d, const DecodeLaunch& L, int device, cudaStream_t st);
int launch_decode(p0p_ctx* c, const KP& p);

}  // namespace p0p
