// p0p_gemm: argument validation (the reference's thrown errors plus the range checks WebGPU's bounded
// bindings gave it for free), kernel choice, launch.  Replaces gemm(gpu, a) of src/ops/gemm.js:268-327.
// There is no dispatch splitting: the reference cuts work into <= 0.2 s dispatches for the browser GPU
// watchdog (src/ops/gemm.js:286-292), which a CUDA stream does not need.
#include <cstring>
#include <cstddef>
#include "ctx.h"
#include "k_generic.cuh"
#include "k_aux.cuh"
#include "k_decode.cuh"
#include "umma_launch.cuh"

using namespace p0p;

namespace {

struct Need { const char* name; const p0p_buf* buf; uint64_t off_bytes; uint64_t bytes; };

inline bool live(const p0p_ctx* c, const p0p_buf* b) { return b && c->bufs.count(const_cast<p0p_buf*>(b)); }

}  // namespace

extern "C" int p0p_last_kernel(const p0p_ctx* c) { return c ? c->last_kernel : 0; }
extern "C" uint64_t p0p_launch_count(const p0p_ctx* c) { return c ? c->launches : 0; }
extern "C" int p0p_last_plan(const p0p_ctx* c, uint32_t* out8) {
  if (!c || !out8) return -1;
  for (int i = 0; i < 8; i++) out8[i] = c->last_plan[i];
  return 0;
}

extern "C" int p0p_gemm(p0p_ctx* c, const p0p_gemm_args* a_in, double* flops) {
  P0P_ALIVE(c);
  // callers built against the argument block without the peer fields pass a shorter struct_size: the rest reads as zero
  if (!a_in || a_in->struct_size < offsetof(p0p_gemm_args, n_ypeers)) return fail(c, -1, "gemm: bad argument block");
  p0p_gemm_args a_full;
  memset(&a_full, 0, sizeof a_full);
  memcpy(&a_full, a_in, std::min<size_t>(a_in->struct_size, sizeof a_full));
  const p0p_gemm_args* a = &a_full;
  if (a->n_ypeers > 7u) return fail(c, -1, "gemm: at most 7 peer copies of y");
  if (a->enc > P0P_ENC_F16) return fail(c, -2, "gemm: unsupported weight encoding %u", a->enc);          // src/ops/gemm.js:271
  if (a->xmode > P0P_X_CONV3 || a->epi > P0P_EPI_ONORMGATE) return fail(c, -2, "gemm: unknown prologue or epilogue");
  const uint32_t M = a->M, N = a->N, K = a->K;
  if (K % 32u) return fail(c, -3, "gemm: K must be a multiple of 32");                                    // :283
  if (flops) *flops = 2.0 * M * N * K;                                                                    // :326
  if (!M || !N || !K) return 0;
  if (!live(c, a->x) || !live(c, a->w) || !live(c, a->y)) return fail(c, -4, "gemm: missing binding X, W or Y");   // :313
  const bool conv = a->xmode == P0P_X_CONV || a->xmode == P0P_X_CONV3, xf32 = a->xmode == P0P_X_LNMOD || a->xmode == P0P_X_RMS;
  const bool red128 = a->epi == P0P_EPI_HEADS || a->epi == P0P_EPI_ONORMGATE;
  const uint32_t fl = a->flags;
  if (a->enc == P0P_ENC_Q4 && (a->w_rows % 64u || a->w_cols % 32u)) return fail(c, -5, "q4g32a.t64 needs rows %% 64 == 0 and K %% 32 == 0");
  if (a->enc == P0P_ENC_Q8 && (a->w_rows % 64u || a->w_cols % 64u)) return fail(c, -5, "q8g64s.t64 needs rows %% 64 == 0 and K %% 64 == 0");
  if ((a->x_off | a->w_off | a->y_off) & 15u) return fail(c, -5, "gemm: x.off, w.off and y.off must be multiples of 16 bytes");
  if ((uint64_t)a->wk0 + K > a->w_cols) return fail(c, -5, "gemm: wk0 + K exceeds the weight's %u columns", a->w_cols);
  if (a->enc != P0P_ENC_F16 && (a->wk0 % 32u)) return fail(c, -5, "gemm: wk0 must be a multiple of 32 for quantised weights");
  if (!a->w_rows) return fail(c, -5, "gemm: the weight has no rows");
  if (a->wr0 >= a->w_rows) return fail(c, -5, "gemm: wr0 %u is past the weight's %u rows", a->wr0, a->w_rows);

  KP p{};
  p.M = M; p.N = N; p.K = K; p.ldx = a->ldx ? a->ldx : K; p.kx0 = a->kx0; p.wR0 = a->wr0; p.wR1 = a->wr1;
  p.wG = a->enc == P0P_ENC_Q4 ? a->w_cols / 32u : a->enc == P0P_ENC_Q8 ? a->w_cols / 64u : (a->w_ld ? a->w_ld : a->w_cols);   // :284
  p.wk0 = a->wk0; p.ldy = a->ldy ? a->ldy : N; p.ny0 = a->ny0;
  p.rowOff = a->rowOff; p.Ltot = a->Ltot; p.Hq = a->Hq; p.Hkv = a->Hkv; p.eps = a->eps != 0.0f ? a->eps : 1e-6f;
  p.pvOff = a->pv ? a->pv_off : 0; p.pvStride = a->pv ? a->pv_stride : 0; p.evOff = a->ev ? a->ev_off : 0; p.statOff = a->st ? a->st_off : 0;
  p.Hi = a->Hi; p.Wi = a->Wi; p.Ci = a->Ci; p.Ho = a->Ho; p.Wo = a->Wo; p.stride = a->stride ? a->stride : 1; p.padT = a->padT; p.padL = a->padL; p.ks = a->ks ? a->ks : 1;
  p.Nw = a->w_rows; p.bvOff = a->bv ? a->bv_off : 0; p.bvUp = a->bv ? a->bv_up : 0;
  p.enc = a->enc; p.xmode = a->xmode; p.epi = a->epi; p.flags = fl;

  // ---- extents every binding must cover (bytes from the binding's offset)
  const uint32_t tileN = red128 ? (N + 127u) / 128u * 128u : (N + 3u) / 4u * 4u;   // columns that are computed and may be stored
  if (red128 && (a->wr0 + tileN > a->w_rows + 127u)) { /* clamped rows: fine */ }
  std::vector<Need> need;
  uint64_t xbytes = 0;
  if (conv) {
    if (!a->Ci || a->Ci % 32u) return fail(c, -6, "gemm: conv needs Ci %% 32 == 0");
    if (!a->Hi || !a->Wi || !a->Ho || !a->Wo) return fail(c, -6, "gemm: conv needs Hi, Wi, Ho, Wo");
    if (a->xmode == P0P_X_CONV3) {
      if (K != 27u * a->Ci) return fail(c, -6, "gemm: conv3 needs K == 27 * Ci");
      const uint32_t T = p.stride, HW = a->Ho * a->Wo, otmax = (M - 1u) / HW;
      const int gmin = std::max((int)a->padT - 1, 0) < (int)T - 1 ? std::max((int)a->padT - 1, 0) : (int)T - 1;
      const int gmax = std::min((int)(otmax + a->padT + 1u), (int)T - 1);
      uint64_t itmax;
      if (p.ks > 1u) itmax = p.ks - 1u;
      else { if ((int)a->padL > gmin) return fail(c, -6, "gemm: conv3 padL %u is past the first input frame %d this call reads", a->padL, gmin); itmax = (uint64_t)(gmax - (int)a->padL); }
      xbytes = (itmax + 1u) * a->Hi * a->Wi * (uint64_t)a->Ci * 2u;
      if (fl & P0P_F_PN) need.push_back({"ST", a->st, 0, (itmax + 1u) * a->Hi * a->Wi * 4ull});
    } else {
      if (K != p.ks * p.ks * a->Ci) return fail(c, -6, "gemm: conv needs K == ks * ks * Ci");
      xbytes = (uint64_t)a->Hi * a->Wi * a->Ci * 2u;
      if ((uint64_t)M > (uint64_t)a->Ho * a->Wo) return fail(c, -6, "gemm: conv M exceeds Ho * Wo");
      if (fl & P0P_F_GN) need.push_back({"PV", a->pv, 0, ((uint64_t)p.pvOff + p.pvStride + a->Ci) * 4ull});
    }
  } else {
    xbytes = ((uint64_t)(M - 1u) * p.ldx + p.kx0 + K) * (xf32 ? 4u : 2u);
    if (xf32) {
      need.push_back({"ST", a->st, 0, ((uint64_t)p.statOff + M) * 8ull});
      need.push_back({"PV", a->pv, 0, ((uint64_t)p.pvOff + (a->xmode == P0P_X_LNMOD ? p.pvStride : 0u) + p.kx0 + K) * 4ull});
    }
  }
  need.push_back({"X", a->x, a->x_off, xbytes});
  // weights
  uint64_t rmax;
  if (a->epi == P0P_EPI_SWIGLU) {
    if (N % 2u) return fail(c, -5, "gemm: swiglu needs an even N (gate/up column pairs)");
    rmax = (uint64_t)std::max(a->wr0, a->wr1) + N / 2u - 1u;
    if (rmax >= a->w_rows) return fail(c, -5, "gemm: swiglu rows [%u|%u, +%u) exceed the weight's %u rows", a->wr0, a->wr1, N / 2u, a->w_rows);
  } else rmax = std::min<uint64_t>((uint64_t)a->wr0 + tileN - 1u, a->w_rows - 1u);
  uint64_t wbytes;
  if (a->enc == P0P_ENC_Q4) wbytes = ((rmax >> 6) * p.wG + (a->wk0 + K - 1u) / 32u + 1u) * 1280ull;
  else if (a->enc == P0P_ENC_Q8) wbytes = ((rmax >> 6) * p.wG + (a->wk0 + K - 1u) / 64u + 1u) * 4224ull;
  else wbytes = (rmax * p.wG + a->wk0 + K) * 2ull;
  if (a->w_bytes && wbytes > a->w_bytes) return fail(c, -7, "gemm: the call reads %llu bytes of a weight of %llu bytes", (unsigned long long)wbytes, (unsigned long long)a->w_bytes);
  need.push_back({"W", a->w, a->w_off, wbytes});
  // outputs and epilogue vectors
  uint64_t ybytes;
  if (a->epi == P0P_EPI_HEADS) {
    if (!a->Ltot || (uint64_t)a->rowOff + M > a->Ltot) return fail(c, -8, "gemm: heads needs rowOff + M <= Ltot");
    if (N % 128u) return fail(c, -8, "gemm: heads needs N %% 128 == 0 (one head per 128 columns)");
    ybytes = ((uint64_t)(N / 128u) * a->Ltot) * 256ull;
    need.push_back({"EV", a->ev, 0, ((uint64_t)p.evOff + 256u) * 4ull});
    need.push_back({"RP", a->rp, 0, ((uint64_t)a->rowOff + M) * 512ull});
  } else if (a->epi == P0P_EPI_SWIGLU) {
    ybytes = ((uint64_t)(M - 1u) * p.ldy + p.ny0 + N / 2u) * 2ull;
    if (fl & P0P_F_BIAS) need.push_back({"BV", a->bv, 0, ((uint64_t)p.bvOff + p.bvUp + N / 2u) * 4ull});
  } else {
    const bool yf32 = a->epi == P0P_EPI_F32 || a->epi == P0P_EPI_RESADD;
    ybytes = ((uint64_t)(M - 1u) * p.ldy + p.ny0 + tileN) * (yf32 ? 4ull : 2ull);
    if (a->epi == P0P_EPI_RESADD && (fl & P0P_F_GATE)) need.push_back({"EV", a->ev, 0, ((uint64_t)p.evOff + tileN) * 4ull});
    if (a->epi == P0P_EPI_RESADD && (fl & P0P_F_BIAS)) need.push_back({"BV", a->bv, 0, ((uint64_t)p.bvOff + tileN) * 4ull});
    if (a->epi == P0P_EPI_BIAS) need.push_back({"EV", a->ev, 0, ((uint64_t)p.evOff + tileN) * 4ull});
    if (a->epi == P0P_EPI_ONORMGATE) {
      if (N % 128u) return fail(c, -8, "gemm: onormgate needs N %% 128 == 0");
      need.push_back({"EV", a->ev, 0, ((uint64_t)p.evOff + 128u) * 4ull});
      need.push_back({"GT", a->gt, 0, ((uint64_t)(M - 1u) * a->Ltot + p.ny0 + N) * 2ull});
    }
  }
  need.push_back({"Y", a->y, a->y_off, ybytes});
  for (const Need& n : need) {
    if (!live(c, n.buf)) return fail(c, -4, "gemm: missing binding %s", n.name);                           // :313
    uint64_t avail = n.buf->size > n.off_bytes ? n.buf->size - n.off_bytes : 0;
    if (n.buf == a->x && a->x_size) avail = std::min(avail, a->x_size);
    if (n.buf == a->y && n.name[0] == 'Y' && a->y_size) avail = std::min(avail, a->y_size);
    if (n.bytes > avail) return fail(c, -7, "gemm: binding %s needs %llu bytes, %llu are bound", n.name, (unsigned long long)n.bytes, (unsigned long long)avail);
  }

  p.X = (const char*)a->x->ptr + a->x_off; p.W = (const uint8_t*)a->w->ptr + a->w_off; p.Y = (char*)a->y->ptr + a->y_off;
  p.ST = a->st ? (const float*)a->st->ptr : nullptr; p.PV = a->pv ? (const float*)a->pv->ptr : nullptr;
  p.EV = a->ev ? (const float*)a->ev->ptr : nullptr; p.BV = a->bv ? (const float*)a->bv->ptr : nullptr;
  p.RP = a->rp ? (const float*)a->rp->ptr : nullptr; p.GT = a->gt ? (const __half*)a->gt->ptr : nullptr;
  p.nyp = a->n_ypeers;
  for (uint32_t q = 0; q < a->n_ypeers; q++) {
    const p0p_buf* yb = a->y_peers[q];
    if (!live(c, yb)) return fail(c, -4, "gemm: missing binding y_peers[%u]", q);
    if (yb->size < a->y->size) return fail(c, -7, "gemm: y_peers[%u] is smaller than y", q);
    p.YP[q] = (char*)yb->ptr + a->y_off;
  }
  p.vecx = (a->xmode == P0P_X_F16 && p.ldx % 8u == 0 && p.kx0 % 8u == 0 && ((uintptr_t)p.X & 15u) == 0) ? 1u : 0u;
  p.vecw = (a->enc == P0P_ENC_F16 && p.wG % 8u == 0 && a->wk0 % 8u == 0 && ((uintptr_t)p.W & 15u) == 0) ? 1u : 0u;
  if (a->epi == P0P_EPI_HEADS && ((uintptr_t)p.Y & 15u)) return fail(c, -5, "gemm: heads output must be 16-byte aligned");

  DeviceGuard g(c->device);
  // ---- kernel choice.  conv3 always takes the same kernel and tile whatever M is: a clip run in chunks or
  // from a ring must give the bits of the whole-clip call (test/kernels.test.js:123-145).
  int want = (int)a->force_kernel, used = 0;
  int rc = 0;
  // The streaming kernel wins up to 8 tokens (it never dequantises); from 9 on its second token group doubles its work and
  // the tensor-core kernel (narrow tiles, K-split accumulators, split-K) is faster on every shape measured.
  // (5 to 8 tokens over a small weight, under 16 MB: the stream is too short to pay for the two launches and the split-K
  // reduction; measured 14.7 against 19.3 us at 4096 x 4096.)
  const bool dec_ok = decode_supported(p), um_ok = umma_supported(c, p);
  const uint64_t stream_bytes = (uint64_t)N * K * (a->enc == P0P_ENC_Q4 ? 5u : 8u) / 8u;
  const bool small_weight = p.M >= 5u && stream_bytes <= (16ull << 20);
  if (want == P0P_K_DECODE || (want == P0P_K_AUTO && dec_ok && ((p.M <= 8u && !small_weight) || !um_ok))) {
    if (!dec_ok) return fail(c, -9, "gemm: the decode kernel does not take this configuration");
    rc = launch_decode(c, p); used = P0P_K_DECODE;
  } else if (want == P0P_K_UMMA || (want == P0P_K_AUTO && um_ok)) {
    if (!um_ok) return fail(c, -9, "gemm: the tensor-core kernel does not take this configuration");
    rc = launch_umma(c, p); used = P0P_K_UMMA;
  } else {
    if (p.nyp) return fail(c, -9, "gemm: peer copies of y need the decode or the tensor-core kernel, which do not take this configuration");
    cudaError_t e = launch_generic(p, c->stream);
    if (e != cudaSuccess) return cuda_fail(c, e, "gemm launch");
    c->launches += 1; used = P0P_K_GENERIC;
  }
  if (rc) return rc;
  c->last_kernel = used;
  return 0;
}

extern "C" int p0p_dequant(p0p_ctx* c, uint32_t enc, const p0p_buf* w, uint64_t w_off, uint32_t w_cols, uint32_t w_ld,
                           uint32_t r0, uint32_t nr, uint32_t path, p0p_buf* out, uint64_t out_off) {
  P0P_ALIVE(c);
  if (enc > P0P_ENC_F16) return fail(c, -2, "dequant: unsupported weight encoding %u", enc);
  if (!live(c, w) || !live(c, out)) return fail(c, -4, "dequant: missing binding");
  if (!nr || !w_cols) return 0;
  if ((enc == P0P_ENC_Q4 && w_cols % 32u) || (enc == P0P_ENC_Q8 && w_cols % 64u)) return fail(c, -5, "dequant: column count does not fit the encoding");
  if ((w_off & 15u) || (out_off & 15u)) return fail(c, -5, "dequant: offsets must be multiples of 16 bytes");
  const uint32_t wG = enc == P0P_ENC_Q4 ? w_cols / 32u : enc == P0P_ENC_Q8 ? w_cols / 64u : (w_ld ? w_ld : w_cols);
  const uint64_t rmax = (uint64_t)r0 + nr - 1u;
  const uint64_t wbytes = enc == P0P_ENC_Q4 ? ((rmax >> 6) + 1u) * wG * 1280ull : enc == P0P_ENC_Q8 ? ((rmax >> 6) + 1u) * wG * 4224ull : (rmax * wG + w_cols) * 2ull;
  if (w_off > w->size || wbytes > w->size - w_off) return fail(c, -7, "dequant: the weight range is outside its buffer");
  const uint64_t obytes = (uint64_t)nr * w_cols * 2ull;
  if (out_off > out->size || obytes > out->size - out_off) return fail(c, -7, "dequant: the output range is outside its buffer");
  DeviceGuard g(c->device);
  cudaError_t e = launch_dequant(enc, (const uint8_t*)w->ptr + w_off, wG, w_cols, r0, nr, path, (__half*)((char*)out->ptr + out_off), c->stream);
  if (e != cudaSuccess) return cuda_fail(c, e, "dequant launch");
  c->launches += 1;
  return 0;
}

extern "C" int p0p_rowstats(p0p_ctx* c, const p0p_buf* x, uint64_t x_off, uint32_t ld, uint32_t c0, uint32_t rows, uint32_t cols,
                            uint32_t mode, float eps, p0p_buf* st, uint32_t st_off) {
  P0P_ALIVE(c);
  if (!live(c, x) || !live(c, st)) return fail(c, -4, "rowstats: missing binding");
  if (!rows || !cols) return 0;
  if (!ld) ld = cols;
  if (x_off & 3u) return fail(c, -5, "rowstats: x.off must be a multiple of 4 bytes");
  const uint64_t xb = ((uint64_t)(rows - 1u) * ld + c0 + cols) * 4ull, sb = ((uint64_t)st_off + rows) * 8ull;
  if (x_off > x->size || xb > x->size - x_off || sb > st->size) return fail(c, -7, "rowstats: a range is outside its buffer");
  DeviceGuard g(c->device);
  cudaError_t e = launch_rowstats((const float*)((const char*)x->ptr + x_off), ld, c0, rows, cols, mode, eps, (float*)st->ptr + (size_t)st_off * 2u, c->stream);
  if (e != cudaSuccess) return cuda_fail(c, e, "rowstats launch");
  c->launches += 1;
  return 0;
}
