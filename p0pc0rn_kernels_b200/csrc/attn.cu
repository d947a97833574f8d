// p0p_attention: host entry of the head-128 flash attention (src/ops/attention.js:168-193) — validation, launch.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdlib>

#include "ctx.h"
#include "device_once.h"
#include "k_attn.cuh"
#include "k_attn_tc.cuh"
#include "tmap.h"

using namespace p0p;

extern "C" int p0p_attention(p0p_ctx* c, const p0p_attn_args* a, double* flops) {
  P0P_ALIVE(c);
  if (!a || a->struct_size < offsetof(p0p_attn_args, kernel)) return fail(c, -1, "attention: bad argument block");
  const uint32_t Hq = a->Hq, Hkv = a->Hkv ? a->Hkv : a->Hq, Lq = a->Lq, Lk = a->Lk ? a->Lk : a->Lq;
  const uint32_t ldo = a->ldo ? a->ldo : Hq * 128u;                                            // attention.js:176
  if (flops) *flops = 4.0 * Lq * Lk * 128.0 * Hq;                                             // :192
  if (!Hq || !Lq || !Lk) return 0;
  if (Hq % Hkv) return fail(c, -3, "attention: Hq must be a multiple of Hkv");
  if (a->mode > 2u) return fail(c, -2, "attention: unknown mask mode %u", a->mode);
  const uint32_t nvalid = a->nvalid ? a->nvalid : Lk;                                          // :188
  auto live = [&](const p0p_buf* b) { return b && c->bufs.count(const_cast<p0p_buf*>(b)); };
  if (!live(a->q) || !live(a->k) || !live(a->v) || !live(a->o)) return fail(c, -4, "attention: missing binding");
  const uint64_t qs = (uint64_t)Hq * Lq * 256u, ks = (uint64_t)Hkv * Lk * 256u, os = ((uint64_t)(Lq - 1u) * ldo + (uint64_t)Hq * 128u) * 2u;
  if (a->q_off > a->q->size || qs > a->q->size - a->q_off) return fail(c, -7, "attention: q needs %llu bytes", (unsigned long long)qs);
  if (a->k_off > a->k->size || ks > a->k->size - a->k_off) return fail(c, -7, "attention: k needs %llu bytes", (unsigned long long)ks);
  if (a->v_off > a->v->size || ks > a->v->size - a->v_off) return fail(c, -7, "attention: v needs %llu bytes", (unsigned long long)ks);
  if (a->o_off > a->o->size || os > a->o->size - a->o_off) return fail(c, -7, "attention: o needs %llu bytes", (unsigned long long)os);
  if ((a->q_off | a->k_off | a->v_off) & 15u) return fail(c, -5, "attention: q / k / v offsets must be multiples of 16 bytes");
  if ((a->o_off & 3u) || (ldo & 1u) || ldo < Hq * 128u) return fail(c, -5, "attention: o.off must be a multiple of 4 bytes and o.ld even and at least Hq * 128");
  AttnP p{};
  p.Q = reinterpret_cast<const __half*>((const char*)a->q->ptr + a->q_off); p.K = reinterpret_cast<const __half*>((const char*)a->k->ptr + a->k_off);
  p.V = reinterpret_cast<const __half*>((const char*)a->v->ptr + a->v_off); p.O = reinterpret_cast<__half*>((char*)a->o->ptr + a->o_off);
  p.Lq = Lq; p.Lk = Lk; p.ldo = ldo; p.Hq = Hq; p.Hkv = Hkv; p.mode = a->mode; p.nvalid = nvalid;
  p.scale_log2 = (a->scale > 0.0f ? a->scale : 1.0f / std::sqrt(128.0f)) * 1.4426950408889634f;    // :181
  DeviceGuard g(c->device);
  const uint32_t which = a->struct_size >= offsetof(p0p_attn_args, kernel) + sizeof(uint32_t) ? a->kernel : 0u;
  if (which != 0u && which != P0P_K_ATTN_WARP && which != P0P_K_ATTN_TMEM) return fail(c, -2, "attention: unknown kernel selector %u", which);
  static DeviceOnce once[2];
  // ---- tensor-memory kernel: two tiles of 128 queries per block.  Fewer than 128 queries per head leave most of a tile
  // empty: those calls (decode steps) stay on the warp-level kernel, whose tile is 64 queries.
  if (which == P0P_K_ATTN_TMEM || (which == 0u && Lq >= 128u)) {
    if (!tmap_encoder()) return fail(c, -12, "attention: the driver offers no tensor-map encoder");
    const uint32_t ldv = (Lk + 7u) & ~7u;
    const uint64_t vt_bytes = (uint64_t)Hkv * 128u * ldv * 2u;
    if (int rc = ensure_scratch(c, vt_bytes)) return rc;
    int rc = once[1].run(c->device, [&] { return (int)cudaFuncSetAttribute(k_attn_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATC_SMEM); });
    if (rc) return cuda_fail(c, (cudaError_t)rc, "attention kernel attribute");
    CUtensorMap mq, mk, mv;
    if (!make_map_3d(&mq, p.Q, 128u, Lq, Hq, 128u, (uint64_t)Lq * 128u, 128u) || !make_map_3d(&mk, p.K, 128u, Lk, Hkv, 128u, (uint64_t)Lk * 128u, 128u) ||
        !make_map_3d(&mv, c->scratch, Lk, 128u, Hkv, ldv, (uint64_t)ldv * 128u, 128u))
      return fail(c, -12, "attention: a tensor map could not be encoded");
    k_attn_vt<<<dim3((Lk + 63u) / 64u, Hkv), 256, 0, c->stream>>>(p.V, reinterpret_cast<__half*>(c->scratch), Lk, ldv);
    AttnTcP t{};
    t.O = p.O; t.Lq = Lq; t.Lk = Lk; t.ldo = ldo; t.Hq = Hq; t.Hkv = Hkv; t.mode = a->mode; t.nvalid = nvalid; t.scale_log2 = p.scale_log2; t.status = c->dev_status;
    attn_plan(Lq, Lk, Hq, a->mode, nvalid, (uint32_t)c->prop.multiProcessorCount, t.np, t.ns);
#ifdef P0P_KNOBS
    if (const char* e = getenv("P0P_ATTN_NS")) { const uint32_t T = (Lq + 127u) / 128u; uint32_t s = (uint32_t)atoi(e); if (s <= T && ((T - s) & 1u) == 0u) { t.ns = s; t.np = (T - s) / 2u; } }
#endif
    k_attn_tc<<<Hq * (t.np + t.ns), ATC_THREADS, ATC_SMEM, c->stream>>>(t, mq, mk, mv);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(c, e, "attention launch");
    c->launches += 2;
    c->last_kernel = P0P_K_ATTN_TMEM;
    return 0;
  }
  int rc = once[0].run(c->device, [&] { return (int)cudaFuncSetAttribute(k_attn128, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM); });
  if (rc) return cuda_fail(c, (cudaError_t)rc, "attention kernel attribute");
  k_attn128<<<dim3((Lq + AT_BQ - 1) / AT_BQ, Hq), 128, AT_SMEM, c->stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "attention launch");
  c->launches += 1;
  c->last_kernel = P0P_K_ATTN_WARP;
  return 0;
}
