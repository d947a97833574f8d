// p0p_attention: host entry of the head-128 flash attention (src/ops/attention.js:168-193) — validation, launch.
#include <algorithm>
#include <cmath>

#include "ctx.h"
#include "k_attn.cuh"

using namespace p0p;

extern "C" int p0p_attention(p0p_ctx* c, const p0p_attn_args* a, double* flops) {
  P0P_ALIVE(c);
  if (!a || a->struct_size < sizeof(p0p_attn_args)) return fail(c, -1, "attention: bad argument block");
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
  static bool ready = false;
  if (!ready) {
    cudaError_t e = cudaFuncSetAttribute(k_attn128, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (e != cudaSuccess) return cuda_fail(c, e, "attention kernel attribute");
    ready = true;
  }
  k_attn128<<<dim3((Lq + AT_BQ - 1) / AT_BQ, Hq), 128, AT_SMEM, c->stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "attention launch");
  c->launches += 1;
  return 0;
}
