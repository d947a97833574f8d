// Node.js N-API addon over the C ABI of include/p0p.h.  It is the binding the reference's JavaScript
// (`op(gpu, args)`, src/index.js) attaches to when the WebGPU runtime (src/core/gpu.js) is replaced by libp0p.so.
// Thin by design: every export forwards to one p0p_* call; handles travel as BigInt pointers wrapped in externals.
//
// NOT BUILT OR RUN where this project is developed: the build image has no Node.js and no node_api.h.  Build with
//   node-gyp rebuild   (binding.gyp beside this file; needs libp0p.so on the library path)
#include <node_api.h>

#include <cstring>
#include <string>
#include <vector>

#include "../../include/p0p.h"

namespace {

#define NAPI_OK(call) do { if ((call) != napi_ok) { napi_throw_error(env, nullptr, "p0p addon: N-API call failed: " #call); return nullptr; } } while (0)

napi_value throw_ctx(napi_env env, p0p_ctx* c, int rc) {
  std::string msg = c ? p0p_last_error(c) : "p0p: no context";
  // negative = bad argument (the reference throws Error), positive = CUDA error (the reference throws GpuError)
  napi_throw_error(env, rc > 0 ? "GpuError" : "Error", msg.c_str());
  return nullptr;
}
template <class T> T* unwrap(napi_env env, napi_value v) { void* p = nullptr; napi_get_value_external(env, v, &p); return static_cast<T*>(p); }
napi_value wrap(napi_env env, void* p) { napi_value v; napi_create_external(env, p, nullptr, nullptr, &v); return v; }
uint32_t u32(napi_env env, napi_value o, const char* k, uint32_t dflt = 0) {
  bool has = false; napi_has_named_property(env, o, k, &has); if (!has) return dflt;
  napi_value v; napi_get_named_property(env, o, k, &v); napi_valuetype t; napi_typeof(env, v, &t);
  if (t != napi_number) return dflt; double d = 0; napi_get_value_double(env, v, &d); return (uint32_t)d;
}
double f64(napi_env env, napi_value o, const char* k, double dflt = 0) {
  bool has = false; napi_has_named_property(env, o, k, &has); if (!has) return dflt;
  napi_value v; napi_get_named_property(env, o, k, &v); napi_valuetype t; napi_typeof(env, v, &t);
  if (t != napi_number) return dflt; double d = 0; napi_get_value_double(env, v, &d); return d;
}
p0p_buf* bufp(napi_env env, napi_value o, const char* k) {
  bool has = false; napi_has_named_property(env, o, k, &has); if (!has) return nullptr;
  napi_value v; napi_get_named_property(env, o, k, &v); napi_valuetype t; napi_typeof(env, v, &t);
  return t == napi_external ? unwrap<p0p_buf>(env, v) : nullptr;
}

// open(device) -> external ctx
napi_value Open(napi_env env, napi_callback_info info) {
  size_t argc = 1; napi_value a[1]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  int32_t dev = 0; if (argc) napi_get_value_int32(env, a[0], &dev);
  p0p_ctx* c = nullptr; p0p_opts o{sizeof(p0p_opts), 0, nullptr};
  int rc = p0p_open(dev, &o, &c);
  if (rc) { napi_throw_error(env, "GpuError", "no CUDA device with sm_100 available"); return nullptr; }
  return wrap(env, c);
}
napi_value Close(napi_env env, napi_callback_info info) {
  size_t argc = 1; napi_value a[1]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_close(unwrap<p0p_ctx>(env, a[0])); return nullptr;
}
// alloc(ctx, bytes) -> {handle, size}
napi_value Alloc(napi_env env, napi_callback_info info) {
  size_t argc = 2; napi_value a[2]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_ctx* c = unwrap<p0p_ctx>(env, a[0]); double bytes = 0; napi_get_value_double(env, a[1], &bytes);
  p0p_buf* b = nullptr; int rc = p0p_alloc(c, (uint64_t)bytes, &b); if (rc) return throw_ctx(env, c, rc);
  napi_value o, sz; napi_create_object(env, &o); napi_create_double(env, (double)p0p_buf_size(b), &sz);
  napi_set_named_property(env, o, "handle", wrap(env, b)); napi_set_named_property(env, o, "size", sz); return o;
}
napi_value Free(napi_env env, napi_callback_info info) {
  size_t argc = 2; napi_value a[2]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_free(unwrap<p0p_ctx>(env, a[0]), unwrap<p0p_buf>(env, a[1])); return nullptr;
}
// write(ctx, buf, dstOff, arrayBufferOrView)
napi_value Write(napi_env env, napi_callback_info info) {
  size_t argc = 4; napi_value a[4]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_ctx* c = unwrap<p0p_ctx>(env, a[0]); double off = 0; napi_get_value_double(env, a[2], &off);
  void* data = nullptr; size_t len = 0; bool is_ab = false; napi_is_arraybuffer(env, a[3], &is_ab);
  if (is_ab) napi_get_arraybuffer_info(env, a[3], &data, &len);
  else { napi_typedarray_type t; napi_value ab; size_t boff; size_t n; NAPI_OK(napi_get_typedarray_info(env, a[3], &t, &n, &data, &ab, &boff));
         static const size_t esz[] = {1, 1, 1, 2, 2, 4, 4, 4, 8, 8, 8}; len = n * esz[t]; }
  int rc = p0p_write(c, unwrap<p0p_buf>(env, a[1]), (uint64_t)off, data, len); if (rc) return throw_ctx(env, c, rc);
  return nullptr;
}
// read(ctx, buf, off, size) -> ArrayBuffer
napi_value Read(napi_env env, napi_callback_info info) {
  size_t argc = 4; napi_value a[4]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_ctx* c = unwrap<p0p_ctx>(env, a[0]); double off = 0, size = 0; napi_get_value_double(env, a[2], &off); napi_get_value_double(env, a[3], &size);
  void* data = nullptr; napi_value ab; NAPI_OK(napi_create_arraybuffer(env, (size_t)size, &data, &ab));
  int rc = p0p_read(c, unwrap<p0p_buf>(env, a[1]), (uint64_t)off, data, (uint64_t)size); if (rc) return throw_ctx(env, c, rc);
  return ab;
}
napi_value Sync(napi_env env, napi_callback_info info) {
  size_t argc = 1; napi_value a[1]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_ctx* c = unwrap<p0p_ctx>(env, a[0]); int rc = p0p_sync(c); if (rc) return throw_ctx(env, c, rc); return nullptr;
}
// gemm(ctx, flat) -> flops; `flat` is the argument object flattened by gemm.js to the fields of p0p_gemm_args
napi_value Gemm(napi_env env, napi_callback_info info) {
  size_t argc = 2; napi_value a[2]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  p0p_ctx* c = unwrap<p0p_ctx>(env, a[0]); napi_value o = a[1];
  p0p_gemm_args g; std::memset(&g, 0, sizeof g); g.struct_size = sizeof g;
#define U(f) g.f = u32(env, o, #f)
  U(enc); U(xmode); U(epi); U(flags); U(M); U(N); U(K); U(ldx); U(kx0); U(wr0); U(wr1); U(wk0); U(w_rows); U(w_cols); U(w_ld); U(ldy); U(ny0);
  U(rowOff); U(Ltot); U(Hq); U(Hkv); U(pv_off); U(pv_stride); U(ev_off); U(st_off); U(bv_off); U(bv_up); U(Hi); U(Wi); U(Ci); U(Ho); U(Wo);
  U(stride); U(padT); U(padL); U(ks); U(tile_bm); U(tile_bn); U(acc_f16);
#undef U
  g.eps = (float)f64(env, o, "eps", 1e-6);
  g.x = bufp(env, o, "x"); g.w = bufp(env, o, "w"); g.y = bufp(env, o, "y"); g.st = bufp(env, o, "st"); g.pv = bufp(env, o, "pv");
  g.ev = bufp(env, o, "ev"); g.bv = bufp(env, o, "bv"); g.rp = bufp(env, o, "rp"); g.gt = bufp(env, o, "gt");
  g.x_off = (uint64_t)f64(env, o, "x_off"); g.w_off = (uint64_t)f64(env, o, "w_off"); g.y_off = (uint64_t)f64(env, o, "y_off");
  g.w_bytes = (uint64_t)f64(env, o, "w_bytes"); g.x_size = (uint64_t)f64(env, o, "x_size"); g.y_size = (uint64_t)f64(env, o, "y_size");
  {   // y.peers: externals of buffers opened with ipcOpen (multi-GPU extension; absent in the reference's argument object)
    bool has = false; napi_has_named_property(env, o, "y_peers", &has);
    if (has) {
      napi_value arr; napi_get_named_property(env, o, "y_peers", &arr); uint32_t n = 0; napi_get_array_length(env, arr, &n);
      for (uint32_t i = 0; i < n && i < 7u; i++) { napi_value e; napi_get_element(env, arr, i, &e); g.y_peers[i] = unwrap<p0p_buf>(env, e); g.n_ypeers = i + 1u; }
    }
  }
  double flops = 0; int rc = p0p_gemm(c, &g, &flops); if (rc) return throw_ctx(env, c, rc);
  napi_value r; napi_create_double(env, flops, &r); return r;
}
napi_value F2h(napi_env env, napi_callback_info info) {
  size_t argc = 1; napi_value a[1]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  double v = 0; napi_get_value_double(env, a[0], &v); napi_value r; napi_create_uint32(env, p0p_f2h((float)v), &r); return r;
}
napi_value H2f(napi_env env, napi_callback_info info) {
  size_t argc = 1; napi_value a[1]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  uint32_t h = 0; napi_get_value_uint32(env, a[0], &h); napi_value r; napi_create_double(env, p0p_h2f((uint16_t)h), &r); return r;
}
// packQ(bits, Float32Array W, rows, K, Float32Array deq | null) -> Uint8Array bytes (as ArrayBuffer)
napi_value PackQ(napi_env env, napi_callback_info info) {
  size_t argc = 5; napi_value a[5]; NAPI_OK(napi_get_cb_info(env, info, &argc, a, nullptr, nullptr));
  uint32_t bits = 4, rows = 0, K = 0; napi_get_value_uint32(env, a[0], &bits); napi_get_value_uint32(env, a[2], &rows); napi_get_value_uint32(env, a[3], &K);
  napi_typedarray_type t; size_t n; void* W; napi_value ab; size_t boff; NAPI_OK(napi_get_typedarray_info(env, a[1], &t, &n, &W, &ab, &boff));
  void* deq = nullptr; napi_valuetype dt; napi_typeof(env, a[4], &dt);
  if (dt == napi_object) NAPI_OK(napi_get_typedarray_info(env, a[4], &t, &n, &deq, &ab, &boff));
  const size_t bytes = (size_t)p0p_encoded_bytes(bits == 4 ? P0P_ENC_Q4 : P0P_ENC_Q8, rows, K);
  void* out = nullptr; napi_value oab; NAPI_OK(napi_create_arraybuffer(env, bytes, &out, &oab));
  int rc = bits == 4 ? p0p_pack_q4((const float*)W, rows, K, (uint8_t*)out, (float*)deq) : p0p_pack_q8((const float*)W, rows, K, (uint8_t*)out, (float*)deq);
  if (rc) { napi_throw_error(env, nullptr, bits == 4 ? "q4g32a.t64 needs rows % 64 == 0 and K % 32 == 0" : "q8g64s.t64 needs rows % 64 == 0 and K % 64 == 0"); return nullptr; }
  return oab;
}

napi_value Init(napi_env env, napi_value exports) {
  const napi_property_descriptor d[] = {
    {"open", nullptr, Open, nullptr, nullptr, nullptr, napi_default, nullptr}, {"close", nullptr, Close, nullptr, nullptr, nullptr, napi_default, nullptr},
    {"alloc", nullptr, Alloc, nullptr, nullptr, nullptr, napi_default, nullptr}, {"free", nullptr, Free, nullptr, nullptr, nullptr, napi_default, nullptr},
    {"write", nullptr, Write, nullptr, nullptr, nullptr, napi_default, nullptr}, {"read", nullptr, Read, nullptr, nullptr, nullptr, napi_default, nullptr},
    {"sync", nullptr, Sync, nullptr, nullptr, nullptr, napi_default, nullptr}, {"gemm", nullptr, Gemm, nullptr, nullptr, nullptr, napi_default, nullptr},
    {"f2h", nullptr, F2h, nullptr, nullptr, nullptr, napi_default, nullptr}, {"h2f", nullptr, H2f, nullptr, nullptr, nullptr, napi_default, nullptr},
    {"packQ", nullptr, PackQ, nullptr, nullptr, nullptr, napi_default, nullptr},
  };
  napi_define_properties(env, exports, sizeof d / sizeof d[0], d);
  return exports;
}

}  // namespace

NAPI_MODULE(p0p_addon, Init)
