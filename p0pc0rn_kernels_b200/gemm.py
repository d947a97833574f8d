"""gemm(gpu, a): the host-side mirror of the reference op (src/ops/gemm.js:268-327).  The argument object is the
reference's, as a dict:

  w: {buf, off, enc: 'q4g32a.t64' | 'q8g64s.t64' | 'f16', bytes, rows, cols, ld?}
  x: {buf, off, ld, k0, mode: 'f16' | 'lnmod' | 'rms', size?};  y: {buf, off, ld, n0, size?};  M, N, K
  wr0, wr1, wk0;  epi: 'f16' | 'f32' | 'resadd' | 'swiglu' | 'heads' | 'bias' | 'onormgate'
  ev {buf, off (floats)}, stats {buf, off (rows)}, pv {buf, off, stride (floats)}, bv {buf, off, up (floats)}, gt {buf}
  res, store, act: 'silu' | 'gelu';  heads {Ltot, Hq, Hkv, rowOff, eps, ropeMode, rope {buf}}
  conv {kind: 'conv' | 'conv3', Hi, Wi, Ci, Ho, Wo, stride, padT, padL, ks, up2, gn, pn};  tile {BM, BN};  acc

Returns 2*M*N*K.  Bad arguments raise ValueError with the reference's message where it has one.
"""
from __future__ import annotations

import ctypes as C

from ._lib import (ENC, EPI, F_BIAS, F_GATE, F_GELU, F_GN, F_PN, F_RES, F_ROPE_HALF, F_STORE, F_UP2, K_AUTO, K_DECODE, K_GENERIC, K_UMMA, XMODE,
                   GemmArgs, lib)

DEFAULT_TILE = {"BM": 64, "BN": 128}   # src/ops/gemm.js:22 (kept for callers; the CUDA kernels pick their own tiles)
_KERNELS = {None: K_AUTO, "auto": K_AUTO, "generic": K_GENERIC, "decode": K_DECODE, "umma": K_UMMA}


def _h(t):
    return t["buf"].handle if t and t.get("buf") is not None else None


def gemm(gpu, a: dict) -> float:
    enc = a["w"].get("enc")
    if enc not in ENC:
        raise ValueError("gemm: unsupported weight encoding " + str(enc))             # src/ops/gemm.js:271
    cv = a.get("conv") or None
    x, y, w = a["x"], a["y"], a["w"]
    h = a.get("heads") or {}
    g = GemmArgs()
    g.struct_size = C.sizeof(GemmArgs)
    g.enc = ENC[enc]
    g.xmode = XMODE["conv3" if cv.get("kind") == "conv3" else "conv"] if cv else XMODE[x.get("mode") or "f16"]
    epi = a.get("epi") or "f16"
    if epi not in EPI:
        raise ValueError("gemm: unknown epilogue " + str(epi))
    g.epi = EPI[epi]
    fl = 0
    if a.get("ev") and epi == "resadd": fl |= F_GATE                                   # :277
    if a.get("res"): fl |= F_RES
    if a.get("store"): fl |= F_STORE
    if cv and cv.get("gn"): fl |= F_GN
    if cv and cv.get("up2"): fl |= F_UP2
    if cv and cv.get("pn"): fl |= F_PN
    if a.get("bv"): fl |= F_BIAS
    if (a.get("act") or "silu") == "gelu": fl |= F_GELU
    if h.get("ropeMode") == "half": fl |= F_ROPE_HALF
    g.flags = fl
    g.M, g.N, g.K = int(a["M"]), int(a["N"]), int(a["K"])
    g.ldx = int(x.get("ld") or a["K"]); g.kx0 = int(x.get("k0") or 0)                  # :317
    g.wr0 = int(a.get("wr0") or 0); g.wr1 = int(a.get("wr1") or 0); g.wk0 = int(a.get("wk0") or 0)
    g.w_rows = int(w["rows"]); g.w_cols = int(w["cols"]); g.w_ld = int(w.get("ld") or 0)
    g.ldy = int(y.get("ld") or a["N"]); g.ny0 = int(y.get("n0") or 0)                  # :318
    g.rowOff = int(h.get("rowOff") or 0); g.Ltot = int(h.get("Ltot") or 0); g.Hq = int(h.get("Hq") or 0); g.Hkv = int(h.get("Hkv") or 0)
    g.eps = float(h.get("eps") or 1e-6)                                                # :319
    pv, ev, st, bv = a.get("pv"), a.get("ev"), a.get("stats"), a.get("bv")
    g.pv_off = int(pv.get("off") or 0) if pv else 0; g.pv_stride = int(pv.get("stride") or 0) if pv else 0   # :320
    g.ev_off = int(ev.get("off") or 0) if ev else 0; g.st_off = int(st.get("off") or 0) if st else 0
    g.bv_off = int(bv.get("off") or 0) if bv else 0; g.bv_up = int(bv.get("up") or 0) if bv else 0           # :322
    c = cv or {}
    g.Hi = int(c.get("Hi") or 0); g.Wi = int(c.get("Wi") or 0); g.Ci = int(c.get("Ci") or 0); g.Ho = int(c.get("Ho") or 0); g.Wo = int(c.get("Wo") or 0)
    g.stride = int(c.get("stride") or 1); g.padT = int(c.get("padT") or 0); g.padL = int(c.get("padL") or 0); g.ks = int(c.get("ks") or 1)   # :321
    t = a.get("tile") or {}
    g.tile_bm = int(t.get("BM") or 0); g.tile_bn = int(t.get("BN") or 0)
    if t and (g.tile_bm % 32 or g.tile_bn % 64 or (g.tile_bm // 8) * (g.tile_bn // 8) > 256):
        raise ValueError(f"bad tile {g.tile_bm}x{g.tile_bn}")                           # src/ops/gemm.js:31
    g.acc_f16 = 1 if (a.get("acc") or (gpu.tune or {}).get("acc")) == "f16" else 0
    g.force_kernel = _KERNELS[a.get("kernel")]
    g.x, g.w, g.y = _h(x), _h(w), _h(y)
    g.st, g.pv, g.ev, g.bv = _h(st), _h(pv), _h(ev), _h(bv)
    g.rp = _h(h.get("rope")); g.gt = _h(a.get("gt"))
    g.x_off = int(x.get("off") or 0); g.w_off = int(w.get("off") or 0); g.y_off = int(y.get("off") or 0)
    g.w_bytes = int(w.get("bytes") or 0)
    g.x_size = int(x["size"]) if x.get("size") is not None else 0
    g.y_size = int(y["size"]) if y.get("size") is not None else 0
    peers = y.get("peers") or []          # not in the reference: the other ranks' copies of y (Gpu.ipcOpen), stored to as well
    if len(peers) > 7: raise ValueError("gemm: at most 7 peer copies of y")
    g.n_ypeers = len(peers)
    for i, pb in enumerate(peers): g.y_peers[i] = pb.handle.value if hasattr(pb.handle, "value") else pb.handle
    fl_out = C.c_double()
    gpu._check(lib.p0p_gemm(gpu._h, C.byref(g), C.byref(fl_out)))
    return fl_out.value
