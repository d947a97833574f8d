"""Shared builders for the parity tests: a case is a dict of op arguments; ``build`` makes its seeded host arrays,
``run_gpu`` runs it through the public API (C ABI underneath), ``run_oracle`` through the CPU oracle, ``check``
applies the gates.

Gates (vs the float64-accumulating oracle): cosine similarity > 0.9995 (the reference's own pass criterion,
test/kernels.test.js:228), relative L2 <= 4e-3 (its tuning sweep's bound, bench/sweep.js:33) and
max |err| <= 2e-2 * max |ref| (the fp16 tolerance the task states).  Output words the op must not touch are
poisoned with NaN bit patterns before the run and have to come back untouched.
"""
from __future__ import annotations

import numpy as np

import oracle as O

COS_MIN, REL_L2_MAX, MAX_ABS_REL = 0.9995, 4e-3, 2e-2
ENC_NAMES = {"q4": "q4g32a.t64", "q8": "q8g64s.t64", "f16": "f16"}


def encode(enc, W0, rows, cols):
    """-> (bytes uint8, values the reference's CPU check multiplies with)"""
    if enc == "q4g32a.t64":
        return O.pack_q4(W0, rows, cols)
    if enc == "q8g64s.t64":
        return O.pack_q8(W0, rows, cols)
    Wd = O.round_f16(W0)
    return O.to_f16(Wd).view(np.uint8), Wd


def rope_table(L, seed=5):
    """[L][64][cos, sin] f32, the layout of ropeWan / ropeGemma (src/ops/video2.js:154-172)"""
    ang = np.random.default_rng(seed).uniform(-np.pi, np.pi, (L, 64)).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32).reshape(-1)


def build(c: dict) -> dict:
    """Seeded host arrays of a case.  Keys of c: enc, M, N, K, xmode, epi and the optional fields of the op."""
    c = dict(c); c.pop("expect", None)
    enc = ENC_NAMES.get(c["enc"], c["enc"])
    M, N, K = c["M"], c["N"], c["K"]
    seed = c.get("seed", 7)
    epi = c.get("epi", "f16"); xmode = c.get("xmode", "f16")
    conv = c.get("conv")
    wk0 = c.get("wk0", 0); wr0 = c.get("wr0", 0)
    w_cols = c.get("w_cols", wk0 + K)
    if epi == "swiglu":
        half = N // 2; wr1 = c.get("wr1", wr0 + half); w_rows = c.get("w_rows", max(wr0, wr1) + half)
    else:
        wr1 = 0; w_rows = c.get("w_rows", wr0 + N)
    if enc != "f16": w_rows = -(-w_rows // 64) * 64
    w_ld = c.get("w_ld", 0)
    W0 = O.randn(w_rows * (w_ld or w_cols), seed + 4, c.get("w_scale", 0.05))
    if enc == "f16" and w_ld:
        Wd = O.round_f16(W0); Wb = O.to_f16(Wd).view(np.uint8)
    else:
        Wb, Wd = encode(enc, W0, w_rows, w_cols)
    h = {"enc": enc, "M": M, "N": N, "K": K, "epi": epi, "xmode": xmode, "conv": conv, "wk0": wk0, "wr0": wr0, "wr1": wr1, "w_rows": w_rows,
         "w_cols": w_cols, "w_ld": w_ld, "W": np.ascontiguousarray(Wb), "Wd": Wd, "kernel": c.get("kernel"), "name": c.get("name", ""),
         "res": c.get("res", False), "store": c.get("store", False), "act": c.get("act", "silu"), "tile": c.get("tile"), "acc": c.get("acc"),
         "w_off": c.get("w_off", 0), "x_off": c.get("x_off", 0), "y_off": c.get("y_off", 0), "peers": c.get("peers", 0)}
    # ---- X
    ldx = c.get("ldx", K); kx0 = c.get("kx0", 0)
    h["ldx"], h["kx0"] = ldx, kx0
    if conv:
        n_in = c["x_elems"]
        Xf = O.round_f16(O.randn(n_in, seed)); h["X"] = O.to_f16(Xf); h["Xf"] = Xf
        if conv.get("pn"):
            vox = n_in // conv["Ci"]
            h["ST"] = (1.0 / np.sqrt((Xf.reshape(vox, -1) ** 2).mean(1) + 1e-6)).astype(np.float32)
        if conv.get("gn"):
            Ci = conv["Ci"]
            h["PV"] = np.concatenate([O.randn(Ci, seed + 20, 0.2) + 1.0, O.randn(Ci, seed + 21, 0.3)]).astype(np.float32); h["pv_stride"] = Ci
    elif xmode == "f16":
        Xf = O.round_f16(O.randn(M * ldx, seed)); h["X"] = O.to_f16(Xf); h["Xf"] = Xf
    else:
        Xf = O.round_f16(O.randn(M * ldx, seed)) * np.float32(c.get("x_scale", 1.0)) + np.float32(c.get("x_shift", 0.0))
        h["X"] = Xf.astype(np.float32); h["Xf"] = h["X"]
        st_off = c.get("st_off", 0)
        st = O.rowstats(h["X"].reshape(M, ldx)[:, kx0:kx0 + K].copy(), M, K, K, rms=(xmode == "rms"), eps=1e-6)
        h["ST"] = np.concatenate([np.full(st_off * 2, 77.0, np.float32), st]); h["st_off"] = st_off
        pv_off = c.get("pv_off", 0); Kt = kx0 + K
        if xmode == "rms":
            h["PV"] = np.concatenate([np.full(pv_off, 9.0, np.float32), (O.randn(Kt, seed + 20, 0.1) + 1.0).astype(np.float32)]); h["pv_stride"] = 0
        else:
            sc = O.round_f16(O.randn(Kt, seed + 20, 0.5)); sh = O.round_f16(O.randn(Kt, seed + 21, 0.5))
            h["PV"] = np.concatenate([np.full(pv_off, 9.0, np.float32), sc, sh]).astype(np.float32); h["pv_stride"] = Kt
        h["pv_off"] = pv_off
    # ---- epilogue vectors and Y
    ldy = c.get("ldy"); ny0 = c.get("ny0", 0)
    ev_off = c.get("ev_off", 0); bv_off = c.get("bv_off", 0)
    if epi == "heads":
        hd = dict(c["heads"]); Ltot = hd["Ltot"]
        h["heads"] = hd
        h["EV"] = np.concatenate([np.full(ev_off, 3.0, np.float32), (O.randn(256, seed + 30, 0.1) + 1.0).astype(np.float32)])
        h["RP"] = rope_table(Ltot, seed + 31)
        ysz, ydt = (N // 128) * Ltot * 128, np.uint16
    elif epi == "swiglu":
        ldy = ldy or N // 2; ysz, ydt = M * ldy, np.uint16
        if c.get("bias"): h["BV"] = np.concatenate([np.full(bv_off, 3.0, np.float32), O.randn(N, seed + 32, 0.5)]).astype(np.float32); h["bv_up"] = N // 2
    else:
        ldy = ldy or N
        ydt = np.float32 if epi in ("f32", "resadd") else np.uint16; ysz = M * ldy
        if epi == "resadd" and c.get("gate"): h["EV"] = np.concatenate([np.full(ev_off, 3.0, np.float32), O.randn(N, seed + 30, 0.5)]).astype(np.float32)
        if epi == "resadd" and c.get("bias"): h["BV"] = np.concatenate([np.full(bv_off, 3.0, np.float32), O.randn(N, seed + 32, 0.5)]).astype(np.float32)
        if epi == "bias": h["EV"] = np.concatenate([np.full(ev_off, 3.0, np.float32), O.randn(N, seed + 30, 0.5)]).astype(np.float32)
        if epi == "onormgate":
            Ltot = c["Ltot"]; h["heads"] = {"Ltot": Ltot, "eps": 1e-6}
            h["EV"] = np.concatenate([np.full(ev_off, 3.0, np.float32), (O.randn(128, seed + 30, 0.1) + 1.0).astype(np.float32)])
            h["GT"] = O.to_f16(O.randn(M * Ltot, seed + 33))
    h["ldy"], h["ny0"], h["ev_off"], h["bv_off"] = ldy, ny0, ev_off, bv_off
    # Y starts as NaN poison, or as data where the epilogue reads it
    if (epi == "resadd" and not h["store"]) or (epi == "bias" and h["res"]):
        y0 = O.randn(ysz, seed + 40)
        h["Y0"] = y0.astype(np.float32) if ydt == np.float32 else O.to_f16(y0)
    else:
        h["Y0"] = np.full(ysz, 0xFFFFFFFF, np.uint32).view(np.float32) if ydt == np.float32 else np.full(ysz, 0xFFFF, np.uint16)
    return h


def _opt(h, k, d=None):
    return h[k] if k in h else d


def run_oracle(h: dict, threads: int = 0) -> np.ndarray:
    Y = h["Y0"].copy()
    O.gemm(enc=h["enc"], X=h["X"], W=h["W"], Y=Y, M=h["M"], N=h["N"], K=h["K"], w_rows=h["w_rows"], w_cols=h["w_cols"], w_ld=h["w_ld"],
           xmode=h["xmode"], epi=h["epi"], ldx=h["ldx"], kx0=h["kx0"], wr0=h["wr0"], wr1=h["wr1"], wk0=h["wk0"], ldy=h["ldy"], ny0=h["ny0"],
           ST=_opt(h, "ST"), st_off=_opt(h, "st_off", 0), PV=_opt(h, "PV"), pv_off=_opt(h, "pv_off", 0), pv_stride=_opt(h, "pv_stride", 0),
           EV=_opt(h, "EV"), ev_off=h["ev_off"], BV=_opt(h, "BV"), bv_off=h["bv_off"], bv_up=_opt(h, "bv_up", 0), RP=_opt(h, "RP"), GT=_opt(h, "GT"),
           res=h["res"], store=h["store"], act=h["act"], heads=_opt(h, "heads"), conv=h["conv"], threads=threads)
    return Y


def gemm_args(gpu, h: dict, bufs: dict) -> dict:
    a = {"w": {"enc": h["enc"], "buf": bufs["W"], "off": h["w_off"], "bytes": h["W"].nbytes, "rows": h["w_rows"], "cols": h["w_cols"]},
         "x": {"buf": bufs["X"], "off": h["x_off"]}, "y": {"buf": bufs["Y"], "off": h["y_off"]}, "M": h["M"], "N": h["N"], "K": h["K"]}
    if h["w_ld"]: a["w"]["ld"] = h["w_ld"]
    if h["ldx"] != h["K"]: a["x"]["ld"] = h["ldx"]
    if h["kx0"]: a["x"]["k0"] = h["kx0"]
    if h["xmode"] != "f16" and not h["conv"]: a["x"]["mode"] = h["xmode"]
    if h["epi"] != "f16": a["epi"] = h["epi"]
    if h["ldy"] != h["N"]: a["y"]["ld"] = h["ldy"]        # the reference's default row stride is N, for swiglu too (src/ops/gemm.js:318)
    if h["ny0"]: a["y"]["n0"] = h["ny0"]
    for k in ("wr0", "wr1", "wk0"):
        if h[k]: a[k] = h[k]
    if "ST" in h: a["stats"] = {"buf": bufs["ST"], "off": _opt(h, "st_off", 0)}
    if "PV" in h: a["pv"] = {"buf": bufs["PV"], "off": _opt(h, "pv_off", 0), "stride": _opt(h, "pv_stride", 0)}
    if "EV" in h: a["ev"] = {"buf": bufs["EV"], "off": h["ev_off"]}
    if "BV" in h: a["bv"] = {"buf": bufs["BV"], "off": h["bv_off"], "up": _opt(h, "bv_up", 0)}
    if "GT" in h: a["gt"] = {"buf": bufs["GT"]}
    if "heads" in h:
        a["heads"] = dict(h["heads"])
        if "RP" in h: a["heads"]["rope"] = {"buf": bufs["RP"]}
    if h["conv"]: a["conv"] = dict(h["conv"])
    for k in ("res", "store"):
        if h[k]: a[k] = True
    if h["act"] != "silu": a["act"] = h["act"]
    if h["tile"]: a["tile"] = h["tile"]
    if h["acc"]: a["acc"] = h["acc"]
    if h["kernel"]: a["kernel"] = h["kernel"]
    return a


def run_gpu(gpu, h: dict, gemm=None) -> np.ndarray:
    import p0pc0rn_kernels_b200 as P
    gemm = gemm or P.gemm
    bufs = {}
    try:
        for k in ("X", "W", "ST", "PV", "EV", "BV", "RP", "GT"):
            if k in h:
                pad = h.get(k.lower() + "_off", 0) if k in ("X", "W") else 0
                data = h[k] if not pad else np.concatenate([np.full(pad, 0xAB, np.uint8), np.ascontiguousarray(h[k]).view(np.uint8).reshape(-1)])
                bufs[k] = gpu.upload(data, k)
        y0 = h["Y0"] if not h["y_off"] else np.concatenate([np.full(h["y_off"], 0xAB, np.uint8), h["Y0"].view(np.uint8).reshape(-1)])
        bufs["Y"] = gpu.upload(y0, "Y")
        args = gemm_args(gpu, h, bufs)
        npeers = int(h.get("peers") or 0)
        for q in range(npeers): bufs[f"YP{q}"] = gpu.upload(y0, f"Y peer {q}")          # same starting bytes as Y (read-modify-write epilogues)
        if npeers: args["y"]["peers"] = [bufs[f"YP{q}"] for q in range(npeers)]
        fl = gemm(gpu, args)
        assert fl == 2.0 * h["M"] * h["N"] * h["K"]
        raw = gpu.read(bufs["Y"], h["y_off"], h["Y0"].nbytes)
        for q in range(npeers):
            assert np.array_equal(gpu.read(bufs[f"YP{q}"], 0, y0.nbytes), gpu.read(bufs["Y"], 0, y0.nbytes)), f"peer copy {q} of y differs from y"
        if h["y_off"]:
            head = gpu.read(bufs["Y"], 0, h["y_off"])
            assert (head == 0xAB).all(), "bytes before y.off were written"
        return raw.view(h["Y0"].dtype).copy()
    finally:
        for b in bufs.values(): gpu.free(b)


def as_float(y: np.ndarray) -> np.ndarray:
    return y if y.dtype == np.float32 else O.from_f16(y)


def check(got: np.ndarray, want: np.ndarray, label: str = ""):
    """poisoned words untouched; written words within the gates.  Returns (cos, rel_l2, max_abs)."""
    if want.dtype == np.float32:
        poison = want.view(np.uint32) == 0xFFFFFFFF; gp = got.view(np.uint32) == 0xFFFFFFFF
    else:
        poison = want == 0xFFFF; gp = got == 0xFFFF
    assert np.array_equal(poison, gp), f"{label}: the set of written outputs differs ({int((poison != gp).sum())} words)"
    g = as_float(got)[~poison].astype(np.float64); w = as_float(want)[~poison].astype(np.float64)
    assert np.isfinite(g).all(), f"{label}: non-finite outputs"
    cos = float((g * w).sum() / np.sqrt(max(1e-30, (g * g).sum() * (w * w).sum())))
    rel = float(np.sqrt(((g - w) ** 2).sum() / max(1e-30, (w * w).sum())))
    mx = float(np.abs(g - w).max()) if g.size else 0.0
    ref = float(np.abs(w).max()) if w.size else 0.0
    assert cos > COS_MIN, f"{label}: cosine {cos}"
    assert rel <= REL_L2_MAX, f"{label}: relative L2 {rel}"
    assert mx <= MAX_ABS_REL * ref + 1e-6, f"{label}: max abs error {mx} vs {ref}"
    return cos, rel, mx
