"""CPU oracle for the p0pc0rn-kernels `gemm` path — TEST INFRASTRUCTURE ONLY.

A ctypes view of ``libp0p_oracle.so`` (built from ``p0p_oracle.c`` by ``oracle/Makefile``), which restates in
plain C the reference's fp16 helpers (src/core/gpu.js:275-299), seeded generators and CPU multiplications
(test/kernels.test.js:12-29, 52-65), weight encoders (src/convert/encode.js:56-122) and the shader arithmetic
of every gemm prologue/epilogue (src/ops/gemm.js:60-101, 143-172, 191-254).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module, and only
as the checker.  The product package never does.

Pinning status: "parity unpinned" beyond the reference's few stored known-answer constants — the reference
holds no golden vectors for this path and no JavaScript engine exists where this runs.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libp0p_oracle.so")

X_MODES = {"f16": 0, "lnmod": 1, "rms": 2, "conv": 3, "conv3": 4}
EPIS = {"f16": 0, "f32": 1, "resadd": 2, "swiglu": 3, "heads": 4, "bias": 5, "onormgate": 6}
ENCS = {"q4g32a.t64": 0, "q8g64s.t64": 1, "f16": 2}
F_GATE, F_RES, F_STORE, F_GN, F_UP2, F_PN, F_BIAS, F_GELU, F_ROPE_HALF = 1, 2, 4, 8, 16, 32, 64, 128, 256


def build(force: bool = False) -> str:
    """Compile the oracle library if it is missing or older than its source."""
    src = os.path.join(_HERE, "p0p_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libp0p_oracle.so"], check=True, capture_output=True)
    return _SO


class _Args(C.Structure):
    _fields_ = ([(n, C.c_uint32) for n in ("enc", "xmode", "epi", "flags", "M", "N", "K", "ldx", "kx0", "wR0", "wR1", "wG", "wk0",
                                            "ldy", "ny0", "rowOff", "Ltot", "Hq", "Hkv")]
                + [("eps", C.c_float)]
                + [(n, C.c_uint32) for n in ("pvOff", "pvStride", "evOff", "statOff", "Hi", "Wi", "Ci", "Ho", "Wo", "stride", "padT",
                                              "padL", "ks", "Nw", "bvOff", "bvUp")]
                + [(n, C.c_void_p) for n in ("X", "W", "Y", "ST", "PV", "EV", "BV", "RP", "GT")]
                + [("threads", C.c_int)])


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_f2h.restype = C.c_uint16; L.orc_f2h.argtypes = [C.c_float]
        L.orc_h2f.restype = C.c_float; L.orc_h2f.argtypes = [C.c_uint16]
        L.orc_f8.restype = C.c_float; L.orc_f8.argtypes = [C.c_int, C.c_uint8]
        L.orc_pack_q4.restype = C.c_int; L.orc_pack_q8.restype = C.c_int; L.orc_gemm.restype = C.c_int
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------- fp16 / generators
def f2h(v: float) -> int:
    return int(lib().orc_f2h(C.c_float(v)))


def h2f(h: int) -> float:
    return float(lib().orc_h2f(C.c_uint16(h)))


def to_f16(a) -> np.ndarray:
    a = _f32(a).ravel(); o = np.empty(a.size, np.uint16); lib().orc_to_f16(_p(a), _p(o), C.c_size_t(a.size)); return o


def from_f16(h) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16).ravel(); o = np.empty(h.size, np.float32); lib().orc_from_f16(_p(h), _p(o), C.c_size_t(h.size)); return o


def round_f16(a) -> np.ndarray:
    a = _f32(a).ravel(); o = np.empty_like(a); lib().orc_round_f16(_p(a), _p(o), C.c_size_t(a.size)); return o


def to_bf16(a) -> np.ndarray:
    a = _f32(a).ravel(); o = np.empty(a.size, np.uint16); lib().orc_to_bf16(_p(a), _p(o), C.c_size_t(a.size)); return o


def from_bf16(h) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16).ravel(); o = np.empty(h.size, np.float32); lib().orc_from_bf16(_p(h), _p(o), C.c_size_t(h.size)); return o


def f8(e4m3: bool, byte: int) -> float:
    return float(lib().orc_f8(1 if e4m3 else 0, C.c_uint8(byte)))


def randn(n: int, seed: int, scale: float = 1.0) -> np.ndarray:
    o = np.empty(n, np.float32); lib().orc_randn(_p(o), C.c_size_t(n), C.c_uint32(seed & 0xFFFFFFFF), C.c_double(scale)); return o


def rng_u32(n: int, seed: int) -> np.ndarray:
    o = np.empty(n, np.uint32); lib().orc_rng_u32(_p(o), C.c_size_t(n), C.c_uint32(seed & 0xFFFFFFFF)); return o


# ---------------------------------------------------------------- encoders
def pack_q4(W, rows: int, K: int):
    """-> (bytes uint8[rows*K*5/8], deq float32[rows*K])"""
    W = _f32(W).ravel(); out = np.zeros(rows * K * 5 // 8, np.uint8); deq = np.empty(rows * K, np.float32)
    if lib().orc_pack_q4(_p(W), C.c_uint32(rows), C.c_uint32(K), _p(out), _p(deq)):
        raise ValueError("q4g32a.t64 needs rows % 64 == 0 and K % 32 == 0")
    return out, deq


def pack_q8(W, rows: int, K: int):
    W = _f32(W).ravel(); out = np.zeros(rows * K * 33 // 32, np.uint8); deq = np.empty(rows * K, np.float32)
    if lib().orc_pack_q8(_p(W), C.c_uint32(rows), C.c_uint32(K), _p(out), _p(deq)):
        raise ValueError("q8g64s.t64 needs rows % 64 == 0 and K % 64 == 0")
    return out, deq


def reorder_conv_rows(W, rows: int, I: int, taps: int) -> np.ndarray:
    W = _f32(W).ravel(); o = np.empty_like(W); lib().orc_reorder_conv_rows(_p(W), _p(o), C.c_uint32(rows), C.c_uint32(I), C.c_uint32(taps)); return o


def dequant(enc: str, Wbytes, r0: int, nr: int, K: int, ld: int = 0):
    """tile values as the shader forms them: (fp16 bits uint16[nr*K], fp32 before rounding float32[nr*K])"""
    Wb = np.ascontiguousarray(Wbytes).view(np.uint8).ravel(); h = np.empty(nr * K, np.uint16); f = np.empty(nr * K, np.float32)
    lib().orc_dequant(C.c_int(ENCS[enc]), _p(Wb), C.c_uint32(r0), C.c_uint32(nr), C.c_uint32(K), C.c_uint32(ld), _p(h), _p(f)); return h, f


# ---------------------------------------------------------------- the reference tests' CPU multiplications
def cpu_gemm(X, W, M: int, N: int, K: int, threads: int = 1) -> np.ndarray:
    X = _f32(X).ravel(); W = _f32(W).ravel(); Y = np.empty(M * N, np.float32)
    lib().orc_cpu_gemm(_p(X), _p(W), _p(Y), C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), C.c_int(threads)); return Y


def cpu_conv3(X, Wt, T: int, H: int, Wd: int, Cc: int, N: int, threads: int = 1) -> np.ndarray:
    X = _f32(X).ravel(); Wt = _f32(Wt).ravel(); Y = np.empty(T * H * Wd * N, np.float32)
    lib().orc_cpu_conv3(_p(X), _p(Wt), _p(Y), C.c_uint32(T), C.c_uint32(H), C.c_uint32(Wd), C.c_uint32(Cc), C.c_uint32(N), C.c_int(threads)); return Y


def compare(got, want):
    """-> (cos, maxErr) as test/kernels.test.js:16-21"""
    got = _f32(got).ravel(); want = _f32(want).ravel(); out = (C.c_double * 2)()
    lib().orc_compare(_p(got), _p(want), C.c_size_t(want.size), out); return float(out[0]), float(out[1])


def rowstats(X, rows: int, cols: int, ld: int | None = None, rms: bool = False, eps: float = 1e-6) -> np.ndarray:
    X = _f32(X).ravel(); ST = np.empty(rows * 2, np.float32)
    lib().orc_rowstats(_p(X), C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(ld or cols), C.c_int(1 if rms else 0), C.c_float(eps), _p(ST)); return ST


def pixstats(X16, V: int, Cc: int, eps: float = 1e-8) -> np.ndarray:
    """pixstats of src/ops/video.js:301-318 on fp16 bits [V][C] -> float32 [V]"""
    X16 = np.ascontiguousarray(X16, np.uint16).ravel(); R = np.empty(V, np.float32)
    lib().orc_pixstats(_p(X16), C.c_uint32(V), C.c_uint32(Cc), C.c_float(eps), _p(R)); return R


def gn_partial(X16, pix: int, Cc: int) -> np.ndarray:
    """gnPartial of src/ops/misc.js:50-73 -> float32 [ceil(pix/64)][32][4] = (n, mean, M2, 0)"""
    X16 = np.ascontiguousarray(X16, np.uint16).ravel(); nwg = -(-pix // 64); PT = np.zeros(nwg * 32 * 4, np.float32)
    lib().orc_gn_partial(_p(X16), C.c_uint32(pix), C.c_uint32(Cc), C.c_uint32(0), _p(PT)); return PT


def gn_finalize(PT, nwg: int, Cc: int, gamma, beta, eps: float = 1e-6) -> np.ndarray:
    """gnFinalize of src/ops/misc.js:75-104 -> float32 [2][C] = a, b"""
    PT = _f32(PT).ravel(); gamma = _f32(gamma).ravel(); beta = _f32(beta).ravel(); AB = np.empty(2 * Cc, np.float32)
    lib().orc_gn_finalize(_p(PT), C.c_uint32(nwg), C.c_uint32(Cc), C.c_float(eps), _p(gamma), _p(beta), _p(AB)); return AB


def cpu_attn(Q, Kt, V, *, Hq: int, Hkv: int | None = None, Lq: int, Lk: int | None = None, D: int = 128, mode: int = 0, nvalid: int | None = None,
             scale: float | None = None, cap: float = 0.0, threads: int = 0) -> np.ndarray:
    """cpuAttn of test/kernels.test.js:32-48 -> O float32 [Lq][Hq*D]"""
    Hkv = Hkv or Hq; Lk = Lk or Lq; nvalid = nvalid or Lk
    Q, Kt, V = _f32(Q).ravel(), _f32(Kt).ravel(), _f32(V).ravel()
    O_ = np.empty(Lq * Hq * D, np.float32)
    lib().orc_cpu_attn(_p(Q), _p(Kt), _p(V), _p(O_), C.c_uint32(Hq), C.c_uint32(Hkv), C.c_uint32(Lq), C.c_uint32(Lk), C.c_uint32(D), C.c_uint32(mode),
                       C.c_uint32(nvalid), C.c_double(scale if scale is not None else 1.0 / np.sqrt(D)), C.c_double(cap), C.c_int(threads or max_threads()))
    return O_


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------- the whole op
def gemm(*, enc: str, X, W, Y, M: int, N: int, K: int, w_rows: int, w_cols: int, w_ld: int = 0, xmode: str = "f16", epi: str = "f16",
         ldx: int | None = None, kx0: int = 0, wr0: int = 0, wr1: int = 0, wk0: int = 0, ldy: int | None = None, ny0: int = 0,
         ST=None, st_off: int = 0, PV=None, pv_off: int = 0, pv_stride: int = 0, EV=None, ev_off: int = 0, BV=None, bv_off: int = 0,
         bv_up: int = 0, RP=None, GT=None, res: bool = False, store: bool = False, act: str = "silu", heads: dict | None = None,
         conv: dict | None = None, threads: int = 0) -> None:
    """Run the restated op on host arrays; Y (a numpy array of the output dtype) is updated in place.

    Arguments carry the meaning of the reference's gemm() argument object (src/ops/gemm.js:259-267); X, W, Y are
    the arrays *from* the x/w/y byte offsets on.
    """
    a = _Args()
    h = heads or {}; c = conv or {}
    a.enc = ENCS[enc]
    a.xmode = X_MODES["conv3" if c.get("kind") == "conv3" else "conv"] if conv else X_MODES[xmode]
    a.epi = EPIS[epi]
    fl = 0
    if EV is not None and epi == "resadd": fl |= F_GATE
    if res: fl |= F_RES
    if store: fl |= F_STORE
    if c.get("gn"): fl |= F_GN
    if c.get("up2"): fl |= F_UP2
    if c.get("pn"): fl |= F_PN
    if BV is not None: fl |= F_BIAS
    if act == "gelu": fl |= F_GELU
    if h.get("ropeMode") == "half": fl |= F_ROPE_HALF
    a.flags = fl
    a.M, a.N, a.K = M, N, K
    a.ldx = ldx or K; a.kx0 = kx0; a.wR0 = wr0; a.wR1 = wr1
    a.wG = w_cols // 32 if enc.startswith("q4") else w_cols // 64 if enc.startswith("q8") else (w_ld or w_cols)
    a.wk0 = wk0; a.ldy = ldy or N; a.ny0 = ny0
    a.rowOff = h.get("rowOff", 0); a.Ltot = h.get("Ltot", 0); a.Hq = h.get("Hq", 0); a.Hkv = h.get("Hkv", 0); a.eps = h.get("eps", 1e-6) or 1e-6
    a.pvOff = pv_off; a.pvStride = pv_stride; a.evOff = ev_off; a.statOff = st_off
    a.Hi = c.get("Hi", 0); a.Wi = c.get("Wi", 0); a.Ci = c.get("Ci", 0); a.Ho = c.get("Ho", 0); a.Wo = c.get("Wo", 0)
    a.stride = c.get("stride", 1) or 1; a.padT = c.get("padT", 0); a.padL = c.get("padL", 0); a.ks = c.get("ks", 1) or 1
    a.Nw = w_rows; a.bvOff = bv_off; a.bvUp = bv_up
    keep = []
    def ptr(arr, dt=None):
        if arr is None: return None
        arr2 = np.ascontiguousarray(arr) if dt is None else np.ascontiguousarray(arr, dtype=dt)
        keep.append(arr2); return arr2.ctypes.data
    a.X = ptr(X); a.W = ptr(np.ascontiguousarray(W).view(np.uint8))
    assert Y.flags["C_CONTIGUOUS"]; a.Y = Y.ctypes.data
    a.ST = ptr(ST, np.float32); a.PV = ptr(PV, np.float32); a.EV = ptr(EV, np.float32); a.BV = ptr(BV, np.float32)
    a.RP = ptr(RP, np.float32); a.GT = ptr(GT, np.uint16)
    a.threads = threads or max_threads()
    rc = lib().orc_gemm(C.byref(a))
    if rc: raise RuntimeError(f"oracle gemm failed ({rc})")
