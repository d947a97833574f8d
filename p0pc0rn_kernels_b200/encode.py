"""Weight conversion on the CPU: safetensors reading, the encodings of the reference's docs/FORMAT.md, convolution
weight reordering and the per-tensor encoding rule — the host-side mirror of src/convert/encode.js.  The
quantisers run in the native library (``p0p_pack_q4`` / ``p0p_pack_q8``)."""
from __future__ import annotations

import ctypes as C
import json
import re

import numpy as np

from ._lib import lib

MANIFEST_FORMAT = "p0pc0rn-kernels.weights/1"      # src/convert/encode.js:134
_BYTES = {"F32": 4, "F16": 2, "BF16": 2, "F8_E4M3": 1, "F8_E5M2": 1}


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


# ------------------------------------------------------------------ safetensors (src/convert/encode.js:17-52)
def safetensorsHeader(data):
    u8 = np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
    n = int(u8[:8].view("<u8")[0])
    if n > 100e6 or 8 + n > u8.size:
        raise ValueError("safetensors: bad or truncated header")
    return {"header": json.loads(bytes(u8[8:8 + n]).decode()), "dataStart": 8 + n}


def safetensorsList(header):
    ts = [{"name": k, "dtype": t["dtype"], "shape": t["shape"], "begin": t["data_offsets"][0], "end": t["data_offsets"][1]}
          for k, t in header.items() if k != "__metadata__"]
    return sorted(ts, key=lambda t: t["begin"])


def dtypeBytes(dt):
    if dt not in _BYTES:
        raise ValueError("unsupported dtype " + dt + " (F32, F16, BF16, F8_E4M3, F8_E5M2)")
    return _BYTES[dt]


def _f8_table(e4m3: bool) -> np.ndarray:
    t = np.empty(256, np.float32)
    for i in range(256):
        s = -1.0 if i & 0x80 else 1.0
        e = (i >> 3) & 15 if e4m3 else (i >> 2) & 31
        m = i & 7 if e4m3 else i & 3
        mb, bias = (3, 7) if e4m3 else (2, 15)
        if e4m3 and e == 15 and m == 7: t[i] = np.nan
        elif not e4m3 and e == 31: t[i] = np.nan if m else s * np.inf
        else: t[i] = s * ((m / (1 << mb)) * 2.0 ** (1 - bias) if e == 0 else (1 + m / (1 << mb)) * 2.0 ** (e - bias))
    return t


_E4M3 = None
_E5M2 = None


def toFloat32(dtype, data) -> np.ndarray:
    """raw tensor bytes of a dtype -> float32 array"""
    global _E4M3, _E5M2
    u8 = np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    dtypeBytes(dtype)
    if dtype == "F32": return u8.view("<f4").astype(np.float32)
    if dtype == "F8_E4M3":
        _E4M3 = _E4M3 if _E4M3 is not None else _f8_table(True); return _E4M3[u8]
    if dtype == "F8_E5M2":
        _E5M2 = _E5M2 if _E5M2 is not None else _f8_table(False); return _E5M2[u8]
    h = u8.view("<u2")
    if dtype == "BF16": return (h.astype(np.uint32) << 16).view(np.float32)
    o = np.empty(h.size, np.float32)
    hc = np.ascontiguousarray(h)
    lib.p0p_from_f16(hc.ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p), h.size)
    return o


# ------------------------------------------------------------------ encodings (src/convert/encode.js:56-106)
def packQ4(W, rows, K, deq=None) -> np.ndarray:
    if rows % 64 or K % 32:
        raise ValueError("q4g32a.t64 needs rows % 64 == 0 and K % 32 == 0")
    W = _f32(W); out = np.zeros(rows * K * 5 // 8, np.uint8)
    lib.p0p_pack_q4(W.ctypes.data_as(C.c_void_p), rows, K, out.ctypes.data_as(C.c_void_p), deq.ctypes.data_as(C.c_void_p) if deq is not None else None)
    return out


def packQ8(W, rows, K, deq=None) -> np.ndarray:
    if rows % 64 or K % 64:
        raise ValueError("q8g64s.t64 needs rows % 64 == 0 and K % 64 == 0")
    W = _f32(W); out = np.zeros(rows * K * 33 // 32, np.uint8)
    lib.p0p_pack_q8(W.ctypes.data_as(C.c_void_p), rows, K, out.ctypes.data_as(C.c_void_p), deq.ctypes.data_as(C.c_void_p) if deq is not None else None)
    return out


def packF16(W) -> np.ndarray:
    W = _f32(W); o = np.empty(W.size, np.uint16)
    lib.p0p_to_f16(W.ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p), W.size)
    return o.view(np.uint8)


def packF32(W) -> np.ndarray:
    return _f32(W).copy().view(np.uint8)


def tileBytes(enc, K):
    return (K // 32) * 1280 if enc == "q4g32a.t64" else (K // 64) * 4224 if enc == "q8g64s.t64" else 64 * K * 2 if enc == "f16" else 64 * K * 4


def encodeRows(enc, W, rows, K) -> np.ndarray:
    W = _f32(W)
    if enc == "q4g32a.t64": return packQ4(W, rows, K)
    if enc == "q8g64s.t64": return packQ8(W, rows, K)
    if enc == "f16": return packF16(W[: rows * K])
    if enc == "f32": return packF32(W[: rows * K])
    raise ValueError("unknown encoding " + str(enc))


# ------------------------------------------------------------------ layout and the encoding rule (src/convert/encode.js:111-133)
def matrixOf(shape):
    shape = list(shape)
    if len(shape) == 4: return {"rows": shape[0], "cols": shape[1] * shape[2] * shape[3], "layout": "OHWI"}
    if len(shape) == 5: return {"rows": shape[0], "cols": shape[1] * shape[2] * shape[3] * shape[4], "layout": "OTHWI"}
    if len(shape) <= 1: return {"rows": 1, "cols": shape[0] if shape else 1, "layout": "vector"}
    return {"rows": int(np.prod(shape[:-1])), "cols": shape[-1], "layout": "row-major"}


def reorderConvRows(W, rows, shape) -> np.ndarray:
    """rows of a convolution weight OIHW / OITHW (I * taps) -> (taps * I)"""
    W = _f32(W); I = shape[1]; taps = int(np.prod(shape[2:]))
    out = np.empty(rows * I * taps, np.float32)
    lib.p0p_reorder_conv_rows(W.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), rows, I, taps)
    return out


def chooseEncoding(name, shape, opts=None):
    opts = opts or {}
    bits = opts.get("bits") or 4
    m = matrixOf(shape)
    f32, keep = opts.get("f32"), opts.get("keep")
    if f32 and re.search(f32, name): return "f32"
    if m["layout"] == "vector": return "f32"
    if (keep and re.search(keep, name)) or bits == 16: return "f16"
    if bits == 4 and m["rows"] % 64 == 0 and m["cols"] % 32 == 0: return "q4g32a.t64"
    if bits in (4, 8) and m["rows"] % 64 == 0 and m["cols"] % 64 == 0: return "q8g64s.t64"
    return "f16"
