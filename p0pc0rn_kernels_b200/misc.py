"""Producers of the statistics that gemm's fused prologues read — host-side mirrors of the reference ops:

  rowstats                         per-row (mean, rstd) of an fp32 matrix -> `stats` of the rms / lnmod prologues (src/ops/misc.js:16-44)
  pixstats                         per-voxel PixelNorm factor of an fp16 tensor -> `stats` of conv3's `pn`          (src/ops/video.js:301-318)
  gnPartial / gnFinalize / groupnormStats   exact GroupNorm(32) statistics of an HWC fp16 tensor -> `pv` (a, b per channel) of conv's `gn`
                                   (src/ops/misc.js:50-120)
"""
from __future__ import annotations

import ctypes as C
import math

from ._lib import lib


def rowstats(gpu, a: dict) -> None:
    """a: {x: {buf, off (bytes), ld (floats), c0}, rows, cols, mode: 'ln' | 'rms', eps, st: {buf, off (rows)}}"""
    x, st = a["x"], a["st"]
    gpu._check(lib.p0p_rowstats(gpu._h, x["buf"].handle, int(x.get("off") or 0), int(x.get("ld") or a["cols"]), int(x.get("c0") or 0),
                                int(a["rows"]), int(a["cols"]), 1 if a.get("mode") == "rms" else 0, float(a["eps"]), st["buf"].handle,
                                int(st.get("off") or 0)))


def pixstats(gpu, a: dict) -> None:
    """a: {x: {buf, off (bytes)}, V, C, eps (default 1e-8), r: {buf}, ro (floats)}: r[ro + v] = rsqrt(mean_c x[v][c]^2 + eps)"""
    x = a["x"]
    gpu._check(lib.p0p_pixstats(gpu._h, x["buf"].handle, int(x.get("off") or 0), int(a["V"]), int(a["C"]), float(a.get("eps") or 1e-8),
                                a["r"]["buf"].handle, int(a.get("ro") or 0)))


def gnPartBytes(pix: int) -> int:
    """bytes of partial rows for `pix` pixels (src/ops/misc.js:106)"""
    return math.ceil(pix / 64) * 512


def gnPartial(gpu, a: dict) -> int:
    """a: {x: {buf, off}, pix, C, part: buf, wgOff}: partial statistics into part rows [wgOff, wgOff + ceil(pix / 64)); returns the row count"""
    x = a["x"]; n = C.c_uint32()
    gpu._check(lib.p0p_gn_partial(gpu._h, x["buf"].handle, int(x.get("off") or 0), int(a["pix"]), int(a["C"]), a["part"].handle, int(a.get("wgOff") or 0), C.byref(n)))
    return int(n.value)


def gnFinalize(gpu, a: dict) -> None:
    """a: {part: buf, nwg, C, eps, gb: {buf, gOff, bOff (bytes)}, ab: {buf, off (floats)}}: a[C], b[C] with GN(x) = a * x + b per channel"""
    gb, ab = a["gb"], a["ab"]
    gpu._check(lib.p0p_gn_finalize(gpu._h, a["part"].handle, int(a["nwg"]), int(a["C"]), float(a.get("eps") or 1e-6), gb["buf"].handle,
                                   int(gb.get("gOff") or 0) // 4, int(gb.get("bOff") or 0) // 4, ab["buf"].handle, int(ab.get("off") or 0)))


def groupnormStats(gpu, a: dict) -> None:
    """Exact GroupNorm(32) statistics of x -> ab.  a: {x, pix, C, part: scratch of gnPartBytes(pix), gb, ab, eps}"""
    nwg = gnPartial(gpu, {"x": a["x"], "pix": a["pix"], "C": a["C"], "part": a["part"]})
    gnFinalize(gpu, {"part": a["part"], "nwg": nwg, "C": a["C"], "gb": a["gb"], "ab": a["ab"], "eps": a.get("eps")})
