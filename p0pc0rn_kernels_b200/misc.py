"""rowstats: per-row (mean, rstd) of an fp32 matrix, the producer of the `stats` input of gemm's fused norm
prologues — host-side mirror of src/ops/misc.js:16-44."""
from __future__ import annotations

from ._lib import lib


def rowstats(gpu, a: dict) -> None:
    """a: {x: {buf, off (bytes), ld (floats), c0}, rows, cols, mode: 'ln' | 'rms', eps, st: {buf, off (rows)}}"""
    x, st = a["x"], a["st"]
    gpu._check(lib.p0p_rowstats(gpu._h, x["buf"].handle, int(x.get("off") or 0), int(x.get("ld") or a["cols"]), int(x.get("c0") or 0),
                                int(a["rows"]), int(a["cols"]), 1 if a.get("mode") == "rms" else 0, float(a["eps"]), st["buf"].handle,
                                int(st.get("off") or 0)))
