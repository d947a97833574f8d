"""defaultTune / calibrate / TUNE_TABLE — kept so that code written against src/core/tune.js runs unchanged.
The reference measures throughput to cut work into dispatches short enough for a browser's GPU watchdog; a
CUDA stream has no such limit, so calibrate() only reports rates and tile choices do not change results."""
from __future__ import annotations

import time

import numpy as np

TUNE_TABLE: list = []          # src/core/tune.js:18-22: entries match browser adapters; none applies to CUDA


def tuneEntry(g, table=None):
    info = g.info or {}
    for e in (TUNE_TABLE if table is None else table):
        if all(str(v).lower() in str(info.get(k, "")).lower() for k, v in (e.get("match") or {}).items()):
            return e
    return None


def defaultTune(g, o=None):
    o = o or {}
    t = (tuneEntry(g, o.get("table")) or {}).get("tune") or {}
    g.tune = {"acc": o.get("acc") or t.get("acc") or "f16", "vaeAcc": o.get("vaeAcc") or "f16"}
    if o.get("gemm") or t.get("gemm"):
        g.tune["gemm"] = dict(t.get("gemm") or {}, **(o.get("gemm") or {}))
    return g.tune


def calibrate(g):
    """times the q4 GEMM of src/core/tune.js:39-58 (1024 x 3072 x 3072) and sets gpu.rate / gpu.calib"""
    from .gemm import gemm
    M, N, K = 1024, 3072, 3072
    recs = (N // 64) * (K // 32)
    rs = np.random.default_rng(12345)
    u = rs.integers(0, 2 ** 32, recs * 320, dtype=np.uint32).reshape(recs, 320)
    u[:, 256:] = (0x2000 | ((0xA800 | (np.arange(64, dtype=np.uint32) & 0x3F)) << 16))[None, :]
    h = ((rs.integers(0, 2 ** 16, M * K, dtype=np.uint32) & 0x83FF) | 0x3400).astype(np.uint16)
    W, X, Y = g.upload(u), g.upload(h), g.buffer(M * N * 2)
    try:
        def run():
            gemm(g, {"w": {"buf": W, "off": 0, "bytes": W._pf, "enc": "q4g32a.t64", "rows": N, "cols": K}, "x": {"buf": X}, "M": M, "N": N, "K": K,
                     "epi": "f16", "y": {"buf": Y}})
        run(); g.done()
        t0 = time.perf_counter()
        for _ in range(4): run()
        g.done()
        dt = (time.perf_counter() - t0) / 4
        r = 2.0 * M * N * K / dt
        g.rate.update(mm=r, mm32=r, mm16=r)
        g.calib = {"gemmF32Gflops": round(r / 1e9), "gemmF16Gflops": round(r / 1e9), "attnGflops": None}
    finally:
        for b in (W, X, Y): g.free(b)
    return g.calib
