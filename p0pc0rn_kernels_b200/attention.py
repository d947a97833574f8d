"""attention(gpu, args): head-128 flash attention — host-side mirror of src/ops/attention.js:168-193."""
from __future__ import annotations

import ctypes as C

from ._lib import AttnArgs, lib


def attention(gpu, a: dict) -> float:
    """a: {q: {buf, off}, k, v, o: {buf, off, ld}, Hq, Hkv, Lq, Lk, scale, mode, nvalid}; returns 4 * Lq * Lk * 128 * Hq.
    Q [Hq][Lq][128], K / V [Hkv][Lk][128] f16 head-major; O [Lq][o.ld] f16 token-major.  The reference's tuning fields
    (cfg, cfgF) are accepted and ignored.  `kernel` ('warp' | 'tmem', for tests) forces one of the two kernels."""
    g = AttnArgs()
    g.struct_size = C.sizeof(AttnArgs)
    g.Hq = int(a["Hq"]); g.Hkv = int(a.get("Hkv") or a["Hq"]); g.Lq = int(a["Lq"]); g.Lk = int(a.get("Lk") or a["Lq"])
    g.ldo = int(a["o"].get("ld") or g.Hq * 128); g.mode = int(a.get("mode") or 0); g.nvalid = int(a.get("nvalid") or g.Lk)
    g.scale = float(a["scale"]) if a.get("scale") is not None else 0.0
    for name in ("q", "k", "v", "o"):
        t = a[name]
        setattr(g, name, t["buf"].handle.value if hasattr(t["buf"].handle, "value") else t["buf"].handle)
        setattr(g, name + "_off", int(t.get("off") or 0))
    g.kernel = {None: 0, "warp": 16, "tmem": 17}[a.get("kernel")]
    fl = C.c_double(0.0)
    gpu._check(lib.p0p_attention(gpu._h, C.byref(g), C.byref(fl)))
    return fl.value
