"""Load a converted model (manifest.json + weight shards) onto the GPU: each shard becomes one buffer and each
tensor a view the ops take directly — the host-side mirror of src/weights.js."""
from __future__ import annotations

import json
import os

import numpy as np

from .encode import MANIFEST_FORMAT


def _model_of(manifest, bufs, gpu):
    class Model:
        def __init__(self): self.manifest = manifest
        def names(self): return list(manifest["tensors"].keys())
        def tensor(self, name):
            """a weight for gemm's `w`: {enc, buf, off, bytes, rows, cols} (+ shape, layout) (src/weights.js:38-41)"""
            t = manifest["tensors"].get(name)
            if not t: raise KeyError("no tensor " + name)
            return {"enc": t["enc"], "buf": bufs[t["file"]], "off": t["offset"], "bytes": t["bytes"], "rows": t["rows"], "cols": t["cols"],
                    "shape": t["shape"], "layout": t["layout"]}
        def vector(self, name):
            """an fp32 vector as the ops take it: {buf, off} with off counted in floats (src/weights.js:43-47)"""
            t = manifest["tensors"].get(name)
            if not t: raise KeyError("no tensor " + name)
            if t["enc"] != "f32": raise ValueError(name + " is " + t["enc"] + ", not f32")
            return {"buf": bufs[t["file"]], "off": t["offset"] // 4}
        def free(self):
            for b in bufs.values(): gpu.free(b)
    return Model()


def loadWeights(gpu, base, opts=None):
    """base: the folder holding manifest.json; opts: {onProgress(doneBytes, totalBytes)} (src/weights.js:10-25)"""
    opts = opts or {}
    with open(os.path.join(base, "manifest.json")) as f:
        manifest = json.load(f)
    if manifest.get("format") != MANIFEST_FORMAT:
        raise ValueError("not a converted model (format " + str(manifest.get("format")) + ")")
    total = sum(s["bytes"] for s in manifest["shards"]); bufs = {}; done = 0
    try:
        for s in manifest["shards"]:
            data = np.fromfile(os.path.join(base, s["file"]), np.uint8)
            if data.size != s["bytes"]:
                raise ValueError(f"{s['file']}: {data.size} bytes, the manifest says {s['bytes']}")
            bufs[s["file"]] = gpu.upload(data, s["file"]); done += s["bytes"]
            if opts.get("onProgress"): opts["onProgress"](done, total)
    except Exception:
        for b in bufs.values(): gpu.free(b)
        raise
    return _model_of(manifest, bufs, gpu)


def uploadWeights(gpu, manifest, shards):
    """the same from shards already in memory ({file: uint8 array}) (src/weights.js:28-31)"""
    bufs = {s["file"]: gpu.upload(shards[s["file"]], s["file"]) for s in manifest["shards"]}
    return _model_of(manifest, bufs, gpu)
