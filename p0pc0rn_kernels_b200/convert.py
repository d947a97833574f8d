"""Converter core: safetensors sources -> weight shards in the kernels' encodings + a manifest — the host-side
mirror of src/convert/convert.js (docs/FORMAT.md, "Converted models").  Tensors stream in blocks of whole
64-row tiles, every tensor starts on a 256-byte boundary of its shard, shards roll over at shardBytes."""
from __future__ import annotations

import json

import numpy as np

from .encode import (MANIFEST_FORMAT, chooseEncoding, dtypeBytes, encodeRows, matrixOf, reorderConvRows, safetensorsHeader, safetensorsList,
                     tileBytes, toFloat32)

ALIGN = 256                       # src/convert/convert.js:10
_SUPPORTED = {"F32", "F16", "BF16", "F8_E4M3", "F8_E5M2"}


def encodedBytes(enc, rows, cols):
    return (rows // 64) * tileBytes(enc, cols) if enc in ("q4g32a.t64", "q8g64s.t64") else rows * cols * (2 if enc == "f16" else 4)


def convert(sources, out, opts=None):
    """sources: [{file, header, dataStart, read(offset, length) -> bytes}]; out: object with begin(name), write(bytes), end().
    opts: {bits, keep, f32, shardBytes, onTensor}.  Returns the manifest (src/convert/convert.js:15-44)."""
    opts = opts or {}
    shardBytes = opts.get("shardBytes") or 512 * 2 ** 20
    tensors, shards, skipped = {}, [], {}
    cur = None

    def close():
        nonlocal cur
        if cur is None: return
        out.end(); shards.append({"file": cur["file"], "bytes": cur["bytes"]}); cur = None

    def open_():
        nonlocal cur
        if cur is not None: close()
        cur = {"file": "weights-%05d.bin" % (len(shards) + 1), "bytes": 0}
        out.begin(cur["file"])

    def put(u8):
        out.write(u8); cur["bytes"] += len(u8)

    for src in sources:
        for t in safetensorsList(src["header"]):
            if t["name"] in tensors: raise ValueError("tensor " + t["name"] + " appears twice")
            if t["dtype"] not in _SUPPORTED:
                skipped[t["name"]] = t["dtype"]; continue
            m = matrixOf(t["shape"]); enc = chooseEncoding(t["name"], t["shape"], opts)
            size = encodedBytes(enc, m["rows"], m["cols"]); eb = dtypeBytes(t["dtype"])
            if t["end"] - t["begin"] != m["rows"] * m["cols"] * eb:
                raise ValueError(f"tensor {t['name']}: {t['end'] - t['begin']} bytes for shape [{','.join(map(str, t['shape']))}] {t['dtype']}")
            if cur is None or (cur["bytes"] > 0 and -(-cur["bytes"] // ALIGN) * ALIGN + size > shardBytes): open_()
            pad = (ALIGN - cur["bytes"] % ALIGN) % ALIGN
            if pad: put(bytes(pad))
            entry = {"enc": enc, "dtype": t["dtype"], "shape": t["shape"], "rows": m["rows"], "cols": m["cols"], "layout": m["layout"],
                     "file": cur["file"], "offset": cur["bytes"], "bytes": size}
            conv = m["layout"] in ("OHWI", "OTHWI")
            block = max(64, (4 * 2 ** 20) // max(1, m["cols"]) // 64 * 64)
            for r0 in range(0, m["rows"], block):
                nr = min(block, m["rows"] - r0)
                raw = src["read"](src["dataStart"] + t["begin"] + r0 * m["cols"] * eb, nr * m["cols"] * eb)
                W = toFloat32(t["dtype"], raw)
                if conv: W = reorderConvRows(W, nr, t["shape"])
                put(encodeRows(enc, W, nr, m["cols"]).tobytes())
            if cur["bytes"] - entry["offset"] != size:
                raise ValueError(f"tensor {t['name']}: wrote {cur['bytes'] - entry['offset']} of {size} bytes")
            tensors[t["name"]] = entry
            if opts.get("onTensor"): opts["onTensor"](t["name"], entry)
    close()
    return {"format": MANIFEST_FORMAT, "sources": [s["file"] for s in sources], "bits": opts.get("bits") or 4, "tensors": tensors,
            "shards": shards, "skipped": skipped}


def convertSafetensors(buffer, opts=None, file="model.safetensors"):
    """one safetensors file in memory -> {manifest, shards: {name: uint8 array}} (src/convert/convert.js:48-54)"""
    u8 = np.frombuffer(buffer, np.uint8) if not isinstance(buffer, np.ndarray) else buffer.view(np.uint8).reshape(-1)
    hd = safetensorsHeader(u8)
    files, state = {}, {}

    class _Out:
        def begin(self, n): state["name"] = n; state["parts"] = []
        def write(self, b): state["parts"].append(bytes(b))
        def end(self): files[state["name"]] = np.frombuffer(b"".join(state["parts"]), np.uint8)

    manifest = convert([{"file": file, "header": hd["header"], "dataStart": hd["dataStart"], "read": lambda off, ln: u8[off:off + ln]}], _Out(), opts)
    return {"manifest": manifest, "shards": files}


def writeSafetensors(tensors, metadata=None) -> np.ndarray:
    """build a safetensors file in memory from {name: {dtype, shape, data}} (src/convert/convert.js:57-66)"""
    header, off = {}, 0
    if metadata: header["__metadata__"] = metadata
    datas = []
    for name, t in tensors.items():
        d = np.ascontiguousarray(t["data"]).view(np.uint8).reshape(-1)
        header[name] = {"dtype": t["dtype"], "shape": list(t["shape"]), "data_offsets": [off, off + d.size]}
        off += d.size; datas.append(d)
    js = json.dumps(header, separators=(",", ":")).encode()
    js += b" " * ((8 - ((8 + len(js)) % 8)) % 8)
    return np.concatenate([np.frombuffer(np.uint64(len(js)).tobytes(), np.uint8), np.frombuffer(js, np.uint8), *datas]) if datas else \
        np.concatenate([np.frombuffer(np.uint64(len(js)).tobytes(), np.uint8), np.frombuffer(js, np.uint8)])
