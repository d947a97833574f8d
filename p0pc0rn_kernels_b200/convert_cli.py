"""Command line of the converter — the host-side mirror of tools/convert.mjs:9-62:

    python -m p0pc0rn_kernels_b200.convert_cli <model.safetensors | model folder | files...> --out <folder>
           [--bits 4|8|16] [--keep <regex>] [--f32 <regex>] [--shard-mb 512] [--dry-run]

    --bits 4   matrices that fit 64-row tiles -> q4g32a.t64 (8 -> q8g64s.t64, 16 -> fp16); everything else -> fp16; vectors -> fp32
    --keep     tensors whose names match stay fp16 (default "embed": embeddings are looked up by row, not multiplied)
    --f32      tensors whose names match are stored fp32

Writes shards of at most --shard-mb plus manifest.json (docs/FORMAT.md).  Tensors stream in blocks, so models larger than memory
convert.  Exit status 2 on a usage error, like the reference."""
from __future__ import annotations

import datetime
import json
import os
import re
import sys
import time

import numpy as np

from .convert import convert, encodedBytes
from .encode import chooseEncoding, matrixOf, safetensorsHeader, safetensorsList

USAGE = ("usage: python -m p0pc0rn_kernels_b200.convert_cli <model.safetensors | folder | files...> --out <folder> [--bits 4|8|16] "
         "[--keep <regex>] [--f32 <regex>] [--shard-mb 512] [--dry-run]")


def main(argv=None, out=sys.stdout, err=sys.stderr) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)

    def flag(k, d):
        if k not in argv: return d
        i = argv.index(k)
        v = argv[i + 1] if i + 1 < len(argv) else d
        del argv[i:i + 2]
        return v

    OUT, KEEP, F32 = flag("--out", None), flag("--keep", "embed"), flag("--f32", None)
    try:
        BITS, SHARD = int(flag("--bits", 4)), float(flag("--shard-mb", 512))
    except ValueError:
        BITS, SHARD = 0, 512
    DRY = "--dry-run" in argv
    if DRY: argv.remove("--dry-run")
    if not argv or (not OUT and not DRY) or BITS not in (4, 8, 16):
        print(USAGE, file=err)
        return 2
    opts = {"bits": BITS, "keep": re.compile(KEEP) if KEEP else None, "f32": re.compile(F32) if F32 else None, "shardBytes": int(SHARD * 2 ** 20)}
    files = []
    for p in argv:
        files += [os.path.join(p, f) for f in sorted(os.listdir(p)) if f.endswith(".safetensors")] if os.path.isdir(p) else [p]
    if not files:
        print("no .safetensors files found", file=err)
        return 2

    handles, sources = [], []
    for f in files:
        fd = open(f, "rb"); handles.append(fd)
        n = int(np.frombuffer(fd.read(8), np.uint64)[0])
        fd.seek(0)
        hd = safetensorsHeader(np.frombuffer(fd.read(8 + n), np.uint8))

        def read(off, ln, fd=fd):
            fd.seek(off)
            b = fd.read(ln)
            if len(b) != ln: raise IOError("unexpected end of file")
            return np.frombuffer(b, np.uint8)
        sources.append({"file": os.path.basename(f), "header": hd["header"], "dataStart": hd["dataStart"], "read": read})

    mb = lambda b: f"{b / 1e6:.1f} MB"
    try:
        if DRY:
            total = {}
            for s in sources:
                for t in safetensorsList(s["header"]):
                    enc = chooseEncoding(t["name"], t["shape"], opts); m = matrixOf(t["shape"])
                    e = total.setdefault(enc, {"n": 0, "bytes": 0})
                    e["n"] += 1; e["bytes"] += encodedBytes(enc, m["rows"], m["cols"])
            for enc, e in total.items():
                print(f"{enc:<12} {e['n']:>5} tensors  {mb(e['bytes'])}", file=out)
            return 0

        os.makedirs(OUT, exist_ok=True)
        state = {"fd": None, "n": 0}

        class _Out:
            def begin(self, name): state["fd"] = open(os.path.join(OUT, name), "wb")
            def write(self, b): state["fd"].write(bytes(b))
            def end(self): state["fd"].close(); state["fd"] = None

        t0 = time.time()

        def on_tensor(name, e):
            state["n"] += 1
            if state["n"] % 50 == 0: print(f"{state['n']} tensors, {time.time() - t0:.0f} s", file=out)

        manifest = convert(sources, _Out(), dict(opts, onTensor=on_tensor))
        manifest["created"] = datetime.datetime.now(datetime.timezone.utc).isoformat()
        with open(os.path.join(OUT, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
        by = {}
        for e in manifest["tensors"].values(): by[e["enc"]] = by.get(e["enc"], 0) + 1
        total = sum(sh["bytes"] for sh in manifest["shards"])
        print(f"converted {len(manifest['tensors'])} tensors in {time.time() - t0:.0f} s: {mb(total)} in {len(manifest['shards'])} shard(s); "
              + ", ".join(f"{v} {k}" for k, v in by.items())
              + (f"; skipped {len(manifest['skipped'])} non-float tensors" if manifest["skipped"] else ""), file=out)
        return 0
    finally:
        for fd in handles: fd.close()


if __name__ == "__main__":
    sys.exit(main())
