"""Builds the native library of this package in-tree: ``libp0p.so`` (CUDA kernels for sm_100a + the C ABI of
``include/p0p.h``).  nvcc cross-compiles without a GPU.

    python p0pc0rn_kernels_b200/build.py [--force]

Each source file is compiled to an object under ``build/`` (in parallel), then the objects are linked.  Run it as a
script (or load it by path): importing the package needs the library this builds."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libp0p.so")
SOURCES = ["runtime.cu", "gemm.cu", "decode.cu", "umma_q4.cu", "umma_q8.cu", "umma_f16.cu", "decode_finish.cu", "attn.cu", "stats.cu", "peer.cu", "noalloc.cu", "host_codec.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=default,-ffp-contract=off", "-Xptxas", "-v"]


def _headers() -> list[str]:
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [os.path.join(HERE, "..", "include", "p0p.h")]


def _obj(src: str) -> str:
    return os.path.join(OBJ, os.path.splitext(src)[0] + ".o")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def stale() -> bool:
    return _stale(LIB, [os.path.join(CSRC, s) for s in SOURCES] + _headers())


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None, lib: str | None = None) -> str:
    """Compile libp0p.so if it is missing or older than its sources; returns its path.  ``extra_flags`` (e.g. ``-D`` switches)
    and ``lib`` build a variant next to the regular library, with objects of its own."""
    out = lib or LIB
    objdir = OBJ if lib is None else os.path.splitext(lib)[0] + "_obj"
    if not force and lib is None and not stale():
        return out
    os.makedirs(objdir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    heads = _headers()
    logs: dict[str, str] = {}

    def compile_one(src: str):
        path, obj = os.path.join(CSRC, src), os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        if not force and not _stale(obj, [path] + heads):
            return obj, 0
        cmd = [nvcc, *NVCC_FLAGS, *(extra_flags or []), "-c", "-o", obj, path]
        r = subprocess.run(cmd, capture_output=True, text=True)
        logs[src] = " ".join(cmd) + "\n" + r.stdout + r.stderr
        return obj, r.returncode

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, SOURCES))
    log = "\n".join(logs[s] for s in SOURCES if s in logs)
    with open(os.path.join(objdir, "build.log"), "w") as f:
        f.write(log)
    if any(rc for _, rc in results):
        sys.stderr.write(log)
        raise RuntimeError("nvcc failed building libp0p.so")
    link = [nvcc, "-shared", "-o", out, *[o for o, _ in results]]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed linking libp0p.so")
    if verbose:
        print(log)
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
