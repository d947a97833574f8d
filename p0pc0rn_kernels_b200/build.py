"""Builds the native library of this package in-tree: ``libp0p.so`` (CUDA kernels for sm_100a + the C ABI of
``include/p0p.h``).  nvcc cross-compiles without a GPU.

    python p0pc0rn_kernels_b200/build.py [--force]

Run it as a script (or load it by path): importing the package needs the library this builds."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libp0p.so")
SOURCES = ["runtime.cu", "gemm.cu", "attn.cu", "noalloc.cu", "host_codec.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC,-fvisibility=default,-ffp-contract=off", "-Xptxas", "-v"]


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES]


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "p0p.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile libp0p.so if it is missing or older than its sources; returns its path."""
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB, *sources()]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    with open(os.path.join(HERE, "build.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if r.returncode != 0:
        sys.stderr.write(log)
        raise RuntimeError("nvcc failed building libp0p.so")
    if verbose:
        print(log)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
