"""Writes the golden fixtures of this folder.

The reference stores no golden vectors for the gemm path and cannot be run where this project is built (it is
JavaScript; there is no JavaScript engine), so these fixtures come from the CPU oracle (oracle/p0p_oracle.c),
itself pinned on the reference's stored known-answer constants and layout identities (tests/test_oracle.py).
They freeze the oracle: an accidental change to it, or a kernel compared against a drifted oracle, shows up as a
fixture mismatch.  Each fixture restates one of the reference's own test cases (test/kernels.test.js) by seed.

    python tests/golden/make_golden.py          # rewrite every fixture
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def _sha(a) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def gemm_encodings(O):
    """test/kernels.test.js:72-84: M32 N128 K256, seeds 7 / 11 (0.05): encoder bytes (hashed) and fp16 outputs"""
    M, N, K = 32, 128, 256
    X = O.round_f16(O.randn(M * K, 7)); W0 = O.randn(N * K, 11, 0.05)
    b4, d4 = O.pack_q4(W0, N, K); b8, d8 = O.pack_q8(W0, N, K); Wd = O.round_f16(W0)
    return {"x_head": X[:16], "w_head": W0[:16], "q4_sha": _sha(b4), "q8_sha": _sha(b8), "q4_rec0": b4[:1280], "q8_rec0": b8[:4224],
            "y_f16": O.to_f16(O.cpu_gemm(X, Wd, M, N, K)), "y_q4": O.to_f16(O.cpu_gemm(X, d4, M, N, K)), "y_q8": O.to_f16(O.cpu_gemm(X, d8, M, N, K))}


def partial_tiles(O):
    """test/kernels.test.js:85-92: M33 N192 K256, seeds 17 / 19"""
    M, N, K = 33, 192, 256
    X = O.round_f16(O.randn(M * K, 17)); Wd = O.round_f16(O.randn(N * K, 19, 0.05))
    return {"y": O.to_f16(O.cpu_gemm(X, Wd, M, N, K))}


def conv3_clip(O):
    """test/kernels.test.js:95-112: T5 H6 W6 C32 N128, seeds 31 / 33 (0.03)"""
    T, H, W, C, N = 5, 6, 6, 32, 128
    X = O.round_f16(O.randn(T * H * W * C, 31)); Wt = O.round_f16(O.randn(N * 27 * C, 33, 0.03))
    return {"y": O.to_f16(O.cpu_conv3(X, Wt, T, H, W, C, N))}


def fused_variants(O):
    """outputs of the oracle's restatement of the shader arithmetic for the fused cases the reference never tests"""
    import cases as CS
    out = {}
    for name, c in (("rms_swiglu", dict(enc="q4", M=8, N=128, K=128, xmode="rms", epi="swiglu")),
                    ("lnmod_heads", dict(enc="q8", M=8, N=384, K=128, xmode="lnmod", epi="heads", heads=dict(Ltot=8, Hq=1, Hkv=1, rowOff=0, eps=1e-6))),
                    ("resadd_gate", dict(enc="q4", M=8, N=128, K=128, epi="resadd", gate=True))):
        y = CS.run_oracle(CS.build(c))
        out[name] = y.view(np.uint32) if y.dtype == np.float32 else y
    return out


CASES = {"gemm_encodings": gemm_encodings, "partial_tiles": partial_tiles, "conv3_clip": conv3_clip, "fused_variants": fused_variants}

if __name__ == "__main__":
    import oracle as O
    O.build()
    for name, fn in CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **fn(O))
        print("wrote", name)
