"""The producers of the statistics gemm's fused prologues read, CUDA against the CPU oracle: pixstats (src/ops/video.js:301-318),
gnPartial / gnFinalize (src/ops/misc.js:50-120); then the two fused prologues fed by them instead of by host-computed vectors:
conv3 with PixelNorm (`pn`) and the 2-D convolution with GroupNorm (`gn`).  fp32 statistics: relative tolerance 1e-5 (the
summation order differs from the shader's; both are fp32 sums of a few thousand terms)."""
import numpy as np
import pytest

import cases as CS

pytestmark = pytest.mark.gpu


def P():
    import p0pc0rn_kernels_b200 as P_
    return P_


@pytest.mark.parametrize("V,C", [(90, 32), (1000, 128), (4097, 64), (33, 512), (50, 36)])
def test_pixstats(gpu, oracle, V, C):
    O = oracle
    X = O.to_f16(O.randn(V * C, 3) * 1.5 + 0.25)
    xb, rb = gpu.upload(X), gpu.upload(np.full(V + 5, 7.0, np.float32))
    try:
        P().pixstats(gpu, {"x": {"buf": xb}, "V": V, "C": C, "eps": 1e-8, "r": {"buf": rb}, "ro": 3})
        got = gpu.read(rb, 0, (V + 5) * 4).view(np.float32)
        assert (got[:3] == 7.0).all() and (got[3 + V:] == 7.0).all(), "words outside [ro, ro + V) were written"
        np.testing.assert_allclose(got[3:3 + V], O.pixstats(X, V, C, 1e-8), rtol=1e-5)
    finally:
        for b in (xb, rb): gpu.free(b)


@pytest.mark.parametrize("pix,C", [(64, 32), (100, 64), (1000, 128), (14720, 128), (200, 512), (129, 256)])
def test_groupnorm_stats(gpu, oracle, pix, C):
    O = oracle
    X = O.to_f16(O.randn(pix * C, 5) * 2.0 + np.tile(np.linspace(-1, 1, C, dtype=np.float32), pix))
    gamma, beta = (1.0 + O.randn(C, 6, 0.2)).astype(np.float32), O.randn(C, 7, 0.3)
    xb = gpu.upload(X); part = gpu.buffer(P().gnPartBytes(pix)); gb = gpu.upload(np.concatenate([gamma, beta])); ab = gpu.buffer((2 * C + 4) * 4)
    try:
        nwg = P().gnPartial(gpu, {"x": {"buf": xb}, "pix": pix, "C": C, "part": part})
        assert nwg == -(-pix // 64)
        pt = gpu.read(part, 0, nwg * 512).view(np.float32)
        want_pt = O.gn_partial(X, pix, C)
        np.testing.assert_allclose(pt, want_pt, rtol=2e-5, atol=2e-5)
        P().gnFinalize(gpu, {"part": part, "nwg": nwg, "C": C, "eps": 1e-6, "gb": {"buf": gb, "gOff": 0, "bOff": C * 4}, "ab": {"buf": ab, "off": 4}})
        got = gpu.read(ab, 16, 2 * C * 4).view(np.float32)
        np.testing.assert_allclose(got, O.gn_finalize(want_pt, nwg, C, gamma, beta, 1e-6), rtol=2e-5, atol=2e-5)
        # the statistics are those of the whole tensor (float64 reference), whatever the chunking
        xf = O.from_f16(X).astype(np.float64).reshape(pix, 32, C // 32)
        mean, var = xf.mean((0, 2)), xf.var((0, 2))
        a = np.repeat(1.0 / np.sqrt(var + 1e-6), C // 32) * gamma
        np.testing.assert_allclose(got[:C], a, rtol=1e-4)
        np.testing.assert_allclose(got[C:], beta - np.repeat(mean, C // 32) * a, rtol=1e-4, atol=1e-4)
    finally:
        for b in (xb, part, gb, ab): gpu.free(b)


def test_groupnorm_partials_of_separate_calls_merge(gpu, oracle):
    """two bands of an image written to consecutive partial rows (wgOff) give the statistics of the whole image (src/ops/misc.js:52-53)"""
    O = oracle
    pix, C = 640, 64
    X = O.to_f16(O.randn(pix * C, 9))
    xb = gpu.upload(X); part = gpu.buffer(P().gnPartBytes(pix)); part2 = gpu.buffer(P().gnPartBytes(pix))
    try:
        n = P().gnPartial(gpu, {"x": {"buf": xb}, "pix": pix, "C": C, "part": part})
        n1 = P().gnPartial(gpu, {"x": {"buf": xb}, "pix": 256, "C": C, "part": part2})
        n2 = P().gnPartial(gpu, {"x": {"buf": xb, "off": 256 * C * 2}, "pix": pix - 256, "C": C, "part": part2, "wgOff": n1})
        assert n1 + n2 == n
        assert np.array_equal(gpu.read(part, 0, n * 512), gpu.read(part2, 0, n * 512))
    finally:
        for b in (xb, part, part2): gpu.free(b)


@pytest.mark.parametrize("kernel", [None, "generic"])
def test_conv3_pixelnorm_from_pixstats(gpu, oracle, kernel):
    """conv3 with the fused PixelNorm + SiLU, its `stats` produced by pixstats on the GPU"""
    O = oracle
    c = dict(name="conv3 pn", enc="f16", M=3 * 5 * 6, N=64, K=27 * 32, x_elems=3 * 5 * 6 * 32, w_scale=0.03, epi="bias", kernel=kernel,
             conv=dict(kind="conv3", Hi=5, Wi=6, Ci=32, Ho=5, Wo=6, stride=3, padT=0, padL=0, ks=1, pn=True))
    h = CS.build(c)
    V = 3 * 5 * 6
    xb, rb = gpu.upload(h["X"]), gpu.buffer(V * 4)
    try:
        P().pixstats(gpu, {"x": {"buf": xb}, "V": V, "C": 32, "eps": 1e-6, "r": {"buf": rb}})
        st = gpu.read(rb, 0, V * 4).view(np.float32).copy()
    finally:
        for b in (xb, rb): gpu.free(b)
    np.testing.assert_allclose(st, h["ST"], rtol=1e-5)
    h["ST"] = st                                   # the GPU's own statistics feed both the kernel and the oracle
    CS.check(CS.run_gpu(gpu, h), CS.run_oracle(h), "conv3 pn from pixstats")


@pytest.mark.parametrize("Ci,kernel", [(32, None), (64, None), (64, "generic")])
def test_conv_groupnorm_from_gn_stats(gpu, oracle, Ci, kernel):
    """2-D convolution with the fused GroupNorm-apply + SiLU, its (a, b) produced by gnPartial + gnFinalize on the GPU"""
    O = oracle
    Hh = 16
    c = dict(name="conv gn", enc="f16", M=Hh * Hh, N=64, K=9 * Ci, x_elems=Hh * Hh * Ci, w_scale=0.03, epi="bias", kernel=kernel,
             conv=dict(kind="conv", Hi=Hh, Wi=Hh, Ci=Ci, Ho=Hh, Wo=Hh, stride=1, padT=1, padL=1, ks=3, gn=True))
    h = CS.build(c)
    gamma, beta = (1.0 + O.randn(Ci, 6, 0.2)).astype(np.float32), O.randn(Ci, 7, 0.3)
    pix = Hh * Hh
    xb = gpu.upload(h["X"]); part = gpu.buffer(P().gnPartBytes(pix)); gb = gpu.upload(np.concatenate([gamma, beta])); ab = gpu.buffer(2 * Ci * 4)
    try:
        P().groupnormStats(gpu, {"x": {"buf": xb}, "pix": pix, "C": Ci, "part": part, "gb": {"buf": gb, "gOff": 0, "bOff": Ci * 4}, "ab": {"buf": ab}, "eps": 1e-6})
        pv = gpu.read(ab, 0, 2 * Ci * 4).view(np.float32).copy()
    finally:
        for b in (xb, part, gb, ab): gpu.free(b)
    h["PV"] = pv; h["pv_stride"] = Ci
    CS.check(CS.run_gpu(gpu, h), CS.run_oracle(h), "conv gn from groupnormStats")
