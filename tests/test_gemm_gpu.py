"""Parity of the CUDA gemm path with the CPU oracle, through the public API (C ABI underneath).

The first block restates the reference's own GEMM-family tests one for one (test/kernels.test.js:72-145,
198-221): same shapes, seeds, generators and pass criterion, plus the tighter gates of tests/cases.py.  The
second block covers what the reference's tests leave out: every fused prologue and epilogue and the sub-range
arguments, against the oracle's restatement of the shader arithmetic (src/ops/gemm.js:60-101, 191-254)."""
import numpy as np
import pytest

import cases as CS

pytestmark = pytest.mark.gpu

KERNELS = [None, "generic"]   # None = the library's own choice


def P():
    import p0pc0rn_kernels_b200 as P_
    return P_


# ------------------------------------------------------------------------------------------------ reference cases
@pytest.mark.parametrize("acc", ["f32", "f16"])
@pytest.mark.parametrize("enc", ["f16", "q4g32a.t64", "q8g64s.t64"])
@pytest.mark.parametrize("kernel", KERNELS)
def test_ref_gemm_encodings(gpu, oracle, enc, acc, kernel):
    """GEMM, three weight encodings x two accumulate modes: M32 N128 K256, seeds 7 / 11 (0.05) (test/kernels.test.js:72-84)"""
    O = oracle
    M, N, K = 32, 128, 256
    X = O.round_f16(O.randn(M * K, 7)); W0 = O.randn(N * K, 11, 0.05)
    Wb, Wd = CS.encode(enc, W0, N, K)
    wb, xb, yb = gpu.upload(Wb), gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        a = {"w": {"enc": enc, "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K, "acc": acc}
        if kernel: a["kernel"] = kernel
        P().gemm(gpu, a)
        got = P().fromF16(gpu.read(yb, 0, M * N * 2).view(np.uint16))
        want = O.cpu_gemm(X, Wd, M, N, K)
        cos, _ = O.compare(got, want)
        assert cos > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), f"gemm {enc}")
    finally:
        for b in (wb, xb, yb): gpu.free(b)


@pytest.mark.parametrize("kernel", KERNELS)
def test_ref_partial_tiles(gpu, oracle, kernel):
    """GEMM, partial tiles M33 N192 K256 f16, seeds 17 / 19 (test/kernels.test.js:85-92)"""
    O = oracle
    M, N, K = 33, 192, 256
    X = O.round_f16(O.randn(M * K, 17)); Wd = O.round_f16(O.randn(N * K, 19, 0.05))
    wb, xb, yb = gpu.upload(P().toF16(Wd)), gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        a = {"w": {"enc": "f16", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K}
        if kernel: a["kernel"] = kernel
        P().gemm(gpu, a)
        got = P().fromF16(gpu.read(yb, 0, M * N * 2).view(np.uint16))
        want = O.cpu_gemm(X, Wd, M, N, K)
        assert O.compare(got, want)[0] > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), "partial tiles")
    finally:
        for b in (wb, xb, yb): gpu.free(b)


C3 = {"T": 5, "H": 6, "W": 6, "C": 32, "N": 128}   # test/kernels.test.js:95


def conv3_setup(gpu, O, seed_x=31, seed_w=33):
    T, H, W, C, N = (C3[k] for k in "THWCN")
    X = O.round_f16(O.randn(T * H * W * C, seed_x)); Wt = O.round_f16(O.randn(N * 27 * C, seed_w, 0.03))
    return {"X": X, "Wt": Wt, "xb": gpu.upload(P().toF16(X)), "wb": gpu.upload(P().toF16(Wt))}


def conv3(gpu, s, x, y, t0, nf, padL=0, ks=1, tile=None, kernel=None):
    """output frames [t0, t0 + nf) of the clip (test/kernels.test.js:101-105)"""
    T, H, W, C, N = (C3[k] for k in "THWCN")
    a = {"w": {"enc": "f16", "buf": s["wb"], "off": 0, "bytes": s["wb"]._pf, "rows": N, "cols": 27 * C}, "x": x, "y": y, "M": nf * H * W, "N": N, "K": 27 * C,
         "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": t0, "padL": padL, "ks": ks}}
    if tile: a["tile"] = tile
    if kernel: a["kernel"] = kernel
    P().gemm(gpu, a)


@pytest.mark.parametrize("tile", [None, {"BM": 128, "BN": 128}, {"BM": 64, "BN": 64}, {"BM": 32, "BN": 128}, {"BM": 128, "BN": 64}])
@pytest.mark.parametrize("kernel", KERNELS)
def test_ref_conv3(gpu, oracle, tile, kernel):
    """3x3x3 convolution over a THWC clip, and at the tiles the tuning table can pick (test/kernels.test.js:106-122)"""
    O = oracle
    T, H, W, C, N = (C3[k] for k in "THWCN")
    s = conv3_setup(gpu, O); yb = gpu.buffer(T * H * W * N * 2)
    try:
        conv3(gpu, s, {"buf": s["xb"]}, {"buf": yb}, 0, T, tile=tile, kernel=kernel)
        got = P().fromF16(gpu.read(yb, 0, T * H * W * N * 2).view(np.uint16))
        want = O.cpu_conv3(s["X"], s["Wt"], T, H, W, C, N)
        assert O.compare(got, want)[0] > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), "conv3")
    finally:
        for b in (s["xb"], s["wb"], yb): gpu.free(b)


@pytest.mark.parametrize("kernel", KERNELS)
def test_ref_conv3_chunks_bit_identical(gpu, oracle, kernel):
    """conv3 in time chunks of 2 frames = the whole clip, bit for bit (test/kernels.test.js:123-131)"""
    O = oracle
    T, H, W, C, N = (C3[k] for k in "THWCN")
    s = conv3_setup(gpu, O); n = T * H * W * N
    ya, yb = gpu.buffer(n * 2), gpu.buffer(n * 2); fx, fy = H * W * C * 2, H * W * N * 2
    try:
        conv3(gpu, s, {"buf": s["xb"]}, {"buf": ya}, 0, T, kernel=kernel)
        for t0 in range(0, T, 2):
            padL = max(0, t0 - 1)
            conv3(gpu, s, {"buf": s["xb"], "off": padL * fx}, {"buf": yb, "off": t0 * fy}, t0, min(2, T - t0), padL, kernel=kernel)
        a, b = gpu.read(ya, 0, n * 2).view(np.uint16), gpu.read(yb, 0, n * 2).view(np.uint16)
        assert np.array_equal(a, b), "chunked conv3 DIFFERS from the whole clip"
    finally:
        for x in (s["xb"], s["wb"], ya, yb): gpu.free(x)


@pytest.mark.parametrize("kernel", KERNELS)
def test_ref_conv3_ring_bit_identical(gpu, oracle, kernel):
    """conv3 from a ring of 3 frames = the whole clip, bit for bit (test/kernels.test.js:132-145)"""
    O = oracle
    T, H, W, C, N = (C3[k] for k in "THWCN")
    s = conv3_setup(gpu, O); n = T * H * W * N
    ya, yb = gpu.buffer(n * 2), gpu.buffer(n * 2); fx, fy = H * W * C, H * W * N * 2
    ring = gpu.buffer(3 * fx * 2); X16 = P().toF16(s["X"])
    try:
        conv3(gpu, s, {"buf": s["xb"]}, {"buf": ya}, 0, T, kernel=kernel)
        for t in range(T):
            for g in sorted({max(0, t - 1), t, min(T - 1, t + 1)}):
                gpu.device.queue.writeBuffer(ring, (g % 3) * fx * 2, X16, g * fx, fx)
            conv3(gpu, s, {"buf": ring}, {"buf": yb, "off": t * fy}, t, 1, 0, 3, kernel=kernel)
            gpu.done()   # the ring is rewritten for the next frame
        a, b = gpu.read(ya, 0, n * 2).view(np.uint16), gpu.read(yb, 0, n * 2).view(np.uint16)
        assert np.array_equal(a, b), "ring conv3 DIFFERS from the whole clip"
    finally:
        for x in (s["xb"], s["wb"], ya, yb, ring): gpu.free(x)


# ---- conv3 on the tensor-core kernel: clips whose channel count lets a 64-k step stay inside one tap ---------------------
TC_CLIPS = [
    dict(name="128-token tiles, fp16 weights", T=5, H=8, W=16, C=64, N=128, enc="f16"),
    dict(name="384-token tiles (two multiplies per step), fp16 weights, bias", T=4, H=8, W=48, C=64, N=128, enc="f16", bias=True),
    dict(name="q4 weights (operand in tensor memory), 256 output channels", T=4, H=4, W=32, C=128, N=256, enc="q4"),
    dict(name="q8 weights, 320-token tiles", T=3, H=4, W=80, C=64, N=128, enc="q8"),
]


@pytest.mark.gpu
@pytest.mark.parametrize("clip", TC_CLIPS, ids=[c["name"] for c in TC_CLIPS])
def test_conv3_tensor_core(gpu, oracle, clip):
    """conv3 through the tcgen05 kernel (the clip read by 4-D tensor-map boxes, zero padding from the out-of-range fill):
    against the CPU convolution, and whole clip == 2-frame chunks == ring of 3 frames bit for bit"""
    O = oracle
    T, H, W, C, N, enc = (clip[k] for k in ("T", "H", "W", "C", "N", "enc"))
    K = 27 * C
    X = O.round_f16(O.randn(T * H * W * C, 131)); W0 = O.randn(N * K, 133, 0.03)
    if enc == "f16": Wref = O.round_f16(W0); wbytes = P().toF16(Wref); encn = "f16"
    elif enc == "q4": wbytes, Wref = O.pack_q4(W0, N, K); encn = "q4g32a.t64"
    else: wbytes, Wref = O.pack_q8(W0, N, K); encn = "q8g64s.t64"
    bias = O.randn(N, 135, 0.1) if clip.get("bias") else None
    xb, wb = gpu.upload(P().toF16(X)), gpu.upload(wbytes)
    n = T * H * W * N; fx, fy = H * W * C, H * W * N * 2
    ya, yb, yc, ring = gpu.buffer(n * 2), gpu.buffer(n * 2), gpu.buffer(n * 2), gpu.buffer(3 * fx * 2)
    bb = gpu.upload(bias) if bias is not None else None
    X16 = P().toF16(X)

    def run(x, y, t0, nf, padL=0, ks=1):
        a = {"w": {"enc": encn, "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": x, "y": y, "M": nf * H * W, "N": N, "K": K,
             "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": t0, "padL": padL, "ks": ks}}
        if bb is not None: a["epi"] = "bias"; a["ev"] = {"buf": bb}
        P().gemm(gpu, a)
        assert P()._lib.KERNEL_NAMES.get(gpu.lastKernel) == "umma", "conv3 did not take the tensor-core kernel"

    try:
        run({"buf": xb}, {"buf": ya}, 0, T)
        got = P().fromF16(gpu.read(ya, 0, n * 2).view(np.uint16))
        want = O.cpu_conv3(X, Wref, T, H, W, C, N)
        if bias is not None: want = (want.reshape(-1, N) + bias[None, :]).astype(np.float32).ravel()
        assert O.compare(got, want)[0] > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), "conv3 tensor core")
        for t0 in range(0, T, 2):
            padL = max(0, t0 - 1)
            run({"buf": xb, "off": padL * fx * 2}, {"buf": yb, "off": t0 * fy}, t0, min(2, T - t0), padL)
        for t in range(T):
            for g in sorted({max(0, t - 1), t, min(T - 1, t + 1)}):
                gpu.device.queue.writeBuffer(ring, (g % 3) * fx * 2, X16, g * fx, fx)
            run({"buf": ring}, {"buf": yc, "off": t * fy}, t, 1, 0, 3)
            gpu.done()
        a, b, c = (gpu.read(y, 0, n * 2).view(np.uint16) for y in (ya, yb, yc))
        assert np.array_equal(a, b), "chunked conv3 DIFFERS from the whole clip"
        assert np.array_equal(a, c), "ring conv3 DIFFERS from the whole clip"
    finally:
        for x in (xb, wb, ya, yb, yc, ring, bb):
            if x is not None: gpu.free(x)


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("clip", [dict(T=5, H=6, W=6, C=32, N=128), dict(T=6, H=8, W=16, C=64, N=128)], ids=["general kernel", "tensor-core kernel"])
def test_conv3_split_by_frames_is_the_whole_clip(gpu, oracle, clip, world):
    """the multi-GPU form of conv3: every rank's frame range (run here one after the other on one GPU) writes the bits of the
    whole-clip call"""
    O = oracle
    T, H, W, C, N = (clip[k] for k in "THWCN")
    X = O.round_f16(O.randn(T * H * W * C, 31)); Wt = O.round_f16(O.randn(N * 27 * C, 33, 0.03)); bias = O.randn(N, 35, 0.1)
    xb, wb, bb = gpu.upload(P().toF16(X)), gpu.upload(P().toF16(Wt)), gpu.upload(bias)
    n = T * H * W * N
    ya, yb = gpu.buffer(n * 2), gpu.upload(np.full(n, 0xFFFF, np.uint16))
    whole = {"w": {"enc": "f16", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": 27 * C}, "x": {"buf": xb}, "y": {"buf": ya}, "M": T * H * W, "N": N, "K": 27 * C,
             "epi": "bias", "ev": {"buf": bb}, "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": 0, "padL": 0, "ks": 1}}
    try:
        P().gemm(gpu, whole)
        for r in range(world):
            a = P().conv3_frame_shard(dict(whole, y={"buf": yb}), r, world)
            if a is not None: P().gemm(gpu, a)
        a_, b_ = gpu.read(ya, 0, n * 2).view(np.uint16), gpu.read(yb, 0, n * 2).view(np.uint16)
        assert np.array_equal(a_, b_), "the frame shards DIFFER from the whole clip"
    finally:
        for b in (xb, wb, bb, ya, yb): gpu.free(b)


def test_ref_converted_bf16_linear_q4(gpu, oracle):
    """a BF16 linear layer, converted to 4-bit, through the GEMM (test/kernels.test.js:198-209)"""
    O = oracle
    M, N, K = 32, 192, 512
    Wb16 = O.to_bf16(O.randn(N * K, 81, 0.05)); X = O.round_f16(O.randn(M * K, 83))
    file = P().writeSafetensors({"layers.0.mlp.up_proj.weight": {"dtype": "BF16", "shape": [N, K], "data": Wb16.view(np.uint8)}})
    r = P().convertSafetensors(file, {"bits": 4}); model = P().uploadWeights(gpu, r["manifest"], r["shards"])
    w = model.tensor("layers.0.mlp.up_proj.weight")
    _, deq = O.pack_q4(O.from_bf16(Wb16), N, K)
    xb, yb = gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        assert w["enc"] == "q4g32a.t64"
        P().gemm(gpu, {"w": w, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K})
        got = P().fromF16(gpu.read(yb, 0, M * N * 2).view(np.uint16)); want = O.cpu_gemm(X, deq, M, N, K)
        assert O.compare(got, want)[0] > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), "converted q4")
    finally:
        model.free(); gpu.free(xb); gpu.free(yb)


def test_ref_converted_conv3_weight(gpu, oracle):
    """a 3x3x3 conv weight in PyTorch layout [O, I, kt, kh, kw] through the 3D convolution (test/kernels.test.js:210-221)"""
    O = oracle
    T, H, W, C, N = (C3[k] for k in "THWCN")
    src = O.round_f16(O.randn(N * C * 27, 87, 0.03)); X = O.round_f16(O.randn(T * H * W * C, 89))
    file = P().writeSafetensors({"decoder.conv.weight": {"dtype": "F16", "shape": [N, C, 3, 3, 3], "data": P().toF16(src).view(np.uint8)}})
    r = P().convertSafetensors(file, {"bits": 16}); model = P().uploadWeights(gpu, r["manifest"], r["shards"]); w = model.tensor("decoder.conv.weight")
    ref = src.reshape(N, C, 27).transpose(0, 2, 1).reshape(-1).copy()   # ref[n][tap][c] = src[n][c][tap]
    xb, yb = gpu.upload(P().toF16(X)), gpu.buffer(T * H * W * N * 2)
    try:
        P().gemm(gpu, {"w": w, "x": {"buf": xb}, "y": {"buf": yb}, "M": T * H * W, "N": N, "K": 27 * C,
                       "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": 0, "padL": 0, "ks": 1}})
        got = P().fromF16(gpu.read(yb, 0, T * H * W * N * 2).view(np.uint16)); want = O.cpu_conv3(X, ref, T, H, W, C, N)
        assert O.compare(got, want)[0] > 0.9995
        CS.check(P().toF16(got), O.to_f16(want), "converted conv3")
    finally:
        model.free(); gpu.free(xb); gpu.free(yb)


def test_readme_quick_start(gpu):
    """README.md:52-63: 0.5 x 0.01 over K = 512 is about 2.56 everywhere"""
    M, N, K = 64, 256, 512
    x = gpu.upload(P().toF16(np.full(M * K, 0.5, np.float32))); w = gpu.upload(P().toF16(np.full(N * K, 0.01, np.float32))); y = gpu.buffer(M * N * 2)
    try:
        P().gemm(gpu, {"w": {"enc": "f16", "buf": w, "off": 0, "bytes": N * K * 2, "rows": N, "cols": K}, "x": {"buf": x}, "y": {"buf": y}, "M": M, "N": N, "K": K})
        out = P().fromF16(gpu.read(y, 0, M * N * 2).view(np.uint16))
        assert np.allclose(out, 2.56, atol=5e-3)
    finally:
        for b in (x, w, y): gpu.free(b)


# ------------------------------------------------------------------------------------------------ beyond the reference's tests
HEADS = {"Ltot": 80, "Hq": 2, "Hkv": 1, "rowOff": 8, "eps": 1e-6}
EXTRA = [
    dict(name="f32 store", enc="q4", M=40, N=128, K=256, epi="f32"),
    dict(name="resadd plain", enc="q4", M=40, N=192, K=256, epi="resadd"),
    dict(name="resadd gate+bias", enc="q8", M=40, N=192, K=256, epi="resadd", gate=True, bias=True, ev_off=8, bv_off=4),
    dict(name="resadd store", enc="f16", M=40, N=128, K=256, epi="resadd", gate=True, store=True),
    dict(name="swiglu", enc="q4", M=40, N=256, K=256, epi="swiglu"),
    dict(name="swiglu bias rows", enc="q4", M=40, N=256, K=256, epi="swiglu", bias=True, wr0=64, wr1=256, w_rows=448),
    dict(name="geglu", enc="q8", M=24, N=256, K=256, epi="swiglu", act="gelu"),
    dict(name="bias", enc="f16", M=40, N=128, K=256, epi="bias", ev_off=16),
    dict(name="bias+res", enc="q4", M=40, N=128, K=256, epi="bias", res=True),
    dict(name="heads interleaved", enc="q8", M=40, N=512, K=256, epi="heads", heads=dict(HEADS)),
    dict(name="heads half", enc="q4", M=40, N=512, K=256, epi="heads", heads=dict(HEADS, ropeMode="half")),
    dict(name="onormgate", enc="q4", M=24, N=256, K=256, epi="onormgate", Ltot=256),
    dict(name="rms", enc="q4", M=40, N=128, K=256, xmode="rms", st_off=3, pv_off=8),
    dict(name="lnmod", enc="q8", M=40, N=128, K=256, xmode="lnmod", x_shift=0.7),
    dict(name="rms+swiglu", enc="q4", M=40, N=256, K=512, xmode="rms", epi="swiglu"),
    dict(name="lnmod+heads", enc="q8", M=40, N=384, K=256, xmode="lnmod", epi="heads", heads=dict(Ltot=40, Hq=1, Hkv=1, rowOff=0, eps=1e-6)),
    dict(name="sub-ranges", enc="q4", M=20, N=128, K=128, ldx=320, kx0=64, wk0=128, w_cols=384, wr0=64, w_rows=256, ldy=200, ny0=40),
    dict(name="sub-ranges f16 ld", enc="f16", M=20, N=128, K=128, ldx=320, kx0=64, wk0=128, w_cols=256, w_ld=264, wr0=3, w_rows=140, ldy=200, ny0=40),
    dict(name="byte offsets", enc="q8", M=20, N=128, K=128, x_off=256, w_off=512, y_off=768),
    dict(name="M=1", enc="q4", M=1, N=256, K=512),
    dict(name="M=16 q8", enc="q8", M=16, N=256, K=512),
    dict(name="tail columns", enc="f16", M=17, N=100, K=96, w_rows=100),
]
CONV = [
    dict(name="conv3x3", enc="f16", M=8 * 8, N=64, K=9 * 32, x_elems=8 * 8 * 32, w_scale=0.03,
         conv=dict(kind="conv", Hi=8, Wi=8, Ci=32, Ho=8, Wo=8, stride=1, padT=1, padL=1, ks=3)),
    dict(name="conv3x3 stride2", enc="f16", M=4 * 4, N=64, K=9 * 32, x_elems=8 * 8 * 32, w_scale=0.03,
         conv=dict(kind="conv", Hi=8, Wi=8, Ci=32, Ho=4, Wo=4, stride=2, padT=1, padL=1, ks=3)),
    dict(name="conv1x1", enc="q4", M=8 * 8, N=64, K=64, x_elems=8 * 8 * 64, conv=dict(kind="conv", Hi=8, Wi=8, Ci=64, Ho=8, Wo=8, stride=1, padT=0, padL=0, ks=1)),
    dict(name="conv up2+gn", enc="f16", M=16 * 16, N=64, K=9 * 32, x_elems=8 * 8 * 32, w_scale=0.03, epi="bias",
         conv=dict(kind="conv", Hi=8, Wi=8, Ci=32, Ho=16, Wo=16, stride=1, padT=1, padL=1, ks=3, up2=True, gn=True)),
    dict(name="conv3 pn", enc="f16", M=3 * 5 * 6, N=64, K=27 * 32, x_elems=3 * 5 * 6 * 32, w_scale=0.03, epi="bias",
         conv=dict(kind="conv3", Hi=5, Wi=6, Ci=32, Ho=5, Wo=6, stride=3, padT=0, padL=0, ks=1, pn=True)),
]
# 2-D convolutions the tensor-core kernel takes (Ci % 64 == 0, whole tiles of whole output rows): the image read by tensor-map
# boxes whose element strides are the convolution's stride, zero padding from the out-of-range fill
CONV_TC = [
    dict(name="tc conv3x3 c64 f16", enc="f16", M=16 * 16, N=128, K=9 * 64, x_elems=16 * 16 * 64, w_scale=0.03, epi="bias",
         conv=dict(kind="conv", Hi=16, Wi=16, Ci=64, Ho=16, Wo=16, stride=1, padT=1, padL=1, ks=3)),
    dict(name="tc conv3x3 stride2 c64 q4", enc="q4", M=8 * 8, N=128, K=9 * 64, x_elems=16 * 16 * 64,
         conv=dict(kind="conv", Hi=16, Wi=16, Ci=64, Ho=8, Wo=8, stride=2, padT=1, padL=1, ks=3)),
    dict(name="tc conv1x1 c128 q8", enc="q8", M=16 * 24, N=192, K=128, x_elems=16 * 24 * 128, epi="f32",
         conv=dict(kind="conv", Hi=16, Wi=24, Ci=128, Ho=16, Wo=24, stride=1, padT=0, padL=0, ks=1)),
    dict(name="tc conv5x5 pad2 c64 q8 wide image", enc="q8", M=12 * 40, N=64, K=25 * 64, x_elems=12 * 40 * 64,
         conv=dict(kind="conv", Hi=12, Wi=40, Ci=64, Ho=12, Wo=40, stride=1, padT=2, padL=2, ks=5)),
    dict(name="tc conv3x3 gn c64 f16", enc="f16", M=16 * 16, N=64, K=9 * 64, x_elems=16 * 16 * 64, w_scale=0.03, epi="bias",
         conv=dict(kind="conv", Hi=16, Wi=16, Ci=64, Ho=16, Wo=16, stride=1, padT=1, padL=1, ks=3, gn=True)),
    dict(name="tc conv3x3 stride2 unpadded c128 f16", enc="f16", M=8 * 8, N=128, K=9 * 128, x_elems=17 * 17 * 128, w_scale=0.03,
         conv=dict(kind="conv", Hi=17, Wi=17, Ci=128, Ho=8, Wo=8, stride=2, padT=0, padL=0, ks=3)),
    dict(name="tc conv3x3 c64 q4 320 tokens per tile", enc="q4", M=32 * 40, N=256, K=9 * 64, x_elems=32 * 40 * 64, epi="bias", res=True,
         conv=dict(kind="conv", Hi=32, Wi=40, Ci=64, Ho=32, Wo=40, stride=1, padT=1, padL=1, ks=3)),
]


@pytest.mark.parametrize("case", CONV_TC, ids=lambda c: c["name"])
def test_conv_tensor_core(gpu, oracle, case):
    """the 2-D implicit-GEMM convolution on the tcgen05 kernel, against the oracle, and equal in kind to the CUDA-core kernel"""
    h = CS.build(dict(case))
    got = CS.run_gpu(gpu, h)
    assert P()._lib.KERNEL_NAMES.get(gpu.lastKernel) == "umma", "the convolution did not take the tensor-core kernel"
    want = CS.run_oracle(h)
    CS.check(got, want, case["name"])
    CS.check(CS.run_gpu(gpu, CS.build(dict(case, kernel="generic"))), want, case["name"] + " (generic)")


@pytest.mark.parametrize("case", EXTRA + CONV, ids=lambda c: c["name"])
@pytest.mark.parametrize("kernel", KERNELS + ["umma"])
def test_fused_variants(gpu, oracle, case, kernel):
    h = CS.build(dict(case, kernel=kernel))
    try:
        got = CS.run_gpu(gpu, h)
    except ValueError as e:
        if kernel == "umma" and "does not take" in str(e):
            pytest.skip("outside the tensor-core kernel's conditions")
        raise
    want = CS.run_oracle(h)
    CS.check(got, want, case["name"])


UMMA = [
    dict(name="u q4 M300", enc="q4", M=300, N=384, K=512),
    dict(name="u q8 M520 3 token tiles", enc="q8", M=520, N=256, K=1024),
    dict(name="u f16 M200 ld", enc="f16", M=200, N=320, K=448, w_ld=456, w_cols=456, wr0=5, w_rows=330),
    dict(name="u q4 M17", enc="q4", M=17, N=256, K=256),
    dict(name="u split-K q4 M64 K4096", enc="q4", M=64, N=256, K=4096),
    dict(name="u split-K q8 M300 resadd", enc="q8", M=300, N=128, K=2048, epi="resadd"),
    dict(name="u split-K lnmod+heads", enc="q8", M=100, N=384, K=1536, xmode="lnmod", epi="heads", heads=dict(Ltot=128, Hq=1, Hkv=1, rowOff=7, eps=1e-6)),
    dict(name="u split-K rms+swiglu bias", enc="q4", M=40, N=512, K=2048, xmode="rms", epi="swiglu", bias=True),
    dict(name="u split-K f16 weights ragged K split", enc="f16", M=90, N=256, K=1600),
    dict(name="u split-K of the last round only (149 tiles)", enc="q4", M=64, N=128 * 149, K=1024),
    dict(name="u split-K of the last round only, rms+swiglu (150 tiles)", enc="q8", M=100, N=2 * 64 * 150, K=512, xmode="rms", epi="swiglu"),
    dict(name="u split-K of the last round only, wide tiles resadd (2 x 75 tiles)", enc="q4", M=600, N=128 * 75, K=768, epi="resadd"),
    # quantised weights, tiles up to 128 tokens, 32 k-steps or more per unit (one tile per SM: no split): pipeline steps of 256 k, the
    # last step of the k loop short by one, two and three k-steps; above 64 tokens with a single accumulator buffer
    dict(name="u q4 M16 256-k steps, tail of one k-step", enc="q4", M=16, N=128 * 148, K=64 * 33),
    dict(name="u q4 M100 256-k steps, tail of two k-steps, rms+swiglu", enc="q4", M=100, N=2 * 64 * 148, K=64 * 34, xmode="rms", epi="swiglu"),
    dict(name="u q4 M64 256-k steps, tail of three k-steps, resadd", enc="q4", M=64, N=128 * 148, K=64 * 35, epi="resadd"),
    dict(name="u q8 M48 256-k steps, tail of two k-steps", enc="q8", M=48, N=128 * 148, K=64 * 34),
    dict(name="u q8 M90 256-k steps, tail of three k-steps, rms+swiglu", enc="q8", M=90, N=2 * 64 * 148, K=64 * 35, xmode="rms", epi="swiglu"),
    dict(name="u q4 M384 one wide tile, ring wrap", enc="q4", M=384, N=640, K=1280),
    dict(name="u q8 M777 wide tiles, many", enc="q8", M=777, N=2560, K=448, epi="resadd"),
    dict(name="u q4 M250 single accumulator, narrow", enc="q4", M=250, N=1280, K=192, epi="swiglu"),
    dict(name="u f16 M3 (small M, fp16 weights)", enc="f16", M=3, N=256, K=512),
    dict(name="u q4 many tiles (two accumulators, ring wrap)", enc="q4", M=1024, N=6144, K=320),
    dict(name="u q8 many tiles", enc="q8", M=700, N=5120, K=192),
    dict(name="u rms+swiglu M512", enc="q4", M=512, N=1024, K=1024, xmode="rms", epi="swiglu"),
    dict(name="u swiglu bias rows tail", enc="q8", M=130, N=320, K=256, epi="swiglu", bias=True, wr0=64, wr1=320, w_rows=512),
    dict(name="u lnmod+heads M300", enc="q8", M=300, N=1152, K=512, xmode="lnmod", epi="heads", heads=dict(Ltot=320, Hq=4, Hkv=2, rowOff=10, eps=1e-6)),
    dict(name="u heads half M200", enc="q4", M=200, N=512, K=256, epi="heads", heads=dict(Ltot=200, Hq=2, Hkv=1, rowOff=0, eps=1e-6, ropeMode="half")),
    dict(name="u resadd gate+bias M260", enc="q4", M=260, N=384, K=256, epi="resadd", gate=True, bias=True),
    dict(name="u f32 tail columns", enc="q4", M=70, N=200, K=128, epi="f32", w_rows=256),
    dict(name="u bias+res M90", enc="f16", M=90, N=256, K=128, epi="bias", res=True),
    dict(name="u onormgate M64", enc="q4", M=64, N=256, K=256, epi="onormgate", Ltot=256),
    dict(name="u sub-ranges", enc="q4", M=50, N=128, K=128, ldx=328, kx0=72, wk0=160, w_cols=384, wr0=64, w_rows=256, ldy=200, ny0=40),
    dict(name="u sub-ranges q8", enc="q8", M=50, N=128, K=128, ldx=328, kx0=72, wk0=128, w_cols=384, wr0=64, w_rows=256, ldy=200, ny0=40),
]


@pytest.mark.parametrize("case", UMMA, ids=lambda c: c["name"])
def test_tensor_core_kernel(gpu, oracle, case):
    """the tcgen05 / TMEM kernel against the oracle; it is also what the library picks for these shapes, and it is
    deterministic run to run"""
    from p0pc0rn_kernels_b200._lib import K_UMMA
    h = CS.build(dict(case, kernel="umma"))
    got = CS.run_gpu(gpu, h)
    assert gpu.lastKernel == K_UMMA
    CS.check(got, CS.run_oracle(h), case["name"])
    got2 = CS.run_gpu(gpu, CS.build(dict(case)))
    assert gpu.lastKernel == K_UMMA and np.array_equal(got, got2)
    if "256-k steps" in case["name"]:
        assert gpu.lastPlan["KW"] == 4 and gpu.lastPlan["S"] == 1, gpu.lastPlan


def test_tensor_core_matches_general_kernel_bits_of_weights(gpu, oracle):
    """identity tokens turn the multiply into a read-out of the operand tiles: the tensor-core kernel's dequantised
    weights equal f16(deq) bit for bit (fp32 accumulation of one non-zero product per output is exact)"""
    O = oracle
    K, N = 256, 256
    for enc, scale in (("q4g32a.t64", 0.05), ("q8g64s.t64", 0.05), ("q4g32a.t64", 1.0), ("q8g64s.t64", 1.0)):      # packed conversions and their fallbacks
        W0 = O.randn(N * K, 11, scale); Wb, deq = CS.encode(enc, W0, N, K)
        X = np.eye(K, dtype=np.float32)
        wb, xb, yb = gpu.upload(Wb), gpu.upload(P().toF16(X)), gpu.buffer(K * N * 2)
        try:
            P().gemm(gpu, {"w": {"enc": enc, "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": K, "N": N, "K": K, "kernel": "umma"})
            got = gpu.read(yb, 0, K * N * 2).view(np.uint16).reshape(K, N)
            assert np.array_equal(got, O.to_f16(deq).reshape(N, K).T), enc
        finally:
            for b in (wb, xb, yb): gpu.free(b)


DECODE = [
    dict(name="d q4 M1", enc="q4", M=1, N=256, K=512),
    dict(name="d q8 M1", enc="q8", M=1, N=256, K=512),
    dict(name="d q4 M2 long K", enc="q4", M=2, N=128, K=4096 + 1024),
    dict(name="d q8 M3 long K", enc="q8", M=3, N=192, K=4096 + 768),
    dict(name="d q4 M5 K768", enc="q4", M=5, N=320, K=768),
    dict(name="d q4 M8", enc="q4", M=8, N=512, K=1024),
    dict(name="d q8 M9", enc="q8", M=9, N=256, K=1280),
    dict(name="d q4 M16", enc="q4", M=16, N=1024, K=2048),
    dict(name="d q8 M16", enc="q8", M=16, N=256, K=1536),
    dict(name="d q4 M13 tail cols", enc="q4", M=13, N=100, K=256, w_rows=128),
    dict(name="d rms+swiglu M1", enc="q4", M=1, N=512, K=1024, xmode="rms", epi="swiglu"),
    dict(name="d rms+swiglu M16 rows", enc="q4", M=16, N=256, K=512, xmode="rms", epi="swiglu", bias=True, wr0=64, wr1=256, w_rows=448, st_off=2, pv_off=4),
    dict(name="d geglu q8 M4", enc="q8", M=4, N=256, K=256, epi="swiglu", act="gelu"),
    dict(name="d resadd M1", enc="q4", M=1, N=256, K=1024, epi="resadd"),
    dict(name="d resadd gate+bias M7", enc="q8", M=7, N=192, K=256, epi="resadd", gate=True, bias=True, ev_off=8, bv_off=4),
    dict(name="d f32 M3", enc="q4", M=3, N=128, K=256, epi="f32"),
    dict(name="d bias+res M6", enc="q4", M=6, N=128, K=256, epi="bias", res=True),
    dict(name="d lnmod+heads M12", enc="q8", M=12, N=384, K=256, xmode="lnmod", epi="heads", heads=dict(Ltot=20, Hq=1, Hkv=1, rowOff=3, eps=1e-6)),
    dict(name="d heads half M5", enc="q4", M=5, N=512, K=256, epi="heads", heads=dict(Ltot=8, Hq=2, Hkv=1, rowOff=1, eps=1e-6, ropeMode="half")),
    dict(name="d onormgate M4", enc="q4", M=4, N=256, K=256, epi="onormgate", Ltot=256),
    dict(name="d sub-ranges M4", enc="q4", M=4, N=128, K=256, ldx=448, kx0=64, wk0=160, w_cols=512, wr0=64, w_rows=256, ldy=200, ny0=40),
    dict(name="d sub-ranges q8 M4", enc="q8", M=4, N=128, K=256, ldx=456, kx0=66, wk0=128, w_cols=512, wr0=64, w_rows=256, ldy=200, ny0=40),
    dict(name="d byte offsets M2", enc="q8", M=2, N=128, K=256, x_off=256, w_off=512, y_off=768),
    # more units than resident blocks: the stages are dealt out evenly and units are shared by two blocks (part 0 / part 1 of the
    # partial sums), with a short last k-block; and so many units that the ranges are rounded to whole units again
    dict(name="d q4 M3 shared units, short last k-block", enc="q4", M=3, N=64 * 300, K=4096 + 1024),
    dict(name="d q8 M1 shared units, short last k-block", enc="q8", M=1, N=64 * 500, K=2048 + 256),
    dict(name="d q4 M2 shared units, rms+swiglu", enc="q4", M=2, N=2 * 64 * 250, K=4096, xmode="rms", epi="swiglu"),
    dict(name="d q4 M2 whole-unit ranges (1800 units)", enc="q4", M=2, N=64 * 1800, K=512),
    dict(name="d K not a stage multiple -> general kernel", enc="q4", M=2, N=128, K=384, expect="generic"),
]


@pytest.mark.parametrize("case", DECODE, ids=lambda c: c["name"])
def test_decode_kernel(gpu, oracle, case):
    """the decode-sized kernel (M <= 16: bulk-copy weight stream, raw codes on the tensor cores, split-K) against the oracle"""
    from p0pc0rn_kernels_b200._lib import K_DECODE, K_UMMA
    if case.get("expect") == "generic":                          # shapes the kernel does not take are refused when forced and served otherwise
        with pytest.raises(ValueError, match="does not take"):
            CS.run_gpu(gpu, CS.build(dict(case, kernel="decode")))
        h = CS.build(dict(case)); got = CS.run_gpu(gpu, h)
        CS.check(got, CS.run_oracle(h), case["name"])
        return
    h = CS.build(dict(case, kernel="decode"))
    got = CS.run_gpu(gpu, h)
    assert gpu.lastKernel == K_DECODE
    plan = gpu.lastPlan
    if "shared units" in case["name"]:                           # the blocks' ranges are not whole units: some unit has two parts
        assert not plan["whole"] and plan["G"] < plan["units"] and (plan["T"] % plan["G"] or (plan["T"] // plan["G"]) % (plan["KC"] // 256)), plan
    if "whole-unit ranges" in case["name"]: assert plan["whole"] and plan["units"] >= 4 * plan["G"], plan
    CS.check(got, CS.run_oracle(h), case["name"])
    h2 = CS.build(dict(case))                                   # the library's own pick: this kernel up to 8 tokens, the tensor-core kernel from 9
    got2 = CS.run_gpu(gpu, h2)
    if case["M"] <= 4:
        assert gpu.lastKernel == K_DECODE and np.array_equal(got, got2), "not deterministic run to run"
    else:                                                       # 5..8 tokens: this kernel unless the weight is small; 9 and more: the tensor-core kernel
        assert gpu.lastKernel in (K_DECODE, K_UMMA) and (case["M"] <= 8 or gpu.lastKernel == K_UMMA)
        if gpu.lastKernel == K_DECODE: assert np.array_equal(got, got2), "not deterministic run to run"
        else: CS.check(got2, CS.run_oracle(h2), case["name"] + " (library's pick)")


PEERS = [
    dict(name="p decode M3 swiglu", enc="q4", M=3, N=256, K=512, epi="swiglu", peers=2),
    dict(name="p decode M1 resadd", enc="q8", M=1, N=128, K=256, epi="resadd", peers=1),
    dict(name="p umma rms+swiglu (row-wise stores)", enc="q4", M=100, N=512, K=512, xmode="rms", epi="swiglu", ldy=1024, ny0=256, peers=3),
    dict(name="p umma resadd (fp32 rows)", enc="q4", M=300, N=256, K=512, epi="resadd", ldy=512, ny0=128, peers=2),
    dict(name="p umma split-K heads", enc="q8", M=100, N=384, K=1536, xmode="lnmod", epi="heads", heads=dict(Ltot=128, Hq=1, Hkv=1, rowOff=7, eps=1e-6), peers=1),
    dict(name="p umma scalar stores (odd ld)", enc="q4", M=40, N=100, K=256, w_rows=128, ldy=110, peers=7),
]


@pytest.mark.parametrize("case", PEERS, ids=lambda c: c["name"])
def test_peer_copies_of_y(gpu, oracle, case):
    """every store to y is repeated into the peer copies (here: other buffers of the same GPU), bit for bit, on both kernels"""
    h = CS.build(dict(case))
    got = CS.run_gpu(gpu, h)                  # run_gpu compares the peer buffers with y
    CS.check(got, CS.run_oracle(h), case["name"])


def test_peer_copies_refused_on_general_kernel(gpu):
    h = CS.build(dict(name="p generic", enc="q4", M=2, N=128, K=96, peers=1))        # K % 64 != 0: only the general kernel takes it
    with pytest.raises(ValueError, match="peer copies"):
        CS.run_gpu(gpu, h)


# scales on both sides of the packed conversions' conditions (q4: scale < 2^-4 and the exactness window; q8: scale < 2^-8), down to
# subnormal scales and minima
@pytest.mark.parametrize("enc,scale", [("q4g32a.t64", 0.05), ("q8g64s.t64", 0.05), ("q4g32a.t64", 1.0), ("q4g32a.t64", "offset"), ("f16", 0.05),
                                       ("q4g32a.t64", 0.02), ("q4g32a.t64", 2e-5), ("q4g32a.t64", 0.3), ("q8g64s.t64", 1.0), ("q8g64s.t64", 0.02), ("q8g64s.t64", 1e-4)])
@pytest.mark.parametrize("path", [0, 1])
def test_dequant_bit_exact(gpu, oracle, enc, scale, path):
    """every tile value the kernels multiply with equals f16(deq) of the encoder, bit for bit (docs/FORMAT.md)"""
    import ctypes as C
    from p0pc0rn_kernels_b200._lib import ENC, lib
    O = oracle
    N, K = 192, 256
    if scale == "offset":   # groups that sit far from zero: min >> scale, where a single fp16 fma could double-round
        W0 = (1.0 + 1e-4 * O.randn(N * K, 3)).astype(np.float32) * np.repeat(np.float32(10.0) ** np.random.default_rng(1).integers(-3, 3, N * K // 32), 32).astype(np.float32)
    else:
        W0 = O.randn(N * K, 11, scale)
    Wb, deq = CS.encode(enc, W0, N, K)
    wb, ob = gpu.upload(Wb), gpu.buffer(N * K * 2)
    try:
        gpu._check(lib.p0p_dequant(gpu._h, ENC[enc], wb.handle, 0, K, 0, 0, N, path, ob.handle, 0))
        got = gpu.read(ob, 0, N * K * 2).view(np.uint16)
        assert np.array_equal(got, O.to_f16(deq)), f"{int((got != O.to_f16(deq)).sum())} of {N * K} tile values differ"
    finally:
        gpu.free(wb); gpu.free(ob)


def test_recorded_sequence(gpu, oracle):
    """op calls recorded into a graph (the Runner's batching, src/core/gpu.js:203-257) replay to the same bits"""
    h = CS.build(dict(enc="q4", M=4, N=256, K=512, xmode="rms", epi="swiglu"))
    want = CS.run_gpu(gpu, h)
    bufs = {k: gpu.upload(h[k], k) for k in ("X", "W", "ST", "PV")}
    bufs["Y"] = gpu.upload(h["Y0"], "Y")
    try:
        a = CS.gemm_args(gpu, h, bufs)
        P().gemm(gpu, a)                                  # first call sizes scratch memory
        gpu.upload(h["Y0"], "", bufs["Y"], 0)
        g = gpu.record(lambda: P().gemm(gpu, a))
        assert np.array_equal(gpu.read(bufs["Y"]).view(np.uint16)[: h["Y0"].size], h["Y0"]), "recording must not run the op"
        g.launch(); g.launch()
        assert np.array_equal(gpu.read(bufs["Y"]).view(np.uint16)[: h["Y0"].size], want)
        g.free()
    finally:
        for b in bufs.values(): gpu.free(b)


def test_rowstats(gpu, oracle):
    O = oracle
    rows, cols = 37, 1000
    X = (O.randn(rows * cols, 5) + 0.3).astype(np.float32)
    xb, sb = gpu.upload(X), gpu.buffer((rows + 2) * 8)
    try:
        for mode in ("ln", "rms"):
            P().rowstats(gpu, {"x": {"buf": xb}, "rows": rows, "cols": cols, "mode": mode, "eps": 1e-6, "st": {"buf": sb, "off": 2}})
            got = gpu.read(sb, 16, rows * 8).view(np.float32)
            want = O.rowstats(X, rows, cols, rms=(mode == "rms"))
            assert np.allclose(got, want, rtol=2e-5, atol=1e-6)
    finally:
        gpu.free(xb); gpu.free(sb)


def test_errors(gpu):
    """bad arguments raise with the reference's messages (src/ops/gemm.js:271, 283, 313); the context stays usable"""
    b = gpu.buffer(4096)
    try:
        with pytest.raises(ValueError, match="unsupported weight encoding"):
            P().gemm(gpu, {"w": {"enc": "q2", "buf": b, "rows": 64, "cols": 32}, "x": {"buf": b}, "y": {"buf": b}, "M": 1, "N": 64, "K": 32})
        with pytest.raises(ValueError, match="K must be a multiple of 32"):
            P().gemm(gpu, {"w": {"enc": "f16", "buf": b, "rows": 8, "cols": 48}, "x": {"buf": b}, "y": {"buf": b}, "M": 1, "N": 8, "K": 48})
        with pytest.raises(ValueError, match="missing binding"):
            P().gemm(gpu, {"w": {"enc": "f16", "buf": b, "rows": 8, "cols": 32}, "x": {"buf": b, "mode": "rms"}, "y": {"buf": b}, "M": 1, "N": 8, "K": 32})
        with pytest.raises(ValueError, match="bytes"):
            P().gemm(gpu, {"w": {"enc": "f16", "buf": b, "rows": 64, "cols": 64}, "x": {"buf": b}, "y": {"buf": b}, "M": 64, "N": 64, "K": 64, "epi": "f32"})
        with pytest.raises(ValueError, match="bad tile"):
            P().gemm(gpu, {"w": {"enc": "f16", "buf": b, "rows": 8, "cols": 32}, "x": {"buf": b}, "y": {"buf": b}, "M": 1, "N": 8, "K": 32, "tile": {"BM": 48, "BN": 64}})
        gpu.done()
        assert not gpu.lost
    finally:
        gpu.free(b)


def test_buffers(gpu):
    """zero-filled buffers, 16-byte rounding, same-size pool reuse, double free (src/core/gpu.js:87-139)"""
    a = gpu.buffer(100)
    assert a._pf == 112 and not gpu.read(a).any()
    gpu.upload(np.full(100, 7, np.uint8), "", a, 4)
    assert gpu.read(a, 4, 100).tolist() == [7] * 100
    s0 = gpu.poolStats()
    gpu.free(a); gpu.free(a)
    b = gpu.buffer(100)
    assert not gpu.read(b).any(), "a pooled buffer must come back cleared"
    assert gpu.poolStats()["reuses"] >= s0["reuses"]
    gpu.free(b)
    with pytest.raises(ValueError):
        gpu.read(b.__class__(gpu, b.handle, 16), 0, 16)


def test_shareable_buffers_and_read_into(gpu):
    """the two buffer extensions: memory other processes can map (zeroed, never pooled, exportable) and reads into the caller's array"""
    a = gpu.buffer(1000, "shared", shareable=True)
    assert a._pf == 1008 and not gpu.read(a).any()
    gpu.upload(np.arange(1000, dtype=np.uint8), "", a, 0)
    out = np.zeros(1000, np.uint8)
    got = gpu.read(a, 0, 1000, out=out)
    assert got is out and out.tolist() == [i % 256 for i in range(1000)]
    assert len(gpu.ipcExport(a)) == 64
    b = gpu.buffer(1000)
    with pytest.raises(ValueError, match="shareable"):
        gpu.ipcExport(b)                                  # the stream-ordered pool's memory has no handle
    with pytest.raises(ValueError):
        gpu.read(a, 0, 1000, out=np.zeros(10, np.uint8))
    s0 = gpu.poolStats()
    gpu.free(a); gpu.free(b)
    c = gpu.buffer(1000, "shared", shareable=True)        # a new allocation, cleared
    assert not gpu.read(c).any()
    gpu.free(c)
    assert gpu.poolStats()["alive"] <= s0["alive"]
