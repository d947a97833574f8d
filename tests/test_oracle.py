"""The CPU oracle against everything that pins it without a GPU: the reference's stored known-answer constants
(test/convert.test.mjs:44-47, README.md:63), the byte-layout identities of docs/FORMAT.md, IEEE fp16 as numpy
implements it, hand-computed generator outputs, the chunk / ring identities of conv3, compositions of pinned
pieces, and the committed golden fixtures."""
import os

import numpy as np
import pytest

import cases as CS

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_dtype_known_answers(oracle):
    """test/convert.test.mjs:44-47"""
    O = oracle
    assert O.f8(True, 0x38) == 1 and O.f8(True, 0xC0) == -2
    assert O.f8(False, 0x3C) == 1
    assert O.from_bf16(np.array([0x3F80, 0xC000], np.uint16)).tolist() == [1, -2]
    assert O.from_f16(np.array([0x3C00, 0xC000], np.uint16)).tolist() == [1, -2]


def test_f16_matches_ieee(oracle):
    O = oracle
    allh = np.arange(65536, dtype=np.uint16)
    f = O.from_f16(allh); ref = allh.view(np.float16).astype(np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(f[ok].view(np.uint32), ref[ok].view(np.uint32)) and np.isnan(f[~ok]).all()
    assert np.array_equal(O.to_f16(f[ok]), allh[ok])                          # round trip
    rs = np.random.default_rng(0)
    x = (rs.standard_normal(300000) * 10.0 ** rs.integers(-9, 5, 300000)).astype(np.float32)
    assert np.array_equal(O.to_f16(x), x.astype(np.float16).view(np.uint16))
    # ties, overflow, subnormal edges, NaN (src/core/gpu.js:279: NaN -> sign | 0x7e00)
    np.seterr(over='ignore')
    edge = np.array([65504, 65519.99, 65520, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -14, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11, -0.0], np.float32)
    assert np.array_equal(O.to_f16(edge), edge.astype(np.float16).view(np.uint16))
    assert O.f2h(float("nan")) & 0x7FFF == 0x7E00 and O.f2h(float("inf")) == 0x7C00 and O.f2h(float("-inf")) == 0xFC00


def test_rng_hand_computed(oracle):
    """xorshift32 with an arithmetic middle shift (test/kernels.test.js:12): seed 7 -> 0x1CE0E7 worked by hand;
    a seed whose first shift sets bit 31 exercises the sign-extending shift."""
    O = oracle
    assert int(O.rng_u32(1, 7)[0]) == 0x1CE0E7
    def py(seed, n):
        s = seed & 0xFFFFFFFF or 1; out = []
        for _ in range(n):
            s ^= (s << 13) & 0xFFFFFFFF
            si = s - (1 << 32) if s & 0x80000000 else s
            s ^= (si >> 17) & 0xFFFFFFFF
            s ^= (s << 5) & 0xFFFFFFFF
            out.append(s)
        return out
    for seed in (1, 7, 11, 0x7FFFF, 0xDEADBEEF, 0):
        assert O.rng_u32(64, seed).tolist() == py(seed, 64)
    r = O.randn(200001, 7)
    assert abs(float(r.mean())) < 0.01 and abs(float(r.std()) - 1) < 0.01
    assert np.allclose(O.randn(1000, 11, 0.05), O.randn(1000, 11) * 0.05, rtol=1e-6)


def _decode_q4_numpy(b, N, K):
    """docs/FORMAT.md:20-27 decoded with numpy, independent of the C restatement"""
    G = K // 32; rec = b.reshape(N // 64, G, 1280)
    codes = rec[:, :, :1024].reshape(N // 64, G, 64, 16)
    q = np.stack([codes & 15, codes >> 4], -1).reshape(N // 64, G, 64, 32).astype(np.float32)
    sm = rec[:, :, 1024:].copy().view(np.uint16).reshape(N // 64, G, 64, 2)
    s = sm[..., 0].view(np.float16).astype(np.float32)[..., None]; mn = sm[..., 1].view(np.float16).astype(np.float32)[..., None]
    return (q * s + mn).astype(np.float32).transpose(0, 2, 1, 3).reshape(N, K)


def _decode_q8_numpy(b, N, K):
    G = K // 64; rec = b.reshape(N // 64, G, 4224)
    q = rec[:, :, :4096].copy().view(np.int8).reshape(N // 64, G, 64, 64).astype(np.float32)
    s = rec[:, :, 4096:].copy().view(np.float16).astype(np.float32).reshape(N // 64, G, 64, 1)
    return (q * s).astype(np.float32).transpose(0, 2, 1, 3).reshape(N, K)


@pytest.mark.parametrize("scale", [0.02, 0.05, 1.0, 30.0])
def test_format_layout_and_quantiser(oracle, scale):
    """sizes 5/8 and 33/32 bytes per weight, record offsets, and the quantiser's own guarantees (docs/FORMAT.md)"""
    O = oracle
    N, K = 192, 256
    W = O.randn(N * K, 11, scale)
    b4, d4 = O.pack_q4(W, N, K); b8, d8 = O.pack_q8(W, N, K)
    assert b4.size == N * K * 5 // 8 and b8.size == N * K * 33 // 32
    assert np.array_equal(_decode_q4_numpy(b4, N, K).reshape(-1), d4)
    assert np.array_equal(_decode_q8_numpy(b8, N, K).reshape(-1), d8)
    h, f = O.dequant("q4g32a.t64", b4, 0, N, K); assert np.array_equal(f, d4) and np.array_equal(h, O.to_f16(d4))
    h, f = O.dequant("q8g64s.t64", b8, 0, N, K); assert np.array_equal(f, d8) and np.array_equal(h, O.to_f16(d8))
    # half a quantisation step (plus the fp16 rounding of the minimum / scale)
    s4 = np.repeat(b4.reshape(-1, 1280)[:, 1024:].copy().view(np.uint16)[:, 0::2].view(np.float16).astype(np.float32).reshape(N // 64, K // 32, 64).transpose(0, 2, 1).reshape(-1), 32)
    assert (np.abs(d4 - W) <= 0.5 * s4 * 1.01 + np.abs(W) * 2.0 ** -10).all()
    # a tile-aligned row range is one contiguous byte range
    sub, dsub = O.pack_q4(W[64 * K:128 * K], 64, K)
    assert np.array_equal(sub, b4[(K // 32) * 1280:2 * (K // 32) * 1280]) and np.array_equal(dsub, d4[64 * K:128 * K])
    with pytest.raises(ValueError): O.pack_q4(W, 100, K)
    with pytest.raises(ValueError): O.pack_q8(W, 64, 96)


def test_constant_and_zero_groups(oracle):
    """s == 0 -> 1 (src/convert/encode.js:64, 84)"""
    O = oracle
    W = np.zeros(64 * 64, np.float32); W[:32] = 0.375
    b, d = O.pack_q4(W, 64, 64); assert np.array_equal(d, W)
    assert b[1024:1028].view(np.uint16)[0] == 0x3C00          # scale 1.0 stored for the constant group
    # a constant that fp16 rounds UP puts the minimum above the maximum: the scale comes out negative and
    # the codes saturate, yet the group still decodes to within an fp16 step (src/convert/encode.js:64-68)
    W2 = np.full(64 * 32, 0.37, np.float32); b2, d2 = O.pack_q4(W2, 64, 32)
    assert np.abs(d2 - 0.37).max() < 2e-4
    b, d = O.pack_q8(W, 64, 64); assert np.allclose(d, W, atol=2e-3)
    assert b.reshape(-1, 4224)[0, 4096:].copy().view(np.float16)[1] == 1.0


def test_reorder_conv_rows(oracle):
    O = oracle
    rows, I, taps = 5, 6, 27
    W = np.arange(rows * I * taps, dtype=np.float32)
    assert np.array_equal(O.reorder_conv_rows(W, rows, I, taps), W.reshape(rows, I, taps).transpose(0, 2, 1).reshape(-1))


def test_cpu_gemm_against_numpy(oracle):
    O = oracle
    M, N, K = 32, 128, 256
    X = O.round_f16(O.randn(M * K, 7)); W = O.randn(N * K, 11, 0.05)
    want = (X.reshape(M, K).astype(np.float64) @ W.reshape(N, K).astype(np.float64).T).astype(np.float32).reshape(-1)
    got = O.cpu_gemm(X, W, M, N, K)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    assert np.array_equal(got, O.cpu_gemm(X, W, M, N, K, threads=4))
    assert O.compare(got, want)[0] > 0.999999
    # README.md:63: 512 x 0.5 x 0.01 ~ 2.56
    y = O.cpu_gemm(O.round_f16(np.full(64 * 512, 0.5, np.float32)), O.round_f16(np.full(256 * 512, 0.01, np.float32)), 64, 256, 512)
    assert np.allclose(y, 2.56, atol=2e-3)


def test_cpu_conv3_against_numpy(oracle):
    O = oracle
    T, H, W, C, N = 4, 5, 6, 8, 16
    X = O.round_f16(O.randn(T * H * W * C, 31)); Wt = O.round_f16(O.randn(N * 27 * C, 33, 0.03))
    Xp = X.reshape(T, H, W, C).astype(np.float64)
    Xp = np.concatenate([Xp[:1], Xp, Xp[-1:]], 0); Xp = np.pad(Xp, ((0, 0), (1, 1), (1, 1), (0, 0)))
    Wk = Wt.reshape(N, 3, 3, 3, C).astype(np.float64); want = np.zeros((T, H, W, N))
    for kt in range(3):
        for ky in range(3):
            for kx in range(3):
                want += np.einsum("thwc,nc->thwn", Xp[kt:kt + T, ky:ky + H, kx:kx + W], Wk[:, kt, ky, kx])
    assert np.allclose(O.cpu_conv3(X, Wt, T, H, W, C, N), want.reshape(-1), rtol=1e-5, atol=1e-5)


def test_oracle_gemm_equals_cpu_refs(oracle):
    """the full restatement reduces to the reference tests' CPU multiplications for the plain cases"""
    O = oracle
    for enc in ("f16", "q4", "q8"):
        h = CS.build(dict(enc=enc, M=32, N=128, K=256, seed=7))
        got = O.from_f16(CS.run_oracle(h)); want = O.cpu_gemm(h["Xf"], h["Wd"], 32, 128, 256)
        assert O.compare(got, want)[0] > 0.99999 and np.abs(got - want).max() < 4e-3
    T, H, W, C, N = 5, 6, 6, 32, 128
    h = CS.build(dict(enc="f16", M=T * H * W, N=N, K=27 * C, x_elems=T * H * W * C, w_scale=0.03, seed=31,
                      conv=dict(kind="conv3", Hi=H, Wi=W, Ci=C, Ho=H, Wo=W, stride=T, padT=0, padL=0, ks=1)))
    got = O.from_f16(CS.run_oracle(h)); want = O.cpu_conv3(h["Xf"], h["Wd"], T, H, W, C, N)
    assert np.array_equal(CS.run_oracle(h), O.to_f16(want))


def test_conv3_chunks_and_ring_identity_on_cpu(oracle):
    """index arithmetic of src/ops/gemm.js:68-80: 2-frame chunks from a buffer offset and a ring of 3 frames give the
    bits of the whole clip (test/kernels.test.js:123-145)"""
    O = oracle
    T, H, W, C, N = 5, 6, 6, 32, 64
    X = O.to_f16(O.round_f16(O.randn(T * H * W * C, 31))); Wt = O.round_f16(O.randn(N * 27 * C, 33, 0.03)); Wb = O.to_f16(Wt).view(np.uint8)
    def run(Xin, Y, t0, nf, padL, ks):
        O.gemm(enc="f16", X=Xin, W=Wb, Y=Y, M=nf * H * W, N=N, K=27 * C, w_rows=N, w_cols=27 * C, epi="f16",
               conv=dict(kind="conv3", Hi=H, Wi=W, Ci=C, Ho=H, Wo=W, stride=T, padT=t0, padL=padL, ks=ks))
    whole = np.zeros(T * H * W * N, np.uint16); run(X, whole, 0, T, 0, 1)
    chunks = np.zeros_like(whole); fx, fy = H * W * C, H * W * N
    for t0 in range(0, T, 2):
        padL = max(0, t0 - 1); nf = min(2, T - t0)
        y = np.zeros(nf * fy, np.uint16); run(X[padL * fx:], y, t0, nf, padL, 1); chunks[t0 * fy:(t0 + nf) * fy] = y
    assert np.array_equal(whole, chunks)
    ring = np.zeros(3 * fx, np.uint16); out = np.zeros_like(whole)
    for t in range(T):
        for g in {max(0, t - 1), t, min(T - 1, t + 1)}: ring[(g % 3) * fx:(g % 3 + 1) * fx] = X[g * fx:(g + 1) * fx]
        y = np.zeros(fy, np.uint16); run(ring, y, t, 1, 0, 3); out[t * fy:(t + 1) * fy] = y
    assert np.array_equal(whole, out)


def test_fused_variants_compose_from_pinned_pieces(oracle):
    """rms + swiglu equals RMS-scale -> fp16 -> the pinned plain multiplication -> SiLU(gate) * up, and
    lnmod + resadd(gate) likewise: the unpinned prologues / epilogues agree with a composition of pinned parts"""
    O = oracle
    M, K, half = 24, 256, 64
    h = CS.build(dict(enc="q4", M=M, N=2 * half, K=K, xmode="rms", epi="swiglu"))
    got = O.from_f16(CS.run_oracle(h)).reshape(M, half)
    X = h["X"].reshape(M, K); rstd = h["ST"][1::2][:, None]; gamma = h["PV"][:K][None, :]
    Xn = O.round_f16((X * rstd * gamma).astype(np.float32))
    Wt = O.from_f16(O.dequant(h["enc"], h["W"], 0, h["w_rows"], K)[0])
    Y = O.cpu_gemm(Xn, Wt, M, h["w_rows"], K).reshape(M, -1)
    g, u = Y[:, :half], Y[:, half:2 * half]
    want = O.round_f16((g / (1 + np.exp(-g)) * u).astype(np.float32)).reshape(M, half)
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-3
    h = CS.build(dict(enc="q8", M=M, N=128, K=K, xmode="lnmod", epi="resadd", gate=True, x_shift=0.5))
    got = CS.run_oracle(h).reshape(M, 128)
    X = h["X"].reshape(M, K); mean = h["ST"][0::2][:, None]; rstd = h["ST"][1::2][:, None]; sc = h["PV"][:K][None]; sh = h["PV"][K:2 * K][None]
    Xn = O.round_f16(((X - mean) * rstd * (1 + sc) + sh).astype(np.float32))
    Wt = O.from_f16(O.dequant(h["enc"], h["W"], 0, h["w_rows"], K)[0])
    want = h["Y0"].reshape(M, 128) + h["EV"][None, :128] * O.cpu_gemm(Xn, Wt, M, 128, K).reshape(M, 128)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_heads_properties(oracle):
    """Q/K sections are unit-RMS before the norm weight and RoPE is a rotation (norm preserving); V passes through"""
    O = oracle
    hd = dict(Ltot=40, Hq=1, Hkv=1, rowOff=0, eps=1e-6)
    for mode in (None, "half"):
        h = CS.build(dict(enc="q8", M=40, N=384, K=256, epi="heads", heads=dict(hd, **({"ropeMode": mode} if mode else {}))))
        h["EV"][:] = 1.0
        Y = O.from_f16(CS.run_oracle(h)).reshape(3, 40, 128)
        assert np.allclose((Y[:2] ** 2).mean(-1), 1.0, atol=5e-3)
        plain = CS.build(dict(enc="q8", M=40, N=384, K=256)); yp = O.from_f16(CS.run_oracle(plain)).reshape(40, 3, 128)
        assert np.array_equal(O.to_f16(Y[2]), O.to_f16(yp[:, 2]))


def test_rowstats(oracle):
    O = oracle
    X = (O.randn(7 * 300, 3) * 2 + 0.5).astype(np.float32).reshape(7, 300)
    st = O.rowstats(X, 7, 300).reshape(7, 2)
    assert np.allclose(st[:, 0], X.mean(1), rtol=1e-5) and np.allclose(st[:, 1], 1 / np.sqrt(X.var(1) + 1e-6), rtol=1e-5)
    st = O.rowstats(X, 7, 300, rms=True).reshape(7, 2)
    assert (st[:, 0] == 0).all() and np.allclose(st[:, 1], 1 / np.sqrt((X ** 2).mean(1) + 1e-6), rtol=1e-5)


@pytest.mark.parametrize("name", sorted(f[:-4] for f in os.listdir(GOLDEN) if f.endswith(".npz")) if os.path.isdir(GOLDEN) else [])
def test_golden_fixtures(oracle, name):
    """committed outputs (tests/golden/make_golden.py wrote them) still come out of the oracle bit for bit"""
    import sys
    if GOLDEN not in sys.path: sys.path.insert(0, GOLDEN)
    import make_golden
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = make_golden.CASES[name](oracle)
    for k in z.files:
        assert np.array_equal(z[k], out[k]), f"{name}:{k}"


# ---------------------------------------------------------------- statistics producers (pixstats, GroupNorm) against numpy float64
def test_pixstats_restatement_against_numpy(oracle):
    """src/ops/video.js:301-318: rstd per voxel over the channels"""
    O = oracle
    V, C = 77, 96
    X = O.to_f16(O.randn(V * C, 3) * 2.0 + 0.5)
    xf = O.from_f16(X).astype(np.float64).reshape(V, C)
    np.testing.assert_allclose(O.pixstats(X, V, C, 1e-8), 1.0 / np.sqrt((xf ** 2).mean(1) + 1e-8), rtol=2e-7)


@pytest.mark.parametrize("pix,C", [(64, 32), (200, 128), (1000, 512)])
def test_groupnorm_restatement_against_numpy(oracle, pix, C):
    """src/ops/misc.js:50-104: chunk partials merged by Chan's formula = the statistics of the whole tensor"""
    O = oracle
    X = O.to_f16(O.randn(pix * C, 5) * 1.5 + np.tile(np.linspace(-2, 2, C, dtype=np.float32), pix))
    gamma, beta = (1.0 + O.randn(C, 6, 0.2)).astype(np.float32), O.randn(C, 7, 0.3)
    PT = O.gn_partial(X, pix, C); nwg = -(-pix // 64)
    pt = PT.reshape(nwg, 32, 4)
    assert pt[:, :, 0].sum() == pix * C                                   # the counts cover every element once
    AB = O.gn_finalize(PT, nwg, C, gamma, beta, 1e-6)
    xf = O.from_f16(X).astype(np.float64).reshape(pix, 32, C // 32)
    mean, var = xf.mean((0, 2)), xf.var((0, 2))
    a = np.repeat(1.0 / np.sqrt(var + 1e-6), C // 32) * gamma
    np.testing.assert_allclose(AB[:C], a, rtol=2e-5)
    np.testing.assert_allclose(AB[C:], beta - np.repeat(mean, C // 32) * a, rtol=2e-4, atol=2e-5)
