"""attention (head 128), the step after the 'heads' projection: the reference's cases (test/kernels.test.js:148-165) and wider ones,
through the C ABI against the CPU restatement of cpuAttn."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ATT = [   # test/kernels.test.js:149-151
    dict(label="no mask", Hq=2, Hkv=2, Lq=96, Lk=96, mode=0),
    dict(label="causal + valid length 80, GQA 4:2", Hq=4, Hkv=2, Lq=96, Lk=96, mode=1, nvalid=80),
    dict(label="valid length 77 of 100 keys, 64 queries", Hq=2, Hkv=2, Lq=64, Lk=100, mode=2, nvalid=77),
]
MORE = [
    dict(label="ragged tiles, GQA 6:2", Hq=6, Hkv=2, Lq=150, Lk=333, mode=0),
    dict(label="causal, long", Hq=2, Hkv=1, Lq=300, Lk=300, mode=1, nvalid=300),
    dict(label="one query", Hq=3, Hkv=3, Lq=1, Lk=70, mode=2, nvalid=33),
    dict(label="custom scale, output row stride", Hq=2, Hkv=2, Lq=70, Lk=130, mode=0, scale=0.05, ldo=2 * 128 + 64),
]


WIDE = [   # several blocks of two 128-query tiles, key tiles of 128, a last block with one tile, ragged ends
    dict(label="700 x 700, causal + valid length 650", Hq=2, Hkv=1, Lq=700, Lk=700, mode=1, nvalid=650),
    dict(label="384 x 520, GQA 4:2", Hq=4, Hkv=2, Lq=384, Lk=520, mode=0),
    dict(label="257 x 1000, valid length 901", Hq=2, Hkv=2, Lq=257, Lk=1000, mode=2, nvalid=901),
    dict(label="wide score range (the running maximum moves by more than the lazy threshold)", Hq=2, Hkv=2, Lq=300, Lk=640, mode=0, qstd=4.0),
    dict(label="512 x 512, output rows not 16-byte aligned", Hq=1, Hkv=1, Lq=512, Lk=512, mode=0, ldo=128 + 6),
]


@pytest.mark.parametrize("kernel", ["warp", "tmem"])
@pytest.mark.parametrize("c", ATT + MORE + WIDE, ids=lambda c: c["label"])
def test_attention_head128(gpu, oracle, c, kernel):
    import p0pc0rn_kernels_b200 as P
    O = oracle
    D, Hq, Hkv, Lq, Lk = 128, c["Hq"], c["Hkv"], c["Lq"], c["Lk"]
    Q = O.round_f16(O.randn(Hq * Lq * D, 21, c.get("qstd", 0.5))); Kt = O.round_f16(O.randn(Hkv * Lk * D, 22, 0.5)); V = O.round_f16(O.randn(Hkv * Lk * D, 23))
    ldo = c.get("ldo", Hq * D)
    qb, kb, vb = gpu.upload(P.toF16(Q)), gpu.upload(P.toF16(Kt)), gpu.upload(P.toF16(V))
    ob = gpu.upload(np.full(Lq * ldo, 0x7E01, np.uint16))                                    # NaN poison: only the head columns may change
    try:
        a = {"q": {"buf": qb}, "k": {"buf": kb}, "v": {"buf": vb}, "o": {"buf": ob, "ld": ldo}, "Lq": Lq, "Lk": Lk, "Hq": Hq, "Hkv": Hkv,
             "mode": c["mode"], "nvalid": c.get("nvalid"), "kernel": kernel}
        if "scale" in c: a["scale"] = c["scale"]
        fl = P.attention(gpu, a)
        assert fl == 4.0 * Lq * Lk * 128 * Hq
        assert gpu.lastKernel == {"warp": 16, "tmem": 17}[kernel]
        raw = gpu.read(ob, 0, Lq * ldo * 2).view(np.uint16).reshape(Lq, ldo)
        assert (raw[:, Hq * D:] == 0x7E01).all(), "columns past the heads were written"
        got = P.fromF16(np.ascontiguousarray(raw[:, :Hq * D]).ravel())
        want = O.cpu_attn(Q, Kt, V, Hq=Hq, Hkv=Hkv, Lq=Lq, Lk=Lk, mode=c["mode"], nvalid=c.get("nvalid"), scale=c.get("scale"))
        cos, maxabs = O.compare(got, want)[:2]
        assert cos > 0.9995, (cos, maxabs)                                                      # the reference's gate (test/kernels.test.js:228)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    finally:
        for b in (qb, kb, vb, ob): gpu.free(b)


def test_attention_dit_shape(gpu, oracle):
    """24 heads x 3600 tokens (the attention after the DiT projection): the library's own choice of kernel, two heads checked."""
    import p0pc0rn_kernels_b200 as P
    O = oracle
    D, H, L = 128, 24, 3600
    Q = O.round_f16(O.randn(H * L * D, 31, 0.5)); Kt = O.round_f16(O.randn(H * L * D, 32, 0.5)); V = O.round_f16(O.randn(H * L * D, 33))
    qb, kb, vb, ob = gpu.upload(P.toF16(Q)), gpu.upload(P.toF16(Kt)), gpu.upload(P.toF16(V)), gpu.buffer(L * H * D * 2)
    try:
        P.attention(gpu, {"q": {"buf": qb}, "k": {"buf": kb}, "v": {"buf": vb}, "o": {"buf": ob}, "Lq": L, "Lk": L, "Hq": H, "Hkv": H, "mode": 0})
        assert gpu.lastKernel == 17
        got = P.fromF16(gpu.read(ob, 0, L * H * D * 2).view(np.uint16)).reshape(L, H, D)
        assert np.isfinite(got).all()
        for h in (0, 23):
            sl = slice(h * L * D, (h + 1) * L * D)
            want = O.cpu_attn(Q[sl], Kt[sl], V[sl], Hq=1, Hkv=1, Lq=L, Lk=L, mode=0).reshape(L, D)
            cos = O.compare(got[:, h].ravel(), want.ravel())[0]
            assert cos > 0.9995, (h, cos)
            assert np.abs(got[:, h] - want).max() <= 2e-2 * np.abs(want).max()
    finally:
        for b in (qb, kb, vb, ob): gpu.free(b)


def test_attention_errors(gpu):
    import p0pc0rn_kernels_b200 as P
    b = gpu.buffer(1024)
    with pytest.raises(ValueError, match="needs"):
        P.attention(gpu, {"q": {"buf": b}, "k": {"buf": b}, "v": {"buf": b}, "o": {"buf": b}, "Lq": 64, "Lk": 64, "Hq": 2})
    with pytest.raises(ValueError, match="multiple of Hkv"):
        P.attention(gpu, {"q": {"buf": b}, "k": {"buf": b}, "v": {"buf": b}, "o": {"buf": b}, "Lq": 1, "Lk": 1, "Hq": 3, "Hkv": 2})
    gpu.free(b)
