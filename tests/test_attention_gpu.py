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


@pytest.mark.parametrize("c", ATT + MORE, ids=lambda c: c["label"])
def test_attention_head128(gpu, oracle, c):
    import p0pc0rn_kernels_b200 as P
    O = oracle
    D, Hq, Hkv, Lq, Lk = 128, c["Hq"], c["Hkv"], c["Lq"], c["Lk"]
    Q = O.round_f16(O.randn(Hq * Lq * D, 21, 0.5)); Kt = O.round_f16(O.randn(Hkv * Lk * D, 22, 0.5)); V = O.round_f16(O.randn(Hkv * Lk * D, 23))
    ldo = c.get("ldo", Hq * D)
    qb, kb, vb = gpu.upload(P.toF16(Q)), gpu.upload(P.toF16(Kt)), gpu.upload(P.toF16(V))
    ob = gpu.upload(np.full(Lq * ldo, 0x7E01, np.uint16))                                    # NaN poison: only the head columns may change
    try:
        a = {"q": {"buf": qb}, "k": {"buf": kb}, "v": {"buf": vb}, "o": {"buf": ob, "ld": ldo}, "Lq": Lq, "Lk": Lk, "Hq": Hq, "Hkv": Hkv,
             "mode": c["mode"], "nvalid": c.get("nvalid")}
        if "scale" in c: a["scale"] = c["scale"]
        fl = P.attention(gpu, a)
        assert fl == 4.0 * Lq * Lk * 128 * Hq
        raw = gpu.read(ob, 0, Lq * ldo * 2).view(np.uint16).reshape(Lq, ldo)
        assert (raw[:, Hq * D:] == 0x7E01).all(), "columns past the heads were written"
        got = P.fromF16(np.ascontiguousarray(raw[:, :Hq * D]).ravel())
        want = O.cpu_attn(Q, Kt, V, Hq=Hq, Hkv=Hkv, Lq=Lq, Lk=Lk, mode=c["mode"], nvalid=c.get("nvalid"), scale=c.get("scale"))
        cos, maxabs = O.compare(got, want)[:2]
        assert cos > 0.9995, (cos, maxabs)                                                      # the reference's gate (test/kernels.test.js:228)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
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
