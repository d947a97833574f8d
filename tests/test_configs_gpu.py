"""Parity at the shapes of the baseline's own configurations (not scaled-down stand-ins), CUDA path against the CPU oracle:

  C1  plain q4 GEMM M64 N1024 K1024, weights N(0, 0.02) quantised by convertSafetensors and loaded by uploadWeights
  C2  LLM MLP block, q4: rms + gate/up K4096 -> 2 x 14336 (swiglu), down K14336 -> 4096 (resadd), M in {1, 16, 512}
  C3  DiT projection, q8: 3600 tokens, lnmod, K3072 -> 9216, heads epilogue (24 + 24 + 24 heads of 128)
  C4  conv3 over a 13 x 92 x 160 x 128 clip, fp16 weights in the converter's layout, bias; whole clip = 4-frame chunks out of a
      ring of 6 frames, bit for bit
  C5  two corners of the large-shape sweep: q4 M128 16384 x 16384, and q4 M8192 4096 x 4096 on a sample of rows

Inputs are seeded with the restated generators of the reference's tests (test/kernels.test.js:12-15); the gates are those of
tests/cases.py (cos > 0.9995 as test/kernels.test.js:228, relative L2 <= 4e-3, max |err| <= 2e-2 max |ref|)."""
import numpy as np
import pytest

import cases as CS

pytestmark = pytest.mark.gpu

HID, FF = 4096, 14336


def P():
    import p0pc0rn_kernels_b200 as P_
    return P_


def test_c1_plain_q4_through_the_converter(gpu, oracle):
    O = oracle
    M, N, K = 64, 1024, 1024
    X = O.round_f16(O.randn(M * K, 7)); W0 = O.randn(N * K, 11, 0.02)
    file = P().writeSafetensors({"layer.weight": {"dtype": "F32", "shape": [N, K], "data": W0.view(np.uint8)}})
    r = P().convertSafetensors(file, {"bits": 4}); model = P().uploadWeights(gpu, r["manifest"], r["shards"]); w = model.tensor("layer.weight")
    assert w["enc"] == "q4g32a.t64" and w["rows"] == N and w["cols"] == K
    Wb, Wd = O.pack_q4(W0, N, K)
    xb, yb = gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        assert np.array_equal(gpu.read(w["buf"], w["off"], w["bytes"]), Wb), "converter bytes differ from packQ4"
        P().gemm(gpu, {"w": w, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K})
        got = gpu.read(yb, 0, M * N * 2).view(np.uint16)
        want = O.cpu_gemm(X, Wd, M, N, K, threads=O.max_threads())
        assert O.compare(P().fromF16(got), want)[0] > 0.9995
        CS.check(got.copy(), O.to_f16(want), "C1")
    finally:
        for b in (xb, yb): gpu.free(b)
        model.free()


@pytest.fixture(scope="module")
def mlp_weights(oracle):
    """gate|up [28672][4096] and down [4096][14336], N(0, 0.02), quantised to q4 by the oracle's packer"""
    O = oracle
    gu = O.pack_q4(O.randn(2 * FF * HID, 11, 0.02), 2 * FF, HID)[0]
    dn = O.pack_q4(O.randn(HID * FF, 13, 0.02), HID, FF)[0]
    return gu, dn


@pytest.mark.parametrize("M", [1, 16, 512])
def test_c2_mlp_block(gpu, oracle, mlp_weights, M):
    """both GEMMs of the block at the benchmarked shapes: 448 column tiles with the last round split along K (gate/up), the
    split-K down GEMM; decode kernel at M = 1"""
    O = oracle
    gu, dn = mlp_weights
    X = (O.round_f16(O.randn(M * HID, 7))).astype(np.float32)
    gamma = (1.0 + O.randn(HID, 21, 0.1)).astype(np.float32)
    ST = O.rowstats(X, M, HID, rms=True, eps=1e-6)
    wg, wd = gpu.upload(gu), gpu.upload(dn)
    xb, gb, stb = gpu.upload(X), gpu.upload(gamma), gpu.buffer(M * 8)
    hb = gpu.upload(np.full(M * FF, 0xFFFF, np.uint16))
    try:
        P().rowstats(gpu, {"x": {"buf": xb}, "rows": M, "cols": HID, "mode": "rms", "eps": 1e-6, "st": {"buf": stb}})
        st_gpu = gpu.read(stb, 0, M * 8).view(np.float32)
        assert np.allclose(st_gpu, ST, rtol=2e-6, atol=0)
        P().gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wg, "off": 0, "bytes": gu.nbytes, "rows": 2 * FF, "cols": HID}, "x": {"buf": xb, "mode": "rms"},
                       "y": {"buf": hb, "ld": FF}, "M": M, "N": 2 * FF, "K": HID, "wr0": 0, "wr1": FF, "epi": "swiglu", "stats": {"buf": stb}, "pv": {"buf": gb}})
        h_gpu = gpu.read(hb, 0, M * FF * 2).view(np.uint16).copy()
        h_ref = np.full(M * FF, 0xFFFF, np.uint16)
        O.gemm(enc="q4g32a.t64", X=X, W=gu, Y=h_ref, M=M, N=2 * FF, K=HID, w_rows=2 * FF, w_cols=HID, xmode="rms", epi="swiglu", wr0=0, wr1=FF, ldy=FF, ST=ST, PV=gamma)
        CS.check(h_gpu, h_ref, f"C2 gate/up M={M}")
        # down GEMM on the GPU's own hidden row (what the block feeds it), residual add in place on the fp32 stream
        R0 = O.randn(M * HID, 41)
        rb = gpu.upload(R0)
        P().gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wd, "off": 0, "bytes": dn.nbytes, "rows": HID, "cols": FF}, "x": {"buf": hb}, "y": {"buf": rb}, "M": M, "N": HID, "K": FF, "epi": "resadd"})
        r_gpu = gpu.read(rb, 0, M * HID * 4).view(np.float32).copy(); gpu.free(rb)
        r_ref = R0.copy()
        O.gemm(enc="q4g32a.t64", X=h_gpu, W=dn, Y=r_ref, M=M, N=HID, K=FF, w_rows=HID, w_cols=FF, epi="resadd")
        CS.check(r_gpu, r_ref, f"C2 down M={M}")
    finally:
        for b in (wg, wd, xb, gb, stb, hb): gpu.free(b)
        gpu.drainPool()


def test_c3_dit_projection(gpu, oracle):
    c = dict(name="C3", enc="q8", M=3600, N=9216, K=3072, xmode="lnmod", epi="heads", w_scale=0.02, heads=dict(Ltot=3600, Hq=24, Hkv=24, rowOff=0, eps=1e-6))
    h = CS.build(c)
    got = CS.run_gpu(gpu, h)
    assert P()._lib.KERNEL_NAMES.get(gpu.lastKernel) == "umma"
    CS.check(got, CS.run_oracle(h), "C3")
    gpu.drainPool()


def test_c4_conv3_clip_whole_and_ring_chunks(gpu, oracle):
    O = oracle
    T, H, W, C, N = 13, 92, 160, 128, 128
    K = 27 * C; fx = H * W * C; fy = H * W * N
    X = O.round_f16(O.randn(T * fx, 31))
    w5 = O.randn(N * C * 27, 33, 0.03)                                   # [N][C][3][3][3] as a checkpoint holds it
    Wk = O.round_f16(O.reorder_conv_rows(w5, N, C, 27))                  # -> [N][(kt ky kx) C], the kernel's layout (reorderConvRows)
    bias = O.randn(N, 35, 0.1)
    xb, wb, bb = gpu.upload(P().toF16(X)), gpu.upload(P().toF16(Wk)), gpu.upload(bias)
    ya, yb, ring = gpu.buffer(T * fy * 2), gpu.buffer(T * fy * 2), gpu.buffer(6 * fx * 2)

    def conv(xbuf, xoff, ybuf, yoff, t0, nf, padL, ks):
        P().gemm(gpu, {"w": {"enc": "f16", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xbuf, "off": xoff}, "y": {"buf": ybuf, "off": yoff},
                       "M": nf * H * W, "N": N, "K": K, "epi": "bias", "ev": {"buf": bb},
                       "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": t0, "padL": padL, "ks": ks}})
    try:
        conv(xb, 0, ya, 0, 0, T, 0, 1)
        assert P()._lib.KERNEL_NAMES.get(gpu.lastKernel) == "umma"
        have = set()
        for t0 in range(0, T, 4):
            nf = min(4, T - t0)
            for g in range(max(0, t0 - 1), min(T - 1, t0 + nf) + 1):                     # frames t0-1 .. t0+nf into their ring slots
                if g not in have:
                    gpu.device.queue.writeBuffer(ring, (g % 6) * fx * 2, P().toF16(X[g * fx:(g + 1) * fx])); have.add(g)
            conv(ring, 0, yb, t0 * fy * 2, t0, nf, 0, 6)
            gpu.done()
        a, b = gpu.read(ya, 0, T * fy * 2).view(np.uint16), gpu.read(yb, 0, T * fy * 2).view(np.uint16)
        assert np.array_equal(a, b), "4-frame chunks out of a ring of 6 DIFFER from the whole clip"
        want = np.zeros(T * fy, np.uint16)
        O.gemm(enc="f16", X=O.to_f16(X), W=O.to_f16(Wk), Y=want, M=T * H * W, N=N, K=K, w_rows=N, w_cols=K, epi="bias", EV=bias,
               conv={"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": 0, "padL": 0, "ks": 1})
        CS.check(a.copy(), want, "C4")
    finally:
        for x in (xb, wb, bb, ya, yb, ring): gpu.free(x)
        gpu.drainPool()


def _tiled_q4(O, rows, cols, seed, slab_rows=2048):
    """N(0, 0.02) weights, q4: a slab of rows drawn and encoded once, repeated down the tensor (records are independent 64 x 32
    blocks, so the repeated bytes are a valid tensor with the same value distribution); returns (bytes, dequantised slab)"""
    W0 = O.randn(slab_rows * cols, seed, 0.02)
    b, d = O.pack_q4(W0, slab_rows, cols)
    return np.tile(b, rows // slab_rows), d


def test_c5_sweep_corner_m128_16384(gpu, oracle):
    O = oracle
    M, N, K = 128, 16384, 16384
    Wb, Wd = _tiled_q4(O, N, K, 11)
    X = O.round_f16(O.randn(M * K, 7))
    wb, xb, yb = gpu.upload(Wb), gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        P().gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wb, "off": 0, "bytes": Wb.nbytes, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K})
        got = gpu.read(yb, 0, M * N * 2).view(np.uint16).reshape(M, N)
        ref = O.cpu_gemm(X, Wd, M, 2048, K, threads=O.max_threads()).reshape(M, 2048)     # the slab's columns repeat every 2048
        for rep in (0, 3, 7):
            CS.check(np.ascontiguousarray(got[:, rep * 2048:(rep + 1) * 2048]).ravel(), O.to_f16(ref.ravel()), f"C5 M128 16384^2 columns {rep * 2048}+")
    finally:
        for b in (wb, xb, yb): gpu.free(b)
        gpu.drainPool()


def test_c5_sweep_corner_m8192_4096_row_sample(gpu, oracle):
    O = oracle
    M, N, K = 8192, 4096, 4096
    Wb, Wd = O.pack_q4(O.randn(N * K, 11, 0.02), N, K)
    X = O.round_f16(O.randn(M * K, 7))
    wb, xb, yb = gpu.upload(Wb), gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
    try:
        P().gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wb, "off": 0, "bytes": Wb.nbytes, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K})
        got = gpu.read(yb, 0, M * N * 2).view(np.uint16).reshape(M, N)
        rows = np.array(sorted(set(O.rng_u32(96, 5) % M) | {0, 383, 384, M - 1}))          # a sample of token rows, tile edges included
        ref = O.cpu_gemm(X.reshape(M, K)[rows].copy(), Wd, len(rows), N, K, threads=O.max_threads())
        CS.check(np.ascontiguousarray(got[rows]).ravel(), O.to_f16(ref), "C5 M8192 4096^2 row sample")
    finally:
        for b in (wb, xb, yb): gpu.free(b)
        gpu.drainPool()
