"""Host-side logic that needs no GPU: the native library loads and exports every symbol include/p0p.h declares,
its host codecs agree with the oracle bit for bit, the converter mirrors the reference's converter tests
(test/convert.test.mjs), and the N-shard byte ranges reassemble the full problem (2 gloo ranks on CPU)."""
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def P():
    import importlib.util
    spec = importlib.util.spec_from_file_location("p0p_build", os.path.join(ROOT, "p0pc0rn_kernels_b200", "build.py"))
    build = importlib.util.module_from_spec(spec); spec.loader.exec_module(build)
    build.build()          # no-op when libp0p.so is newer than its sources
    import p0pc0rn_kernels_b200 as P_
    return P_


def test_library_exports_every_declared_symbol(P):
    import ctypes
    from p0pc0rn_kernels_b200._lib import LIB_PATH, SYMBOLS
    hdr = open(os.path.join(ROOT, "include", "p0p.h")).read()
    declared = sorted(set(re.findall(r"\b(p0p_[a-z0-9_]+)\s*\(", hdr)))
    assert declared and sorted(SYMBOLS) == declared, set(SYMBOLS) ^ set(declared)
    L = ctypes.CDLL(LIB_PATH)
    for s in declared:
        assert hasattr(L, s), s
    assert L.p0p_abi_version() == 1


def test_argument_block_layout_matches_header(P, tmp_path):
    """the ctypes transcription of p0p_gemm_args has the header's size and field offsets (checked by compiling the header with gcc)"""
    import ctypes as C, subprocess, shutil
    if not shutil.which("gcc"): pytest.skip("no gcc")
    from p0pc0rn_kernels_b200._lib import GemmArgs
    fields = ["struct_size", "M", "eps", "force_kernel", "x", "gt", "x_off", "y_size", "n_ypeers", "y_peers"]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "p0p.h"\nint main(void){printf("%zu", sizeof(p0p_gemm_args));'
                   + "".join(f'printf(" %zu", offsetof(p0p_gemm_args, {f}));' for f in fields) + "return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include"), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert got[0] == C.sizeof(GemmArgs)
    assert got[1:] == [getattr(GemmArgs, f).offset for f in fields]


def test_no_gpu_fails_loudly(P):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(P.GpuError):
        P.createGpu()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "p0pc0rn_kernels_b200")
    for dp, _, fs in os.walk(pkg):
        for f in fs:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".js", ".cc")):
                txt = open(os.path.join(dp, f)).read()
                assert "import oracle" not in txt and "from oracle" not in txt and "p0p_oracle" not in txt, f


def test_fp16_codec_matches_oracle(P, oracle):
    O = oracle
    rs = np.random.default_rng(0)
    x = (rs.standard_normal(400000) * 10.0 ** rs.integers(-9, 6, 400000)).astype(np.float32)
    x = np.concatenate([x, np.array([0, -0.0, 65504, 65519.99, 65520, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -14, np.inf, -np.inf], np.float32)])
    assert np.array_equal(P.toF16(x), O.to_f16(x))
    assert P.f2h(float("nan")) == O.f2h(float("nan")) == 0x7E00
    allh = np.arange(65536, dtype=np.uint16); a, b = P.fromF16(allh), O.from_f16(allh); ok = ~np.isnan(b)
    assert np.array_equal(a[ok].view(np.uint32), b[ok].view(np.uint32)) and np.isnan(a[~ok]).all()
    assert P.h2f(0x3C00) == 1.0 and P.h2f(0xC000) == -2.0


@pytest.mark.parametrize("seed,scale", [(11, 0.05), (5, 1.0), (9, 1e-4), (3, 3000.0), (4, 1e-7)])
def test_encoders_match_oracle(P, oracle, seed, scale):
    O = oracle
    N, K = 192, 256
    W = O.randn(N * K, seed, scale)
    if seed == 5: W[: 64] = 0.37; W[64:128] = 0.0                     # constant and zero groups
    d = np.empty(N * K, np.float32)
    b = P.packQ4(W, N, K, d); bo, do = O.pack_q4(W, N, K); assert np.array_equal(b, bo) and np.array_equal(d.view(np.uint32), do.view(np.uint32))
    b = P.packQ8(W, N, K, d); bo, do = O.pack_q8(W, N, K); assert np.array_equal(b, bo) and np.array_equal(d.view(np.uint32), do.view(np.uint32))
    assert np.array_equal(P.packF16(W).view(np.uint16), O.to_f16(W))
    assert np.array_equal(P.reorderConvRows(W[: 4 * 8 * 27], 4, [4, 8, 3, 3, 3]), O.reorder_conv_rows(W[: 4 * 8 * 27], 4, 8, 27))
    with pytest.raises(ValueError, match="rows % 64"): P.packQ4(W, 100, K)
    with pytest.raises(ValueError, match="K % 64"): P.packQ8(W, 64, 96)


def test_dtype_known_answers(P):
    """test/convert.test.mjs:44-47"""
    f8 = P.toFloat32("F8_E4M3", np.array([0x38, 0xC0], np.uint8)); assert f8.tolist() == [1, -2]
    assert P.toFloat32("F8_E5M2", np.array([0x3C], np.uint8))[0] == 1
    assert P.toFloat32("BF16", np.array([0x3F80, 0xC000], np.uint16).view(np.uint8)).tolist() == [1, -2]
    assert P.toFloat32("F16", np.array([0x3C00, 0xC000], np.uint16).view(np.uint8)).tolist() == [1, -2]
    with pytest.raises(ValueError, match="unsupported dtype"): P.toFloat32("I64", np.zeros(8, np.uint8))


def test_converter(P, oracle):
    """encoding choice, shard roll-over, 256-byte alignment, bytes equal to the encoders', conv layout (test/convert.test.mjs:29-81)"""
    O = oracle
    S = {"qkv": O.randn(192 * 256, 1, 0.05), "mlp": O.randn(128 * 128, 2, 0.05), "conv": O.randn(64 * 32 * 9, 3, 0.05), "conv3": O.randn(64 * 32 * 27, 4, 0.05),
         "norm": O.randn(256, 5), "emb": O.randn(100 * 64, 6), "odd": O.randn(100 * 30, 7)}
    fp8 = (np.arange(64 * 64) % 120).astype(np.uint8)
    T = {"blocks.0.attn.qkv.weight": {"dtype": "BF16", "shape": [192, 256], "data": O.to_bf16(S["qkv"])},
         "blocks.0.mlp.weight": {"dtype": "F32", "shape": [128, 128], "data": S["mlp"]},
         "decoder.conv.weight": {"dtype": "F16", "shape": [64, 32, 3, 3], "data": O.to_f16(S["conv"])},
         "decoder.conv3.weight": {"dtype": "F16", "shape": [64, 32, 3, 3, 3], "data": O.to_f16(S["conv3"])},
         "blocks.0.norm.weight": {"dtype": "F32", "shape": [256], "data": S["norm"]},
         "embed_tokens.weight": {"dtype": "BF16", "shape": [100, 64], "data": O.to_bf16(S["emb"])},
         "odd.weight": {"dtype": "F32", "shape": [100, 30], "data": S["odd"]},
         "fp8.weight": {"dtype": "F8_E4M3", "shape": [64, 64], "data": fp8},
         "position_ids": {"dtype": "I64", "shape": [8], "data": np.zeros(64, np.uint8)}}
    file = P.writeSafetensors(T, {"format": "pt"})
    hd = P.safetensorsHeader(file); assert hd["dataStart"] % 8 == 0 and hd["header"]["__metadata__"] == {"format": "pt"}
    r = P.convertSafetensors(file, {"bits": 4, "keep": "embed", "shardBytes": 64 * 1024}); m, shards = r["manifest"], r["shards"]
    assert m["format"] == P.MANIFEST_FORMAT == "p0pc0rn-kernels.weights/1"
    want = {"blocks.0.attn.qkv.weight": "q4g32a.t64", "blocks.0.mlp.weight": "q4g32a.t64", "decoder.conv.weight": "q4g32a.t64", "decoder.conv3.weight": "q4g32a.t64",
            "blocks.0.norm.weight": "f32", "embed_tokens.weight": "f16", "odd.weight": "f16", "fp8.weight": "q4g32a.t64"}
    for k, enc in want.items(): assert m["tensors"][k]["enc"] == enc, k
    assert m["skipped"] == {"position_ids": "I64"} and "position_ids" not in m["tensors"]
    assert len(m["shards"]) > 1
    for s in m["shards"]: assert shards[s["file"]].size == s["bytes"]
    sl = lambda name, mm=m, ss=shards: ss[mm["tensors"][name]["file"]][mm["tensors"][name]["offset"]: mm["tensors"][name]["offset"] + mm["tensors"][name]["bytes"]]
    for k, t in m["tensors"].items(): assert t["offset"] % 256 == 0 and t["offset"] + t["bytes"] <= shards[t["file"]].size
    assert np.array_equal(sl("blocks.0.attn.qkv.weight"), O.pack_q4(O.from_bf16(O.to_bf16(S["qkv"])), 192, 256)[0])
    assert np.array_equal(sl("blocks.0.mlp.weight"), O.pack_q4(S["mlp"], 128, 128)[0])
    assert np.array_equal(sl("fp8.weight"), O.pack_q4(np.array([O.f8(True, int(b)) for b in fp8], np.float32), 64, 64)[0])
    assert np.array_equal(sl("blocks.0.norm.weight"), S["norm"].view(np.uint8))
    assert np.array_equal(sl("embed_tokens.weight").view(np.uint16), O.to_f16(O.from_bf16(O.to_bf16(S["emb"]))))
    assert np.array_equal(sl("odd.weight").view(np.uint16), O.to_f16(S["odd"]))
    r16 = P.convertSafetensors(file, {"bits": 16}); m16, s16 = r16["manifest"], r16["shards"]
    for name, src, taps in (("decoder.conv.weight", S["conv"], 9), ("decoder.conv3.weight", S["conv3"], 27)):
        got = sl(name, m16, s16).view(np.uint16).reshape(64, taps, 32)
        assert m16["tensors"][name]["layout"] == ("OHWI" if taps == 9 else "OTHWI")
        assert np.array_equal(got, O.to_f16(src).reshape(64, 32, taps).transpose(0, 2, 1))
    r8 = P.convertSafetensors(file, {"bits": 8}); t8 = r8["manifest"]["tensors"]["blocks.0.mlp.weight"]
    assert t8["enc"] == "q8g64s.t64" and np.array_equal(sl("blocks.0.mlp.weight", r8["manifest"], r8["shards"]), O.pack_q8(S["mlp"], 128, 128)[0])
    assert P.encodedBytes("q4g32a.t64", 128, 128) == 128 * 128 * 5 // 8 and P.encodedBytes("q8g64s.t64", 128, 128) == 128 * 128 * 33 // 32


def test_load_weights_from_disk_without_gpu(P, tmp_path):
    class FakeGpu:
        def __init__(self): self.up = {}
        def upload(self, data, label=""): self.up[label] = np.array(data); return label
        def free(self, b): self.up.pop(b, None)
    W = np.arange(64 * 32, dtype=np.float32) / 1000
    r = P.convertSafetensors(P.writeSafetensors({"a.weight": {"dtype": "F32", "shape": [64, 32], "data": W}, "a.bias": {"dtype": "F32", "shape": [64], "data": W[:64]}}))
    import json
    (tmp_path / "manifest.json").write_text(json.dumps(r["manifest"]))
    for f, b in r["shards"].items(): b.tofile(tmp_path / f)
    g = FakeGpu(); model = P.loadWeights(g, str(tmp_path))
    w = model.tensor("a.weight"); v = model.vector("a.bias")
    assert w["enc"] == "q4g32a.t64" and w["rows"] == 64 and w["cols"] == 32 and w["off"] % 256 == 0 and v["off"] * 4 % 256 == 0
    with pytest.raises(ValueError): model.vector("a.weight")
    model.free(); assert not g.up
    (tmp_path / "manifest.json").write_text(json.dumps(dict(r["manifest"], format="other")))
    with pytest.raises(ValueError, match="not a converted model"): P.loadWeights(g, str(tmp_path))


def test_shard_rows_are_byte_slices(P, oracle):
    O = oracle
    N, K = 512, 256
    W = O.randn(N * K, 3, 0.05)
    for enc, pack in (("q4g32a.t64", O.pack_q4), ("q8g64s.t64", O.pack_q8)):
        full, _ = pack(W, N, K)
        for world in (1, 2, 4, 8):
            parts = [P.shard_bytes(full, enc, N, K, r, world) for r in range(world)]
            assert np.array_equal(np.concatenate(parts), full)
            for r in range(world):
                s = P.shard_rows(enc, N, K, r, world)
                assert s["row0"] == r * N // world and np.array_equal(parts[r], pack(W[s["row0"] * K:(s["row0"] + s["rows"]) * K], s["rows"], K)[0])
        with pytest.raises(ValueError): P.shard_rows(enc, 192, K, 0, 8)
    s = P.shard_rows("f16", 100, 30, 1, 4); assert s == {"row0": 25, "rows": 25, "off": 25 * 60, "bytes": 25 * 60}
    # gate|up: a rank's shard is again [gate | up]
    half = 256; Wgu = O.randn(2 * half * K, 5, 0.05); full, _ = O.pack_q4(Wgu, 2 * half, K)
    sh = P.shard_swiglu_bytes(full, "q4g32a.t64", half, K, 1, 2)
    want = np.concatenate([O.pack_q4(Wgu[128 * K:256 * K], 128, K)[0], O.pack_q4(Wgu[(half + 128) * K:(half + 256) * K], 128, K)[0]])
    assert np.array_equal(sh, want)


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, 'tests'))
import numpy as np, torch, torch.distributed as dist
import oracle as O, p0pc0rn_kernels_b200 as P, cases as CS
dist.init_process_group('gloo', init_method='tcp://127.0.0.1:{port}', rank=int(sys.argv[1]), world_size=2)
rank, world = dist.get_rank(), 2
M, N, K = 5, 256, 128
X = O.to_f16(O.round_f16(O.randn(M * K, 7))); W0 = O.randn(N * K, 11, 0.05)
for enc, pack in (('q4g32a.t64', O.pack_q4), ('q8g64s.t64', O.pack_q8)):
    full, _ = pack(W0, N, K)
    Yfull = np.zeros(M * N, np.uint16); O.gemm(enc=enc, X=X, W=full, Y=Yfull, M=M, N=N, K=K, w_rows=N, w_cols=K)
    s = P.shard_rows(enc, N, K, rank, world); mine = P.shard_bytes(full, enc, N, K, rank, world)
    Yloc = np.zeros(M * s['rows'], np.uint16); O.gemm(enc=enc, X=X, W=mine, Y=Yloc, M=M, N=s['rows'], K=K, w_rows=s['rows'], w_cols=K)
    got = P.all_gather_columns(torch.from_numpy(Yloc.view(np.float16).reshape(M, s['rows']))).numpy().view(np.uint16).reshape(-1)
    assert np.array_equal(got, Yfull), enc
    got1 = P.all_gather_columns(torch.from_numpy(Yloc.view(np.float16).reshape(M, s['rows'])[:1].copy())).numpy().view(np.uint16).reshape(-1)
    assert np.array_equal(got1, Yfull[:N]), enc
# conv3 split by output frames: each rank's chunk call (the oracle stands in for the device) and the gather of the frames
T, H, W, C, N = 5, 4, 4, 32, 64
Xc = O.to_f16(O.round_f16(O.randn(T * H * W * C, 31))); Wc = O.to_f16(O.round_f16(O.randn(N * 27 * C, 33, 0.03)))
whole = {{"w": {{"enc": "f16"}}, "x": {{"off": 0}}, "y": {{"off": 0}}, "M": T * H * W, "N": N, "K": 27 * C,
         "conv": {{"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": 0, "padL": 0, "ks": 1}}}}
Yw = np.zeros(T * H * W * N, np.uint16)
O.gemm(enc="f16", X=Xc, W=Wc, Y=Yw, M=T * H * W, N=N, K=27 * C, w_rows=N, w_cols=27 * C, conv=whole["conv"])
a = P.conv3_frame_shard(whole, rank, world)
t0, nf = P.shard_frames(T, rank, world)
Yl = np.zeros(nf * H * W * N, np.uint16)
O.gemm(enc="f16", X=Xc[a["x"]["off"] // 2:], W=Wc, Y=Yl, M=a["M"], N=N, K=27 * C, w_rows=N, w_cols=27 * C, conv=a["conv"])
assert a["y"]["off"] == t0 * H * W * N * 2
got = P.all_gather_frames(torch.from_numpy(Yl.view(np.float16).reshape(nf, H * W * N)), T).numpy().view(np.uint16).reshape(-1)
assert np.array_equal(got, Yw), 'conv3 frames'
dist.barrier(); dist.destroy_process_group()
print('rank', rank, 'ok')
"""


def test_n_sharding_two_ranks_gloo(P, tmp_path):
    """the N-partition on 2 CPU ranks (gloo): each rank multiplies its byte-sliced shard (the oracle stands in for
    the device), the all-gather of the column blocks equals the unsharded result bit for bit, M == 1 included"""
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    script = tmp_path / "worker.py"; script.write_text(_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in o, o


@pytest.mark.parametrize("T,world", [(13, 8), (13, 2), (5, 3), (4, 8), (1, 2)])
def test_conv3_frame_shards_cover_the_clip(P, oracle, T, world):
    """the frame ranges tile [0, T); each rank's chunk arguments give, on the oracle, the frames of the whole-clip call bit for
    bit - with the rank addressing the whole clip, and with the rank holding only its frames plus the halo"""
    O = oracle
    H, W, C, N = 3, 4, 32, 64
    X = O.to_f16(O.round_f16(O.randn(T * H * W * C, 31))); Wt = O.to_f16(O.round_f16(O.randn(N * 27 * C, 33, 0.03)))
    whole = {"w": {"enc": "f16"}, "x": {"off": 0}, "y": {"off": 0, "ld": N}, "M": T * H * W, "N": N, "K": 27 * C,
             "conv": {"kind": "conv3", "Hi": H, "Wi": W, "Ci": C, "Ho": H, "Wo": W, "stride": T, "padT": 0, "padL": 0, "ks": 1}}
    Yw = np.zeros(T * H * W * N, np.uint16)
    O.gemm(enc="f16", X=X, W=Wt, Y=Yw, M=T * H * W, N=N, K=27 * C, w_rows=N, w_cols=27 * C, conv=whole["conv"])
    cover, Ys, Yl = [], np.zeros_like(Yw), np.zeros_like(Yw)
    fx = H * W * C
    for r in range(world):
        t0, nf = P.shard_frames(T, r, world); cover += list(range(t0, t0 + nf))
        a = P.conv3_frame_shard(whole, r, world)
        assert (a is None) == (nf == 0)
        if a is None: continue
        O.gemm(enc="f16", X=X[a["x"]["off"] // 2:], W=Wt, Y=Ys[a["y"]["off"] // 2:], M=a["M"], N=N, K=27 * C, w_rows=N, w_cols=27 * C, conv=a["conv"])
        b = P.conv3_frame_shard(whole, r, world, local_input=True)
        mine = X[b["in0"] * fx:(b["in0"] + b["nin"]) * fx].copy()                       # only the frames the rank reads
        assert b["x"]["off"] == 0 and b["nin"] <= nf + 2
        O.gemm(enc="f16", X=mine, W=Wt, Y=Yl[b["y"]["off"] // 2:], M=b["M"], N=N, K=27 * C, w_rows=N, w_cols=27 * C, conv=b["conv"])
    assert cover == list(range(T))
    assert np.array_equal(Ys, Yw) and np.array_equal(Yl, Yw)
    with pytest.raises(ValueError): P.conv3_frame_shard(dict(whole, conv=dict(whole["conv"], ks=3)), 0, 2)


def test_converter_command_line(P, oracle, tmp_path):
    """the CLI (tools/convert.mjs:9-62): usage errors exit 2, --dry-run lists encodings, a run writes the shards and manifest that
    convertSafetensors gives for the same file, and loadWeights-style reading of the folder sees the same tensors"""
    import io
    from p0pc0rn_kernels_b200 import convert_cli
    O = oracle
    T = {"blocks.0.attn.qkv.weight": {"dtype": "BF16", "shape": [192, 256], "data": O.to_bf16(O.randn(192 * 256, 1, 0.05))},
         "blocks.0.norm.weight": {"dtype": "F32", "shape": [256], "data": O.randn(256, 5)},
         "embed_tokens.weight": {"dtype": "BF16", "shape": [100, 64], "data": O.to_bf16(O.randn(100 * 64, 6))},
         "ids": {"dtype": "I64", "shape": [4], "data": np.arange(4, dtype=np.int64)}}
    src = tmp_path / "model.safetensors"; src.write_bytes(P.writeSafetensors(T).tobytes())
    out, err = io.StringIO(), io.StringIO()
    assert convert_cli.main([], out, err) == 2 and "usage" in err.getvalue()
    assert convert_cli.main([str(src)], out, err) == 2                                   # no --out and no --dry-run
    assert convert_cli.main([str(src), "--out", str(tmp_path / "o"), "--bits", "5"], out, err) == 2
    out = io.StringIO()
    assert convert_cli.main([str(src), "--dry-run", "--bits", "8"], out, err) == 0
    listing = out.getvalue()
    assert "q8g64s.t64" in listing and "f32" in listing and "f16" in listing
    out = io.StringIO()
    assert convert_cli.main([str(tmp_path), "--out", str(tmp_path / "o"), "--bits", "4", "--shard-mb", "512"], out, err) == 0          # a folder of .safetensors files
    assert out.getvalue().startswith("converted 3 tensors") and "skipped 1 non-float tensors" in out.getvalue()
    want = P.convertSafetensors(src.read_bytes(), {"bits": 4, "keep": __import__("re").compile("embed")})
    man = json.load(open(tmp_path / "o" / "manifest.json"))
    assert man["tensors"] == want["manifest"]["tensors"] and man["shards"] == want["manifest"]["shards"] and "created" in man
    for sh in man["shards"]:
        assert np.array_equal(np.fromfile(tmp_path / "o" / sh["file"], np.uint8), want["shards"][sh["file"]])
