#!/usr/bin/env python
"""Benchmark of the B200 gemm path on the LLM MLP block of the baseline's configs (q4 weights):

    RMSNorm prologue -> gate/up GEMM  K=4096 -> 2 x 14336, SwiGLU epilogue -> down GEMM  K=14336 -> 4096, residual add

One step = one pass of the block over M tokens (default 512): row statistics, the fused gate/up GEMM, the fused
down GEMM.  `value` is TFLOP/s (2*M*N*K of both GEMMs over the device time of K steps, inputs resident in HBM);
`e2e` is the same through the public API with HOST buffers (page-locked host -> device copy of the tokens and a
device -> host read of the result inside the timed region; the steps run as a three-stream pipeline - upload, block,
read-back over a ring of residual buffers - and the plain one-after-the-other loop is reported beside it).
Decode-sized M (1, 16) is measured next to it and reported as GB/s of the weight stream in `cases`.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m 512]

With N > 1 (one process per GPU under torchrun) both weights are split column-wise (N) across the ranks; every rank's
epilogue stores its columns of the SwiGLU output and of the block output into all ranks' buffers (peer stores over
NVLink) and the library's own flag barrier orders the ranks (NCCL all-gathers with P0P_BENCH_GATHER=nccl).  The
problem is fixed, so scaling is "strong".  `--impl reference` times the reference's CPU path (the oracle port, all
host threads) on the same bounded sample as the `cpu_baseline` leg.

Every loop that holds a cross-rank operation runs a number of iterations that is the same on every rank by
construction (a command-line value, or a value all-reduced first), never a per-rank clock.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HID, FF = 4096, 14336
METRIC, UNIT = "q4 dequant-GEMM TFLOP/s (LLM MLP block: rms+gate/up swiglu, down resadd)", "TFLOP/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "tensor": d["bf16_tflops"], "tensor_sustained": d.get("bf16_tflops_sustained"), "src": "measured"}
    return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "src": "fallback"}


def block_flops(M):
    return 2.0 * M * (2 * FF) * HID + 2.0 * M * HID * FF


def block_bytes(M):
    """algorithmic bytes of one block pass: weights once, fp32 tokens in, fp16 hidden out+in, fp32 residual read+write, stats, gamma"""
    w = (2 * FF * HID + HID * FF) * 5 // 8
    return w + M * HID * 4 + 2 * M * FF * 2 + 2 * M * HID * 4 + M * 8 + HID * 4


def synth_q4(rows, cols, seed, P, tile_rows=2048):
    """N(0, 0.02) weights quantised to q4g32a.t64.  A 2048-row slab is drawn and encoded, then repeated down the
    tensor: records are independent 64 x 32 blocks, so the repeated bytes are a valid tensor with the same value
    distribution (documented stand-in: the configs name no dataset)."""
    rs = np.random.default_rng(seed)
    tr = min(tile_rows, rows)
    slab = P.packQ4((rs.standard_normal(tr * cols) * 0.02).astype(np.float32), tr, cols)
    reps = -(-rows // tr)
    return np.tile(slab, reps)[: rows * cols * 5 // 8]


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs"""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try: self.proc.wait(timeout=5)
            except Exception: pass
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"): reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


_CPU_INPUTS = {}


def cpu_sample(M_rows, gu_cols, dn_cols, threads, seed=3, reps=1):
    """the reference's CPU path on a bounded sample of the block: M_rows tokens, the first gu_cols hidden columns of
    the gate/up GEMM (RMS prologue, SwiGLU) and the first dn_cols output columns of the down GEMM (residual add).
    Returns (flops, seconds) of `reps` passes; the inputs of a sample size are generated once and reused."""
    import oracle as O
    key = (M_rows, gu_cols, dn_cols, seed)
    if key not in _CPU_INPUTS:
        rs = np.random.default_rng(seed)
        X = O.round_f16(rs.standard_normal(M_rows * HID).astype(np.float32))
        gamma = (1 + 0.1 * rs.standard_normal(HID)).astype(np.float32)
        Wgu, _ = O.pack_q4((rs.standard_normal(2 * gu_cols * HID) * 0.02).astype(np.float32), 2 * gu_cols, HID)
        Wdn, _ = O.pack_q4((rs.standard_normal(dn_cols * FF) * 0.02).astype(np.float32), dn_cols, FF)
        Hfull = O.to_f16(rs.standard_normal(M_rows * FF).astype(np.float32))
        _CPU_INPUTS[key] = (X, gamma, Wgu, Wdn, Hfull)
    X, gamma, Wgu, Wdn, Hfull = _CPU_INPUTS[key]
    t0 = time.perf_counter()
    for _ in range(reps):
        ST = O.rowstats(X, M_rows, HID, rms=True)
        Hh = np.zeros(M_rows * gu_cols, np.uint16)
        O.gemm(enc="q4g32a.t64", X=X, W=Wgu, Y=Hh, M=M_rows, N=2 * gu_cols, K=HID, w_rows=2 * gu_cols, w_cols=HID, xmode="rms", epi="swiglu",
               wr0=0, wr1=gu_cols, ldy=gu_cols, ST=ST, PV=gamma, threads=threads)
        R = X[: M_rows * HID].reshape(M_rows, HID)[:, :dn_cols].copy()
        O.gemm(enc="q4g32a.t64", X=Hfull, W=Wdn, Y=R, M=M_rows, N=dn_cols, K=FF, w_rows=dn_cols, w_cols=FF, epi="resadd", threads=threads)
    dt = time.perf_counter() - t0
    fl = reps * (2.0 * M_rows * (2 * gu_cols) * HID + 2.0 * M_rows * dn_cols * FF)
    return fl, dt


CPU_SAMPLE = (512, FF // 2, HID // 2)      # tokens, hidden columns of gate/up, output columns of down: the bounded sample both CPU legs time


def cpu_sample_text(rows, gu, dn):
    return f"{rows} tokens x {gu} of {FF} hidden columns (gate/up, rms+swiglu) + {dn} of {HID} output columns (down, resadd), float64 accumulate"


def run_reference(args, rank):
    """--impl reference: the reference's own CPU implementation of the path (oracle port; the reference is JavaScript
    and no JavaScript engine exists here), all host threads, the bounded sample of CPU_SAMPLE per step; the
    single-thread rate (the reference's cpuGemm is single-threaded, test/kernels.test.js:29) beside it."""
    if rank != 0:
        return
    import oracle as O
    O.build()
    thr = max(O.max_threads(), len(os.sched_getaffinity(0)))       # torchrun pins OMP_NUM_THREADS to 1: the host's cores are still there
    rows, gu, dn = min(args.m, CPU_SAMPLE[0]), CPU_SAMPLE[1], CPU_SAMPLE[2]
    for _ in range(min(args.warmup, 2)): cpu_sample(1, 256, 128, thr)
    t = 0.0; fl = 0.0
    for _ in range(args.steps):
        f, d = cpu_sample(rows, gu, dn, thr); fl += f; t += d
    v = fl / t / 1e12
    f1, d1 = cpu_sample(128, 1024, 512, 1)
    sample = cpu_sample_text(rows, gu, dn)
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": t / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64 accumulate of f16 products",
                      "data": "synthetic", "config": {"workload": f"LLM MLP block q4, M={args.m} (configs[1]); CPU sample per step: {sample}"},
                      "cpu_baseline": {"value": v, "unit": UNIT, "cores": thr, "kind": "port", "sample": sample, "single_thread_value": f1 / d1 / 1e12},
                      "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}), flush=True)


def run_shapes(args, P, torch, gpu, stream, dev, pk, rank, world):
    """Plain GEMMs (no prologue, fp16 store) of given shapes, N-sharded over the ranks (no gather): one JSON line per
    shape with TFLOP/s, GB/s of the algorithmic bytes and both roofline fractions.  Weights are rotated so that
    every launch streams from HBM."""
    if args.sweep:
        shapes = [(e, m, n, k) for e in ("q4", "q8") for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336), (16384, 16384)) for m in (1, 16, 128, 1024, 8192)]
    else:
        shapes = [(t.split(":")[0], int(t.split(":")[1]), int(t.split(":")[2]), int(t.split(":")[3])) for t in args.shape.split(",")]
    rs = np.random.default_rng(7)
    for enc, M, N, K in shapes:
        encn = {"q4": "q4g32a.t64", "q8": "q8g64s.t64", "f16": "f16"}[enc]
        nl = N // world
        slab_rows = min(nl, 1024)
        W0 = (rs.standard_normal(slab_rows * K) * 0.02).astype(np.float32)
        slab = P.packQ4(W0, slab_rows, K) if enc == "q4" else P.packQ8(W0, slab_rows, K) if enc == "q8" else P.packF16(W0)
        wbytes = np.tile(slab, -(-nl // slab_rows))[: P.encodedBytes(encn, nl, K)]
        copies = max(2, min(8, int(np.ceil(300e6 / wbytes.nbytes))))
        Ws = [gpu.upload(wbytes) for _ in range(copies)]
        xb = gpu.upload(P.toF16(rs.standard_normal(M * K).astype(np.float32))); yb = gpu.buffer(M * nl * 2)
        def call(i):
            a = {"w": {"enc": encn, "buf": Ws[i], "off": 0, "bytes": wbytes.nbytes, "rows": nl, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": nl, "K": K}
            if args.kernel: a["kernel"] = args.kernel
            P.gemm(gpu, a)
        gs = []
        for i in range(copies):
            call(i); call(i); torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream): call(i)
            gs.append(g)
        fam = P._lib.KERNEL_NAMES.get(gpu.lastKernel)
        reps = max(args.steps, 10)
        for s in range(max(3, args.warmup)): gs[s % copies].replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(reps): gs[s % copies].replay()
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        fl = 2.0 * M * nl * K; by = wbytes.nbytes + M * K * 2 + M * nl * 2
        if rank == 0:
            print(json.dumps({"shape": {"enc": enc, "M": M, "N": N, "K": K, "n_gpus": world}, "family": fam, "ms": ms, "TFLOP/s": fl * world / (ms * 1e-3) / 1e12,
                              "GB/s": by * world / (ms * 1e-3) / 1e9, "frac_hbm": by / (ms * 1e-3) / 1e9 / pk["hbm"], "frac_tensor": fl / (ms * 1e-3) / 1e12 / pk["tensor"],
                              "weight_copies": copies}), flush=True)
        for b in Ws + [xb, yb]: gpu.free(b)
        gpu.drainPool()
    torch.cuda.synchronize()
    sys.stdout.flush()


def run_configs(args, P, torch, gpu, stream, dev, pk, rank, world):
    """The two other single-GPU configurations of the baseline, one JSON line each:
    dit_qkv  q8 projection of 3600 tokens, hidden 3072 -> 9216 with the LayerNorm + modulation prologue and the QK-norm + RoPE
             head-split epilogue (24 + 24 + 24 heads of 128);
    conv3    3x3x3 convolution of a 13 x 92 x 160 x 128 clip to 128 channels (fp16 weights in the converter's layout, bias),
             run whole and as 4-frame chunks out of a ring of 6 frames; the two outputs must be bit-identical."""
    rs = np.random.default_rng(11)

    def graph_time(fn, reps):
        fn(); fn(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream): fn()
        for _ in range(3): g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps): g.replay()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for name in args.config.split(","):
        if name == "dit_qkv":
            M, K, N, H = 3600, 3072, 9216, 24
            x = gpu.upload(rs.standard_normal(M * K).astype(np.float32)); st = gpu.buffer(M * 8)
            pv = gpu.upload(P.fromF16(P.toF16((rs.standard_normal(2 * K) * 0.5).astype(np.float32))))        # scale | shift, fp16-rounded values held as f32
            slab = P.packQ8((rs.standard_normal(1024 * K) * 0.02).astype(np.float32), 1024, K)
            wbytes = np.tile(slab, N // 1024)
            Ws = [gpu.upload(wbytes) for _ in range(5)]                                                      # 5 x 29 MB > L2
            ev = gpu.upload((1 + 0.1 * rs.standard_normal(256)).astype(np.float32))
            ang = rs.uniform(0, 6.28, M * 64).astype(np.float32)
            rp = gpu.upload(np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32).ravel())
            y = gpu.buffer(3 * H * M * 128 * 2)
            P.rowstats(gpu, {"x": {"buf": x}, "rows": M, "cols": K, "mode": "ln", "eps": 1e-6, "st": {"buf": st}})
            i = [0]
            def call():
                i[0] = (i[0] + 1) % len(Ws)
                a = {"w": {"enc": "q8g64s.t64", "buf": Ws[i[0]], "off": 0, "bytes": wbytes.nbytes, "rows": N, "cols": K}, "x": {"buf": x, "mode": "lnmod"},
                     "y": {"buf": y}, "M": M, "N": N, "K": K, "epi": "heads", "stats": {"buf": st}, "pv": {"buf": pv, "off": 0, "stride": K}, "ev": {"buf": ev},
                     "heads": {"Ltot": M, "Hq": H, "Hkv": H, "rowOff": 0, "eps": 1e-6, "rope": {"buf": rp}}}
                if args.kernel: a["kernel"] = args.kernel
                P.gemm(gpu, a)
            # one graph per weight copy would need five graphs; the kernel is 0.2 ms, so eager launches on the stream are timed instead
            for _ in range(5): call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(args.steps, 10)
            e0.record()
            for _ in range(reps): call()
            e1.record(); torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            fl = 2.0 * M * N * K; by = wbytes.nbytes + M * K * 4 + M * N * 2 + M * 8 + 2 * K * 4 + M * 128 * 4
            print(json.dumps({"config": "dit_qkv (configs[2])", "family": P._lib.KERNEL_NAMES.get(gpu.lastKernel), "M": M, "N": N, "K": K, "ms": ms,
                              "TFLOP/s": fl / (ms * 1e-3) / 1e12, "GB/s": by / (ms * 1e-3) / 1e9, "frac_tensor": fl / (ms * 1e-3) / 1e12 / pk["tensor"]}), flush=True)
            for b in Ws + [x, st, pv, ev, rp, y]: gpu.free(b)
            gpu.drainPool()
        elif name == "attention":
            # the attention that consumes the DiT projection's heads: 24 heads of 128 over 3600 tokens, no mask
            H, L = 24, 3600
            q = gpu.upload(P.toF16((rs.standard_normal(H * L * 128) * 0.5).astype(np.float32))); k = gpu.upload(P.toF16((rs.standard_normal(H * L * 128) * 0.5).astype(np.float32)))
            v = gpu.upload(P.toF16(rs.standard_normal(H * L * 128).astype(np.float32))); o = gpu.buffer(L * H * 128 * 2)
            def call(): P.attention(gpu, {"q": {"buf": q}, "k": {"buf": k}, "v": {"buf": v}, "o": {"buf": o}, "Lq": L, "Lk": L, "Hq": H, "Hkv": H, "mode": 0})
            ms = graph_time(call, max(3, min(args.steps, 20)))
            fl = 4.0 * L * L * 128 * H
            print(json.dumps({"config": "attention after dit_qkv (24 heads x 3600 tokens x 128, no mask)", "family": {16: "warp-level mma.sync flash attention", 17: "tcgen05 flash attention (V transposed by a pre-pass, inside the timed call)"}.get(gpu.lastKernel), "ms": ms,
                              "TFLOP/s": fl / (ms * 1e-3) / 1e12, "frac_tensor": fl / (ms * 1e-3) / 1e12 / pk["tensor"]}), flush=True)
            for b in (q, k, v, o): gpu.free(b)
        elif name == "conv3":
            T, Hh, Ww, C, N = 13, 92, 160, 128, 128
            K = 27 * C; fx = Hh * Ww * C; fy = Hh * Ww * N
            clip_t = (torch.randn(T * fx, device=dev, dtype=torch.float32)).to(torch.float16)
            clip = gpu.wrap(clip_t.data_ptr(), clip_t.numel() * 2)
            w5 = (rs.standard_normal(N * C * 27) * 0.03).astype(np.float32)                                   # [N][C][3][3][3] as a checkpoint holds it
            wk = P.reorderConvRows(w5, N, [N, C, 3, 3, 3])                                                              # -> [N][(kt ky kx) C], the kernel's layout
            wb = gpu.upload(P.toF16(wk)); bias = gpu.upload((rs.standard_normal(N) * 0.1).astype(np.float32))
            ya_t = torch.zeros(T * fy, device=dev, dtype=torch.float16); yb_t = torch.zeros(T * fy, device=dev, dtype=torch.float16)
            ya, yb = gpu.wrap(ya_t.data_ptr(), T * fy * 2), gpu.wrap(yb_t.data_ptr(), T * fy * 2)
            ring_t = torch.zeros(6 * fx, device=dev, dtype=torch.float16); ring = gpu.wrap(ring_t.data_ptr(), 6 * fx * 2)

            def conv(xbuf, xoff, ybuf, yoff, t0, nf, padL, ks):
                a = {"w": {"enc": "f16", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xbuf, "off": xoff}, "y": {"buf": ybuf, "off": yoff},
                     "M": nf * Hh * Ww, "N": N, "K": K, "epi": "bias", "ev": {"buf": bias},
                     "conv": {"kind": "conv3", "Hi": Hh, "Wi": Ww, "Ci": C, "Ho": Hh, "Wo": Ww, "stride": T, "padT": t0, "padL": padL, "ks": ks}}
                if args.kernel: a["kernel"] = args.kernel
                P.gemm(gpu, a)

            def whole(): conv(clip, 0, ya, 0, 0, T, 0, 1)
            def chunks():
                have = set()
                for t0 in range(0, T, 4):
                    nf = min(4, T - t0)
                    for g in range(max(0, t0 - 1), min(T - 1, t0 + nf) + 1):                                   # frames t0-1 .. t0+nf into their ring slots
                        if g not in have:
                            ring_t[(g % 6) * fx:(g % 6 + 1) * fx].copy_(clip_t[g * fx:(g + 1) * fx]); have.add(g)
                    conv(ring, 0, yb, t0 * fy * 2, t0, nf, 0, 6)
            reps = max(3, min(args.steps, 20))
            ms_w = graph_time(whole, reps); fam = P._lib.KERNEL_NAMES.get(gpu.lastKernel)
            ms_c = graph_time(chunks, reps)
            torch.cuda.synchronize()
            same = bool(torch.equal(ya_t.view(torch.int16), yb_t.view(torch.int16)))
            if world > 1:
                # N = 128 output channels do not split along N: the ranks split the OUTPUT FRAMES (one-frame halo through padT / padL),
                # every rank holding the clip; each rank's frames must hold the bits of the whole-clip call
                import torch.distributed as dist
                yc_t = torch.zeros(T * fy, device=dev, dtype=torch.float16); yc = gpu.wrap(yc_t.data_ptr(), T * fy * 2)
                wa = {"w": {"enc": "f16", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": clip, "off": 0}, "y": {"buf": yc, "off": 0},
                      "M": T * Hh * Ww, "N": N, "K": K, "epi": "bias", "ev": {"buf": bias},
                      "conv": {"kind": "conv3", "Hi": Hh, "Wi": Ww, "Ci": C, "Ho": Hh, "Wo": Ww, "stride": T, "padT": 0, "padL": 0, "ks": 1}}
                mine = P.conv3_frame_shard(wa, rank, world); t0f, nff = P.shard_frames(T, rank, world)
                def shard():
                    if mine is not None: P.gemm(gpu, mine)
                ms_s = graph_time(shard, reps) if mine is not None else 0.0
                tt = torch.tensor([ms_s], device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); ms_s = float(tt.item())
                ok = torch.tensor([1 if torch.equal(yc_t[t0f * fy:(t0f + nff) * fy].view(torch.int16), ya_t[t0f * fy:(t0f + nff) * fy].view(torch.int16)) else 0], device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if rank == 0:
                    fl_ = 2.0 * T * Hh * Ww * N * K
                    print(json.dumps({"config": "conv3 (configs[3]) split by output frames", "n_gpus": world, "frames_per_rank": [P.shard_frames(T, r, world)[1] for r in range(world)],
                                      "ms": ms_s, "TFLOP/s": fl_ / (ms_s * 1e-3) / 1e12, "speedup_vs_one_gpu_whole_clip": ms_w / ms_s,
                                      "frame_shards_bit_identical_to_whole": bool(ok.item())}), flush=True)
            fl = 2.0 * T * Hh * Ww * N * K; by = T * fx * 2 + N * K * 2 + T * fy * 2 + N * 4
            if rank == 0: print(json.dumps({"config": "conv3 (configs[3])", "family": fam, "M": T * Hh * Ww, "N": N, "K": K, "ms_whole": ms_w, "ms_chunks_of_4_from_ring_of_6": ms_c,
                              "TFLOP/s_whole": fl / (ms_w * 1e-3) / 1e12, "TFLOP/s_chunks": fl / (ms_c * 1e-3) / 1e12, "GB/s_whole": by / (ms_w * 1e-3) / 1e9,
                              "frac_tensor_whole": fl / (ms_w * 1e-3) / 1e12 / pk["tensor"], "chunks_bit_identical_to_whole": same}), flush=True)
    torch.cuda.synchronize()
    sys.stdout.flush()


# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this
# command, see profiles/), keyed by (call, tokens, kernel family, ranks, kernel plan).  A launch whose plan differs from the
# captured one reports null rather than a stale figure.
TRAFFIC = {
    # dram__bytes_read.sum + dram__bytes_write.sum of the k_gemm_umma launch of the gate/up call (the norm pre-pass adds 12.6 MB)
    ("gate_up", 512, "umma", 1): {"bytes": 81271296.0, "plan": "448 tiles of 128 x 256, last round split along K", "captured_at": "71786ec"},
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=512, help="tokens per step of the headline (512 = the tensor-bound case of the config)")
    ap.add_argument("--copies", type=int, default=3, help="weight copies rotated through so that every step streams from HBM")
    ap.add_argument("--rounds", type=int, default=5, help="the headline is the median of this many rounds of --steps steps")
    ap.add_argument("--skip-cases", action="store_true", help="only the headline (for profiler captures)")
    ap.add_argument("--kernel", default=None, help="force a kernel family (generic | decode | umma)")
    ap.add_argument("--shape", default=None, help="enc:M:N:K[,enc:M:N:K...]  time plain GEMMs of these shapes instead of the block (q4|q8|f16)")
    ap.add_argument("--config", default=None, help="dit_qkv | conv3 | attention [,…]: time the baseline's other single-GPU configurations instead of the block")
    ap.add_argument("--sweep", action="store_true", help="the large-shape sweep of the baseline's configs (q4/q8, M in 1..8192, four (N,K))")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1)); local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch
    import torch.distributed as dist
    import p0pc0rn_kernels_b200 as P
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        # a short time-out: should the ranks ever disagree on a collective, the run ends with an error instead of spinning
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # every launch of the library and every torch op / event below shares ONE non-default stream
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    gpu = P.createGpu({"device": local, "stream": stream.cuda_stream})
    pk = peaks()

    try:
        if args.shape or args.sweep:
            run_shapes(args, P, torch, gpu, stream, dev, pk, rank, world)
        elif args.config:
            run_configs(args, P, torch, gpu, stream, dev, pk, rank, world)
        else:
            run_block(args, P, torch, dist, gpu, stream, dev, pk, rank, world, local)
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush(); sys.stderr.flush()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()


def run_block(args, P, torch, dist, gpu, stream, dev, pk, rank, world, local):
    # ---- model state: this rank's column shard of both weights (the whole weights at N = 1), `copies` times
    ffl, hidl = FF // world, HID // world
    gu_full = synth_q4(2 * FF, HID, 1, P); dn_full = synth_q4(HID, FF, 2, P)
    gu_mine = P.shard_swiglu_bytes(gu_full, "q4g32a.t64", FF, HID, rank, world)
    dn_mine = P.shard_bytes(dn_full, "q4g32a.t64", HID, FF, rank, world)
    del gu_full, dn_full
    Wgu = [gpu.upload(gu_mine, f"gate_up.{i}") for i in range(args.copies)]
    Wdn = [gpu.upload(dn_mine, f"down.{i}") for i in range(args.copies)]
    gamma = gpu.upload((1 + 0.1 * np.random.default_rng(4).standard_normal(HID)).astype(np.float32), "gamma")
    w_bytes = gu_mine.nbytes + dn_mine.nbytes
    Mmax = max(args.m, 16)

    def wrap(t):
        return gpu.wrap(t.data_ptr(), t.numel() * t.element_size())

    st_t = torch.zeros(Mmax * 2, dtype=torch.float32, device=dev); st = wrap(st_t)
    class DevView:
        """a library buffer as a torch tensor (no copy), through the CUDA array interface"""
        def __init__(self, buf, n, typestr):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (buf.ptr, False), "version": 2}

    # the residual stream and the full hidden row live in library buffers (cudaMalloc), so that other ranks can map them
    xb = gpu.buffer(Mmax * HID * 4, "residual", shareable=world > 1); x_t = torch.as_tensor(DevView(xb, Mmax * HID, "<f4"), device=dev)      # residual stream (fp32)
    hl_t = torch.zeros(Mmax * ffl, dtype=torch.float16, device=dev); hl = wrap(hl_t)                # this rank's SwiGLU columns (gather path)
    if world == 1: hf, hf_t = hl, hl_t
    else: hf = gpu.buffer(Mmax * FF * 2, "hidden", shareable=True); hf_t = torch.as_tensor(DevView(hf, Mmax * FF, "<f2"), device=dev)   # the full hidden row
    # ---- N > 1: every rank maps the others' hidden and residual buffers and flag blocks; the epilogues then store each rank's
    # columns into all copies (peer stores over NVLink) and the library's flag barrier orders the ranks, instead of an all-gather
    # plus re-layout.  Every rank runs the same collectives here whatever fails locally: a failure travels as data.
    hf_peers, x_peers, flag_peers, flags, fused = [], [], [None] * world, None, False
    if world > 1 and os.environ.get("P0P_BENCH_GATHER", "") != "nccl":
        mine, err = None, None
        try:
            flags = gpu.buffer(gpu.PEER_FLAG_BYTES, "flags", shareable=True)
            mine = (gpu.ipcExport(hf), gpu.ipcExport(xb), gpu.ipcExport(flags))
        except Exception as e:
            err = str(e)
        every = [None] * world
        dist.all_gather_object(every, mine)
        if all(h is not None for h in every):
            try:
                for r, (hh, hx, hfl) in enumerate(every):
                    if r != rank:
                        hf_peers.append(gpu.ipcOpen(hh, Mmax * FF * 2, f"hidden@{r}")); x_peers.append(gpu.ipcOpen(hx, Mmax * HID * 4, f"residual@{r}"))
                        flag_peers[r] = gpu.ipcOpen(hfl, gpu.PEER_FLAG_BYTES, f"flags@{r}")
                fused = True
            except Exception as e:                                               # no peer access on this box: the NCCL gather path below
                err = str(e)
        ok_t = torch.tensor([1 if fused else 0], device=dev); dist.all_reduce(ok_t, op=dist.ReduceOp.MIN); fused = bool(ok_t.item())
        if not fused:
            if rank == 0: print(f"peer mapping failed ({err}); using NCCL all-gathers", file=sys.stderr)
            hf_peers, x_peers = [], []
    BARRIER_CYCLES = 10_000_000_000          # bounded wait of the flag barrier: seconds, far above any skew between ranks in lockstep
    x_host = np.random.default_rng(5).standard_normal(Mmax * HID).astype(np.float32)
    x_t.copy_(torch.from_numpy(x_host))
    launches = {"n": 0}

    def order_ranks():
        """every rank's columns are in every copy once all ranks are past this point of their streams"""
        if fused: gpu.peerBarrier(flags, flag_peers, rank, world, BARRIER_CYCLES)

    def block(M, i, gather=True, xb=xb, xp=None):
        """one pass of the MLP block over M tokens with weight copy i (xb: the residual stream it updates in place; xp: the other
        ranks' copies of that buffer)"""
        xp = x_peers if xp is None else xp
        P.rowstats(gpu, {"x": {"buf": xb}, "rows": M, "cols": HID, "mode": "rms", "eps": 1e-6, "st": {"buf": st}})
        yh = {"buf": hf, "ld": FF, "n0": rank * ffl, "peers": hf_peers} if fused else {"buf": hl, "ld": ffl}
        a = {"w": {"enc": "q4g32a.t64", "buf": Wgu[i], "off": 0, "bytes": gu_mine.nbytes, "rows": 2 * ffl, "cols": HID}, "x": {"buf": xb, "mode": "rms"},
             "y": yh, "M": M, "N": 2 * ffl, "K": HID, "wr0": 0, "wr1": ffl, "epi": "swiglu", "stats": {"buf": st}, "pv": {"buf": gamma}}
        if args.kernel: a["kernel"] = args.kernel
        P.gemm(gpu, a)
        if fused and gather: order_ranks()
        elif world > 1 and gather:
            hf_t[: M * FF].view(M, FF).copy_(P.all_gather_columns(hl_t[: M * ffl].view(M, ffl)))
        # residual add, in place, into this rank's columns of the (replicated) fp32 residual stream
        a = {"w": {"enc": "q4g32a.t64", "buf": Wdn[i], "off": 0, "bytes": dn_mine.nbytes, "rows": hidl, "cols": FF}, "x": {"buf": hf},
             "y": {"buf": xb, "ld": HID, "n0": rank * hidl, "peers": xp if fused else []}, "M": M, "N": hidl, "K": FF, "epi": "resadd"}
        if args.kernel: a["kernel"] = args.kernel
        P.gemm(gpu, a)
        if fused and gather: order_ranks()
        elif world > 1 and gather:
            xv = x_t[: M * HID].view(M, HID)
            xv.copy_(P.all_gather_columns(xv[:, rank * hidl:(rank + 1) * hidl]))

    def graphs_of(fn):
        """one CUDA graph per weight copy holding the launches fn(i) makes (launch-bound steps would otherwise time the host)"""
        gs = []
        for i in range(args.copies):
            fn(i); fn(i)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn(i)
            gs.append(g)
        return gs

    def run_steps(gs, steps):
        """exactly `steps` graph replays bracketed by barrier + synchronize on both sides; device time, max over ranks"""
        torch.cuda.synchronize()
        if world > 1: dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps): gs[s % args.copies].replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1: dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
        return ms / steps

    def timed(M, steps, warmup, rounds, gather=True):
        """median over `rounds` rounds of exactly `steps` steps each (the weight copies rotate through every round)"""
        l0 = gpu.launches
        block(M, 0, gather)
        per_step = gpu.launches - l0
        gs = graphs_of(lambda i: block(M, i, gather))
        for s in range(warmup): gs[s % args.copies].replay()
        per_round = [run_steps(gs, steps) for _ in range(rounds)]
        launches["n"] = per_step * steps
        return float(np.median(per_round)), per_round, gs

    def one_gemm(M, which, i):
        if which == "gate_up":
            a = {"w": {"enc": "q4g32a.t64", "buf": Wgu[i], "off": 0, "bytes": gu_mine.nbytes, "rows": 2 * ffl, "cols": HID}, "x": {"buf": xb, "mode": "rms"},
                 "y": {"buf": hl, "ld": ffl}, "M": M, "N": 2 * ffl, "K": HID, "wr0": 0, "wr1": ffl, "epi": "swiglu", "stats": {"buf": st}, "pv": {"buf": gamma}}
        else:
            a = {"w": {"enc": "q4g32a.t64", "buf": Wdn[i], "off": 0, "bytes": dn_mine.nbytes, "rows": hidl, "cols": FF}, "x": {"buf": hf},
                 "y": {"buf": xb, "ld": HID, "n0": rank * hidl}, "M": M, "N": hidl, "K": FF, "epi": "resadd"}
        if args.kernel: a["kernel"] = args.kernel
        P.gemm(gpu, a)

    def kernel_ms(M, which, reps):
        """average device time of ONE gemm call of the block (gate/up or down): graphs of that call alone (no cross-rank
        operation inside), replayed back to back over the rotating weight copies, CUDA events around the run"""
        P.rowstats(gpu, {"x": {"buf": xb}, "rows": M, "cols": HID, "mode": "rms", "eps": 1e-6, "st": {"buf": st}})
        gs = graphs_of(lambda i: one_gemm(M, which, i))
        fam = gpu.lastKernel
        for s in range(3): gs[s % args.copies].replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(reps): gs[s % args.copies].replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, fam

    # ---- headline: the median of `rounds` rounds of K timed steps at M = args.m
    M = args.m
    sampler = ClockSampler(local)
    if rank == 0: sampler.start()
    ms, per_round, gs_head = timed(M, args.steps, max(3, args.warmup), max(1, args.rounds))
    n_launch = launches["n"]
    gu_ms, gu_kernel = kernel_ms(M, "gate_up", max(20, min(100, args.steps)))
    # keep the GPU under the same load until the sampler (200 ms period) has a few readings of the clocks.  The replay count
    # comes from `ms`, which was all-reduced above: the same on every rank (each replay holds cross-rank barriers).
    n_load = int(min(20000, max(50, 1.2 / (ms * 1e-3))))
    for s in range(n_load): gs_head[s % args.copies].replay()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    value = block_flops(M) / (ms * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers: upload tokens, run, read the result
    import ctypes as C
    from p0pc0rn_kernels_b200._lib import lib
    hp = C.c_void_p(); gpu._check(lib.p0p_host_alloc(gpu._h, M * HID * 4, C.byref(hp)))
    pin_in = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_float)), shape=(M * HID,)); pin_in[:] = x_host[: M * HID]
    out_bytes = M * HID * 4
    hq = C.c_void_p(); gpu._check(lib.p0p_host_alloc(gpu._h, out_bytes, C.byref(hq)))
    pin_out = np.ctypeslib.as_array(C.cast(hq, C.POINTER(C.c_uint8)), shape=(out_bytes,))       # page-locked destination of the step's result

    def e2e_step(i):
        gpu.upload(pin_in, "", xb, 0)           # the step's tokens (fp32 residual stream), page-locked host -> device
        block(M, i)
        return gpu.read(xb, 0, out_bytes, out=pin_out)       # the updated residual stream, device -> page-locked host

    for s in range(3): e2e_step(s % args.copies)
    torch.cuda.synchronize()
    if world > 1: dist.barrier()
    t0 = time.perf_counter()
    n_e2e = max(5, min(args.steps, 30))
    for s in range(n_e2e): e2e_step(s % args.copies)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); e2e_ms = float(t.item())
    h2d = M * HID * 4
    e2e = {"value": block_flops(M) / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": out_bytes, "ms_per_step": e2e_ms,
           "pipeline": "none: upload, block, read-back one after the other on one stream"}
    # ---- the same steps as a serving loop would run them: three contexts of the library on three streams (upload / block /
    # read-back) over a ring of three residual buffers, so that step i's block runs while step i + 1's tokens arrive and step
    # i - 1's result leaves.  Every step still makes its own host -> device copy from page-locked memory and its own device ->
    # host read through the public API, inside the timed region.  N > 1: every rank maps the others' three buffers (the down
    # GEMM stores into the peers' copy of the step's buffer); the barriers inside each step keep the ranks in lockstep, so a
    # buffer is only written by peers between its owner's upload and its owner's read-back.  (With the NCCL gather path the
    # plain loop stays.)
    NB = 3
    pipe_ok = world == 1 or fused
    xbs, xps = [], [[] for _ in range(NB)]
    if pipe_ok:
        mine, err = None, None
        try:
            xbs = [gpu.buffer(M * HID * 4, f"residual.{b}", shareable=world > 1) for b in range(NB)]
            if world > 1: mine = [gpu.ipcExport(b) for b in xbs]
        except Exception as e:
            err = str(e); pipe_ok = False
        if world > 1:
            every = [None] * world
            dist.all_gather_object(every, mine)
            if pipe_ok and all(h is not None for h in every):
                try:
                    for r in range(world):
                        if r != rank:
                            for b in range(NB): xps[b].append(gpu.ipcOpen(every[r][b], M * HID * 4, f"residual.{b}@{r}"))
                except Exception as e:
                    err = str(e); pipe_ok = False
            else: pipe_ok = False
            ok_t = torch.tensor([1 if pipe_ok else 0], device=dev); dist.all_reduce(ok_t, op=dist.ReduceOp.MIN); pipe_ok = bool(ok_t.item())
            if not pipe_ok and rank == 0: print(f"pipelined end-to-end leg skipped ({err})", file=sys.stderr)
    if pipe_ok:
        s_up, s_dn = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        g_up = P.createGpu({"device": local, "stream": s_up.cuda_stream}); g_dn = P.createGpu({"device": local, "stream": s_dn.cuda_stream})
        up_view = [g_up.wrap(b.ptr, M * HID * 4) for b in xbs]; dn_view = [g_dn.wrap(b.ptr, M * HID * 4) for b in xbs]
        hu = C.c_void_p(); g_up._check(lib.p0p_host_alloc(g_up._h, M * HID * 4, C.byref(hu)))
        pin_up = np.ctypeslib.as_array(C.cast(hu, C.POINTER(C.c_float)), shape=(M * HID,)); pin_up[:] = x_host[: M * HID]
        pin_dn = []
        for b in range(NB):
            hd = C.c_void_p(); g_dn._check(lib.p0p_host_alloc(g_dn._h, out_bytes, C.byref(hd)))
            pin_dn.append(np.ctypeslib.as_array(C.cast(hd, C.POINTER(C.c_uint8)), shape=(out_bytes,)))
        graphs = {}
        for b in range(NB):
            for i in range(args.copies):
                block(M, i, True, xbs[b], xps[b]); torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream): block(M, i, True, xbs[b], xps[b])
                graphs[(b, i)] = g
        ev_up = [torch.cuda.Event() for _ in range(NB)]; ev_c = [torch.cuda.Event() for _ in range(NB)]; ev_dn = [torch.cuda.Event() for _ in range(NB)]

        def enqueue(sidx):
            b = sidx % NB
            s_up.wait_event(ev_dn[b])                                    # the buffer's previous result has left
            g_up.upload(pin_up, "", up_view[b], 0); ev_up[b].record(s_up)
            stream.wait_event(ev_up[b]); graphs[(b, sidx % args.copies)].replay(); ev_c[b].record(stream)

        def collect(sidx):
            b = sidx % NB
            s_dn.wait_event(ev_c[b])
            g_dn.read(dn_view[b], 0, out_bytes, out=pin_dn[b]); ev_dn[b].record(s_dn)

        def pipelined(n):
            for sidx in range(n):
                enqueue(sidx)
                if sidx >= NB - 1: collect(sidx - (NB - 1))
            for sidx in range(max(0, n - (NB - 1)), n): collect(sidx)

        pipelined(6); torch.cuda.synchronize()
        n_p = max(10, min(args.steps, 60))
        if world > 1: dist.barrier()
        t0 = time.perf_counter(); pipelined(n_p); torch.cuda.synchronize()
        p_ms = (time.perf_counter() - t0) / n_p * 1e3
        # the pipelined result is the plain loop's: same tokens in, same bits out
        same = bool(np.array_equal(pin_dn[(n_p - 1) % NB], pin_out))
        if world > 1:
            t = torch.tensor([p_ms, 0.0 if same else 1.0], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); p_ms = float(t[0].item()); same = float(t[1].item()) == 0.0
        e2e = {"value": block_flops(M) / (p_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": out_bytes, "ms_per_step": p_ms,
               "pipeline": "3 streams (upload / block / read-back) over a ring of 3 residual buffers; every step copies its tokens in and its result out",
               "unpipelined": {"value": block_flops(M) / (e2e_ms * 1e-3) / 1e12, "ms_per_step": e2e_ms}, "matches_unpipelined_bits": same}
        for v in up_view: g_up.free(v)
        for v in dn_view: g_dn.free(v)
        del graphs
        torch.cuda.synchronize()
        if world > 1: dist.barrier()               # nobody unmaps a buffer a peer's last step may still store into
        for b in range(NB):
            for q in xps[b]: gpu.free(q)
        for b in xbs: gpu.free(b)

    # ---- N > 1: one more block from the same tokens, checked.  Every rank's copy of the hidden row and of the residual must
    # hold the same bits (each rank wrote its columns into all copies): element-wise MAX and MIN over the ranks agree.  Rank 0
    # also compares the residual with the same block run unsharded on its own GPU.  A failed check ends the run non-zero.
    check = None
    if world > 1:
        x_t[: M * HID].copy_(torch.from_numpy(x_host[: M * HID])); torch.cuda.synchronize(); dist.barrier()
        block(M, 0); torch.cuda.synchronize(); dist.barrier()
        identical = {}
        for name, tns in (("hidden", hf_t[: M * FF].view(torch.int16).to(torch.int32)), ("residual", x_t[: M * HID].view(torch.int32).clone())):
            hi, lo = tns.clone(), tns.clone()
            dist.all_reduce(hi, op=dist.ReduceOp.MAX); dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            identical[name] = bool(torch.equal(hi, lo))
        rel = None
        if rank == 0:
            got = x_t[: M * HID].clone()
            Wg = gpu.upload(synth_q4(2 * FF, HID, 1, P), "gate_up.full"); Wd = gpu.upload(synth_q4(HID, FF, 2, P), "down.full")
            x2 = gpu.upload(x_host[: M * HID], "x.full"); h2 = gpu.buffer(M * FF * 2); x2_t = torch.as_tensor(DevView(x2, M * HID, "<f4"), device=dev)
            P.rowstats(gpu, {"x": {"buf": x2}, "rows": M, "cols": HID, "mode": "rms", "eps": 1e-6, "st": {"buf": st}})
            P.gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": Wg, "off": 0, "bytes": Wg._pf, "rows": 2 * FF, "cols": HID}, "x": {"buf": x2, "mode": "rms"}, "y": {"buf": h2, "ld": FF},
                         "M": M, "N": 2 * FF, "K": HID, "wr0": 0, "wr1": FF, "epi": "swiglu", "stats": {"buf": st}, "pv": {"buf": gamma}})
            P.gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": Wd, "off": 0, "bytes": Wd._pf, "rows": HID, "cols": FF}, "x": {"buf": h2}, "y": {"buf": x2, "ld": HID},
                         "M": M, "N": HID, "K": FF, "epi": "resadd"})
            torch.cuda.synchronize()
            rel = float(((got - x2_t).double().norm() / x2_t.double().norm()).item())
            for bfr in (Wg, Wd, x2, h2): gpu.free(bfr)
        dist.barrier()
        check = {"replicas_bit_identical": identical["residual"], "hidden_replicas_bit_identical": identical["hidden"], "rel_l2_vs_unsharded_on_rank0": rel}
        bad = torch.tensor([0 if (identical["residual"] and identical["hidden"] and (rank != 0 or (rel is not None and rel <= 1e-3))) else 1], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            if rank == 0: print(f"MULTI-GPU CHECK FAILED: {check}", file=sys.stderr)
            raise SystemExit(3)

    # ---- decode-sized cases of the same config (HBM-bound): GB/s of the algorithmic bytes
    cases = []
    if not args.skip_cases:
        for Mc in (1, 16):
            msc, _, _ = timed(Mc, max(20, args.steps), 5, 3, gather=True)
            gbs = block_bytes(Mc) / world / (msc * 1e-3) / 1e9 if world > 1 else block_bytes(Mc) / (msc * 1e-3) / 1e9
            kms, kk = kernel_ms(Mc, "gate_up", 60)
            dms, _ = kernel_ms(Mc, "down", 60)
            db = (hidl * FF * 5 // 8) + Mc * FF * 2 + 2 * Mc * hidl * 4
            kb = (2 * ffl * HID * 5 // 8) + Mc * HID * 4 + Mc * ffl * 2
            cases.append({"M": Mc, "ms_per_step": msc, "GB/s": gbs * (world if world > 1 else 1), "TFLOP/s": block_flops(Mc) / (msc * 1e-3) / 1e12,
                          "gate_up_kernel": {"ms": kms, "GB/s": kb / (kms * 1e-3) / 1e9, "frac_hbm": kb / (kms * 1e-3) / 1e9 / pk["hbm"], "family": P._lib.KERNEL_NAMES.get(kk)},
                          "down_kernel": {"ms": dms, "GB/s": db / (dms * 1e-3) / 1e9, "frac_hbm": db / (dms * 1e-3) / 1e9 / pk["hbm"]}})

    # ---- roofline of the dominant kernel (gate/up GEMM: 2/3 of the block's FLOPs)
    gu_flops = 2.0 * M * (2 * ffl) * HID
    fam_name = P._lib.KERNEL_NAMES.get(gu_kernel)
    tr = TRAFFIC.get(("gate_up", M, fam_name, world))
    roof = {"bound": "tensor", "achieved": gu_flops / (gu_ms * 1e-3) / 1e12, "peak": pk["tensor"], "unit": "TFLOP/s", "traffic": tr["bytes"] if tr else None,
            "traffic_source": f"ncu capture at {tr['captured_at']} ({tr['plan']})" if tr else None,
            "kernel": f"gate/up GEMM call ({fam_name} family: norm pre-pass + tensor-core kernel), M={M}", "ms_per_launch": gu_ms, "peak_source": pk["src"] + " (burst cuBLAS bf16)"}
    roof["frac"] = roof["achieved"] / roof["peak"]

    if rank == 0:
        # CPU baseline: the oracle port on a bounded sample (the one --impl reference times), all host threads
        cpu = None
        if world == 1:                       # the CPU baseline is a single-GPU-run figure (and torchrun pins its ranks to one thread)
            import oracle as O
            O.build(); thr = max(O.max_threads(), len(os.sched_getaffinity(0)))
            cpu_sample(1, 256, 128, thr)
            rows, gu, dn = min(M, CPU_SAMPLE[0]), CPU_SAMPLE[1], CPU_SAMPLE[2]
            f, d = cpu_sample(rows, gu, dn, thr, reps=4)
            f1, d1 = cpu_sample(128, 1024, 512, 1)
            cpu = {"value": f / d / 1e12, "unit": UNIT, "cores": thr, "kind": "port", "sample": cpu_sample_text(rows, gu, dn) + f", 4 passes, {d:.1f} s",
                   "single_thread_value": f1 / d1 / 1e12}
        out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
               "rounds": len(per_round), "ms_per_step_rounds": per_round,
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate (q4 weights dequantised in-kernel)",
               "data": "synthetic",
               "config": {"workload": f"LLM MLP block q4, M={M} tokens: rowstats + gate/up K4096->2x14336 (rms, swiglu) + down K14336->4096 (resadd) (configs[1])",
                          "hidden": HID, "ffn": FF, "tokens": M, "partition": f"N-sharded x{world}" + ("" if world == 1 else " + epilogues store each rank's columns into every rank's buffers (peer stores), flag barrier of the library's own" if fused else " + NCCL all-gather of hidden and output"),
                          "l2": f"{args.copies} weight copies rotated ({args.copies * w_bytes / 1e6:.0f} MB per rank > 126 MB L2)",
                          "timing": f"median of {len(per_round)} rounds of {args.steps} steps, each round bracketed by barrier + synchronize"},
               "e2e": e2e, "multi_gpu_check": check, "gpu_launches": n_launch, "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "cases": cases,
               "GB/s": block_bytes(M) / (ms * 1e-3) / 1e9}
        print(json.dumps(out), flush=True)
    torch.cuda.synchronize()
    del gs_head


if __name__ == "__main__":
    main()
