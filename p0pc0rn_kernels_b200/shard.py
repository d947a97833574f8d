"""Column-wise (N) partition of the gemm across GPUs, one process per GPU.

A weight in the tile-major encodings of the reference's docs/FORMAT.md is split on 64-row tile boundaries, so
a rank's rows are ONE contiguous byte range of the encoded tensor (docs/FORMAT.md:20, 41): a shard is uploaded
with a plain byte slice and the unchanged kernel runs on it with ``y.n0`` / ``y.ld`` placing its columns.  The
reference itself is single-device; this module has no counterpart there.

The only collective is the all-gather of the output, and only when the consumer needs the full row
(``all_gather_columns``); it runs through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in CPU tests).

The 3x3x3 convolution (``conv3``) has too few output channels to split along N (128 in the reference's models); it
splits by OUTPUT FRAMES instead: a rank computes frames [t0, t0 + nf) of the clip and reads input frames t0 - 1 ..
t0 + nf, the one-frame halo on each side being what the op's own chunk arguments (``padT`` / ``padL`` / ``x.off``,
src/ops/gemm.js:72-76) express.  A rank's call is the chunked call of the reference's tests
(test/kernels.test.js:123-131), so its frames hold the bits of the whole-clip call.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import ENC, lib


def shard_rows(enc: str, rows: int, cols: int, rank: int, world: int) -> dict:
    """-> {row0, rows, off, bytes}: the row range and the byte range of rank's shard of an encoded weight"""
    r0, nr, bo, nb = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
    rc = lib.p0p_shard_rows(ENC[enc] if enc in ENC else 3, rows, cols, rank, world, C.byref(r0), C.byref(nr), C.byref(bo), C.byref(nb))
    if rc == -1: raise ValueError(f"rank {rank} is not inside a world of {world}")
    if rc: raise ValueError(f"{rows} rows do not split into {world} shards of whole 64-row tiles")
    return {"row0": r0.value, "rows": nr.value, "off": bo.value, "bytes": nb.value}


def shard_weight(w: dict, rank: int, world: int) -> dict:
    """A weight view {enc, buf, off, bytes, rows, cols} of the full tensor -> the view of rank's rows inside the SAME
    buffer (for ranks that hold the whole tensor), plus `row0`."""
    s = shard_rows(w["enc"], w["rows"], w["cols"], rank, world)
    return dict(w, off=(w.get("off") or 0) + s["off"], bytes=s["bytes"], rows=s["rows"], row0=s["row0"])


def shard_bytes(data, enc: str, rows: int, cols: int, rank: int, world: int) -> np.ndarray:
    """the bytes of rank's shard out of the encoded tensor's bytes (what a rank uploads)"""
    s = shard_rows(enc, rows, cols, rank, world)
    u8 = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return u8[s["off"]:s["off"] + s["bytes"]]


def shard_swiglu_bytes(data, enc: str, half_rows: int, cols: int, rank: int, world: int) -> np.ndarray:
    """gate|up weight ([gate rows | up rows], 2*half_rows rows): rank's gate rows followed by its matching up rows,
    so the shard is again a [gate | up] tensor of 2*half_rows/world rows with wr1 = half_rows/world."""
    g = shard_rows(enc, half_rows, cols, rank, world)
    u8 = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    up0 = shard_rows(enc, half_rows, cols, 0, 1)["bytes"]
    return np.concatenate([u8[g["off"]:g["off"] + g["bytes"]], u8[up0 + g["off"]:up0 + g["off"] + g["bytes"]]])


def all_gather_columns(y_local, group=None):
    """[M][n_local] per rank -> [M][n_local * world] on every rank (rank r's columns at r * n_local).

    `ncclAllGather` concatenates along the slowest dimension, so the gather lands in a [world][M][n_local] staging
    tensor and one local permute restores row-major [M][N]; for M == 1 the staging tensor already is the row."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    M, n = y_local.shape
    stage = torch.empty((world * M, n), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stage, y_local.contiguous(), group=group)
    if M == 1:
        return stage.reshape(1, world * n)
    return stage.view(world, M, n).permute(1, 0, 2).reshape(M, world * n)


def shard_frames(T: int, rank: int, world: int) -> tuple:
    """-> (t0, nf): the contiguous range of output frames of rank; the first T % world ranks take one frame more (nf may be 0)"""
    if not 0 <= rank < world: raise ValueError(f"rank {rank} is not inside a world of {world}")
    q, r = divmod(T, world)
    return rank * q + min(rank, r), q + (1 if rank < r else 0)


def conv3_frame_shard(a: dict, rank: int, world: int, local_input: bool = False) -> dict | None:
    """The gemm arguments of rank's output frames, from the arguments `a` of the whole-clip conv3 call (padT = padL = 0,
    ks = 1, stride = T, M = T * Ho * Wo; fp16 output).  None when the rank has no frame.

    The result addresses the whole clip and the whole output (every rank holds both, or maps them): x.off skips to
    the first input frame the rank reads (padL = max(0, t0 - 1)), y.off to its first output frame.  With `local_input`
    the rank holds ONLY its input frames [in0, in0 + nin) in a buffer of its own: x.off stays as given and the extra keys
    `in0` / `nin` say which frames to put there."""
    cv = a["conv"]
    if cv.get("kind") != "conv3" or (cv.get("ks") or 1) != 1 or cv.get("padT") or cv.get("padL"):
        raise ValueError("conv3_frame_shard takes the arguments of a whole-clip conv3 call")
    T, hw = int(cv["stride"]), int(cv["Ho"]) * int(cv["Wo"])
    if a["M"] != T * hw: raise ValueError("conv3_frame_shard: M must be T * Ho * Wo")
    t0, nf = shard_frames(T, rank, world)
    if nf == 0: return None
    padL = max(0, t0 - 1)
    fx = int(cv["Hi"]) * int(cv["Wi"]) * int(cv["Ci"]) * 2                       # bytes of an input frame (fp16 THWC)
    fy = hw * int(a["y"].get("ld") or a["N"]) * 2                                # bytes of an output frame
    b = dict(a, M=nf * hw, conv=dict(cv, padT=t0, padL=padL),
             x=dict(a["x"], off=(a["x"].get("off") or 0) + (0 if local_input else padL * fx)),
             y=dict(a["y"], off=(a["y"].get("off") or 0) + t0 * fy))
    if local_input: b["in0"], b["nin"] = padL, min(T - 1, t0 + nf) - padL + 1
    return b


def all_gather_frames(y_local, T: int, group=None):
    """rank's output frames [nf][frame elements] -> the whole clip's [T][frame elements] on every rank (frame ranges as
    shard_frames gives them; ranks may hold different frame counts, so the gather runs on blocks padded to the largest)"""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    q = -(-T // world)
    pad = torch.zeros((q,) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
    pad[: y_local.shape[0]] = y_local
    stage = torch.empty((world * q,) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stage, pad, group=group)
    parts = []
    for r in range(world):
        _, nf = shard_frames(T, r, world)
        parts.append(stage[r * q: r * q + nf])
    return torch.cat(parts, 0)
