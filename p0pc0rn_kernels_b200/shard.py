"""Column-wise (N) partition of the gemm across GPUs, one process per GPU.

A weight in the tile-major encodings of the reference's docs/FORMAT.md is split on 64-row tile boundaries, so
a rank's rows are ONE contiguous byte range of the encoded tensor (docs/FORMAT.md:20, 41): a shard is uploaded
with a plain byte slice and the unchanged kernel runs on it with ``y.n0`` / ``y.ld`` placing its columns.  The
reference itself is single-device; this module has no counterpart there.

The only collective is the all-gather of the output, and only when the consumer needs the full row
(``all_gather_columns``); it runs through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in CPU tests).
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
