"""Device context, buffers and fp16 helpers: the host-side mirror of the reference's core runtime
(src/core/gpu.js) over the C ABI of ``include/p0p.h``.  Names, argument meaning and error behaviour follow the
reference; what was a Promise there is a plain return value here (the CUDA stream is the in-order queue)."""
from __future__ import annotations

import ctypes as C
import json

import numpy as np

from ._lib import Opts, lib

MB = 1e6


class GpuError(Exception):
    """src/core/gpu.js:12"""


def _bytes_view(data) -> np.ndarray:
    if isinstance(data, (bytes, bytearray, memoryview)):
        return np.frombuffer(data, dtype=np.uint8)
    a = np.ascontiguousarray(data)
    return a.view(np.uint8).reshape(-1)


class Buffer:
    """A device buffer; ``_pf`` is its byte size, as on the reference's GPUBuffer (src/core/gpu.js:106)."""
    __slots__ = ("handle", "_pf", "size", "label", "_gpu")

    def __init__(self, gpu, handle, size, label=""):
        self._gpu = gpu; self.handle = handle; self._pf = size; self.size = size; self.label = label

    @property
    def ptr(self) -> int:
        return lib.p0p_buf_ptr(self.handle) or 0

    def __repr__(self):
        return f"<Buffer {self.label!r} {self._pf} B>"


class _Queue:
    """device.queue.writeBuffer(buf, dstByteOff, data, srcOffset, size): for a typed array source, srcOffset and
    size count ELEMENTS (the WebGPU rule the reference's ring test relies on, test/kernels.test.js:138)."""

    def __init__(self, gpu):
        self._g = gpu

    def writeBuffer(self, buf, dst_off, data, src_off=0, size=None):
        if isinstance(data, np.ndarray):
            flat = np.ascontiguousarray(data).reshape(-1)
            flat = flat[src_off:] if size is None else flat[src_off:src_off + size]
            raw = flat.view(np.uint8)
        else:
            raw = _bytes_view(data); raw = raw[src_off:] if size is None else raw[src_off:src_off + size]
        self._g._write(buf, dst_off, raw)


class _Device:
    def __init__(self, gpu):
        self.queue = _Queue(gpu)


class Gpu:
    """class Gpu of src/core/gpu.js:29-199 for the gemm path."""

    def __init__(self, opts=None):
        self.opts = {"powerPreference": "high-performance", "wantSubgroups": True, "wantF16": True, "maxDispatchSeconds": 0.2, "device": 0}
        self.opts.update(opts or {})
        self.bufs = set()
        self.lostInfo = None
        self.lastError = None
        # dispatch sizing does not exist on CUDA; the fields stay because callers read them (src/ops/gemm.js:288-289)
        self.rate = {"mm": 1.0e15, "mm32": 1.0e15, "mm16": 1.0e15, "attn": 0.5e15, "mem": 6.5e12}
        self.tune = None
        self.calib = None
        self._h = C.c_void_p()
        has_stream = "stream" in self.opts and self.opts["stream"] is not None
        o = Opts(C.sizeof(Opts), 1 if has_stream else 0, self.opts.get("stream") if has_stream else None)
        rc = lib.p0p_open(int(self.opts["device"]), C.byref(o), C.byref(self._h))
        if rc:
            raise GpuError({-2: "no such CUDA device", -3: "an sm_100 (B200) device is required"}.get(rc, f"no CUDA device (error {rc})"))
        n = lib.p0p_describe(self._h, None, 0)
        b = C.create_string_buffer(n)
        lib.p0p_describe(self._h, b, n)
        d = json.loads(b.value.decode())
        self.info = {"vendor": d["vendor"], "architecture": d["architecture"], "device": d["device"], "description": d["device"]}
        self._desc = d
        self.f16 = True; self.subgroups = True; self.sgMin = 32; self.sgMax = 32; self.sgOK16 = True
        self.limits = {"maxBufferSize": d["memMB"] << 20, "maxStorageBufferBindingSize": d["memMB"] << 20,
                       "maxComputeWorkgroupStorageSize": d["wgMem"], "maxComputeInvocationsPerWorkgroup": d["wgInv"]}
        self.device = _Device(self)

    # ---------------------------------------------------------------- errors
    def _check(self, rc: int):
        if rc == 0:
            return
        msg = (lib.p0p_last_error(self._h) or b"").decode()
        self.lastError = msg
        if rc > 0:   # CUDA error
            if lib.p0p_status(self._h):
                self.lostInfo = {"reason": "cuda", "message": msg}
                if self.opts.get("onLost"):
                    try: self.opts["onLost"](self.lostInfo)
                    except Exception: pass
            if self.opts.get("onError"): self.opts["onError"](msg)
            raise GpuError(msg)
        if rc == -10:           # a kernel gave up on a bounded wait: a device-side failure (the context stays usable)
            raise GpuError(msg)
        raise ValueError(msg)   # the reference throws Error(msg) for bad arguments

    @property
    def lost(self) -> bool:
        return bool(self.lostInfo) or bool(lib.p0p_status(self._h))

    def describe(self) -> dict:
        return dict(self.info, f16=True, subgroups=True, sgMin=32, sgMax=32, maxBufferMB=self._desc["memMB"], maxBindMB=self._desc["memMB"],
                    wgMem=self._desc["wgMem"], wgInv=self._desc["wgInv"], sms=self._desc["sms"], l2MB=self._desc["l2MB"])

    # ---------------------------------------------------------------- buffers (src/core/gpu.js:87-148)
    def buffer(self, size, label="", usage=0, shareable=False) -> Buffer:
        """`shareable` (not in the reference): memory other processes can map (ipcExport / ipcOpen); never pooled."""
        h = C.c_void_p()
        rc = (lib.p0p_alloc_shareable if shareable else lib.p0p_alloc)(self._h, int(size), C.byref(h))
        if rc == -2:
            raise GpuError(f"buffer {label} {size} B exceeds maxBufferSize")
        self._check(rc)
        b = Buffer(self, h, lib.p0p_buf_size(h), label)
        self.bufs.add(b)
        return b

    def wrap(self, device_ptr: int, nbytes: int, label="") -> Buffer:
        """Adopt device memory owned elsewhere (for instance a tensor of the host framework)."""
        h = C.c_void_p()
        self._check(lib.p0p_wrap(self._h, C.c_void_p(device_ptr), int(nbytes), C.byref(h)))
        b = Buffer(self, h, int(nbytes), label)
        self.bufs.add(b)
        return b

    def ipcExport(self, b: Buffer) -> bytes:
        """Not in the reference: the 64-byte CUDA IPC handle of a buffer made by buffer() / upload(), for another process on
        the node to map with ipcOpen."""
        h = (C.c_ubyte * 64)()
        self._check(lib.p0p_ipc_export(self._h, b.handle, C.cast(h, C.c_void_p)))
        return bytes(h)

    def ipcOpen(self, handle: bytes, nbytes: int, label="") -> Buffer:
        """Not in the reference: map a buffer another process exported (another GPU of the node); usable as a peer copy of y
        in gemm ({"y": {..., "peers": [...]}}).  free() unmaps it."""
        raw = (C.c_ubyte * 64).from_buffer_copy(handle)
        h = C.c_void_p()
        self._check(lib.p0p_ipc_open(self._h, C.cast(raw, C.c_void_p), int(nbytes), C.byref(h)))
        b = Buffer(self, h, int(nbytes), label)
        self.bufs.add(b)
        return b

    PEER_FLAG_BYTES = 256

    def peerBarrier(self, flags: Buffer, peer_flags: list, rank: int, world: int, wait_cycles: int = 0) -> None:
        """Not in the reference: a stream-ordered barrier between the ranks of one node (p0p_peer_barrier): queue it after a
        gemm that stored into the peers' copies of y and before the call that reads the gathered rows.  `flags`: this rank's
        zeroed flag block (buffer(PEER_FLAG_BYTES, shareable=True)); peer_flags[r]: rank r's block opened with ipcOpen
        (the entry at `rank` is ignored).  Every rank issues the same sequence of barriers."""
        arr = (C.c_void_p * max(8, int(world)))()
        for r in range(min(int(world), len(peer_flags))):
            if r != rank and peer_flags[r] is not None: arr[r] = peer_flags[r].handle
        self._check(lib.p0p_peer_barrier(self._h, flags.handle, arr, int(rank), int(world), int(wait_cycles)))

    def free(self, b):
        if b is None or b not in self.bufs:
            return
        self.bufs.discard(b)
        lib.p0p_free(self._h, b.handle)

    def freeAll(self):
        for b in list(self.bufs):
            self.free(b)
        self.drainPool()

    def drainPool(self):
        lib.p0p_drain_pool(self._h)

    def poolStats(self) -> dict:
        o = (C.c_uint64 * 9)()
        lib.p0p_pool_stats(self._h, o)
        return {"aliveMB": round(o[0] / 1e6), "pooledMB": round(o[1] / 1e6), "bufs": int(o[4]), "pooledN": int(o[5]), "creates": int(o[6]),
                "reuses": int(o[7]), "evictions": int(o[8]), "hwMB": round(o[3] / 1e6), "capMB": None,
                "alive": int(o[0]), "pooled": int(o[1]), "peak": int(o[2]), "hw": int(o[3])}

    @property
    def alive(self) -> int:
        return self.poolStats()["alive"]

    @property
    def peak(self) -> int:
        return self.poolStats()["peak"]

    def resetPeak(self):
        lib.p0p_reset_peak(self._h)

    def _write(self, buf: Buffer, off: int, raw: np.ndarray):
        if raw.size:
            self._check(lib.p0p_write(self._h, buf.handle, int(off), raw.ctypes.data_as(C.c_void_p), raw.size))

    def upload(self, data, label="", dst=None, dstOff=0) -> Buffer:
        """A typed array / bytes into a NEW buffer, or into dst at byte dstOff (src/core/gpu.js:141-148)."""
        raw = _bytes_view(data)
        b = dst or self.buffer(raw.size, label)
        self._write(b, dstOff, raw)
        return b

    def read(self, buf: Buffer, off=0, size=None, out=None) -> np.ndarray:
        """[off, off+size) of a buffer as a uint8 array; waits for queued work (src/core/gpu.js:150-170).  `out` (not in the
        reference): a caller's array of at least `size` bytes to read into, e.g. page-locked memory from p0p_host_alloc."""
        size = buf._pf - off if size is None else size
        if out is None: out = np.empty(int(size), np.uint8)
        elif out.nbytes < size or not out.flags["C_CONTIGUOUS"]: raise ValueError("read: `out` must be a contiguous array of at least `size` bytes")
        if size:
            self._check(lib.p0p_read(self._h, buf.handle, int(off), out.ctypes.data_as(C.c_void_p), int(size)))
        return out

    def done(self):
        """Wait for all queued work (src/core/gpu.js:171-176)."""
        if self.lost:
            raise GpuError("GPU device lost: " + json.dumps(self.lostInfo))
        self._check(lib.p0p_sync(self._h))

    def cap(self, kind="mm"):
        return self.rate[kind] * self.opts["maxDispatchSeconds"]

    # ---------------------------------------------------------------- recorded launch sequences (the Runner's batching, src/core/gpu.js:203-257)
    def record(self, fn) -> "Graph":
        """Run fn() with every op call recorded instead of executed; returns a Graph whose launch() replays them.
        Call fn() once normally first (the first call of a shape sizes the library's scratch memory)."""
        self._check(lib.p0p_capture_begin(self._h))
        try:
            fn()
        finally:
            h = C.c_void_p()
            rc = lib.p0p_capture_end(self._h, C.byref(h))
        self._check(rc)
        return Graph(self, h)

    # ---------------------------------------------------------------- extras the CUDA build adds
    @property
    def stream(self) -> int:
        return lib.p0p_stream(self._h) or 0

    @property
    def lastKernel(self) -> int:
        return lib.p0p_last_kernel(self._h)

    @property
    def lastPlan(self) -> dict:
        """the tensor-core kernel's plan of the last call it served (a test convenience)"""
        out = (C.c_uint32 * 8)()
        self._check(lib.p0p_last_plan(self._h, out))
        v = [int(x) for x in out]
        if self.lastKernel == 2:      # the decode kernel
            return dict(zip(("G", "T", "KC", "S", "whole", "units", "tiles"), v))
        return dict(zip(("BT", "KW", "LOCK", "NS", "NA", "NACC", "S", "T0"), v))

    @property
    def launches(self) -> int:
        return int(lib.p0p_launch_count(self._h))

    def close(self):
        if self._h:
            lib.p0p_close(self._h)
            self._h = C.c_void_p()
            self.bufs.clear()


class Graph:
    """a recorded sequence of op calls"""

    def __init__(self, gpu, handle):
        self._g, self._h = gpu, handle

    def launch(self):
        self._g._check(lib.p0p_graph_launch(self._g._h, self._h))

    def free(self):
        if self._h:
            lib.p0p_graph_free(self._g._h, self._h); self._h = None


def createGpu(opts=None) -> Gpu:
    """createGpu(opts) (src/core/gpu.js:15-20).  Extra option: ``device`` (CUDA ordinal), ``stream`` (a cudaStream_t)."""
    return Gpu(opts)


# ---------------------------------------------------------------- fp16 helpers (src/core/gpu.js:275-299)
def f2h(v: float) -> int:
    return int(lib.p0p_f2h(C.c_float(v)))


def h2f(h: int) -> float:
    return float(lib.p0p_h2f(C.c_uint16(h)))


def toF16(f32arr) -> np.ndarray:
    a = np.ascontiguousarray(f32arr, dtype=np.float32).reshape(-1)
    o = np.empty(a.size, np.uint16)
    lib.p0p_to_f16(a.ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p), a.size)
    return o


def fromF16(u16) -> np.ndarray:
    a = np.ascontiguousarray(u16).view(np.uint16).reshape(-1)
    o = np.empty(a.size, np.float32)
    lib.p0p_from_f16(a.ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p), a.size)
    return o


def view(buffer: Buffer, offset=0, size=None) -> dict:
    size = buffer._pf - offset if size is None else size
    return {"buffer": buffer, "offset": offset, "size": -(-size // 4) * 4}
