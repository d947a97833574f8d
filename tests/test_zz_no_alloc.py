"""p0p_decode_q4_static: the decode-sized q4 multiply for hosts that cannot allocate device memory (a server that
owns the whole GPU arena, a plug-in under a foreign allocator).  It takes raw device pointers and the caller's
stream and keeps its split-K scratch in an array built into the library.  Checked here through the C ABI against
the regular entry point (p0p_gemm), bit for bit, on two calls in a row (the second call finds the shared array
full of the first call's partial sums), plus the refusal of a shape larger than the built-in array, the read-back of
its bounded-wait status word, and a check that warmed-up calls leave the device's free memory where it was."""
import ctypes as C

import numpy as np
import pytest

import cases as CS

pytestmark = pytest.mark.gpu


def _static(gpu, wb, xb, yb, M, N, K):
    from p0pc0rn_kernels_b200._lib import lib
    err = C.create_string_buffer(256)
    rc = lib.p0p_decode_q4_static(int(gpu.opts["device"]), C.c_void_p(gpu.stream), C.c_void_p(wb.ptr), C.c_void_p(xb.ptr), C.c_void_p(yb.ptr), M, N, K, err, 256)
    return rc, err.value.decode()


def _status(gpu):
    from p0pc0rn_kernels_b200._lib import lib
    err = C.create_string_buffer(256)
    return lib.p0p_decode_q4_static_status(int(gpu.opts["device"]), C.c_void_p(gpu.stream), err, 256), err.value.decode()


def _free_bytes(gpu):
    """free device memory as the CUDA runtime reports it (cudaMemGetInfo, through torch: device plumbing only)"""
    import torch
    return torch.cuda.mem_get_info(int(gpu.opts["device"]))[0]


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (5, 256, 2048), (16, 1024, 512)])
def test_static_scratch_matches_regular_entry_point(gpu, oracle, M, N, K):
    import p0pc0rn_kernels_b200 as P
    O = oracle
    X = O.round_f16(O.randn(M * K, 7)); W0 = O.randn(N * K, 11, 0.05)
    Wb, _ = O.pack_q4(W0, N, K)
    wb, xb = gpu.upload(Wb), gpu.upload(P.toF16(X))
    y_ref, y_a, y_b = gpu.buffer(M * N * 2), gpu.upload(np.full(M * N, 0xFFFF, np.uint16)), gpu.upload(np.full(M * N, 0xFFFF, np.uint16))
    try:
        P.gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": y_ref}, "M": M, "N": N, "K": K, "kernel": "decode"})
        want = gpu.read(y_ref, 0, M * N * 2).view(np.uint16)
        for yb in (y_a, y_b):                       # two calls in a row share the built-in array
            rc, msg = _static(gpu, wb, xb, yb, M, N, K)
            assert rc == 0, msg
        assert _status(gpu) == (0, ""), "a bounded wait ran out"
        gpu.done()
        _free_bytes(gpu)                            # (the first query brings up torch's own CUDA state)
        before = _free_bytes(gpu)                   # the calls above have done the per-device set-up: from here on nothing may allocate
        for yb in (y_a, y_b):
            rc, msg = _static(gpu, wb, xb, yb, M, N, K)
            assert rc == 0, msg
        assert _status(gpu) == (0, "")
        assert _free_bytes(gpu) == before, "the entry point changed the device's free memory"
        for yb in (y_a, y_b):
            got = gpu.read(yb, 0, M * N * 2).view(np.uint16)
            assert np.array_equal(got, want)          # same kernel, same plan: identical bits (tolerance of the other tests: cos > 0.9995)
        CS.check(want.copy(), O.to_f16(O.cpu_gemm(X, O.from_f16(O.dequant("q4g32a.t64", Wb, 0, N, K)[0]), M, N, K)), "static scratch")
    finally:
        for b in (wb, xb, y_ref, y_a, y_b): gpu.free(b)


def test_static_scratch_refuses_what_does_not_fit(gpu):
    b = gpu.buffer(4096)
    try:
        rc, msg = _static(gpu, b, b, b, 16, 16384, 16384)      # needs 16 MiB of partial sums, the array holds 8 MiB
        assert rc < 0 and "scratch" in msg
        rc, msg = _static(gpu, b, b, b, 17, 64, 256)
        assert rc < 0 and "M must be" in msg
        rc, msg = _static(gpu, b, b, b, 1, 64, 100)
        assert rc < 0 and "multiple of 256" in msg
        gpu.done()
    finally:
        gpu.free(b)
