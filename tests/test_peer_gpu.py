"""p0p_peer_barrier on one GPU: the barrier's stores and its bounded wait.  A second rank is stood in for by a flag block in
this GPU's own memory that the HOST writes (the rank "arrives" when the host stores its count), so no two kernels ever wait
for one another.  The time-out case is the library's failure-detection path: a wait that nothing satisfies runs out after a
short limit, the next sync reports it (-10) and the context keeps working; nothing traps, faults or spins for long."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def P():
    import p0pc0rn_kernels_b200 as P_
    return P_


def test_barrier_stores_and_passes(gpu):
    mine, peer = gpu.buffer(gpu.PEER_FLAG_BYTES), gpu.buffer(gpu.PEER_FLAG_BYTES)
    try:
        for seq in (1, 2, 3):
            gpu.upload(np.array([seq], np.uint32), "", mine, 4)                 # rank 1 has arrived at barrier `seq` (word 1 of rank 0's block)
            gpu.peerBarrier(mine, [None, peer], 0, 2)
            gpu.done()
            m, p = gpu.read(mine, 0, 256).view(np.uint32), gpu.read(peer, 0, 256).view(np.uint32)
            assert m[0] == seq and m[32] == seq, "rank 0's own arrival and count"
            assert p[0] == seq and p[1] == 0, "rank 0's arrival in rank 1's block, and nothing else"
    finally:
        for b in (mine, peer): gpu.free(b)


def test_bounded_wait_runs_out_and_the_context_stays_usable(gpu, oracle):
    mine, peer = gpu.buffer(gpu.PEER_FLAG_BYTES), gpu.buffer(gpu.PEER_FLAG_BYTES)
    try:
        t0 = time.perf_counter()
        gpu.peerBarrier(mine, [None, peer], 0, 2, wait_cycles=2_000_000)           # nobody writes word 1: the wait ends after ~1 ms
        with pytest.raises(P().GpuError, match="bounded wait"):
            gpu.done()
        assert time.perf_counter() - t0 < 2.0
        assert not gpu.lost
        gpu.done()                                                              # reported once; the context works on
        # a multiply on the same context afterwards
        O = oracle
        M, N, K = 8, 128, 256
        X = O.round_f16(O.randn(M * K, 7)); Wb, Wd = O.pack_q4(O.randn(N * K, 11, 0.05), N, K)
        wb, xb, yb = gpu.upload(Wb), gpu.upload(P().toF16(X)), gpu.buffer(M * N * 2)
        P().gemm(gpu, {"w": {"enc": "q4g32a.t64", "buf": wb, "off": 0, "bytes": wb._pf, "rows": N, "cols": K}, "x": {"buf": xb}, "y": {"buf": yb}, "M": M, "N": N, "K": K})
        got = P().fromF16(gpu.read(yb, 0, M * N * 2).view(np.uint16))
        assert O.compare(got, O.cpu_gemm(X, Wd, M, N, K))[0] > 0.9995
        for b in (wb, xb, yb): gpu.free(b)
    finally:
        for b in (mine, peer): gpu.free(b)


def test_barrier_arguments(gpu):
    mine = gpu.buffer(gpu.PEER_FLAG_BYTES); small = gpu.buffer(64)
    try:
        with pytest.raises(ValueError, match="world"): gpu.peerBarrier(mine, [None] * 9, 0, 9)
        with pytest.raises(ValueError, match="rank"): gpu.peerBarrier(mine, [None, None], 2, 2)
        with pytest.raises(ValueError, match="missing flag block"): gpu.peerBarrier(mine, [None, small], 0, 2)
        gpu.peerBarrier(mine, [None], 0, 1); gpu.done()                          # a group of one: counts, waits for nobody
        assert gpu.read(mine, 0, 256).view(np.uint32)[32] == 1
    finally:
        for b in (mine, small): gpu.free(b)
