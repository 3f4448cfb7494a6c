"""Bounded device-side waits: a wait that nothing satisfies must expire within its budget, leave an error
code in the status word and return with the context usable.  The absent peer is emulated on one GPU by
handing the kernel flag buffers that no kernel ever writes; no kernel here faults, traps or spins forever."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _i64s(values):
    return (ctypes.c_longlong * len(values))(*values)


def test_barrier_wait_expires_with_status_and_context_survives():
    from ttcd_b200 import _native as nv
    nv.load(required=True)
    nv.device_status()                                                     # clear
    mine = torch.zeros(256, dtype=torch.int32, device="cuda")
    ghost = torch.zeros(256, dtype=torch.int32, device="cuda")             # stands for a peer that never arrives
    t0 = time.time()
    nv.call("ttcd_comm_barrier", _i64s([mine.data_ptr(), ghost.data_ptr()]), nv.i32(0), nv.i32(2), nv.i32(0), nv.i32(1),
            nv.i64(300_000_000), nv.stream_ptr())                          # 0.3 s budget
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert nv.device_status() == 501                                       # 500 + the rank that never arrived
    assert int(ghost[0]) == 1                                              # this rank did publish its own arrival
    x = torch.randn(256, 256, device="cuda").bfloat16()
    from ttcd_b200.ops import cuda
    torch.testing.assert_close(cuda.gemm(x, x.t()).view(256, 256).float(), x.float() @ x.float().t(), rtol=2e-2, atol=2e-1)
    assert nv.device_status() == 0


def test_gemm_reduce_scatter_gives_up_on_an_absent_peer():
    from ttcd_b200 import _native as nv
    nv.load(required=True)
    nv.device_status()
    m, n, k = 128, 256, 64
    x = torch.randn(2 * m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda").bfloat16()
    out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    part = [torch.zeros(2 * m, n, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(2)]     # flags[1] is never written
    peer_sum = torch.zeros(m, n, device="cuda")
    sum_flags = torch.zeros(64, device="cuda", dtype=torch.int32)
    t0 = time.time()
    nv.call("ttcd_gemm_rs", nv.ptr(x), nv.ptr(w), nv.ptr(out), _i64s([t.data_ptr() for t in part]),
            _i64s([t.data_ptr() for t in flags]), nv.ptr(peer_sum), nv.ptr(sum_flags), nv.i32(0), nv.i32(2), nv.i64(m), nv.i64(n),
            nv.i64(k), nv.i64(k), nv.i64(k), nv.i64(n), nv.i32(0), nv.i32(1), nv.i64(200_000_000), nv.stream_ptr())
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert nv.device_status() in (641, 635)            # the reducer gave up on peer 1 (or the epilogue on its sum)
    # this rank's partial for the peer's rows was still produced and flagged
    torch.testing.assert_close(part[0][m:].float(), x[m:].float() @ w.float().t(), rtol=2e-2, atol=2e-1)
    assert int(flags[0][1 * 1 * 1]) == 1               # tile (owner 1, block 0, n-tile 0)
    y = torch.randn(512, 512, device="cuda").bfloat16()
    from ttcd_b200.ops import cuda
    torch.testing.assert_close(cuda.gemm(y, y.t()).view(512, 512).float(), y.float() @ y.float().t(), rtol=2e-2, atol=3e-1)
    assert nv.device_status() == 0
