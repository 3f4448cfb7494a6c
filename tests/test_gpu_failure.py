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
            nv.i64(300_000_000), nv.ptr(None), nv.stream_ptr())            # 0.3 s budget
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
    # receive buffers and flags of "rank 0" (this call) and of a peer that never runs: nothing ever arrives in ours
    part = [torch.zeros(m, n, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(2)]
    t0 = time.time()
    nv.call("ttcd_gemm_rs", nv.ptr(x), nv.ptr(w), nv.ptr(out), _i64s([t.data_ptr() for t in part]),
            _i64s([t.data_ptr() for t in flags]), nv.i32(0), nv.i32(2), nv.i64(m), nv.i64(n), nv.i64(k), nv.i64(k), nv.i64(k),
            nv.i64(n), nv.i32(0), nv.i32(1), nv.i64(200_000_000), nv.i32(0), nv.stream_ptr())
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert nv.device_status() == 635                   # the epilogue of this rank's own rows gave up on the peer's tile
    # this rank's tile of the peer's rows was still pushed into the peer's receive buffer and flagged there
    torch.testing.assert_close(part[1].float(), x[m:].float() @ w.float().t(), rtol=2e-2, atol=2e-1)
    assert int(flags[1][0]) == 1                       # slot 0 (the only peer), block 0, n-tile 0
    y = torch.randn(512, 512, device="cuda").bfloat16()
    from ttcd_b200.ops import cuda
    torch.testing.assert_close(cuda.gemm(y, y.t()).view(512, 512).float(), y.float() @ y.float().t(), rtol=2e-2, atol=3e-1)
    assert nv.device_status() == 0


def test_every_unit_with_bounded_waits_exports_its_status_reader():
    """A wait that runs out in any kernel must be visible to ``device_status``: every translation unit that is built
    with bounded waits has a reader, and the list the binding polls names them all."""
    import re
    from pathlib import Path
    from ttcd_b200 import _native as nv
    lib = nv.load(required=True)
    root = Path(__file__).resolve().parents[1] / "csrc"
    with_waits = {re.search(r"TTCD_DEFINE_STATUS_READER\((\w+)\)", f.read_text()).group(1)
                  for f in root.glob("*.cu") if "mbar_wait" in f.read_text() or "atomicCAS(&g_status" in f.read_text()}
    assert with_waits == set(nv.STATUS_UNITS), (with_waits, nv.STATUS_UNITS)
    for unit in nv.STATUS_UNITS:
        assert hasattr(lib, f"ttcd_read_status_{unit}") and hasattr(lib, f"ttcd_set_wait_ns_{unit}")


def test_expired_peer_wait_makes_the_optimizer_kernel_leave_the_weights_alone():
    """What the sharded runtime builds its skip on: the barrier kernel of a rank whose peer never arrives sets the
    fail word, and the fused AdamW + publish kernel that is handed a non-zero skip word changes nothing."""
    from ttcd_b200 import _native as nv
    nv.load(required=True)
    nv.device_status()
    mine = torch.zeros(256, dtype=torch.int32, device="cuda")
    ghost = torch.zeros(256, dtype=torch.int32, device="cuda")
    fail = torch.zeros(1, device="cuda")
    nv.call("ttcd_comm_barrier", _i64s([mine.data_ptr(), ghost.data_ptr()]), nv.i32(0), nv.i32(2), nv.i32(0), nv.i32(1),
            nv.i64(100_000_000), nv.ptr(fail), nv.stream_ptr())
    torch.cuda.synchronize()
    assert float(fail) == 1.0 and nv.device_status() == 501
    n = 4096
    p32 = torch.randn(n, device="cuda")
    g, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    flat = [p32.to(torch.bfloat16).clone() for _ in range(2)]            # the two "ranks'" bf16 parameter buffers
    before = [t.clone() for t in (p32, m, v, *flat)]
    skip = (fail > 0).to(torch.int32)
    coef = torch.ones(1, device="cuda")
    args = lambda sk: (nv.ptr(p32), nv.ptr(g), nv.ptr(m), nv.ptr(v), _i64s([t.data_ptr() for t in flat]), nv.i32(2), nv.i64(0),  # noqa: E731
                       nv.i64(n), nv.f32(1e-2), nv.f32(0.9), nv.f32(0.95), nv.f32(1e-8), nv.f32(0.1), nv.f32(0.1), nv.f32(0.2236),
                       nv.ptr(coef), nv.ptr(sk), nv.stream_ptr())
    nv.call("ttcd_adamw_push", *args(skip))
    torch.cuda.synchronize()
    for t, b in zip((p32, m, v, *flat), before):
        assert torch.equal(t, b)
    nv.call("ttcd_adamw_push", *args(torch.zeros(1, dtype=torch.int32, device="cuda")))
    torch.cuda.synchronize()
    assert not torch.equal(p32, before[0]) and torch.equal(flat[0], flat[1]) and not torch.equal(flat[0], before[3])


def test_check_every_call_mode_names_the_launch_whose_wait_ran_out(monkeypatch):
    """The debugging mode (TTCD_CHECK_EVERY_CALL=1) synchronises after each launch and reads the status words, so an
    expired wait is reported by the call that contained it; healthy launches pass through it unchanged."""
    from ttcd_b200 import _native as nv
    from ttcd_b200.ops import cuda
    nv.load(required=True)
    nv.device_status()
    monkeypatch.setattr(nv, "_CHECK_EVERY_CALL", True)
    x = torch.randn(256, 256, device="cuda").bfloat16()
    torch.testing.assert_close(cuda.gemm(x, x).float().view(256, 256), x.float() @ x.float(), rtol=2e-2, atol=0.5)     # healthy
    mine = torch.zeros(256, dtype=torch.int32, device="cuda")
    ghost = torch.zeros(256, dtype=torch.int32, device="cuda")
    with pytest.raises(nv.NativeError, match="ttcd_comm_barrier.*status 501"):
        nv.call("ttcd_comm_barrier", _i64s([mine.data_ptr(), ghost.data_ptr()]), nv.i32(0), nv.i32(2), nv.i32(0), nv.i32(1),
                nv.i64(100_000_000), nv.ptr(None), nv.stream_ptr())
    assert nv.device_status() == 0                                         # the mode consumed the code
    torch.testing.assert_close(cuda.gemm(x, x).float().view(256, 256), x.float() @ x.float(), rtol=2e-2, atol=0.5)     # still usable
