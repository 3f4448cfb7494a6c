"""`ttcd_rmsnorm_bwd_no_alloc` (csrc/ttcd_no_alloc.h): the RMSNorm backward whose scratch lives in the library
image.  Called through the exported C symbol with ctypes; compared with the regular entry point
`ttcd_rmsnorm_bwd` (caller-provided scratch) on two calls in a row with different data and shapes, so stale
scratch contents from the first call would show in the second.  The file sorts last on purpose: it must pass
alone and after every other GPU test has used the library."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_D, ERR_SHAPE, ERR_TOO_LARGE = 2048, -1, -3


def _lib():
    from ttcd_b200 import _native
    _native.load(required=True)
    lib = ctypes.CDLL(str(_native._LIB_PATH))      # own handle: prototypes set here stay out of the package's
    fn = lib.ttcd_rmsnorm_bwd_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    old = lib.ttcd_rmsnorm_bwd
    old.restype = ctypes.c_int
    old.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn, old


def _case(rows, D, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *shape: torch.randn(*shape, device="cuda", generator=g).bfloat16()
    dy, s, w = mk(rows, D), mk(rows, D), (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    rstd = torch.rsqrt(s.float().pow(2).mean(-1) + 1e-6)
    return dy, s, w, rstd, (mk(rows, D) if with_res else None)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _run_pair(fn, old, rows, D, seed, with_res):
    dy, s, w, rstd, dres = _case(rows, D, seed, with_res)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dx_new, dw_new = torch.empty_like(dy), torch.empty(D, device="cuda", dtype=torch.float32)
    assert fn(_p(dy), _p(s), _p(w), _p(rstd), _p(dres), _p(dx_new), _p(dw_new), rows, D, stream) == 0
    nblk = min(148, (rows + 7) // 8)
    dx_old, part = torch.empty_like(dy), torch.empty(nblk, D, device="cuda", dtype=torch.float32)
    assert old(_p(dy), _p(s), _p(w), _p(rstd), _p(dres), _p(dx_old), _p(part), rows, D, nblk, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dx_new, dx_old)
    torch.testing.assert_close(dw_new, part.sum(0), rtol=1e-5, atol=1e-4)
    # and against plain fp32 PyTorch
    xh = s.float() * rstd[:, None]
    gw = dy.float() * w.float()
    want = rstd[:, None] * (gw - xh * (gw * xh).mean(-1, keepdim=True))
    if dres is not None:
        want = want + dres.float()
    torch.testing.assert_close(dx_new.float(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dw_new, (dy.float() * xh).sum(0), rtol=1e-3, atol=1e-2 * (rows ** 0.5))


def test_two_calls_in_a_row_match_regular_entry_point():
    fn, old = _lib()
    _run_pair(fn, old, rows=4096, D=1024, seed=1, with_res=True)     # fills 148 x 1024 of the array
    _run_pair(fn, old, rows=300, D=2048, seed=2, with_res=False)     # fewer blocks, wider rows: reuses it


def test_limits_are_refused_without_launching():
    fn, _ = _lib()
    dy, s, w, rstd, _ = _case(16, 64, 3, False)
    dx, dw = torch.full_like(dy, 7.0), torch.zeros(64, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(_p(dy), _p(s), _p(w), _p(rstd), None, _p(dx), _p(dw), 16, MAX_D + 8, stream) == ERR_TOO_LARGE
    assert fn(_p(dy), _p(s), _p(w), _p(rstd), None, _p(dx), _p(dw), 16, 60, stream) == ERR_SHAPE
    assert fn(_p(dy), _p(s), _p(w), _p(rstd), None, _p(dx), None, 16, 64, stream) == ERR_SHAPE
    torch.cuda.synchronize()
    assert bool((dx == 7.0).all())


def test_makes_no_device_allocation():
    fn, _ = _lib()
    dy, s, w, rstd, _ = _case(2048, 512, 4, False)
    dx, dw = torch.empty_like(dy), torch.empty(512, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(_p(dy), _p(s), _p(w), _p(rstd), None, _p(dx), _p(dw), 2048, 512, stream) == 0     # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        assert fn(_p(dy), _p(s), _p(w), _p(rstd), None, _p(dx), _p(dw), 2048, 512, stream) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
