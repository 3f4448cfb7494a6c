"""Attention backward (single and dual window) against autograd through the dense fp32 statement."""
import pytest
import torch

from ttcd_b200 import _native, ops
from ttcd_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV, BF = "cuda", torch.bfloat16


@pytest.fixture(autouse=True)
def _status():
    _native.load(required=True)
    yield
    torch.cuda.synchronize()
    assert _native.device_status() == 0, "a bounded device wait expired"


def _check(got, want, name, atol=2e-2, rtol=3e-2):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    bad = (err > atol + rtol * want.abs()).float().mean().item()
    rel = err.norm().item() / max(want.norm().item(), 1e-12)
    assert bad < 1e-3 and rel < 2e-2, f"{name}: rel-rms {rel:.4g}, max err {err.max().item():.4g}, {bad * 100:.3f}% outside tol"


def _inputs(B, T, H, HK, D, Tk=None):
    Tk = T if Tk is None else Tk
    mk = lambda *s: torch.randn(*s, device=DEV).to(BF).requires_grad_()  # noqa: E731
    return mk(B, T, H, D), mk(B, Tk, HK, D), mk(B, Tk, HK, D)


@pytest.mark.parametrize("T,H,HK,D,W", [(128, 2, 1, 128, None), (300, 4, 2, 128, 100), (513, 2, 2, 64, 192),
                                         (1024, 4, 1, 128, 256), (777, 3, 1, 64, None)])
def test_single_window_backward(T, H, HK, D, W):
    q, k, v = _inputs(2, T, H, HK, D)
    o = ops.attention(q, k, v, window=W)
    g = torch.randn_like(o)
    o.backward(g)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref.attention(qf, kf, vf, W).backward(g.float())
    _check(q.grad, qf.grad, "dq")
    _check(k.grad, kf.grad, "dk")
    _check(v.grad, vf.grad, "dv")


@pytest.mark.parametrize("T,H,HK,D,WT,WS", [(512, 2, 1, 128, 256, 128), (1000, 4, 2, 128, 400, 200),
                                             (769, 3, 3, 64, 300, 150), (1536, 2, 1, 128, None, 256),
                                             (700, 2, 2, 128, 256, 256), (2100, 2, 1, 128, 1024, 512)])
def test_dual_window_backward(T, H, HK, D, WT, WS):
    q, k, v = _inputs(1, T, H, HK, D)
    o_t, o_s = ops.dual_window_attention(q, k, v, WT, WS)
    g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    r_t, r_s = ref.dual_window_attention(qf, kf, vf, WT, WS)
    torch.autograd.backward([r_t, r_s], [g_t.float(), g_s.float()])
    _check(q.grad, qf.grad, "dq")
    _check(k.grad, kf.grad, "dk")
    _check(v.grad, vf.grad, "dv")


def test_backward_with_longer_keys():
    q, k, v = _inputs(1, 200, 2, 1, 128, Tk=712)
    o_t, o_s = ops.dual_window_attention(q, k, v, 512, 256)
    g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    r_t, r_s = ref.dual_window_attention(qf, kf, vf, 512, 256)
    torch.autograd.backward([r_t, r_s], [g_t.float(), g_s.float()])
    _check(q.grad, qf.grad, "dq")
    _check(k.grad, kf.grad, "dk")
    _check(v.grad, vf.grad, "dv")


def test_strided_qkv_views_and_packed_sequences():
    B, T, H, HK, D = 1, 640, 4, 2, 128
    qkv = torch.randn(B, T, (H + 2 * HK) * D, device=DEV).to(BF).requires_grad_()
    q = qkv[..., : H * D].view(B, T, H, D)
    k = qkv[..., H * D: (H + HK) * D].view(B, T, HK, D)
    v = qkv[..., (H + HK) * D:].view(B, T, HK, D)
    cu = torch.tensor([0, 200, 640], device=DEV, dtype=torch.int32)
    o = ops.attention(q, k, v, window=128, cu_seqlens=cu)
    g = torch.randn_like(o)
    o.backward(g)
    f = qkv.detach().float().requires_grad_()
    qf = f[..., : H * D].view(B, T, H, D)
    kf = f[..., H * D: (H + HK) * D].view(B, T, HK, D)
    vf = f[..., (H + HK) * D:].view(B, T, HK, D)
    o_r = ref.attention(qf, kf, vf, 128, cu_seqlens=cu)
    o_r.backward(g.float())
    _check(o, o_r, "o", atol=8e-3, rtol=1e-2)
    _check(qkv.grad, f.grad, "dqkv")
