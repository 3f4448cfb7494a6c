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


@pytest.mark.parametrize("B,T,H,HK,D,WT,WS", [(2, 900, 4, 2, 128, 384, 128), (1, 1300, 2, 1, 64, 512, 192)])
def test_dual_backward_batched_and_small_heads(B, T, H, HK, D, WT, WS):
    q, k, v = _inputs(B, T, H, HK, D)
    o_t, o_s = ops.dual_window_attention(q, k, v, WT, WS)
    g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    r_t, r_s = ref.dual_window_attention(qf, kf, vf, WT, WS)
    torch.autograd.backward([r_t, r_s], [g_t.float(), g_s.float()])
    _check(q.grad, qf.grad, "dq")
    _check(k.grad, kf.grad, "dk")
    _check(v.grad, vf.grad, "dv")


@pytest.mark.parametrize("dual", [False, True])
@pytest.mark.parametrize("D,H,HK", [(128, 4, 2), (64, 3, 1)])
def test_packed_documents_one_launch_equals_per_document(dual, D, H, HK):
    """Eight documents of uneven length packed into one 4K row: the in-kernel sequence bounds give what running every
    document on its own gives (forward and backward), with windows shorter and longer than the documents."""
    lens = [37, 700, 129, 1, 1500, 256, 900, 573]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    WT, WS = 512, 192
    q, k, v = _inputs(1, T, H, HK, D)

    def run(qq, kk, vv, cu_seqlens):
        if dual:
            return ops.dual_window_attention(qq, kk, vv, WT, WS, cu_seqlens=cu_seqlens)
        return (ops.attention(qq, kk, vv, window=WT, cu_seqlens=cu_seqlens),)

    launches = _native.launch_count
    outs = run(q, k, v, cu)
    assert _native.launch_count - launches == 1, "a packed row is one forward launch"
    gs = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(list(outs), gs)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    bounds = cu.tolist()
    want = [[] for _ in outs]
    for a, b in zip(bounds[:-1], bounds[1:]):
        if dual:
            r = ref.dual_window_attention(qf[:, a:b], kf[:, a:b], vf[:, a:b], WT, WS)
        else:
            r = (ref.attention(qf[:, a:b], kf[:, a:b], vf[:, a:b], WT),)
        for i, t in enumerate(r):
            want[i].append(t)
    want = [torch.cat(w, dim=1) for w in want]
    torch.autograd.backward(want, [g.float() for g in gs])
    for o, w in zip(outs, want):
        _check(o, w, "o", atol=8e-3, rtol=1e-2)
    _check(q.grad, qf.grad, "dq")
    _check(k.grad, kf.grad, "dk")
    _check(v.grad, vf.grad, "dv")


def test_expired_wait_in_the_backward_is_reported():
    """The dK/dV kernel's wait for key/value tiles that never arrive runs out within its (shortened) budget, the
    kernel returns, the status word of the backward's translation unit says so, and the next call is healthy."""
    import ctypes
    from ttcd_b200.ops import cuda
    lib = _native.load(required=True)
    q, k, v = _inputs(1, 256, 2, 1, 128)
    o, lse = ops.attention(q, k, v, window=128, return_lse=True)
    g = torch.randn_like(o)
    _native.device_status()
    assert lib.ttcd_set_wait_ns_attn_bwd(ctypes.c_longlong(20_000_000)) == 0          # 20 ms
    try:
        cuda.attn_backward(q.detach(), k.detach(), v.detach(), o.detach(), None, lse, None, g, None, 128, 128, 128 ** -0.5,
                           flags=1)
        torch.cuda.synchronize()
        assert _native.device_status() in (301, 304, 311), "the wait ran out but nothing recorded it"
    finally:
        assert lib.ttcd_set_wait_ns_attn_bwd(ctypes.c_longlong(0)) == 0
    dq, dk, dv = cuda.attn_backward(q.detach(), k.detach(), v.detach(), o.detach(), None, lse, None, g, None, 128, 128,
                                    128 ** -0.5)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref.attention(qf, kf, vf, 128).backward(g.float())
    _check(dq, qf.grad, "dq")
    _check(dk, kf.grad, "dk")
    _check(dv, vf.grad, "dv")


@pytest.mark.parametrize("D", [64, 128])
def test_combine_kernel_matches_torch(D):
    """delta_T, delta' = delta_T + r delta_S and dO' = dO_T + r dO_S (r = exp(lse_T - lse_S)) from one kernel."""
    from ttcd_b200._native import call, i32, i64, ptr, stream_ptr
    B, T, H = 2, 333, 3
    mk = lambda: torch.randn(B, T, H, D, device=DEV).to(BF)  # noqa: E731
    o_t, do_t, o_s, do_s = mk(), mk(), mk(), mk()
    lse_s = torch.randn(B, H, T, device=DEV)
    lse_t = lse_s + torch.rand(B, H, T, device=DEV) * 2
    delta_t, delta_p = torch.empty(B, H, T, device=DEV), torch.empty(B, H, T, device=DEV)
    do_p = torch.empty_like(do_t)
    call("ttcd_attn_bwd_combine", ptr(o_t), ptr(do_t), ptr(o_s), ptr(do_s), ptr(lse_t), ptr(lse_s), ptr(delta_t), ptr(delta_p),
         ptr(do_p), i64(B), i32(T), i32(H), i32(D), stream_ptr())
    r = torch.exp(lse_t - lse_s)
    want_t = (o_t.float() * do_t.float()).sum(-1).transpose(1, 2)
    want_s = (o_s.float() * do_s.float()).sum(-1).transpose(1, 2)
    torch.testing.assert_close(delta_t, want_t, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(delta_p, want_t + r * want_s, rtol=1e-4, atol=2e-3)
    want_do = do_t.float() + r.transpose(1, 2).unsqueeze(-1) * do_s.float()
    torch.testing.assert_close(do_p.float(), want_do, rtol=1e-2, atol=1e-2)
