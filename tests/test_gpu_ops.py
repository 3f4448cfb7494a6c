"""Numerics of every hand-written kernel against the fp32 PyTorch statement of the same op."""
import math

import pytest
import torch

from ttcd_b200 import _native, ops
from ttcd_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"
BF = torch.bfloat16


@pytest.fixture(autouse=True)
def _native_required():
    _native.load(required=True)
    yield
    torch.cuda.synchronize()
    assert _native.device_status() == 0, "a bounded device wait expired"


def _close(got, want, atol, rtol, name=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).float().mean().item()
    assert bad == 0.0, f"{name}: max err {err.max().item():.4g}, {bad * 100:.3f}% outside tol, ref max {want.abs().max().item():.4g}"


def _cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-30))


# ------------------------------------------------------------------------------------------- GEMM

@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 320, 192), (1000, 1160, 1032), (4096, 1024, 1024)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, ta, tb):
    from ttcd_b200.ops import cuda
    a = torch.randn((K, M) if ta else (M, K), device=DEV, dtype=BF)
    b = torch.randn((N, K) if tb else (K, N), device=DEV, dtype=BF)
    a_l = a.t() if ta else a
    b_l = b.t() if tb else b
    got = cuda.gemm(a_l, b_l).view(M, N)
    want = a_l.float() @ b_l.float()
    _close(got, want, atol=0.02 * math.sqrt(K), rtol=1.6e-2, name=f"gemm {M}x{N}x{K} ta={ta} tb={tb}")


def test_gemm_batched_fp32_accumulate_rowscale():
    from ttcd_b200.ops import cuda
    Bt, M, N, K = 3, 256, 384, 512
    a = torch.randn(Bt, K, M, device=DEV, dtype=BF)
    b = torch.randn(Bt, K, N, device=DEV, dtype=BF)
    c = torch.randn(Bt, M, N, device=DEV, dtype=torch.float32)
    rs = torch.rand(Bt * M, device=DEV, dtype=BF)
    want = 0.5 * rs.float().view(Bt, M, 1) * (a.float().transpose(1, 2) @ b.float()) + 2.0 * c
    got = cuda.gemm(a.transpose(1, 2), b, alpha=0.5, beta=2.0, c_in=c, row_scale=rs, out=c.clone())
    _close(got, want, atol=0.3, rtol=1e-2, name="batched gemm")


def test_matmul_autograd():
    a = torch.randn(2, 3, 256, 192, device=DEV, dtype=BF, requires_grad=True)
    b = torch.randn(192, 320, device=DEV, dtype=BF, requires_grad=True)
    out = ops.matmul(a, b)
    g = torch.randn_like(out)
    out.backward(g)
    af, bf_ = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    (af @ bf_).backward(g.float())
    _close(out, af @ bf_, 0.3, 1.6e-2, "matmul fwd")
    _close(a.grad, af.grad, 0.4, 1.6e-2, "matmul da")
    _close(b.grad, bf_.grad, 1.5, 1.6e-2, "matmul db")


def test_linear_and_fused_linear_autograd():
    from ttcd_b200.models.layers import _slab_view
    x = torch.randn(2, 200, 256, device=DEV, dtype=BF, requires_grad=True)
    flat = torch.randn((384 + 128 + 128) * 256, device=DEV, dtype=BF) * 0.05
    ws = [flat[: 384 * 256].view(384, 256), flat[384 * 256: 512 * 256].view(128, 256), flat[512 * 256:].view(128, 256)]
    ws = [w.detach().requires_grad_() for w in ws]
    from ttcd_b200.ops import cuda
    outs = cuda.fused_linear(x, ws, _slab_view(ws))
    loss = sum((o.float() * (i + 1)).sum() for i, o in enumerate(outs))
    loss.backward()
    xf = x.detach().float().requires_grad_()
    wf = [w.detach().float().requires_grad_() for w in ws]
    ref_outs = [xf @ w.t() for w in wf]
    sum((o * (i + 1)).sum() for i, o in enumerate(ref_outs)).backward()
    for o, r in zip(outs, ref_outs):
        _close(o, r, 0.05, 1.6e-2, "fused linear fwd")
    _close(x.grad, xf.grad, 0.3, 2e-2, "fused linear dx")
    for w, r in zip(ws, wf):
        _close(w.grad, r.grad, 1.0, 2e-2, "fused linear dw")


# ----------------------------------------------------------------------------------- elementwise

@pytest.mark.parametrize("D", [128, 960, 1024, 2048, 4096, 5120])     # > 2048: the streaming (wide-row) kernels
def test_rmsnorm_fwd_bwd(D):
    x = torch.randn(3, 77, D, device=DEV, dtype=BF, requires_grad=True)
    r = torch.randn(3, 77, D, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(D, device=DEV) * 0.1 + 1).to(BF).requires_grad_()
    y, s = ops.rmsnorm(x, w, 1e-6, residual=r, prenorm=True)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    torch.autograd.backward([y, s], [gy, gs])
    xf, rf, wf = (t.detach().float().requires_grad_() for t in (x, r, w))
    yr, sr = ref.rmsnorm(xf, wf, 1e-6, residual=rf, prenorm=True)
    torch.autograd.backward([yr, sr], [gy.float(), gs.float()])
    _close(y, yr, 2e-2, 1e-2, "rmsnorm y")
    _close(s, sr, 2e-2, 1e-2, "rmsnorm sum")
    _close(x.grad, xf.grad, 4e-2, 2e-2, "rmsnorm dx")
    _close(r.grad, rf.grad, 4e-2, 2e-2, "rmsnorm dres")
    _close(w.grad, wf.grad, 0.3, 3e-2, "rmsnorm dw")


@pytest.mark.parametrize("D", [960, 1024, 2048, 4096])      # one two-input kernel each way; wide rows use the single kernel twice
def test_rmsnorm_dual(D):
    a_t, a_s, r = (torch.randn(2, 50, D, device=DEV, dtype=BF, requires_grad=True) for _ in range(3))
    w = (torch.randn(D, device=DEV) * 0.1 + 1).to(BF).requires_grad_()
    outs = ops.rmsnorm_dual(a_t, a_s, r, w, 1e-6)
    gs = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, gs)
    f = [t.detach().float().requires_grad_() for t in (a_t, a_s, r, w)]
    outs_r = ref.rmsnorm_dual(f[0], f[1], f[2], f[3], 1e-6)
    torch.autograd.backward(outs_r, [g.float() for g in gs])
    for o, o_r in zip(outs, outs_r):
        _close(o, o_r, 3e-2, 1e-2, "dual fwd")
    for t, t_r, n in zip((a_t, a_s, r), f[:3], ("da_t", "da_s", "dres")):
        _close(t.grad, t_r.grad, 6e-2, 2e-2, n)
    _close(w.grad, f[3].grad, 0.5, 3e-2, "dual dw")


@pytest.mark.parametrize("H,HK,D,norm", [(4, 2, 128, True), (15, 5, 64, False), (2, 2, 128, False)])
def test_qk_norm_rope(H, HK, D, norm):
    B, T = 2, 130
    qkv = torch.randn(B, T, (H + 2 * HK) * D, device=DEV, dtype=BF, requires_grad=True)
    q = qkv[..., : H * D].view(B, T, H, D)
    k = qkv[..., H * D: (H + HK) * D].view(B, T, HK, D)
    qw = (torch.rand(D, device=DEV) + 0.5).to(BF).requires_grad_() if norm else None
    kw = (torch.rand(D, device=DEV) + 0.5).to(BF).requires_grad_() if norm else None
    cos, sin = ref.rope_tables(D, 10000.0, 512, device=DEV, dtype=BF)
    qo, ko = ops.qkv_norm_rope(q, k, qw, kw, 1e-5, cos, sin, offset=7)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    torch.autograd.backward([qo, ko], [gq, gk])
    qkv_f = qkv.detach().float().requires_grad_()
    qf = qkv_f[..., : H * D].view(B, T, H, D)
    kf = qkv_f[..., H * D: (H + HK) * D].view(B, T, HK, D)
    qwf = qw.detach().float().requires_grad_() if norm else None
    kwf = kw.detach().float().requires_grad_() if norm else None
    if norm:
        qf, kf = ref.rmsnorm(qf, qwf, 1e-5), ref.rmsnorm(kf, kwf, 1e-5)
    qr, kr = ref.rope(qf, cos, sin, 7), ref.rope(kf, cos, sin, 7)
    torch.autograd.backward([qr, kr], [gq.float(), gk.float()])
    _close(qo, qr, 3e-2, 1.5e-2, "q rope")
    _close(ko, kr, 3e-2, 1.5e-2, "k rope")
    _close(qkv.grad, qkv_f.grad, 6e-2, 3e-2, "dqkv")
    if norm:
        _close(qw.grad, qwf.grad, 1.0, 5e-2, "dqw")
        _close(kw.grad, kwf.grad, 1.0, 5e-2, "dkw")


def test_swiglu():
    gu = torch.randn(300, 2 * 768, device=DEV, dtype=BF, requires_grad=True)
    z = ops.swiglu_packed(gu)
    g = torch.randn_like(z)
    z.backward(g)
    guf = gu.detach().float().requires_grad_()
    zr = ref.swiglu(guf[:, :768], guf[:, 768:])
    zr.backward(g.float())
    _close(z, zr, 2e-2, 1e-2, "swiglu")
    _close(gu.grad, guf.grad, 4e-2, 2e-2, "swiglu grad")


@pytest.mark.parametrize("K,causal,C", [(5, True, 96), (4, True, 64), (5, False, 130), (3, True, 17)])
def test_dwconv(K, causal, C):
    x = torch.randn(2, 3, C, 384, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(384, K, device=DEV) * 0.5).to(BF).requires_grad_()
    y = ops.dwconv_chunked(x, w, causal)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.dwconv_chunked(xf, wf, causal)
    yr.backward(g.float())
    _close(y, yr, 3e-2, 1e-2, "dwconv y")
    _close(x.grad, xf.grad, 5e-2, 2e-2, "dwconv dx")
    _close(w.grad, wf.grad, 0.8, 3e-2, "dwconv dw")


def test_cross_entropy_rows():
    V = 5000 * 8
    logits = (torch.randn(300, V, device=DEV) * 3).to(BF).requires_grad_()
    labels = torch.randint(0, V, (300,), device=DEV)
    labels[::7] = -100
    loss = ops.cross_entropy(logits, labels)
    loss.backward()
    lf = logits.detach().float().requires_grad_()
    lr = ref.cross_entropy(lf, labels)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-3 * max(1.0, abs(lr.item()))
    _close(logits.grad, lf.grad, 2e-5, 2e-2, "dlogits")


def test_linear_cross_entropy():
    N, Hd, V = 700, 256, 4096
    h = (torch.randn(N, Hd, device=DEV) * 0.5).to(BF).requires_grad_()
    w = (torch.randn(V, Hd, device=DEV) * 0.1).to(BF).requires_grad_()
    labels = torch.randint(0, V, (N,), device=DEV)
    labels[-1] = -100
    loss = ops.linear_cross_entropy(h, labels, w, num_chunks=3)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = ref.cross_entropy(hf @ wf.t(), labels)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 5e-3 * abs(lr.item())
    _close(h.grad, hf.grad, 3e-5, 5e-2, "lce dh")
    _close(w.grad, wf.grad, 3e-5, 5e-2, "lce dw")


@pytest.mark.parametrize("smoothing,z", [(0.1, 0.0), (0.0, 1e-3), (0.05, 2e-4)])
def test_cross_entropy_label_smoothing_and_z_loss(smoothing, z):
    V = 4096 + 24                                   # a ragged tail after the vector loop
    logits = (torch.randn(200, V, device=DEV) * 3).to(BF).requires_grad_()
    labels = torch.randint(0, V, (200,), device=DEV)
    labels[::5] = -100
    loss = ops.cross_entropy(logits, labels, label_smoothing=smoothing, z_loss=z)
    loss.backward()
    lf = logits.detach().float().requires_grad_()
    lr = ref.cross_entropy(lf, labels, label_smoothing=smoothing, z_loss=z)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-3 * max(1.0, abs(lr.item())), (loss.item(), lr.item())
    _close(logits.grad, lf.grad, 2e-5, 2e-2, "dlogits")


def test_linear_cross_entropy_with_l2_warp():
    """The l2-warp term (max logit * 1e-4 / valid tokens at each row's arg-max) is added inside the row kernel."""
    N, Hd, V = 600, 256, 4096
    h = (torch.randn(N, Hd, device=DEV) * 0.5).to(BF).requires_grad_()
    w = (torch.randn(V, Hd, device=DEV) * 0.1).to(BF).requires_grad_()
    labels = torch.randint(0, V, (N,), device=DEV)
    labels[:50] = -100
    penalty = 20.0                                  # large enough to stand out from bf16 rounding of the CE part
    plain = ops.linear_cross_entropy(h, labels, w, num_chunks=3)
    g_plain = torch.autograd.grad(plain, [h, w])
    loss = ops.linear_cross_entropy(h, labels, w, num_chunks=3, l2_penalty=penalty)
    loss.backward()
    assert abs(loss.item() - plain.item()) < 1e-6                          # the term touches gradients only
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    # the arg-max column is taken from the bf16 logits the kernel sees (an fp32 product breaks near-ties differently)
    seen = ops.linear(h.detach(), w.detach()).float()
    mx, idx = seen.max(-1, keepdim=True)
    lg = hf @ wf.t()
    total = labels.ne(-100).sum()
    lr = ref.cross_entropy(lg, labels) + (lg.gather(-1, idx) * (mx * penalty / total)).sum()
    lr.backward()
    assert (h.grad - g_plain[0]).abs().max() > 1e-4, "the penalty changed nothing"
    # the warp term is stored in the bf16 gradient of the logits (0.4 % of a value that the large test penalty makes
    # ~0.1), so the absolute tolerance follows the penalty
    _close(h.grad, hf.grad, 2e-3, 5e-2, "lce+l2warp dh")
    _close(w.grad, wf.grad, 2e-3, 5e-2, "lce+l2warp dw")


@pytest.mark.parametrize("rows,K,V", [(300, 256, 4096 + 24), (1024, 128, 1000), (129, 64, 200)])
def test_gemm_epilogue_row_statistics(rows, K, V):
    """The logits GEMM's epilogue leaves (max, sum of exp) per row and column tile; merged they are the row's
    log-sum-exp over the bf16 logits it wrote (ragged last tile, rows past a 128 boundary)."""
    from ttcd_b200.ops import cuda
    h = (torch.randn(rows, K, device=DEV) * 0.5).to(BF)
    w = (torch.randn(V, K, device=DEV) * 0.3).to(BF)
    out = torch.empty(rows, V, device=DEV, dtype=BF)
    parts = cuda._logits_with_lse(h, w, out)
    _close(out, h.float() @ w.float().t(), 0.05, 2e-2, "logits")
    m, s_ = parts[..., 0], parts[..., 1]
    big = m.max(dim=1, keepdim=True).values
    lse = big.squeeze(1) + torch.log((s_ * torch.exp(m - big)).sum(dim=1))
    torch.testing.assert_close(lse, torch.logsumexp(out.float(), dim=-1), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("BH,n,D,Dv", [(3, 5, 32, 32), (2, 7, 128, 64), (2, 3, 256, 96), (5, 1, 64, 128), (2, 4, 256, 128)])
def test_delta_chain_kernels_match_the_loop(BH, n, D, Dv):
    """The chunk-to-chunk chain of the delta rule (one launch per direction) against the same recurrence written as
    a PyTorch loop: corrected values, the state entering every chunk, the final state, and all five gradients."""
    from ttcd_b200.ops import delta_chain as dc
    gen = torch.Generator().manual_seed(BH * 100 + D)
    mk = lambda *sh, sc=0.2: (torch.randn(*sh, generator=gen) * sc).to(DEV).requires_grad_()  # noqa: E731
    mk16 = lambda *sh, sc: (torch.randn(*sh, generator=gen) * sc).bfloat16().float().to(DEV).requires_grad_()  # noqa: E731
    # w and kt are multiplied as bf16 by the kernels: values that bf16 holds exactly, so that the loop sees the same numbers
    w, u, kt, s0 = mk16(BH, n, 64, D, sc=0.1), mk(BH, n, 64, Dv), mk16(BH, n, 64, D, sc=0.1), mk(BH, D, Dv)
    gamma = torch.rand(BH, n, generator=gen).to(DEV).requires_grad_()
    assert dc._native_ok(w, u)
    outs = dc.delta_chain(w, u, kt, gamma, s0)
    want = dc._fwd_torch(*(t.detach() for t in (w, u, kt, gamma, s0)))
    # the running state and the corrected values enter the products rounded to bf16: errors relative to the largest entry
    for a, b, name in zip(outs, want, ("vn", "states", "final")):
        torch.testing.assert_close(a, b, rtol=0, atol=8e-3 * float(b.abs().max()), msg=lambda m, name=name: f"{name}: {m}")
        assert _cos(a, b) > 0.9999, name
    gs = [torch.randn_like(o) for o in outs]
    got = torch.autograd.grad(outs, [w, u, kt, gamma, s0], gs)
    d_vn_tot, ds_next, d_s0 = dc._bwd_torch(w.detach(), kt.detach(), gamma.detach(), *gs)
    states = want[1]
    ref = [-(d_vn_tot @ states.transpose(-1, -2)), d_vn_tot, want[0] @ ds_next.transpose(-1, -2),
           (states * ds_next).sum(dim=(-1, -2)), d_s0]
    for a, b, name in zip(got, ref, ("dw", "du", "dkt", "dgamma", "ds0")):
        torch.testing.assert_close(a, b, rtol=0, atol=8e-3 * float(b.abs().max()), msg=lambda m, name=name: f"{name}: {m}")
        assert _cos(a, b) > 0.9999, name


def _delta_inputs(B, T, H, D, Dv, gated, l2norm, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, D, generator=gen), torch.randn(B, T, H, D, generator=gen)
    if not l2norm:                       # callers that switch the normalisation off pass unit keys
        k = torch.nn.functional.normalize(k, dim=-1)
    v = torch.randn(B, T, H, Dv, generator=gen)
    beta = torch.rand(B, T, H, generator=gen)
    g = -torch.rand(B, T, H, generator=gen) * 0.3 if gated else None
    q, k, v = (t.to(DEV).to(dtype) for t in (q, k, v))
    return q, k, v, beta.to(DEV), None if g is None else g.to(DEV)


@pytest.mark.parametrize("D,Dv,gated,l2norm,dtype", [(64, 64, True, True, torch.float32), (128, 128, False, True, BF),
                                                      (256, 128, True, False, torch.float32), (128, 192, True, True, BF)])
def test_delta_prep_kernels_match_their_statement(D, Dv, gated, l2norm, dtype):
    """The chunk-local kernels of the delta rule (WY factors, scaled keys / queries, intra-chunk scores; and the
    gradients of q, k, v, beta, g from the gradients of those) against the same formulas in float64, on a ragged
    length (the last chunk has 8 of 64 rows)."""
    from ttcd_b200.ops import delta_fused as df
    B, T, H = 2, 200, 3
    q, k, v, beta, g = _delta_inputs(B, T, H, D, Dv, gated, l2norm, dtype, seed=D + Dv)
    scale = D ** -0.5
    assert df.native_ok(q, v)
    dbl = lambda t: None if t is None else t.double()  # noqa: E731
    got = df._prep_fwd(q, k, v, beta, g, scale, l2norm)
    want = df._prep_fwd_torch(dbl(q), dbl(k), dbl(v), dbl(beta), dbl(g), scale, l2norm)
    # the 64 x 64 x 64 products run with TF32 operands (10-bit mantissa): errors relative to the largest entry
    for a, b, name in zip(got, want, ("w", "u", "kt", "q_in", "qk", "gamma")):
        tol = float(b.abs().max()) * {"q_in": 1e-5, "gamma": 1e-5, "kt": 4e-3, "w": 5e-3}.get(name, 2e-3)    # w, kt are stored as bf16
        torch.testing.assert_close(a.double(), b, rtol=0, atol=tol, msg=lambda m, name=name: f"{name}: {m}")
    gen = torch.Generator().manual_seed(7)
    grads = [torch.randn(o.shape, generator=gen).to(DEV) for o in got]
    got_b = df._prep_bwd(q, k, v, beta, g, scale, l2norm, *grads)
    want_b = df._prep_bwd_torch(dbl(q), dbl(k), dbl(v), dbl(beta), dbl(g), scale, l2norm, *(t.double() for t in grads))
    for a, b, name in zip(got_b, want_b, ("dq", "dk", "dv", "dbeta", "dg")):
        if b is None:
            assert a is None
            continue
        tol = float(b.abs().max()) * 4e-3
        torch.testing.assert_close(a.double(), b, rtol=0, atol=tol, msg=lambda m, name=name: f"{name}: {m}")
        assert _cos(a, b) > 0.99999, (name, _cos(a, b))


@pytest.mark.parametrize("gated,keep", [(True, "1"), (False, "0")])
def test_fused_delta_rule_matches_its_cpu_statement(gated, keep, monkeypatch):
    """The whole op on CUDA (kernels + batched products, intermediates kept or rebuilt in backward) against the same op in
    float64 on the CPU: outputs, final state and the gradients of q, k, v, g, beta and the initial state."""
    from ttcd_b200.ops import delta_fused as df
    monkeypatch.setenv("TTCD_DELTA_KEEP", keep)
    B, T, H, D, Dv = 2, 333, 2, 128, 128
    q, k, v, beta, g = _delta_inputs(B, T, H, D, Dv, gated, True, torch.float32, seed=11)
    s0 = (torch.randn(B, H, D, Dv, generator=torch.Generator().manual_seed(5)) * 0.1).to(DEV)
    dev = [None if t is None else t.clone().requires_grad_() for t in (q, k, v, g, beta, s0)]
    cpu = [None if t is None else t.detach().double().cpu().requires_grad_() for t in (q, k, v, g, beta, s0)]
    o, s = df.gated_delta_rule_fused(*dev[:5], None, True, dev[5], True)
    o_ref, s_ref = df.gated_delta_rule_fused(*cpu[:5], None, True, cpu[5], True)
    go, gs = torch.randn_like(o_ref), torch.randn_like(s_ref)
    ((o_ref * go).sum() + (s_ref * gs).sum()).backward()
    ((o * go.to(DEV).float()).sum() + (s * gs.to(DEV).float()).sum()).backward()
    assert _cos(o.cpu().double(), o_ref) > 0.99999 and _cos(s.cpu().double(), s_ref) > 0.99999
    for a, b, name in zip(dev, cpu, ("q", "k", "v", "g", "beta", "s0")):
        if a is not None:
            assert _cos(a.grad.cpu().double(), b.grad) > 0.9999, (name, _cos(a.grad.cpu().double(), b.grad))


def test_adamw_and_sumsq():
    from ttcd_b200.ops import cuda
    n = 100_003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(BF)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    pb = torch.empty(n, device=DEV, dtype=BF)
    coef = torch.tensor([0.5], device=DEV)
    for step in (1, 2, 3):
        cuda.adamw_step(p, g, m, v, pb, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-15, weight_decay=0.1, step=step, coef=coef)
        ref.adamw_step(pr, g, mr, vr, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-15, weight_decay=0.1, step=step, grad_scale=0.5)
    _close(p, pr, 1e-5, 1e-4, "adamw p")
    _close(pb, pr, 1e-2, 1e-2, "adamw bf16 copy")
    out = torch.zeros(1, device=DEV)
    cuda.sumsq(g, out)
    assert abs(out.item() - g.float().pow(2).sum().item()) < 1e-3 * out.item()


def test_newton_schulz():
    g = torch.randn(2, 256, 512, device=DEV, dtype=BF)
    got = ops.newton_schulz(g)
    want = ref.newton_schulz(g.float(), dtype=torch.float32)
    _close(got, want, 0.06, 0.1, "newton-schulz")


# ------------------------------------------------------------------------------------- attention fwd

def _attn_inputs(B, T, H, HK, D, scale=1.0, Tk=None):
    Tk = T if Tk is None else Tk
    q = (torch.randn(B, T, H, D, device=DEV) * scale).to(BF)
    k = (torch.randn(B, Tk, HK, D, device=DEV) * scale).to(BF)
    v = torch.randn(B, Tk, HK, D, device=DEV).to(BF)
    return q, k, v


ATTN_TOL = dict(atol=8e-3, rtol=1e-2)


@pytest.mark.parametrize("T,H,HK,D,W", [(128, 2, 1, 128, None), (257, 4, 2, 128, 100), (513, 2, 2, 64, 192),
                                         (769, 3, 1, 128, 64), (1024, 4, 4, 128, 1024), (2000, 2, 1, 64, None)])
def test_attention_single_window_fwd(T, H, HK, D, W):
    from ttcd_b200.ops import cuda
    q, k, v = _attn_inputs(2, T, H, HK, D)
    with torch.no_grad():
        _, o, _, lse, _ = cuda.attn_forward(q, k, v, W, W, D ** -0.5, False)
    o_r, lse_r = ref.attention(q, k, v, W, return_lse=True)
    _close(o, o_r, name="attn o", **ATTN_TOL)
    _close(lse, lse_r, 2e-2, 1e-3, "attn lse")


@pytest.mark.parametrize("T,H,HK,D,WT,WS", [(512, 2, 1, 128, 256, 128), (1000, 4, 2, 128, 400, 200),
                                             (769, 3, 3, 64, 300, 150), (1536, 2, 1, 128, None, 256),
                                             (700, 2, 2, 128, 256, 256), (900, 2, 1, 128, 320, 288),
                                             (4097, 2, 1, 128, 2048, 1024)])
def test_attention_dual_window_fwd(T, H, HK, D, WT, WS):
    from ttcd_b200.ops import cuda
    q, k, v = _attn_inputs(1, T, H, HK, D)
    with torch.no_grad():
        _, o_t, o_s, lse_t, lse_s = cuda.attn_forward(q, k, v, WT, WS, D ** -0.5, True)
    r_t, l_t = ref.attention(q, k, v, WT, return_lse=True)
    r_s, l_s = ref.attention(q, k, v, WS, return_lse=True)
    _close(o_s, r_s, name="student o", **ATTN_TOL)
    _close(o_t, r_t, name="teacher o", **ATTN_TOL)
    _close(lse_t, l_t, 2e-2, 1e-3, "teacher lse")
    _close(lse_s, l_s, 2e-2, 1e-3, "student lse")


@pytest.mark.parametrize("qk_scale", [0.0, 0.5, 4.0, 16.0])
def test_attention_scale_stress(qk_scale):
    from ttcd_b200.ops import cuda
    q, k, v = _attn_inputs(1, 640, 2, 1, 128, scale=qk_scale)
    with torch.no_grad():
        _, o_t, o_s, _, _ = cuda.attn_forward(q, k, v, 256, 128, 128 ** -0.5, True)
    r_t, r_s = ref.dual_window_attention(q, k, v, 256, 128)
    _close(o_t, r_t, name="teacher", **ATTN_TOL)
    _close(o_s, r_s, name="student", **ATTN_TOL)


def test_attention_cached_prefill_tq_lt_tk():
    from ttcd_b200.ops import cuda
    q, k, v = _attn_inputs(1, 200, 2, 1, 128, Tk=712)
    with torch.no_grad():
        _, o_t, o_s, _, _ = cuda.attn_forward(q, k, v, 512, 256, 128 ** -0.5, True)
    r_t, r_s = ref.dual_window_attention(q, k, v, 512, 256)
    _close(o_t, r_t, name="teacher", **ATTN_TOL)
    _close(o_s, r_s, name="student", **ATTN_TOL)


def test_activation_offload_roundtrip_matches_resident():
    """Saved activations parked in pinned host memory give the same gradients as resident ones."""
    from ttcd_b200.train.activation_offload import OffloadActivations
    torch.manual_seed(0)
    w1 = torch.randn(512, 512, device="cuda", requires_grad=True)
    w2 = torch.randn(512, 512, device="cuda", requires_grad=True)
    x = torch.randn(4096, 512, device="cuda")

    def run(ctx):
        for w in (w1, w2):
            w.grad = None
        with ctx:
            h = torch.tanh(x @ w1)
            y = torch.sigmoid(h @ w2).square().sum()
        y.backward()
        return w1.grad.clone(), w2.grad.clone()

    import contextlib
    ref = run(contextlib.nullcontext())
    off = OffloadActivations(min_offload_bytes=1 << 16, max_fwd_stash=2)
    got = run(off)
    assert off.bytes_offloaded >= 2 * 4096 * 512 * 4
    for a, b in zip(ref, got):
        torch.testing.assert_close(a, b)
    got2 = run(off)          # second pass reuses the pooled host buffers
    torch.testing.assert_close(ref[0], got2[0])


@pytest.mark.parametrize("b,T,with_beta", [(1, 4, True), (2, 3, True), (1, 5, False), (1, 1, True)])
def test_fused_ttt_scan_matches_reference(b, T, with_beta):
    """Batched-GEMM scan with prefix/suffix kernels vs the fp32 statement of the same math: outputs and all
    six gradients."""
    from ttcd_b200.ops import cuda
    from ttcd_b200.ops import reference as ref
    torch.manual_seed(3)
    C, d_i, d_h, lr = 128, 256, 128, 0.3
    mk = lambda *s, scale=1.0: (torch.randn(*s, device="cuda") * scale).bfloat16().requires_grad_()  # noqa: E731
    z_out, z_tgt, z_hat = mk(b, T, C, d_i, scale=0.5), mk(b, T, C, d_i, scale=0.5), mk(b, T, C, d_i, scale=0.5)
    beta = torch.sigmoid(torch.randn(b, T, C, 1, device="cuda")).bfloat16().requires_grad_() if with_beta else None
    w_down, w_upd = mk(d_h, d_i, scale=0.05), mk(d_i, d_h, scale=0.05)
    dy = (torch.randn(b, T, C, d_h, device="cuda") * 0.1).bfloat16()
    inputs = [t for t in (z_out, z_tgt, z_hat, beta, w_down, w_upd) if t is not None]
    y, last = cuda.ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_upd, lr)
    got = torch.autograd.grad(y, inputs, dy, allow_unused=True)
    f = lambda t: None if t is None else t.detach().float().requires_grad_()  # noqa: E731
    fin = [f(t) for t in (z_out, z_tgt, z_hat, beta, w_down, w_upd)]
    y_ref, last_ref = ref.ttt_scan(*fin, lr=lr, update_every=2, state_dtype=torch.float32, return_last_dw_norm=True)
    want = torch.autograd.grad(y_ref, [t for t in fin if t is not None], dy.float(), allow_unused=True)
    assert (y.float() - y_ref).abs().max().item() < 3e-2 * (y_ref.abs().max().item() + 1e-6)     # bf16 operands
    if T > 1:
        torch.testing.assert_close(last.float(), last_ref.float(), rtol=3e-2, atol=1e-2)
    names = [n for n, t in zip(("z_out", "z_tgt", "z_hat", "beta", "w_down", "w_upd"), (z_out, z_tgt, z_hat, beta, w_down, w_upd)) if t is not None]
    for n, a, w in zip(names, got, want):
        if w is None:                      # T == 1: nothing updates, those inputs do not reach the output
            assert a is None or float(a.float().abs().max()) == 0.0, n
            continue
        err = (a.float() - w).abs().max().item()
        ref_mag = w.abs().max().item() + 1e-6
        assert err / ref_mag < 6e-2, (n, err, ref_mag)


def test_split_k_weight_gradient_gemm():
    """Token dimension split into batched slices with fp32 partials == one long-K GEMM."""
    from ttcd_b200.ops import cuda
    torch.manual_seed(5)
    T, n_out, k_in = 8192, 1024, 2048
    assert cuda._split_k_factor(n_out, k_in, T) > 1
    wide = (torch.randn(T, n_out + 512, device="cuda") * 0.1).bfloat16()
    g = wide[:, :n_out]                                   # a column slice of a wider gradient buffer (row stride > width)
    x = (torch.randn(T, k_in, device="cuda") * 0.1).bfloat16()
    got = cuda.gemm_wgrad(g, x)
    want = g.float().t() @ x.float()
    assert got.shape == (n_out, k_in)
    assert (got.float() - want).abs().max().item() < 2e-2 * want.abs().max().item()
    lin = torch.nn.Linear(k_in, n_out, bias=False, device="cuda", dtype=torch.bfloat16)
    xx = x.clone().requires_grad_()
    y = cuda.linear(xx, lin.weight)
    y.backward(wide[:, :n_out].contiguous())
    ref = wide[:, :n_out].float().t() @ x.float()
    assert (lin.weight.grad.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 1024), (3, 304, 1088), (16, 1024, 3072), (5, 151936, 1024)])
def test_small_row_linear_uses_the_weight_streaming_kernel(M, N, K):
    """A handful of rows times a [N, K] weight (the decode step) against fp32 PyTorch; the same call with 17 rows takes
    the tensor-core path and must agree with it."""
    from ttcd_b200 import _native
    from ttcd_b200.ops import cuda
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    before = _native.launch_count
    y = cuda.gemm(x, w.t())
    assert _native.launch_count == before + 1          # one kernel, no padding copies
    want = x.float() @ w.float().t()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)
    x17 = torch.cat([x, torch.randn(17 - M, K, device="cuda").bfloat16()])
    y17 = cuda.gemm(x17, w.t())
    torch.testing.assert_close(y17.reshape(17, N)[:M].float(), y.float(), rtol=2e-2, atol=2e-2)
