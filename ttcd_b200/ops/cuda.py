"""Autograd Functions and launch wrappers for the hand-written sm_100a kernels.

Every function here takes CUDA bf16 tensors and calls ``libttcd_b200.so`` through
``ttcd_b200._native``; forward and backward both run on the native kernels.  Shapes are
validated on the host before a launch (the kernels do no bounds recovery).
"""
from __future__ import annotations

import math

import torch

from .. import _native as nv
from . import reference
from .selective import keep

_BF16 = torch.bfloat16
_SM_BLOCKS = 148 * 2


def _check(t: torch.Tensor, name: str):
    if not (t.is_cuda and t.dtype == _BF16):
        raise TypeError(f"{name} must be a CUDA bf16 tensor, got {t.dtype} on {t.device}")


def _rows2d(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


def _dense_rows(x: torch.Tensor) -> torch.Tensor:
    """2-D view with unit inner stride and a 16-byte aligned row stride (copy only if needed)."""
    x2 = _rows2d(x)
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


# =============================================================================================
# GEMM
# =============================================================================================

def _operand(t: torch.Tensor):
    """Describe a [.., R, C] matrix for the kernel: (tensor, is_row_major, ld, batch_stride)."""
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if t.dim() > 3:
        t = t.reshape(-1, t.shape[-2], t.shape[-1]) if t.is_contiguous() else t.contiguous().view(-1, *t.shape[-2:])
    ok_row = t.stride(-1) == 1 and t.stride(-2) % 8 == 0 and t.stride(-2) >= t.shape[-1]
    ok_col = t.stride(-2) == 1 and t.stride(-1) % 8 == 0 and t.stride(-1) >= t.shape[-2]
    if t.shape[-1] == 1 and t.shape[-2] == 1:
        ok_row, ok_col = False, False
    if not (ok_row or ok_col) or t.data_ptr() % 16 or (t.shape[0] > 1 and t.stride(0) % 8):
        t = t.contiguous()
        ok_row, ok_col = True, False
    row_major = ok_row
    ld = t.stride(-2) if row_major else t.stride(-1)
    return t, row_major, ld, (t.stride(0) if t.shape[0] > 1 else 0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, out_dtype=_BF16, alpha: float = 1.0, beta: float = 0.0,
         c_in: torch.Tensor | None = None, row_scale: torch.Tensor | None = None,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """C[.., M, N] = alpha * rowscale * (a[.., M, K] @ b[.., K, N]) + beta * c_in.

    ``a`` / ``b`` may be transposed views: a row-major a is a K-major A operand, a column-major a
    (i.e. ``x.transpose(-1, -2)`` of a row-major tensor) is MN-major; b row-major [K, N] is an
    MN-major B operand, b = w.transpose(-1, -2) of row-major w [N, K] is K-major.
    """
    _check(a, "a"), _check(b, "b")
    M0, K0, N0 = a.shape[-2], a.shape[-1], b.shape[-1]
    if (M0 <= 16 and a.dim() == 2 and b.dim() == 2 and out_dtype == _BF16 and beta == 0.0 and c_in is None
            and row_scale is None and out is None and K0 % 8 == 0 and b.stride(0) == 1 and b.stride(1) % 8 == 0
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
            and nv.has("ttcd_gemv_small")):
        # a few rows times a [N, K] weight (b is its transposed view): the decode step; one pass over the weight
        y = torch.empty(M0, N0, dtype=_BF16, device=a.device)
        nv.call("ttcd_gemv_small", nv.ptr(a), nv.ptr(b), nv.ptr(y), nv.i32(M0), nv.i32(N0), nv.i32(K0), nv.i64(a.stride(0)),
                nv.i64(b.stride(1)), nv.i64(N0), nv.f32(alpha), nv.stream_ptr())
        return y
    if M0 < 128 or N0 < 128 or K0 < 64:
        # tiny problem: zero-pad up to one tile (TMA boxes must fit inside their tensors)
        if out is not None or c_in is not None or row_scale is not None:
            raise ValueError("gemm with M < 128, N < 128 or K < 64 does not support out/c_in/row_scale")
        Mp, Kp, Np = max(M0, 128), max(K0, 64), max(N0, 128)
        ap = torch.nn.functional.pad(a, (0, Kp - K0, 0, Mp - M0))
        bp = torch.nn.functional.pad(b, (0, Np - N0, 0, Kp - K0))
        full = gemm(ap, bp, out_dtype=out_dtype, alpha=alpha)
        return full[..., :M0, :N0].contiguous()
    a3, a_row, lda, sa = _operand(a)
    b3, b_row, ldb, sb = _operand(b)
    batch = max(a3.shape[0], b3.shape[0])
    M, K = a3.shape[-2], a3.shape[-1]
    K2, N = b3.shape[-2], b3.shape[-1]
    if K != K2:
        raise ValueError(f"gemm shape mismatch: {tuple(a.shape)} @ {tuple(b.shape)}")
    if a3.shape[0] not in (1, batch) or b3.shape[0] not in (1, batch):
        raise ValueError("gemm batch mismatch")
    if a3.shape[0] == 1:
        sa = 0
    if b3.shape[0] == 1:
        sb = 0
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
    c3 = out.view(batch, M, N) if out.dim() != 3 else out
    if c3.stride(-1) != 1:
        raise ValueError("gemm output must be row-major")
    if c_in is not None:
        c_in3 = c_in.view(batch, M, N) if c_in.dim() != 3 else c_in
        if c_in3.stride() != c3.stride() or c_in3.dtype != c3.dtype:
            raise ValueError("c_in must match the output layout and dtype")
    a_mn = 0 if a_row else 1           # A logical [M, K]: row-major => K-major
    b_mn = 1 if b_row else 0           # B given as [K, N]: row-major => N contiguous => MN-major
    nv.call(
        "ttcd_gemm_bf16", nv.ptr(a3), nv.ptr(b3), nv.ptr(c3), nv.ptr(c_in if c_in is not None else None),
        nv.ptr(row_scale), nv.i64(M), nv.i64(N), nv.i64(K), nv.i64(batch), nv.i64(lda), nv.i64(ldb),
        nv.i64(c3.stride(-2)), nv.i64(sa), nv.i64(sb), nv.i64(c3.stride(0) if batch > 1 else M * c3.stride(-2)),
        nv.i32(a_mn), nv.i32(b_mn), nv.i32(1 if c3.dtype == torch.float32 else 0), nv.f32(alpha), nv.f32(beta),
        nv.stream_ptr())
    return out


class GradSlab:
    """Meeting point for the gradients of the column slices of one fused projection (q|k|v): the backward
    kernels of the consumers write straight into one [rows, n_total] buffer, so the projection's backward
    finds its packed gradient in place instead of assembling it with copies.  The forward tags the slices
    (``tag``); whichever backward runs first allocates the buffer."""

    def __init__(self, n_total: int):
        self.n_total = n_total
        self.buf = None

    def get(self, rows: int, device) -> torch.Tensor:
        if self.buf is None or self.buf.shape[0] != rows:
            self.buf = torch.empty(rows, self.n_total, dtype=_BF16, device=device)
        return self.buf

    @staticmethod
    def tag(tensors, widths):
        slab, col = GradSlab(sum(widths)), 0
        for t, w in zip(tensors, widths):
            t._ttcd_grad_slab = (slab, col)
            col += w
        return slab


def _slab_of(t):
    return getattr(t, "_ttcd_grad_slab", None)


class _MatMul(torch.autograd.Function):
    """Batched a @ b with native forward and backward."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        out_shape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2]) + (a.shape[-2], b.shape[-1])
        return keep(lambda: gemm(a, b)).view(out_shape)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        ga = gb = None
        g = g if g.dtype == _BF16 else g.to(_BF16)
        if ctx.needs_input_grad[0]:
            ga = gemm(g, b.transpose(-1, -2))
            ga = _reduce_to(ga.view(torch.broadcast_shapes(g.shape[:-2], b.shape[:-2]) + ga.shape[-2:]), a.shape)
        if ctx.needs_input_grad[1]:
            gb = gemm(a.transpose(-1, -2), g)
            gb = _reduce_to(gb.view(torch.broadcast_shapes(g.shape[:-2], a.shape[:-2]) + gb.shape[-2:]), b.shape)
        return ga, gb


def _reduce_to(t: torch.Tensor, shape) -> torch.Tensor:
    """Sum broadcast batch dims so that t matches ``shape``."""
    if tuple(t.shape) == tuple(shape):
        return t
    while t.dim() > len(shape):
        t = t.sum(0)
    for i, (ts, s) in enumerate(zip(t.shape, shape)):
        if s == 1 and ts != 1:
            t = t.sum(i, keepdim=True)
    return t.reshape(shape)


def matmul(a, b):
    if a.dtype != _BF16:
        a = a.to(_BF16)
    if b.dtype != _BF16:
        b = b.to(_BF16)
    return _MatMul.apply(a, b)


def _split_k_factor(M: int, N: int, K: int, sms: int = 148) -> int:
    """Number of K slices for a weight-gradient GEMM (M, N = weight dims, K = tokens): the output has few tiles
    (64-192 for this model) and would leave a third of the 148 SMs idle or run a mostly empty second wave."""
    tiles = -(-M // 128) * -(-N // (256 if N >= 256 else 128))
    if tiles >= 4 * sms:
        return 1
    best, best_eff = 1, tiles / (-(-tiles // sms) * sms)
    for s_ in range(2, 17):
        if K % (s_ * 64) or K // s_ < 2048:
            continue
        eff = tiles * s_ / (-(-tiles * s_ // sms) * sms)
        if eff > best_eff + 0.02:
            best, best_eff = s_, eff
        if best_eff >= 0.95:
            break
    return best


def gemm_wgrad(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """dW[N_out, K_in] = g[T, N_out]^T @ x[T, K_in] with the token dimension split into slices that run as a
    batched GEMM (fp32 partials, summed once): fills the machine when the weight has few output tiles."""
    T, n_out = g.shape
    k_in = x.shape[1]
    s_ = _split_k_factor(n_out, k_in, T)
    if s_ == 1 or g.stride(1) != 1 or x.stride(1) != 1:
        return gemm(g.transpose(0, 1), x).view(n_out, k_in)
    ts = T // s_
    ga = torch.as_strided(g, (s_, n_out, ts), (ts * g.stride(0), 1, g.stride(0)), g.storage_offset())      # [S, N_out, Ts] view of g^T
    xa = torch.as_strided(x, (s_, ts, k_in), (ts * x.stride(0), x.stride(0), 1), x.storage_offset())
    part = gemm(ga, xa, out_dtype=torch.float32)                                                             # [S, N_out, K_in]
    return part.sum(0).to(_BF16)


_gather_handle = None      # sharded-weights mode: the PendingGather of the projection being run (set by fused_linear)


class _Linear(torch.autograd.Function):
    """y = x @ W^T for one or several weights that share x (one GEMM when they form a slab)."""

    @staticmethod
    def forward(ctx, x, slab, *weights):
        global _gather_handle
        handle, _gather_handle = _gather_handle, None
        x2 = _dense_rows(x)
        if handle is not None and slab is None:
            handle.ensure()            # no single slab to gather into a GEMM: gather first
        w = slab if slab is not None else (weights[0] if len(weights) == 1 else torch.cat(weights, dim=0))
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.splits = [wi.shape[0] for wi in weights]

        def run():
            # sharded weights: this GEMM is the block's first consumer and gathers the block while it multiplies
            y_ = handle.linear(x2, w) if handle is not None else None
            return y_ if y_ is not None else gemm(x2, w.transpose(0, 1))
        y = keep(run).view(x2.shape[0], w.shape[0])
        if handle is not None:
            handle.ensure()            # a replayed (not re-launched) GEMM gathered nothing
        if len(weights) == 1:
            return y.view(*x.shape[:-1], w.shape[0])
        outs, col = [], 0
        for n in ctx.splits:
            outs.append(y[:, col:col + n].view(*x.shape[:-1], n))
            col += n
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        x2, w = ctx.saved_tensors
        n_total = w.shape[0]
        if len(grads) == 1:
            g = _dense_rows(grads[0].to(_BF16))
        elif (g := _adjacent_columns(grads, ctx.splits, n_total)) is not None:
            pass  # the incoming gradients already sit side by side in one buffer
        else:
            # the outputs are column slices of one buffer; rebuild the packed gradient
            g = torch.empty(x2.shape[0], n_total, dtype=_BF16, device=x2.device)
            col = 0
            for gi, n in zip(grads, ctx.splits):
                if gi is None:
                    g[:, col:col + n].zero_()
                else:
                    g[:, col:col + n].copy_(gi.reshape(-1, n))
                col += n
        gx = None
        if ctx.needs_input_grad[0]:
            gx = gemm(g, w).view(ctx.x_shape)
        gw_all = gemm_wgrad(g, x2)
        gws, row = [], 0
        for n in ctx.splits:
            gws.append(gw_all[row:row + n])
            row += n
        return (gx, None, *gws)


def _adjacent_columns(grads, splits, n_total):
    """If the gradients are consecutive column slices of one [rows, n_total] buffer, return it."""
    if any(g is None or g.dtype != _BF16 for g in grads):
        return None
    try:
        views = [g.view(-1, n) for g, n in zip(grads, splits)]
    except RuntimeError:
        return None
    base = views[0]
    expect = base.data_ptr()
    for v, n in zip(views, splits):
        if v.stride() != (n_total, 1) or v.data_ptr() != expect:
            return None
        expect += n * 2
    if base.data_ptr() % 16:
        return None
    return torch.as_strided(base, (base.shape[0], n_total), (n_total, 1))


def linear(x, weight, bias=None):
    _check(x, "x")
    w = weight if weight.dtype == _BF16 else weight.to(_BF16)
    y = _Linear.apply(x, None, w)
    return y if bias is None else y + bias.to(y.dtype)


def fused_linear(x, weights, slab):
    """Several projections of the same input; returns a tuple of column views of one output."""
    global _gather_handle
    ws = [w if w.dtype == _BF16 else w.to(_BF16) for w in weights]
    if any(w.dtype != weights[i].dtype for i, w in enumerate(ws)):
        slab = None
    handle = getattr(weights[0], "_ttcd_gather", None)
    if handle is not None:
        weights[0]._ttcd_gather = None
        _gather_handle = handle if handle.pending else None
    return _Linear.apply(x, slab, *ws)


# =============================================================================================
# RMSNorm
# =============================================================================================

def _rmsnorm_fwd(x2, res2, w, eps, want_sum):
    rows, D = x2.shape
    y = torch.empty_like(x2)
    s = torch.empty_like(x2) if want_sum else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    nv.call("ttcd_rmsnorm_fwd", nv.ptr(x2), nv.ptr(res2), nv.ptr(w), nv.ptr(y), nv.ptr(s), nv.ptr(rstd),
            nv.i64(rows), nv.i32(D), nv.f32(eps), nv.stream_ptr())
    return y, s, rstd


def _rmsnorm_bwd(dy2, s2, w, rstd, dres2):
    rows, D = dy2.shape
    dx = torch.empty_like(dy2)
    nblk = min(_SM_BLOCKS, (rows + 7) // 8)
    dwp = torch.empty(nblk, D, dtype=torch.float32, device=dy2.device) if w is not None else None
    nv.call("ttcd_rmsnorm_bwd", nv.ptr(dy2), nv.ptr(s2), nv.ptr(w), nv.ptr(rstd), nv.ptr(dres2), nv.ptr(dx),
            nv.ptr(dwp), nv.i64(rows), nv.i32(D), nv.i32(nblk), nv.stream_ptr())
    dw = dwp.sum(0) if dwp is not None else None
    return dx, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, prenorm):
        x2 = _rows2d(x).contiguous()
        r2 = _rows2d(residual).contiguous() if residual is not None else None
        w = None if weight is None else weight.to(_BF16).contiguous()
        y, s, rstd = _rmsnorm_fwd(x2, r2, w, eps, want_sum=r2 is not None)
        ctx.save_for_backward(s if s is not None else x2, w, rstd)
        ctx.has_res = r2 is not None
        ctx.prenorm = prenorm
        ctx.wdtype = None if weight is None else weight.dtype
        y = y.view(x.shape)
        if prenorm:
            return y, (s.view(x.shape) if s is not None else x)
        return y

    @staticmethod
    def backward(ctx, dy, dres_out=None):
        s, w, rstd = ctx.saved_tensors
        dy2 = _rows2d(dy).contiguous().to(_BF16)
        dres2 = None
        if ctx.prenorm and dres_out is not None:
            dres2 = _rows2d(dres_out).contiguous().to(_BF16)
        dx, dw = _rmsnorm_bwd(dy2, s, w, rstd, dres2)
        dx = dx.view(dy.shape)
        if dw is not None:
            dw = dw.to(ctx.wdtype)
        return dx, (dx if ctx.has_res else None), dw, None, None


def rmsnorm(x, weight, eps, residual=None, prenorm=False):
    _check(x, "x")
    return _RMSNorm.apply(x, residual, weight, float(eps), bool(prenorm))


class _RMSNormDual(torch.autograd.Function):
    """x = norm(r + a_T), t = norm(r + a_S), r_out = r + a_T with one shared weight: one kernel forward (the residual
    is read once), one kernel backward (d_a_T, d_a_S, d_r and the weight-gradient partial sums of both streams)."""

    @staticmethod
    def forward(ctx, a_t, a_s, residual, weight, eps):
        at2, as2, r2 = (_rows2d(v).contiguous() for v in (a_t, a_s, residual))
        w = weight.to(_BF16).contiguous()
        rows, D = at2.shape
        ctx.fused = D <= 2048
        if ctx.fused:
            x, t, s_t, s_s = (torch.empty_like(at2) for _ in range(4))
            rstd_t = torch.empty(rows, dtype=torch.float32, device=at2.device)
            rstd_s = torch.empty_like(rstd_t)
            nv.call("ttcd_rmsnorm_dual_fwd", nv.ptr(at2), nv.ptr(as2), nv.ptr(r2), nv.ptr(w), nv.ptr(x), nv.ptr(t),
                    nv.ptr(s_t), nv.ptr(s_s), nv.ptr(rstd_t), nv.ptr(rstd_s), nv.i64(rows), nv.i32(D), nv.f32(eps),
                    nv.stream_ptr())
        else:       # wide rows: the single-input streaming kernel, twice
            x, s_t, rstd_t = _rmsnorm_fwd(at2, r2, w, eps, True)
            t, s_s, rstd_s = _rmsnorm_fwd(as2, r2, w, eps, True)
        ctx.save_for_backward(s_t, s_s, w, rstd_t, rstd_s)
        ctx.wdtype = weight.dtype
        shp = a_t.shape
        return x.view(shp), t.view(shp), s_t.view(shp)

    @staticmethod
    def backward(ctx, dx, dt, dres):
        s_t, s_s, w, rstd_t, rstd_s = ctx.saved_tensors
        shp = dx.shape
        dx2, dt2 = _rows2d(dx).contiguous(), _rows2d(dt).contiguous()
        dres2 = None if dres is None else _rows2d(dres).contiguous()
        if not ctx.fused:
            d_at, dw_t = _rmsnorm_bwd(dx2, s_t, w, rstd_t, dres2)
            d_as, dw_s = _rmsnorm_bwd(dt2, s_s, w, rstd_s, None)
            return d_at.view(shp), d_as.view(shp), (d_at + d_as).view(shp), (dw_t + dw_s).to(ctx.wdtype), None
        rows, D = dx2.shape
        d_at, d_as, d_res = (torch.empty_like(dx2) for _ in range(3))
        nblk = min(148, (rows + 7) // 8)
        dwp = torch.empty(nblk, D, dtype=torch.float32, device=dx2.device)
        nv.call("ttcd_rmsnorm_dual_bwd", nv.ptr(dx2), nv.ptr(dt2), nv.ptr(s_t), nv.ptr(s_s), nv.ptr(w), nv.ptr(rstd_t),
                nv.ptr(rstd_s), nv.ptr(dres2), nv.ptr(d_at), nv.ptr(d_as), nv.ptr(d_res), nv.ptr(dwp), nv.i64(rows),
                nv.i32(D), nv.i32(nblk), nv.stream_ptr())
        return d_at.view(shp), d_as.view(shp), d_res.view(shp), dwp.sum(0).to(ctx.wdtype), None


def rmsnorm_dual(a_t, a_s, residual, weight, eps):
    _check(a_t, "a_t")
    return _RMSNormDual.apply(a_t, a_s, residual, weight, float(eps))


# =============================================================================================
# per-head q/k norm + rotary
# =============================================================================================

def _pos_arg(positions, rows, device):
    if positions is None:
        return None
    pos = positions.to(device=device, dtype=torch.int32).reshape(-1)
    if pos.numel() != rows:
        pos = pos.expand(rows // pos.numel(), pos.numel()).reshape(-1)
    return pos.contiguous()


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, qw, kw, eps, cos, sin, offset, positions):
        B, T, H, D = q.shape
        HK = k.shape[2]
        rows = B * T
        tq, tk = _slab_of(q), _slab_of(k)
        ctx.slab = (tq[0], tq[1], tk[1]) if (tq is not None and tk is not None and tq[0] is tk[0] and HK > 0) else None
        if q.stride(-1) != 1 or q.stride(2) != D or k.stride(-1) != 1 or k.stride(2) != D:
            q, k = q.contiguous(), k.contiguous()
        ldq, ldk = q.stride(1), k.stride(1)
        if (B > 1 and (q.stride(0) != T * ldq or k.stride(0) != T * ldk)):
            q, k = q.contiguous(), k.contiguous()
            ldq, ldk = q.stride(1), k.stride(1)
        q_out = torch.empty(B, T, H, D, dtype=_BF16, device=q.device)
        k_out = torch.empty(B, T, HK, D, dtype=_BF16, device=q.device)
        qwb = None if qw is None else qw.to(_BF16).contiguous()
        kwb = None if kw is None else kw.to(_BF16).contiguous()
        half = D // 2 if cos is None else cos.shape[-1]
        pos = _pos_arg(positions, rows, q.device)
        off = 0 if isinstance(offset, torch.Tensor) else int(offset)
        if isinstance(offset, torch.Tensor):
            pos = (torch.arange(T, device=q.device)[None, :] + offset.to(q.device).view(-1, 1)).to(torch.int32).reshape(-1)
        if cos is not None and not getattr(positions, "_ttcd_bounded", False):      # (a static cache checked its bound)
            need = (int(pos.max()) if pos is not None else T - 1 + off) + 1
            if cos.shape[0] < need:
                raise ValueError(f"rotary table has {cos.shape[0]} positions, need {need}")
        if cos is not None:
            cos, sin = cos.contiguous(), sin.contiguous()
        nv.call("ttcd_qk_norm_rope_fwd", nv.ptr(q), nv.i64(ldq), nv.ptr(k), nv.i64(ldk), nv.ptr(q_out), nv.i64(H * D),
                nv.ptr(k_out), nv.i64(HK * D), nv.ptr(qwb), nv.ptr(kwb), nv.ptr(cos), nv.ptr(sin), nv.ptr(pos),
                nv.i64(rows), nv.i32(T), nv.i32(off), nv.i32(H), nv.i32(HK), nv.i32(D), nv.i32(half), nv.f32(eps),
                nv.stream_ptr())
        ctx.save_for_backward(q, k, qwb, kwb, cos, sin, pos)
        ctx.meta = (B, T, H, HK, D, half, off, eps, ldq, ldk,
                    None if qw is None else qw.dtype, None if kw is None else kw.dtype)
        return q_out, k_out

    @staticmethod
    def backward(ctx, dq, dk):
        q, k, qwb, kwb, cos, sin, pos = ctx.saved_tensors
        B, T, H, HK, D, half, off, eps, ldq, ldk, qdt, kdt = ctx.meta
        rows = B * T
        dq, dk = dq.contiguous(), dk.contiguous()
        ldqo, ldko = H * D, HK * D
        if ctx.slab is not None:
            slab, cq, ck = ctx.slab
            buf = slab.get(rows, q.device)
            n_total = slab.n_total
            dq_in = torch.as_strided(buf, (B, T, H, D), (T * n_total, n_total, D, 1), cq)
            dk_in = torch.as_strided(buf, (B, T, HK, D), (T * n_total, n_total, D, 1), ck)
            ldqo = ldko = n_total
        else:
            dq_in = torch.empty(B, T, H, D, dtype=_BF16, device=q.device)
            dk_in = torch.empty(B, T, HK, D, dtype=_BF16, device=q.device)
        nblk = min(_SM_BLOCKS, (rows * (H + HK) + 7) // 8)
        has_w = qwb is not None
        dqw = torch.empty(nblk, D, dtype=torch.float32, device=q.device) if has_w else None
        dkw = torch.empty(nblk, D, dtype=torch.float32, device=q.device) if has_w else None
        nv.call("ttcd_qk_norm_rope_bwd", nv.ptr(dq), nv.i64(H * D), nv.ptr(dk), nv.i64(HK * D), nv.ptr(q), nv.i64(ldq),
                nv.ptr(k), nv.i64(ldk), nv.ptr(dq_in), nv.i64(ldqo), nv.ptr(dk_in), nv.i64(ldko), nv.ptr(qwb),
                nv.ptr(kwb), nv.ptr(cos), nv.ptr(sin), nv.ptr(pos), nv.ptr(dqw), nv.ptr(dkw), nv.i32(nblk),
                nv.i64(rows), nv.i32(T), nv.i32(off), nv.i32(H), nv.i32(HK), nv.i32(D), nv.i32(half), nv.f32(eps),
                nv.stream_ptr())
        gqw = dqw.sum(0).to(qdt) if has_w else None
        gkw = dkw.sum(0).to(kdt) if has_w else None
        return dq_in, dk_in, gqw, gkw, None, None, None, None, None


def qk_norm_rope(q, k, q_weight, k_weight, eps, cos, sin, offset=0, positions=None):
    _check(q, "q"), _check(k, "k")
    return _QKNormRope.apply(q, k, q_weight, k_weight, float(eps), cos, sin, offset, positions)


def rope(x, cos, sin, offset=0, positions=None):
    """Rotary on one tensor (runs the fused kernel with a zero-head partner)."""
    k_dummy = x[:, :, :0]
    out, _ = _QKNormRope.apply(x, k_dummy.reshape(x.shape[0], x.shape[1], 0, x.shape[3]), None, None, 0.0, cos, sin,
                               offset, positions)
    return out


# =============================================================================================
# SwiGLU
# =============================================================================================

class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        d = gate.shape[-1]
        g2, u2 = _rows2d(gate), _rows2d(up)
        if g2.stride(-1) != 1 or g2.stride(0) % 8:
            g2 = g2.contiguous()
        if u2.stride(-1) != 1 or u2.stride(0) % 8:
            u2 = u2.contiguous()
        rows = g2.shape[0]
        z = torch.empty(rows, d, dtype=_BF16, device=gate.device)
        nv.call("ttcd_swiglu_fwd", nv.ptr(g2), nv.ptr(u2), nv.ptr(z), nv.i64(rows), nv.i32(d), nv.i64(g2.stride(0)),
                nv.i64(u2.stride(0)), nv.i64(d), nv.stream_ptr())
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        return z.view(gate.shape)

    @staticmethod
    def backward(ctx, dz):
        g2, u2 = ctx.saved_tensors
        rows, d = g2.shape
        dz2 = _rows2d(dz).contiguous()
        # gradients are written side by side so a fused gate/up GEMM backward can consume one buffer
        packed = torch.empty(rows, 2 * d, dtype=_BF16, device=dz.device)
        dg, du = packed[:, :d], packed[:, d:]
        nv.call("ttcd_swiglu_bwd", nv.ptr(dz2), nv.ptr(g2), nv.ptr(u2), nv.ptr(dg), nv.ptr(du), nv.i64(rows), nv.i32(d),
                nv.i64(d), nv.i64(g2.stride(0)), nv.i64(u2.stride(0)), nv.i64(2 * d), nv.i64(2 * d), nv.stream_ptr())
        return dg.view(ctx.shape), du.view(ctx.shape)


def swiglu(gate, up):
    _check(gate, "gate")
    return _SwiGLU.apply(gate, up)


def swiglu_packed(gate_up):
    d = gate_up.shape[-1] // 2
    return _SwiGLU.apply(gate_up[..., :d], gate_up[..., d:])


# =============================================================================================
# depthwise conv
# =============================================================================================

class _DWConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, causal):
        b, T, C, D = x.shape
        K = w.shape[-1]
        xc = x.contiguous()
        wb = w.to(_BF16).contiguous()
        y = torch.empty_like(xc)
        nv.call("ttcd_dwconv_fwd", nv.ptr(xc), nv.ptr(wb), nv.ptr(y), nv.i64(b * T), nv.i32(C), nv.i32(D), nv.i32(K),
                nv.i32(1 if causal else 0), nv.stream_ptr())
        ctx.save_for_backward(xc, wb)
        ctx.causal = causal
        ctx.wdtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, wb = ctx.saved_tensors
        b, T, C, D = xc.shape
        K = wb.shape[-1]
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        rows_per_block = 64
        nparts = b * T * ((C + rows_per_block - 1) // rows_per_block)
        dwp = torch.empty(nparts, D, K, dtype=torch.float32, device=xc.device) if ctx.needs_input_grad[1] else None
        nv.call("ttcd_dwconv_bwd", nv.ptr(dyc), nv.ptr(xc), nv.ptr(wb), nv.ptr(dx), nv.ptr(dwp), nv.i64(b * T),
                nv.i32(C), nv.i32(D), nv.i32(K), nv.i32(1 if ctx.causal else 0), nv.stream_ptr())
        dw = dwp.sum(0).to(ctx.wdtype) if dwp is not None else None
        return dx, dw, None


def dwconv_chunked(x, w2, causal=True):
    _check(x, "x")
    K = w2.shape[-1]
    if K < 2 or K > 8 or x.shape[-1] % 8:
        return reference.dwconv_chunked(x, w2, causal)
    return _DWConv.apply(x, w2, bool(causal))


# =============================================================================================
# attention
# =============================================================================================

def _attn_layout(t: torch.Tensor):
    """[B, T, H, D] view requirements of the kernel: unit stride on D, heads D apart."""
    B, T, H, D = t.shape
    if t.stride(-1) != 1 or (H > 1 and t.stride(2) != D) or t.stride(1) % 8 or t.data_ptr() % 16 or (
            B > 1 and t.stride(0) % 8):
        t = t.contiguous()
    return t, t.stride(1), (t.stride(0) if B > 1 else T * t.stride(1))


def segment_bounds(cu_seqlens: torch.Tensor, total: int):
    """Per-token (first token of its sequence, one past its last) as int32 tensors, from the boundaries of a packed
    row; computed on the device, nothing synchronises with the host."""
    cu = cu_seqlens.to(torch.int64).reshape(-1)
    pos = torch.arange(total, device=cu.device)
    seg = torch.searchsorted(cu, pos, right=True) - 1
    seg = seg.clamp_(0, cu.numel() - 2)
    return cu[seg].to(torch.int32).contiguous(), cu[seg + 1].clamp(max=total).to(torch.int32).contiguous()


def attn_forward(q, k, v, window_t, window_s, scale, dual, seg=None):
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    if D not in (64, 128):
        raise ValueError(f"head_dim {D} not supported by the attention kernel (64 or 128)")
    if seg is not None and (B != 1 or Tq != Tk):
        raise ValueError("packed sequences need one row of queries and keys of equal length")
    q, ldq, sq = _attn_layout(q)
    k, ldk, sk = _attn_layout(k)
    v, ldv, sv = _attn_layout(v)
    o_t = torch.empty(B, Tq, H, D, dtype=_BF16, device=q.device)
    lse_t = torch.empty(B, H, Tq, dtype=torch.float32, device=q.device)
    o_s = torch.empty_like(o_t) if dual else None
    lse_s = torch.empty_like(lse_t) if dual else None
    nv.call("ttcd_attn_fwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(o_t), nv.ptr(o_s), nv.ptr(lse_t), nv.ptr(lse_s),
            nv.i32(B), nv.i32(Tq), nv.i32(Tk), nv.i32(H), nv.i32(HK), nv.i32(D), nv.i64(ldq), nv.i64(ldk), nv.i64(ldv),
            nv.i64(sq), nv.i64(sk), nv.i64(sv), nv.i32(window_t or 0), nv.i32(window_s or 0), nv.f32(scale),
            nv.ptr(None if seg is None else seg[0]), nv.stream_ptr())
    return (q, k, v), o_t, o_s, lse_t, lse_s


def attn_backward_streams(o_t, o_s, lse_t, lse_s, do_t, do_s):
    """Row statistics of the backward: ``(delta_t, do_c, delta_c)``.  Dual window goes through one softmax: inside the
    student window P_S = r P_T (r = exp(lse_T - lse_S), per row), so the student gradient stream folds into the
    teacher's, dO' = dO_T + r dO_S and delta' = delta_T + r delta_S; one kernel makes delta_T, delta' and dO'."""
    B, Tq, H, D = o_t.shape
    delta_t = torch.empty(B, H, Tq, dtype=torch.float32, device=o_t.device)
    if o_s is None:
        nv.call("ttcd_attn_delta", nv.ptr(o_t), nv.ptr(do_t), nv.ptr(delta_t), nv.i64(B), nv.i32(Tq), nv.i32(H), nv.i32(D),
                nv.stream_ptr())
        return delta_t, None, None
    delta_c = torch.empty_like(delta_t)
    do_c = torch.empty(B, Tq, H, D, dtype=_BF16, device=o_t.device)
    nv.call("ttcd_attn_bwd_combine", nv.ptr(o_t), nv.ptr(do_t), nv.ptr(o_s), nv.ptr(do_s), nv.ptr(lse_t), nv.ptr(lse_s),
            nv.ptr(delta_t), nv.ptr(delta_c), nv.ptr(do_c), nv.i64(B), nv.i32(Tq), nv.i32(H), nv.i32(D), nv.stream_ptr())
    return delta_t, do_c, delta_c


def attn_backward(q, k, v, o_t, o_s, lse_t, lse_s, do_t, do_s, window_t, window_s, scale, dv_slab=None, seg=None,
                  flags: int = 0):
    """dq, dk, dv of the (dual-window) attention; both outputs' gradients are summed in-kernel."""
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    dual = o_s is not None
    q, ldq, sq = _attn_layout(q)
    k, ldk, sk = _attn_layout(k)
    v, ldv, sv = _attn_layout(v)
    do_t = do_t.contiguous()
    do_s = do_s.contiguous() if dual else None
    delta_t, do_c, delta_c = attn_backward_streams(o_t, o_s, lse_t, lse_s, do_t, do_s)
    dq = torch.empty(B, Tq, H, D, dtype=_BF16, device=q.device)
    dk = torch.empty(B, Tk, HK, D, dtype=_BF16, device=q.device)
    ld_dv = sb_dv = 0
    if dv_slab is not None and (dv_slab[1] * 2) % 16 == 0:
        # dV goes straight into the packed q|k|v gradient of the fused projection
        slab, col = dv_slab
        n_total = slab.n_total
        buf = slab.get(B * Tk, q.device)
        dv = torch.as_strided(buf, (B, Tk, HK, D), (Tk * n_total, n_total, D, 1), col)
        ld_dv, sb_dv = n_total, Tk * n_total
    else:
        dv = torch.empty(B, Tk, HK, D, dtype=_BF16, device=q.device)
    nv.call("ttcd_attn_bwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(do_t), nv.ptr(do_c), nv.ptr(lse_t), nv.ptr(delta_t),
            nv.ptr(delta_c), nv.ptr(dq), nv.ptr(dk), nv.ptr(dv), nv.i32(B), nv.i32(Tq), nv.i32(Tk), nv.i32(H), nv.i32(HK),
            nv.i32(D), nv.i64(ldq), nv.i64(ldk), nv.i64(ldv), nv.i64(sq), nv.i64(sk), nv.i64(sv), nv.i64(ld_dv),
            nv.i64(sb_dv), nv.i32(window_t or 0), nv.i32(window_s or 0), nv.f32(scale),
            nv.ptr(None if seg is None else seg[0]), nv.ptr(None if seg is None else seg[1]), nv.i32(flags),
            nv.stream_ptr())
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window_t, window_s, scale, dual, seg_start, seg_end):
        ctx.v_slab = _slab_of(v)
        seg = None if seg_start is None else (seg_start, seg_end)
        qc, kc, vc = (_attn_layout(t)[0] for t in (q, k, v))
        # the kept outputs are o / lse only: q, k, v are rebuilt by the recomputation
        o_t, o_s, lse_t, lse_s = keep(lambda: attn_forward(qc, kc, vc, window_t, window_s, scale, dual, seg)[1:])
        ctx.save_for_backward(qc, kc, vc, o_t, o_s, lse_t, lse_s, seg_start, seg_end)
        ctx.cfg = (window_t, window_s, scale, dual)
        ctx.mark_non_differentiable(lse_t)
        if dual:
            ctx.mark_non_differentiable(lse_s)
            return o_t, o_s, lse_t, lse_s
        return o_t, lse_t

    @staticmethod
    def backward(ctx, *grads):
        qc, kc, vc, o_t, o_s, lse_t, lse_s, seg_start, seg_end = ctx.saved_tensors
        window_t, window_s, scale, dual = ctx.cfg
        do_t = grads[0]
        do_s = grads[1] if dual else None
        if do_t is None:
            do_t = torch.zeros_like(o_t)
        if dual and do_s is None:
            do_s = torch.zeros_like(o_s)
        dq, dk, dv = attn_backward(qc, kc, vc, o_t, o_s, lse_t, lse_s, do_t, do_s, window_t, window_s, scale,
                                   dv_slab=ctx.v_slab, seg=None if seg_start is None else (seg_start, seg_end))
        return dq, dk, dv, None, None, None, None, None, None


def _too_short(q, k) -> bool:
    """Fewer than one 128-row tile of queries or keys: the small-query kernel or the PyTorch statement."""
    return q.shape[1] < 128 or k.shape[1] < 128


_warned_head_dims: set[int] = set()


def _unsupported_head_dim(q) -> bool:
    """The tensor-core attention kernels are built for head_dim 64 and 128 (every recipe of the reference); other
    widths (80 and 96 appear in two of its generic transformer configs) run the PyTorch statement, said once."""
    D = q.shape[-1]
    if D in (64, 128):
        return False
    if D not in _warned_head_dims:
        _warned_head_dims.add(D)
        import warnings
        warnings.warn(f"attention with head_dim {D} runs the PyTorch statement (the native kernels cover 64 and 128)")
    return True


def _packed_args(q, k, cu_seqlens):
    """Packed (varlen) rows are handled inside the kernels: one launch, per-token sequence bounds."""
    if cu_seqlens is None:
        return None, None
    if q.shape[0] != 1 or q.shape[1] != k.shape[1]:
        raise ValueError("cu_seqlens needs a single packed row with as many keys as queries")
    return segment_bounds(cu_seqlens.to(q.device), q.shape[1])


def attention(q, k, v, window=None, scale=None, cu_seqlens=None, return_lse=False):
    _check(q, "q")
    if _unsupported_head_dim(q):
        return reference.attention(q, k, v, window, scale, cu_seqlens, return_lse)
    if _too_short(q, k):
        if cu_seqlens is None and not return_lse and not torch.is_grad_enabled() and attn_small_q_supported(q, k):
            return attn_small_q(q, k, v, window, scale)
        return reference.attention(q, k, v, window, scale, cu_seqlens, return_lse)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    seg_start, seg_end = _packed_args(q, k, cu_seqlens)
    o, lse = _Attention.apply(q, k, v, window, window, scale, False, seg_start, seg_end)
    return (o, lse) if return_lse else o


def dual_window_attention(q, k, v, window_teacher, window_student, scale=None, cu_seqlens=None):
    _check(q, "q")
    if _too_short(q, k) or _unsupported_head_dim(q):
        return reference.dual_window_attention(q, k, v, window_teacher, window_student, scale, cu_seqlens)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    seg_start, seg_end = _packed_args(q, k, cu_seqlens)
    o_t, o_s, _, _ = _Attention.apply(q, k, v, window_teacher, window_student, scale, True, seg_start, seg_end)
    return o_t, o_s


def attn_small_q_supported(q, k) -> bool:
    return (nv.has("ttcd_attn_small_q") and q.shape[-1] in (64, 128) and 1 <= q.shape[1] < 128
            and k.shape[1] >= q.shape[1] and q.shape[2] % k.shape[2] == 0)


def attn_small_q(q, k, v, window=None, scale=None, kv_len=None):
    """Attention of a few query rows (a decode step or a short continuation) over a key/value cache: bottom-right
    aligned causal mask, optional window; forward only (split over the keys, merged by a second pass).  ``kv_len``
    (int32 device tensor of one element) says how many of the key rows are filled and is read by the kernel, so a
    captured launch follows a cache that fills up between replays."""
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    q, ldq, sq = _attn_layout(q)
    k, ldk, sk = _attn_layout(k)
    v, ldv, sv = _attn_layout(v)
    splits = -(-Tk // 256)                  # 256 keys per CTA; the partial results are merged by a second pass
    out = torch.empty(B, Tq, H, D, dtype=_BF16, device=q.device)
    part_o = torch.empty(B, H, Tq, splits, D, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(B, H, Tq, splits, 2, dtype=torch.float32, device=q.device)
    nv.call("ttcd_attn_small_q", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(part_o), nv.ptr(part_ml), nv.i32(B),
            nv.i32(Tq), nv.i32(Tk), nv.i32(H), nv.i32(HK), nv.i32(D), nv.i64(ldq), nv.i64(ldk), nv.i64(ldv), nv.i64(sq),
            nv.i64(sk), nv.i64(sv), nv.i32(window or 0), nv.f32(scale), nv.i32(splits), nv.ptr(kv_len), nv.stream_ptr())
    return out


def lse_merge(o_a, lse_a, o_b, lse_b):
    B, T, H, D = o_a.shape
    out = torch.empty_like(o_a)
    nv.call("ttcd_lse_merge", nv.ptr(o_a.contiguous()), nv.ptr(lse_a.contiguous()), nv.ptr(o_b.contiguous()),
            nv.ptr(lse_b.contiguous()), nv.ptr(out), nv.ptr(None), nv.i64(B), nv.i32(T), nv.i32(H), nv.i32(D),
            nv.stream_ptr())
    return out


# =============================================================================================
# losses
# =============================================================================================

def _ce_rows(logits2, labels, inv_total, ignore_index, write_grad, smoothing=0.0, z_scale=0.0, l2_factor=0.0, lse_part=None):
    """``lse_part`` [rows, tiles, 2] (from ``_logits_with_lse``): the kernel merges it instead of a first pass over the row."""
    rows, V = logits2.shape
    loss_rows = torch.empty(rows, dtype=torch.float32, device=logits2.device)
    nv.call("ttcd_ce_rows", nv.ptr(logits2), nv.ptr(labels), nv.ptr(loss_rows), nv.ptr(None), nv.ptr(inv_total),
            nv.i64(rows), nv.i32(V), nv.i64(logits2.stride(0)), nv.i32(ignore_index), nv.i32(1 if write_grad else 0),
            nv.f32(smoothing), nv.f32(z_scale), nv.f32(l2_factor), nv.ptr(lse_part),
            nv.i32(0 if lse_part is None else lse_part.shape[1]), nv.stream_ptr())
    return loss_rows


def _logits_with_lse(hidden2, w, out):
    """out[rows, V] = hidden2 @ w^T (bf16) and, from the GEMM's epilogue, the (max, sum of exp) of every row per column
    tile: fp32 [rows, tiles, 2].  hidden2 [rows, K] and w [V, K] row-major."""
    rows, K = hidden2.shape
    V = w.shape[0]
    tiles = -(-V // (256 if V >= 256 else 128))
    parts = torch.empty(rows, tiles, 2, dtype=torch.float32, device=hidden2.device)
    nv.call("ttcd_gemm_bf16_lse", nv.ptr(hidden2), nv.ptr(w), nv.ptr(out), nv.i64(rows), nv.i64(V), nv.i64(K),
            nv.i64(hidden2.stride(0)), nv.i64(w.stride(0)), nv.i64(out.stride(0)), nv.i32(0), nv.i32(0), nv.f32(1.0),
            nv.ptr(parts), nv.stream_ptr())
    return parts


class _CrossEntropy(torch.autograd.Function):
    """Mean CE over valid rows; the gradient is computed in the forward, in place on a copy."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, smoothing=0.0, z_scale=0.0):
        lg = logits.contiguous().clone() if logits.requires_grad else logits.contiguous()
        if lg.stride(0) % 8:
            raise ValueError("vocab size must be a multiple of 8 for the CE kernel")
        labels = labels.contiguous().to(torch.int64)
        total = labels.ne(ignore_index).sum().clamp_min(1).to(torch.float32)
        inv_total = (1.0 / total).reshape(1)
        loss_rows = _ce_rows(lg, labels, inv_total, ignore_index, logits.requires_grad, smoothing, z_scale)
        if logits.requires_grad:
            ctx.save_for_backward(lg)
        return (loss_rows.sum() * inv_total).reshape(())

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None, None, None, None


def cross_entropy(logits, labels, ignore_index=-100, label_smoothing=0.0, z_loss=0.0):
    return _CrossEntropy.apply(logits, labels, int(ignore_index), float(label_smoothing), float(z_loss))


def _lce_chunk_rows(n_rows: int, hidden: int, num_chunks: int, sms: int = 148) -> int:
    """Rows per chunk of the chunked lm_head pass: about ``n_rows / num_chunks``, moved (by up to a quarter either way)
    to the multiple of 128 whose dx GEMM ([rows, vocab] x [vocab, hidden]: rows/128 x hidden/256 output tiles, the only
    one of the three GEMMs with few tiles) fills whole waves of the persistent kernel's CTAs; 8192 rows x 1024 would be
    256 tiles = 1.73 waves, 9472 rows are 296 tiles = 2 waves."""
    target = max(1, -(-n_rows // max(1, num_chunks)) // 128)
    total = -(-n_rows // 128)
    if target >= total:
        return total * 128
    n_tiles = max(1, -(-hidden // 256))
    best, best_key = target, None
    for m in range(max(1, target - target // 4), min(total, target + target // 4) + 1):
        tiles = m * n_tiles
        eff = tiles / (-(-tiles // sms) * sms)
        key = (round(eff, 2), -abs(m - target))
        if best_key is None or key > best_key:
            best, best_key = m, key
    return best * 128


class _LinearCrossEntropy(torch.autograd.Function):
    """CE(hidden @ W^T) in token chunks: logits GEMM -> row kernel (LSE + in-place dlogits) ->
    dx and dW GEMMs, so the [tokens, vocab] logits never exist at once and there is no host sync."""

    @staticmethod
    def forward(ctx, hidden, labels, weight, ignore_index, num_chunks, l2_factor=0.0):
        N, Hd = hidden.shape
        V = weight.shape[0]
        hidden = hidden.contiguous()
        w = weight if weight.dtype == _BF16 else weight.to(_BF16)
        labels = labels.contiguous().to(torch.int64)
        total = labels.ne(ignore_index).sum().clamp_min(1).to(torch.float32)
        inv_total = (1.0 / total).reshape(1)
        need_grad = hidden.requires_grad or weight.requires_grad
        chunk = _lce_chunk_rows(N, Hd, num_chunks)
        dx = torch.empty_like(hidden) if need_grad else None
        dw = torch.zeros(V, Hd, dtype=torch.float32, device=hidden.device) if need_grad else None
        loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
        logits = torch.empty(min(chunk + 127, N), V, dtype=_BF16, device=hidden.device)
        # the row statistics come out of the logits GEMM's epilogue (the l2-warp term needs the arg-max: row pass)
        fuse_lse = (l2_factor == 0.0 and nv.has("ttcd_gemm_bf16_lse") and w.is_contiguous() and Hd % 8 == 0
                    and hidden.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
        bounds, s = [], 0
        while s < N:                       # a tail shorter than one 128-row tile joins the chunk before it
            e = N if N - (s + chunk) < 128 else s + chunk
            bounds.append((s, e))
            s = e
        for s, e in bounds:
            lg = logits[: e - s]
            parts = None
            if fuse_lse:
                parts = _logits_with_lse(hidden[s:e], w, lg)
            else:
                gemm(hidden[s:e], w.transpose(0, 1), out=lg.view(1, e - s, V))
            loss_rows = _ce_rows(lg, labels[s:e], inv_total, ignore_index, need_grad, 0.0, 0.0, l2_factor, parts)
            loss = loss + loss_rows.sum()
            if need_grad:
                gemm(lg, w, out=dx[s:e].view(1, e - s, Hd))
                gemm(lg.transpose(0, 1), hidden[s:e], out=dw.view(1, V, Hd), out_dtype=torch.float32, beta=1.0,
                     c_in=dw.view(1, V, Hd))
        if need_grad:
            ctx.save_for_backward(dx, dw.to(weight.dtype))
        return (loss * inv_total).reshape(())

    @staticmethod
    def backward(ctx, g):
        dx, dw = ctx.saved_tensors
        return dx * g.to(dx.dtype), None, dw * g.to(dw.dtype), None, None, None


def linear_cross_entropy(hidden, labels, weight, ignore_index=-100, num_chunks=8, l2_penalty=0.0):
    _check(hidden, "hidden")
    if hidden.shape[0] < 128 or hidden.shape[1] < 64 or weight.shape[0] < 128:       # below one GEMM tile
        return reference.linear_cross_entropy(hidden, labels, weight, None, ignore_index, l2_penalty)
    return _LinearCrossEntropy.apply(hidden, labels, weight, int(ignore_index), int(num_chunks), float(l2_penalty))


# =============================================================================================
# Newton-Schulz (Muon) on the tensor-core GEMM
# =============================================================================================

def newton_schulz(g: torch.Tensor, coeffs=reference.NS_COEFFS) -> torch.Tensor:
    """X <- aX + (bA + cA^2)X with A = XX^T, five fixed coefficient triples, bf16 on tcgen05."""
    squeeze = g.dim() == 2
    x = (g.unsqueeze(0) if squeeze else g).to(_BF16)
    transposed = x.size(1) > x.size(2)
    if transposed:
        x = x.transpose(1, 2).contiguous()
    x = (x / (x.float().norm(dim=(1, 2), keepdim=True) + 1e-7).to(_BF16)).contiguous()
    for a, b, c in coeffs:
        A = gemm(x, x.transpose(1, 2))                                   # X X^T
        Bm = gemm(A, A.transpose(1, 2), alpha=c, beta=b, c_in=A)         # c A^2 + b A   (A symmetric)
        x = gemm(Bm, x, alpha=1.0, beta=a, c_in=x)                        # B X + a X
    if transposed:
        x = x.transpose(1, 2)
    return x.squeeze(0) if squeeze else x


# =============================================================================================
# optimiser helpers
# =============================================================================================

def adamw_step(p32, grad, m, v, p_bf16, *, lr, beta1, beta2, eps, weight_decay, step, coef=None, skip=None):
    """Fused AdamW on a flat fp32 shard; optionally refreshes the bf16 compute copy."""
    n = p32.numel()
    bc1 = 1.0 - beta1 ** step
    bc2_sqrt = math.sqrt(1.0 - beta2 ** step)
    nv.call("ttcd_adamw", nv.ptr(p32), nv.ptr(grad), nv.i32(1 if grad.dtype == _BF16 else 0), nv.ptr(m), nv.ptr(v),
            nv.ptr(p_bf16), nv.i64(n), nv.f32(lr), nv.f32(beta1), nv.f32(beta2), nv.f32(eps), nv.f32(weight_decay),
            nv.f32(bc1), nv.f32(bc2_sqrt), nv.ptr(coef), nv.ptr(skip), nv.stream_ptr())


def sumsq(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x^2); ``out`` is a 1-element fp32 CUDA tensor."""
    nv.call("ttcd_sumsq", nv.ptr(x), nv.i32(1 if x.dtype == _BF16 else 0), nv.i64(x.numel()), nv.ptr(out),
            nv.stream_ptr())


def cast_scale(x: torch.Tensor, y: torch.Tensor, scale: float = 1.0, accumulate: bool = False) -> None:
    kinds = {(_BF16, torch.float32): 0, (torch.float32, _BF16): 1, (torch.float32, torch.float32): 2, (_BF16, _BF16): 3}
    nv.call("ttcd_cast_scale", nv.ptr(x), nv.ptr(y), nv.i64(x.numel()), nv.f32(scale), nv.i32(kinds[(x.dtype, y.dtype)]),
            nv.i32(1 if accumulate else 0), nv.stream_ptr())


# ---------------------------------------------------------------------------------------------
# fast-weight chunk scan
# ---------------------------------------------------------------------------------------------
class _TTTScan(torch.autograd.Function):
    """Grouped fast-weight scan of the TTT layers as batched tensor-core GEMMs with fused epilogues:

        P   = beta * ((z_tgt - z_hat) @ Wu)            one GEMM, beta in the epilogue (row scale)
        dW  = P^T @ z_hat                              one batched GEMM (fp32 out), chunks 0..T-2
        W_i = W_down + lr * sum_{j<i} dW_j             one streaming kernel (prefix + add + cast)
        Y_i = z_out_i @ W_i^T                          one batched GEMM

    with a hand-written backward (five batched GEMMs + the reverse-prefix kernel).  Same math as
    ``reference.ttt_scan`` for the plain configuration (no feature normalisation, fp32 state).

    Context parallel (``cp``: the T chunks are this rank's slice of a longer sequence): every chunk but the
    globally last one updates, the scan starts from ``W_down + sum over earlier ranks of their lr * sum_j dW_j``
    and hands the gradient of that start state back to the earlier ranks.  The two exclusive sums over ranks
    run over peer memory (``cp.exclusive_sum``); everything else is the same kernels.
    """

    @staticmethod
    def forward(ctx, z_out, z_tgt, z_hat, beta, w_down, w_update_t, lr, cp, key):
        b, T, C, d_i = z_out.shape
        d_h = w_down.shape[0]
        z_out, z_tgt, z_hat = z_out.contiguous(), z_tgt.contiguous(), z_hat.contiguous()
        w_down_c = w_down.to(_BF16).contiguous()
        wu = w_update_t.to(_BF16)
        wu = wu if wu.stride(-1) == 1 or wu.stride(-2) == 1 else wu.contiguous()
        sharded = cp is not None and cp.size > 1
        nu = T if (sharded and cp.rank < cp.size - 1) else T - 1       # globally, only the very last chunk never updates
        R = d_h * d_i

        def compute():
            states = torch.empty(b, T, d_h, d_i, dtype=_BF16, device=z_out.device)
            P = None
            last_norm = torch.zeros((), dtype=torch.float32, device=z_out.device)
            if nu > 0:
                diff = z_tgt[:, :nu] - z_hat[:, :nu]
                scale = None if beta is None else beta[:, :nu].reshape(-1).to(_BF16).contiguous()
                P = gemm(diff.reshape(b * nu * C, d_i), wu, row_scale=scale).view(b * nu, C, d_h)
                del diff
                zh_u = z_hat[:, :nu].reshape(b * nu, C, d_i)
                d_w = gemm(P.transpose(-1, -2), zh_u, out_dtype=torch.float32)            # [b*nu, d_h, d_i]
                last_norm = d_w.view(b, nu, -1)[:, -1].norm()
            else:
                d_w = torch.empty(0, dtype=torch.float32, device=z_out.device)
            w_init = None
            if sharded:
                local = (d_w.view(b, nu, R).sum(1) * float(lr)) if nu > 0 else torch.zeros(b, R, device=z_out.device)
                w_init = cp.exclusive_sum(local, key, before=True)       # sum over the ranks before this one
            nv.call("ttcd_ttt_prefix_weights", nv.ptr(d_w if nu > 0 else None), nv.ptr(w_down_c), nv.ptr(w_init),
                    nv.ptr(states), nv.f32(float(lr)), nv.i32(b), nv.i32(T), nv.i64(R), nv.i32(nu), nv.stream_ptr())
            del d_w
            y = gemm(z_out.view(b * T, C, d_i), states.view(b * T, d_h, d_i).transpose(-1, -2)).view(b, T, C, d_h)
            return y, states, P, last_norm

        y, states, P, last_norm = keep(compute)
        ctx.save_for_backward(z_out, z_tgt, z_hat, beta, wu, states, P)
        ctx.lr, ctx.w_dtype, ctx.wu_dtype = float(lr), w_down.dtype, w_update_t.dtype
        ctx.cp, ctx.key, ctx.nu = (cp if sharded else None), key, nu
        ctx.mark_non_differentiable(last_norm)
        return y, last_norm

    @staticmethod
    def backward(ctx, dy, _dnorm):
        z_out, z_tgt, z_hat, beta, wu, states, P = ctx.saved_tensors
        b, T, C, d_i = z_out.shape
        d_h = states.shape[2]
        nu, R, lr, cp = ctx.nu, d_h * d_i, ctx.lr, ctx.cp
        dy3 = dy.to(_BF16).contiguous().view(b * T, C, d_h)
        dz_out = gemm(dy3, states.view(b * T, d_h, d_i)).view(b, T, C, d_i)
        d_states = gemm(dy3.transpose(-1, -2), z_out.view(b * T, C, d_i), out_dtype=torch.float32)       # [b*T, d_h, d_i]
        g_init = None
        if cp is not None:
            # gradient of this rank's start state = sum_i d_states_i; every earlier rank's summed update fed it
            d_start = d_states.view(b, T, R).sum(1)
            g_init = cp.exclusive_sum(d_start, ctx.key, before=False)     # sum over the ranks after this one
        g = torch.empty(b, max(nu, 1), d_h, d_i, dtype=_BF16, device=dy.device)
        d_w_down = torch.empty(d_h, d_i, dtype=torch.float32, device=dy.device)
        nv.call("ttcd_ttt_suffix_grads", nv.ptr(d_states), nv.ptr(g), nv.ptr(d_w_down), nv.ptr(g_init), nv.f32(lr),
                nv.i32(b), nv.i32(T), nv.i64(R), nv.i32(nu), nv.stream_ptr())
        del d_states
        fresh = b == 1 and nu > 0              # every row but the never-updating tail is written below
        dz_tgt = torch.empty_like(z_tgt) if fresh else torch.zeros_like(z_tgt)
        dz_hat = torch.empty_like(z_hat) if fresh else torch.zeros_like(z_hat)
        d_beta = d_wu = None
        if nu > 0:
            g3 = g.view(b * nu, d_h, d_i)
            zh_u = z_hat[:, :nu].reshape(b * nu, C, d_i)
            dP = gemm(zh_u, g3.transpose(-1, -2))                                         # [b*nu, C, d_h]
            if beta is not None:
                bu = beta[:, :nu].reshape(b * nu, C, 1)
                d_beta_u = ((dP.float() * P.float()).sum(-1, keepdim=True) / bu.float().clamp_min(1e-20)).to(beta.dtype)
                d_beta = torch.cat([d_beta_u.view(b, nu, C, 1), torch.zeros_like(beta[:, :T - nu])], dim=1)
                dP = dP * bu.to(_BF16)
            diff = (z_tgt[:, :nu] - z_hat[:, :nu]).reshape(b * nu * C, d_i)
            d_wu = gemm(diff.transpose(-1, -2), dP.view(b * nu * C, d_h)).view(d_i, d_h).to(ctx.wu_dtype)
            del diff
            if b == 1:
                dd = dz_tgt[0, :nu].view(nu, C, d_i)
                gemm(dP.view(nu * C, d_h), wu.transpose(-1, -2), out=dd.view(1, nu * C, d_i))
                gemm(P, g3, alpha=1.0, beta=-1.0, c_in=dd, out=dz_hat[0, :nu].view(nu, C, d_i))
                if nu < T:
                    dz_tgt[0, nu:].zero_()
                    dz_hat[0, nu:].zero_()
            else:
                dd = gemm(dP.view(b * nu * C, d_h), wu.transpose(-1, -2)).view(b * nu, C, d_i)
                dzh = gemm(P, g3, alpha=1.0, beta=-1.0, c_in=dd)
                dz_tgt[:, :nu] = dd.view(b, nu, C, d_i)
                dz_hat[:, :nu] = dzh.view(b, nu, C, d_i)
        return dz_out, dz_tgt, dz_hat, d_beta, d_w_down.to(ctx.w_dtype), d_wu, None, None, None


def ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, lr: float, cp=None, key=None):
    """Returns ``(y [b,T,C,d_h], norm of the last chunk update)``; see ``_TTTScan``."""
    for name, t in (("z_out", z_out), ("z_tgt", z_tgt), ("z_hat", z_hat)):
        _check(t, name)
    return _TTTScan.apply(z_out, z_tgt, z_hat, beta, w_down, w_update_t, float(lr), cp, key)
