"""The chunked (gated) delta rule as ONE differentiable op with a hand-written backward.

Three stages per call, chunks of 64 tokens, everything between them in chunk layout [B*H, n, 64, *] (fp32, except the
chain kernels' tile operands ``w`` and ``kt``, which the GPU path stores as bf16):

1. chunk-local (csrc/delta_prep.cu, one CTA per chunk): row normalisation, decay sums, the unit-lower-triangular
   inverse and the WY factors ``w, u``, the end-scaled keys ``kt``, the decayed queries ``q_in``, the intra-chunk
   scores ``qk`` and the chunk decay ``gamma``;
2. the chain over chunks (csrc/delta_chain.cu): ``vn_i = u_i - w_i S_i``, ``S_{i+1} = gamma_i S_i + kt_i^T vn_i``;
3. the outputs ``o_i = q_in_i S_i + qk_i vn_i`` (two batched products).

Backward runs the three stages in reverse: four batched products for the output stage, the reverse chain, three
more for the chain's operands, and one kernel for the chunk-local part.  The intermediates are kept for backward
within a share of the device memory and rebuilt from q, k, v, g, beta beyond it (stages 1 and 2 again).  On the GPU
every operand of a kernel product is a bf16 or TF32 value and every sum is fp32.

This is the computation of fla/ops/gated_delta_rule/chunk.py (``chunk_gated_delta_rule``) and, with ``g`` None, of
fla/ops/delta_rule/chunk.py (``chunk_delta_rule``).  Off the GPU the same op runs its PyTorch statement of every
stage (``_prep_fwd_torch`` / ``_prep_bwd_torch`` are also the oracle of the kernels' tests).
"""
from __future__ import annotations

import os
import weakref

import torch
import torch.nn.functional as F

from .. import _native as nv
from . import delta_chain as dc
from .reference import _tf32_matmuls

C = 64


def _f(t: torch.Tensor) -> torch.Tensor:
    """fp32 working precision (float64 inputs stay as they are: the PyTorch statement doubles as an exact oracle)."""
    return t if t.dtype == torch.float64 else t.float()


# ------------------------------------------------------------------------------------------------ layouts
def _to_chunks(x: torch.Tensor, n: int) -> torch.Tensor:
    """[B, T, H, W] -> [B*H, n, 64, W] fp32, zero rows beyond T."""
    B, T, H, W = x.shape
    xf = _f(x)
    if n * C != T:
        xf = F.pad(xf, (0, 0, 0, 0, 0, n * C - T))
    return xf.view(B, n, C, H, W).permute(0, 3, 1, 2, 4).reshape(B * H, n, C, W)


def _from_chunks(x: torch.Tensor, B: int, T: int) -> torch.Tensor:
    """[B*H, n, 64, W] -> [B, T, H, W] (a view)."""
    BH, n, _, W = x.shape
    return x.view(B, BH // B, n * C, W)[:, :, :T].transpose(1, 2)


# ------------------------------------------------------------------------------------------------ stage 1 in PyTorch
def _local_terms(q, k, v, beta, g, scale, l2norm):
    B, T, H, D = q.shape
    n = -(-T // C)
    qf, kf = _f(q), _f(k)
    if l2norm:
        qf, kf = F.normalize(qf, dim=-1, eps=1e-6), F.normalize(kf, dim=-1, eps=1e-6)
    qc, kc, vc = _to_chunks(qf * scale, n), _to_chunks(kf, n), _to_chunks(v, n)
    bc = _to_chunks(beta.unsqueeze(-1), n)
    G = (_to_chunks(g.unsqueeze(-1), n) if g is not None else torch.zeros_like(bc)).cumsum(2)
    idx = torch.arange(C, device=q.device)
    low, strict = idx[:, None] >= idx[None, :], idx[:, None] > idx[None, :]
    decay = torch.where(low, (G - G.transpose(-1, -2)).clamp(max=0.0).exp(), G.new_zeros(()))
    eg, to_end = G.exp(), (G[:, :, -1:] - G).exp()
    A, QK = kc @ kc.transpose(-1, -2), qc @ kc.transpose(-1, -2)
    L = torch.where(strict, bc * decay * A, G.new_zeros(()))
    eye = torch.eye(C, device=q.device, dtype=G.dtype)
    Tm = torch.linalg.solve_triangular(eye + L, eye.expand_as(L), upper=False)
    return dict(qc=qc, kc=kc, vc=vc, bc=bc, G=G, decay=decay, eg=eg, to_end=to_end, A=A, QK=QK, L=L, T=Tm, strict=strict)


def _prep_fwd_torch(q, k, v, beta, g, scale, l2norm):
    t = _local_terms(q, k, v, beta, g, scale, l2norm)
    w = t["T"] @ (t["kc"] * t["bc"] * t["eg"])
    u = t["T"] @ (t["vc"] * t["bc"])
    return w, u, t["kc"] * t["to_end"], t["qc"] * t["eg"], t["QK"] * t["decay"], t["eg"][:, :, -1, 0].contiguous()


def _prep_bwd_torch(q, k, v, beta, g, scale, l2norm, d_w, d_u, d_kt, d_qin, d_qk, d_gamma):
    B, T, H, D = q.shape
    t = _local_terms(q, k, v, beta, g, scale, l2norm)
    qc, kc, vc, bc, eg, to_end, decay, A, QK, L, Tm = (t[x] for x in ("qc", "kc", "vc", "bc", "eg", "to_end", "decay", "A", "QK", "L", "T"))
    Tt = Tm.transpose(-1, -2)
    kbg, vb = kc * bc * eg, vc * bc
    d_kbg, d_vb = Tt @ d_w, Tt @ d_u
    d_T = d_w @ kbg.transpose(-1, -2) + d_u @ vb.transpose(-1, -2)
    d_L = -(Tt @ d_T @ Tt) * t["strict"]
    M1, M2 = d_L * bc * decay, d_qk * decay
    E = d_L * L + M2 * QK
    dG = E.sum(-1) - E.sum(-2)
    rk1 = (d_kbg * kc).sum(-1)
    dbeta = (d_L * decay * A).sum(-1) + rk1 * eg[..., 0] + (d_vb * vc).sum(-1)
    dk = (M1 + M1.transpose(-1, -2)) @ kc + M2.transpose(-1, -2) @ qc + d_kbg * bc * eg + d_kt * to_end
    dq = M2 @ kc + d_qin * eg
    dv = d_vb * bc
    r_kt = (d_kt * kc).sum(-1) * to_end[..., 0]
    dG = dG + rk1 * (bc * eg)[..., 0] + (d_qin * qc).sum(-1) * eg[..., 0] - r_kt
    dG[:, :, -1] += r_kt.sum(-1) + d_gamma * eg[:, :, -1, 0]
    dg = dG.flip(-1).cumsum(-1).flip(-1)
    dq, dk, dv = (_from_chunks(x, B, T) for x in (dq, dk, dv))
    dbeta, dg = (_from_chunks(x.unsqueeze(-1), B, T).squeeze(-1) for x in (dbeta, dg))
    qf, kf = _f(q), _f(k)
    if l2norm:          # backward of x -> x / |x| (and of q's scale)
        qn_len, kn_len = qf.norm(dim=-1, keepdim=True).clamp_min(1e-6), kf.norm(dim=-1, keepdim=True).clamp_min(1e-6)
        qn, kn = qf / qn_len, kf / kn_len
        dq = scale * (dq - qn * (qn * dq).sum(-1, keepdim=True)) / qn_len
        dk = (dk - kn * (kn * dk).sum(-1, keepdim=True)) / kn_len
    else:
        dq = dq * scale
    return dq, dk, dv, dbeta, (dg if g is not None else None)


# ------------------------------------------------------------------------------------------------ stage 1 on the GPU
def native_ok(q: torch.Tensor, v: torch.Tensor) -> bool:
    D, Dv = q.shape[-1], v.shape[-1]
    return (q.is_cuda and nv.available() and nv.has("ttcd_delta_prep_fwd") and nv.has("ttcd_delta_chain_fwd")
            and q.dtype in (torch.bfloat16, torch.float32) and D % C == 0 and Dv % C == 0 and D in (64, 128, 256)
            and q.shape[0] * q.shape[2] <= 65535)


def _aligned(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _prep_fwd(q, k, v, beta, g, scale, l2norm):
    if not native_ok(q, v):
        return _prep_fwd_torch(q, k, v, beta, g, scale, l2norm)
    B, T, H, D = q.shape
    Dv, n, dev = v.shape[-1], -(-T // C), q.device
    new = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)  # noqa: E731
    w, kt = (torch.empty(B * H, n, C, D, dtype=torch.bfloat16, device=dev) for _ in range(2))     # the chain's tile operands
    q_in, u = new(B * H, n, C, D), new(B * H, n, C, Dv)
    qk, gamma = new(B * H, n, C, C), new(B * H, n)
    nv.call("ttcd_delta_prep_fwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(beta), nv.ptr(g), nv.ptr(w), nv.ptr(u), nv.ptr(kt),
            nv.ptr(q_in), nv.ptr(qk), nv.ptr(gamma), nv.i32(B), nv.i32(T), nv.i32(H), nv.i32(D), nv.i32(Dv), nv.f32(scale),
            nv.i32(int(l2norm)), nv.i32(int(q.dtype == torch.bfloat16)), nv.stream_ptr())
    return w, u, kt, q_in, qk, gamma


def _prep_bwd(q, k, v, beta, g, scale, l2norm, d_w, d_u, d_kt, d_qin, d_qk, d_gamma):
    if not native_ok(q, v):
        return _prep_bwd_torch(q, k, v, beta, g, scale, l2norm, d_w, d_u, d_kt, d_qin, d_qk, d_gamma)
    B, T, H, D = q.shape
    Dv, dev = v.shape[-1], q.device
    new = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)  # noqa: E731
    dq, dk, dv, dbeta = new(B, T, H, D), new(B, T, H, D), new(B, T, H, Dv), new(B, T, H)
    dg = new(B, T, H) if g is not None else None
    d_w, d_u, d_kt, d_qin, d_qk, d_gamma = (t.contiguous() for t in (d_w, d_u, d_kt, d_qin, d_qk, d_gamma))
    nv.call("ttcd_delta_prep_bwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(beta), nv.ptr(g), nv.ptr(d_w), nv.ptr(d_u),
            nv.ptr(d_kt), nv.ptr(d_qin), nv.ptr(d_qk), nv.ptr(d_gamma), nv.ptr(dq), nv.ptr(dk), nv.ptr(dv), nv.ptr(dbeta),
            nv.ptr(dg), nv.i32(B), nv.i32(T), nv.i32(H), nv.i32(D), nv.i32(Dv), nv.f32(scale), nv.i32(int(l2norm)),
            nv.i32(int(q.dtype == torch.bfloat16)), nv.stream_ptr())
    return dq, dk, dv, dbeta, dg


def _rows_to_tokens(x: torch.Tensor, B: int, T: int, dtype: torch.dtype) -> torch.Tensor:
    """Chunk layout [B*H, n, 64, W] -> token layout [B, T, H, W] in ``dtype``: one pass (layout change and cast)."""
    BH, n, _, W = x.shape
    out = torch.empty(B, T, BH // B, W, dtype=dtype, device=x.device)
    if x.is_cuda and nv.available() and nv.has("ttcd_delta_rows") and x.dtype == torch.float32 \
            and dtype in (torch.bfloat16, torch.float32) and W % 4 == 0:
        nv.call("ttcd_delta_rows", nv.ptr(x.contiguous()), nv.ptr(out), nv.i32(B), nv.i32(T), nv.i32(BH // B), nv.i32(W),
                nv.i32(1), nv.i32(int(dtype == torch.bfloat16)), nv.stream_ptr())
    else:
        out.copy_(_from_chunks(x, B, T))
    return out


def _rows_to_chunks(x: torch.Tensor, n: int, dtype: torch.dtype) -> torch.Tensor:
    """Token layout [B, T, H, W] -> chunk layout [B*H, n, 64, W] in ``dtype`` (fp32 on the GPU), rows beyond T zero."""
    B, T, H, W = x.shape
    if x.is_cuda and nv.available() and nv.has("ttcd_delta_rows") and dtype == torch.float32 \
            and x.dtype in (torch.bfloat16, torch.float32) and W % 4 == 0:
        x = _aligned(x)
        out = torch.empty(B * H, n, C, W, dtype=dtype, device=x.device)
        nv.call("ttcd_delta_rows", nv.ptr(x), nv.ptr(out), nv.i32(B), nv.i32(T), nv.i32(H), nv.i32(W), nv.i32(0),
                nv.i32(int(x.dtype == torch.bfloat16)), nv.stream_ptr())
        return out
    out = x.new_zeros(B, H, n * C, W, dtype=dtype)
    out[:, :, :T].copy_(x.transpose(1, 2))
    return out.view(B * H, n, C, W)


# ------------------------------------------------------------------------------------------------ the op
_KEEP_FRACTION = float(os.environ.get("TTCD_DELTA_KEEP_FRACTION", "0.2"))
_kept_bytes = 0          # bytes of kept intermediates whose backward has not run yet


def _release(nbytes: int) -> None:
    global _kept_bytes
    _kept_bytes -= nbytes


def _keep_intermediates(ctx, q: torch.Tensor, nbytes: int) -> bool:
    """Keep the fp32 intermediates of a call for backward?  ``TTCD_DELTA_KEEP`` = 1 / 0 forces the answer.  Otherwise
    they are kept while all kept sets that still wait for their backward stay within a fifth of the device memory
    (``TTCD_DELTA_KEEP_FRACTION``), so that a deep model keeps them on as many layers as that allows and rebuilds them
    on the rest), and nothing is kept once the process has come within a fifth of the device memory at its peak: a model
    whose other activations fill the device rebuilds everywhere from its second step on."""
    global _kept_bytes
    if not any(ctx.needs_input_grad):
        return False
    mode = os.environ.get("TTCD_DELTA_KEEP", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    if not q.is_cuda:
        return True
    total = torch.cuda.get_device_properties(q.device).total_memory
    if _kept_bytes + nbytes > _KEEP_FRACTION * total:
        return False
    if torch.cuda.max_memory_allocated(q.device) + nbytes > 0.8 * total:      # an earlier step already came close to the limit
        return False
    if torch.cuda.memory_allocated(q.device) + nbytes > 0.5 * total:          # this step's forward is already that large
        return False
    _kept_bytes += nbytes
    weakref.finalize(ctx, _release, nbytes)          # backward done or graph dropped: the set is gone either way
    return True


def _stages_1_2(q, k, v, g, beta, s0, scale, l2norm):
    w, u, kt, q_in, qk, gamma = _prep_fwd(q, k, v, beta, g, scale, l2norm)
    vn, states, final = dc._fwd(w, u, kt, gamma, s0)
    return w, kt, q_in, qk, gamma, vn, states, final


def _flat(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-2], t.shape[-1])


class _FusedDeltaRule(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, s0, scale, l2norm):
        B, T, H, D = q.shape
        Dv = v.shape[-1]
        q, k, v = _aligned(q), _aligned(k), _aligned(v)
        beta32 = _aligned(_f(beta))
        g32 = _aligned(_f(g)) if g is not None else None
        s0_32 = (_f(s0) if s0 is not None else q.new_zeros(B, H, D, Dv, dtype=beta32.dtype)).reshape(B * H, D, Dv).contiguous()
        w, kt, q_in, qk, gamma, vn, states, final = _stages_1_2(q, k, v, g32, beta32, s0_32, scale, l2norm)
        with _tf32_matmuls(q.is_cuda):
            o = torch.baddbmm(torch.bmm(_flat(q_in), _flat(states)), _flat(qk), _flat(vn)).view(B * H, -1, C, Dv)
        kept = (w, kt, q_in, qk, gamma, vn, states)
        if not _keep_intermediates(ctx, q, sum(t.numel() * t.element_size() for t in kept)):
            kept = ()
        ctx.save_for_backward(q, k, v, g32, beta32, s0_32, *kept)
        ctx.scale, ctx.l2norm, ctx.has_kept = scale, l2norm, bool(kept)
        ctx.dtypes = (beta.dtype, None if g is None else g.dtype, None if s0 is None else s0.dtype)
        return _rows_to_tokens(o, B, T, q.dtype), final.view(B, H, D, Dv)

    @staticmethod
    def backward(ctx, d_o, d_final):
        q, k, v, g32, beta32, s0_32, *kept = ctx.saved_tensors
        B, T, H, D = q.shape
        Dv = v.shape[-1]
        if ctx.has_kept:
            w, kt, q_in, qk, gamma, vn, states = kept
        else:
            w, kt, q_in, qk, gamma, vn, states, _ = _stages_1_2(q, k, v, g32, beta32, s0_32, ctx.scale, ctx.l2norm)
        n = w.shape[1]
        do_c = _flat(torch.zeros_like(vn)) if d_o is None else _flat(_rows_to_chunks(d_o, n, vn.dtype))
        d_final = torch.zeros_like(s0_32) if d_final is None else _f(d_final).reshape(B * H, D, Dv)
        with _tf32_matmuls(q.is_cuda):
            # output stage: o = q_in S + qk vn
            d_qin = torch.bmm(do_c, _flat(states).transpose(1, 2)).view_as(q_in)
            d_qk = torch.bmm(do_c, _flat(vn).transpose(1, 2)).view_as(qk)
            d_vn = torch.bmm(_flat(qk).transpose(1, 2), do_c).view_as(vn)
            d_states = torch.bmm(_flat(q_in).transpose(1, 2), do_c).view_as(states)
            del do_c
            # the chain, in reverse
            d_u, ds_next, d_s0, d_gamma = dc._bwd(w, kt, gamma, d_vn, d_states, d_final, states)
            del d_vn, d_states
            d_w = torch.baddbmm(d_u.new_zeros(1, 1, 1), _flat(d_u), _flat(states).transpose(1, 2), beta=0, alpha=-1).view(w.shape)
            d_kt = torch.bmm(_flat(vn), _flat(ds_next).transpose(1, 2)).view(kt.shape)
        del ds_next
        dq, dk, dv, dbeta, dg = _prep_bwd(q, k, v, beta32, g32, ctx.scale, ctx.l2norm, d_w, d_u, d_kt, d_qin, d_qk, d_gamma)
        beta_dtype, g_dtype, s0_dtype = ctx.dtypes
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None if dg is None else dg.to(g_dtype), dbeta.to(beta_dtype),
                None if s0_dtype is None else d_s0.view(B, H, D, Dv).to(s0_dtype), None, None)


def gated_delta_rule_fused(q, k, v, g, beta, scale=None, l2norm: bool = True, initial_state=None,
                           output_final_state: bool = False):
    """q, k [B,T,H,D], v [B,T,H,Dv] (one dtype), g (or None) and beta [B,T,H]; returns (o [B,T,H,Dv] in q's dtype, the
    final state [B,H,D,Dv] fp32 or None).  Differentiable in q, k, v, g, beta and the initial state."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        k, v = k.to(q.dtype), v.to(q.dtype)
    if q.dtype not in (torch.bfloat16, torch.float32, torch.float64):
        q, k, v = q.float(), k.float(), v.float()
    o, final = _FusedDeltaRule.apply(q, k, v, g, beta, initial_state, scale, bool(l2norm))
    return o, (final if output_final_state else None)
