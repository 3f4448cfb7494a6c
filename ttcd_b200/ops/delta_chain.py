"""The sequential part of the chunked (gated) delta rule as one op: the state recurrence over chunks.

For every (batch, head) pair and chunk i, with S_i [D, Dv] the state entering the chunk:

    vn_i    = u_i - w_i S_i                      [C, Dv]   the chunk's corrected values
    S_{i+1} = gamma_i S_i + kt_i^T vn_i          [D, Dv]

(w, u: the chunk's WY factors; kt: keys scaled to the chunk end; gamma: the chunk's total decay).  This is the role
of the reference's ``chunk_gated_delta_rule_fwd_h`` / ``chunk_gated_delta_rule_bwd_dhu`` Triton kernels
(fla/ops/common/chunk_delta_h.py).  Everything else in the rule is batched over chunks; this chain is the only part
with a dependence from chunk to chunk, and the columns of S (the Dv axis) never mix, so a CTA can own a slice of
columns for the whole sequence: one launch per direction instead of a few small launches per chunk.

``delta_chain`` is differentiable (hand-written backward: a reverse chain of the same shape plus batched products)
and runs the CUDA kernels (csrc/delta_chain.cu) on the GPU, plain PyTorch loops elsewhere.
"""
from __future__ import annotations

import torch

from .. import _native as nv


def _fwd_torch(w, u, kt, gamma, s0):
    w, kt = w.to(u.dtype), kt.to(u.dtype)
    BH, n, C, D = w.shape
    S = s0.clone()
    vn = torch.empty_like(u)
    states = u.new_empty(BH, n, D, u.shape[-1])
    for i in range(n):
        states[:, i] = S
        vn[:, i] = u[:, i] - w[:, i] @ S
        S = gamma[:, i, None, None] * S + kt[:, i].transpose(-1, -2) @ vn[:, i]
    return vn, states, S


def _bwd_torch(w, kt, gamma, d_vn, d_states, d_final, states=None):
    w, kt = w.to(d_vn.dtype), kt.to(d_vn.dtype)
    BH, n, C, D = w.shape
    dS = d_final.clone()
    d_vn_tot = torch.empty_like(d_vn)
    dS_next = torch.empty_like(d_states)
    for i in range(n - 1, -1, -1):
        dS_next[:, i] = dS
        d_vn_tot[:, i] = d_vn[:, i] + kt[:, i] @ dS
        dS = gamma[:, i, None, None] * dS + d_states[:, i] - w[:, i].transpose(-1, -2) @ d_vn_tot[:, i]
    if states is None:
        return d_vn_tot, dS_next, dS
    return d_vn_tot, dS_next, dS, (states * dS_next).sum(dim=(-1, -2))


def _native_ok(w, u) -> bool:
    D, Dv = w.shape[-1], u.shape[-1]
    return (w.is_cuda and nv.available() and nv.has("ttcd_delta_chain_fwd") and w.dtype in (torch.float32, torch.bfloat16)
            and u.dtype == torch.float32 and D in (32, 64, 128, 256) and Dv % 32 == 0 and w.shape[2] == 64)


def _tiles(t: torch.Tensor) -> torch.Tensor:
    """w / kt as the kernels take them: contiguous bf16 (exact TF32 operands, half the staging traffic)."""
    return t.to(torch.bfloat16).contiguous()


def _fwd(w, u, kt, gamma, s0):
    if not _native_ok(w, u):
        return _fwd_torch(w, u, kt, gamma, s0)
    BH, n, C, D = w.shape
    Dv = u.shape[-1]
    w, kt = _tiles(w), _tiles(kt)
    u, gamma, s0 = (t.contiguous() for t in (u, gamma, s0))
    vn = torch.empty_like(u)
    states = torch.empty(BH, n, D, Dv, dtype=torch.float32, device=w.device)
    final = torch.empty(BH, D, Dv, dtype=torch.float32, device=w.device)
    nv.call("ttcd_delta_chain_fwd", nv.ptr(w), nv.ptr(u), nv.ptr(kt), nv.ptr(gamma), nv.ptr(s0), nv.ptr(vn), nv.ptr(states),
            nv.ptr(final), nv.i32(BH), nv.i32(n), nv.i32(D), nv.i32(Dv), nv.stream_ptr())
    return vn, states, final


def _bwd(w, kt, gamma, d_vn, d_states, d_final, states=None):
    """The reverse chain; with ``states`` (the forward states) also the gradient of gamma, sum(states * dS_next) per chunk."""
    if not _native_ok(w, d_vn):
        return _bwd_torch(w, kt, gamma, d_vn, d_states, d_final, states)
    BH, n, C, D = w.shape
    Dv = d_vn.shape[-1]
    w, kt = _tiles(w), _tiles(kt)
    gamma, d_vn, d_states, d_final = (t.contiguous() for t in (gamma, d_vn, d_states, d_final))
    d_vn_tot = torch.empty_like(d_vn)
    dS_next = torch.empty_like(d_states)
    d_s0 = torch.empty_like(d_final)
    parts = None if states is None else torch.zeros(BH, n, Dv // 32, dtype=torch.float32, device=w.device)
    # the reverse chain is the forward chain with the roles of w and kt exchanged (and transposed uses)
    nv.call("ttcd_delta_chain_bwd", nv.ptr(w), nv.ptr(kt), nv.ptr(gamma), nv.ptr(d_vn), nv.ptr(d_states), nv.ptr(d_final),
            nv.ptr(d_vn_tot), nv.ptr(dS_next), nv.ptr(d_s0), nv.ptr(None if states is None else states.contiguous()),
            nv.ptr(parts), nv.i32(BH), nv.i32(n), nv.i32(D), nv.i32(Dv), nv.stream_ptr())
    if states is None:
        return d_vn_tot, dS_next, d_s0
    return d_vn_tot, dS_next, d_s0, parts.sum(-1)


class _DeltaChain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, u, kt, gamma, s0):
        vn, states, final = _fwd(w, u, kt, gamma, s0)
        ctx.save_for_backward(w, kt, gamma, vn, states)
        return vn, states, final

    @staticmethod
    def backward(ctx, d_vn, d_states, d_final):
        w, kt, gamma, vn, states = ctx.saved_tensors
        zeros = lambda t, like: torch.zeros_like(like) if t is None else t  # noqa: E731
        d_vn, d_states = zeros(d_vn, vn), zeros(d_states, states)
        d_final = zeros(d_final, states[:, 0])
        d_vn_tot, dS_next, d_s0, d_gamma = _bwd(w, kt, gamma, d_vn, d_states, d_final, states)      # d_gamma [BH, n]
        d_u = d_vn_tot
        d_w = -(d_vn_tot @ states.transpose(-1, -2))                      # [BH, n, C, D]
        d_kt = vn @ dS_next.transpose(-1, -2)                             # [BH, n, C, D]
        return d_w, d_u, d_kt, d_gamma, d_s0


def delta_chain(w, u, kt, gamma, s0):
    """w, kt [BH, n, C, D] (the CUDA kernels multiply them as bf16); u [BH, n, C, Dv]; gamma [BH, n]; s0 [BH, D, Dv] (fp32).  Returns (vn [BH, n, C, Dv], the state
    entering every chunk [BH, n, D, Dv], the final state [BH, D, Dv])."""
    return _DeltaChain.apply(w, u, kt, gamma, s0)
