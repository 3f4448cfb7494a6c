"""Functional op layer.

Each function routes CUDA bf16 tensors to the hand-written sm_100a kernels
(``ttcd_b200.ops.cuda``; autograd Functions with native forward and backward)
and everything else (CPU tensors, fp32) to the PyTorch statements in
``ttcd_b200.ops.reference``.  A CUDA bf16 call with the native library missing
raises instead of silently falling back.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import _native
from . import delta_fused, reference

__all__ = [
    "rmsnorm", "rmsnorm_dual", "qkv_norm_rope", "rope", "swiglu", "swiglu_packed", "linear", "matmul",
    "attention", "dual_window_attention", "lse_merge", "dwconv_chunked", "dwconv_sequence",
    "ttt_scan", "cross_entropy", "linear_cross_entropy", "newton_schulz", "reference",
]


def _cuda():
    from . import cuda  # noqa: WPS433 (lazy: keeps CPU-only imports light)
    return cuda


# -- normalisation -----------------------------------------------------------------

def rmsnorm(x, weight, eps: float, residual=None, prenorm: bool = False):
    if _native.use_native(x):
        return _cuda().rmsnorm(x, weight, eps, residual, prenorm)
    return reference.rmsnorm(x, weight, eps, residual, prenorm)


def rmsnorm_dual(attn_teacher, attn_student, residual, weight, eps: float):
    if _native.use_native(attn_teacher):
        return _cuda().rmsnorm_dual(attn_teacher, attn_student, residual, weight, eps)
    return reference.rmsnorm_dual(attn_teacher, attn_student, residual, weight, eps)


# -- rotary --------------------------------------------------------------------------

def rope(x, cos, sin, offset=0, positions=None):
    if _native.use_native(x):
        return _cuda().rope(x, cos, sin, offset, positions)
    return reference.rope(x, cos, sin, offset, positions)


def qkv_norm_rope(q, k, q_weight, k_weight, eps: float, cos, sin, offset=0, positions=None):
    """Per-head RMSNorm (when weights are given) followed by RoPE on q[B,T,H,D], k[B,T,HK,D]."""
    if _native.use_native(q):
        return _cuda().qk_norm_rope(q, k, q_weight, k_weight, eps, cos, sin, offset, positions)
    if q_weight is not None:
        q = reference.rmsnorm(q, q_weight, eps)
        k = reference.rmsnorm(k, k_weight, eps)
    if cos is not None:
        q = reference.rope(q, cos, sin, offset, positions)
        k = reference.rope(k, cos, sin, offset, positions)
    return q, k


# -- MLP pieces ------------------------------------------------------------------------

def swiglu(gate, up):
    if _native.use_native(gate):
        return _cuda().swiglu(gate, up)
    return reference.swiglu(gate, up)


def swiglu_packed(gate_up):
    """swiglu on a [*, 2*d_i] tensor holding gate then up columns."""
    d = gate_up.shape[-1] // 2
    if _native.use_native(gate_up):
        return _cuda().swiglu_packed(gate_up)
    return reference.swiglu(gate_up[..., :d], gate_up[..., d:])


def linear(x, weight, bias=None):
    if _native.use_native(x):
        return _cuda().linear(x, weight, bias)
    return F.linear(x, weight, bias)


def matmul(a, b):
    """Batched a @ b; transposed views select the operand major mode of the tensor-core kernel."""
    if _native.use_native(a) and b.dtype == torch.bfloat16:
        return _cuda().matmul(a, b)
    return torch.matmul(a, b)


def dwconv_chunked(x, weight, causal: bool = True):
    """x[b,T,C,D], weight [D,K] (or Conv1d layout [D,1,K])."""
    w2 = weight.reshape(weight.shape[0], weight.shape[-1])
    if _native.use_native(x):
        return _cuda().dwconv_chunked(x, w2, causal)
    return reference.dwconv_chunked(x, w2, causal)


def dwconv_sequence(x, weight, bias=None, activation=None, residual=None, cu_seqlens=None):
    w2 = weight.reshape(weight.shape[0], weight.shape[-1])
    if _native.use_native(x) and cu_seqlens is None:
        y = _cuda().dwconv_chunked(x.unsqueeze(1), w2, True).squeeze(1)
        if bias is not None:
            y = y + bias
        if activation in ("silu", "swish"):
            y = F.silu(y)
        if residual is not None:
            y = y + residual
        return y
    return reference.dwconv_sequence(x, w2, bias, activation, residual, cu_seqlens)


# -- attention ---------------------------------------------------------------------------

def attention(q, k, v, window=None, scale=None, cu_seqlens=None, return_lse: bool = False):
    if _native.use_native(q):
        return _cuda().attention(q, k, v, window, scale, cu_seqlens, return_lse)
    return reference.attention(q, k, v, window, scale, cu_seqlens, return_lse)


_DUAL_IMPL = "fused"


def l2_softmax_attention(q, k, v, scale=None, cu_seqlens=None):
    """Causal attention with L2-normalised exponentials (``use_l2_softmax``): PyTorch statement on every device (no
    shipped config enables it)."""
    return reference.l2_softmax_attention(q, k, v, scale, cu_seqlens)


def decode_attention(q, k, v, kv_len, scale=None):
    """One decode step over a fixed-capacity cache: q [B,1,H,D] against the first ``kv_len`` rows (a one-element int32
    device tensor, read on the device) of k, v [B,cap,HK,D], in whatever order they sit (a ring buffer): no positional
    mask, every filled row is visible.  Nothing here reads ``kv_len`` on the host, so the call can be captured."""
    if _native.use_native(q) and q.shape[1] == 1 and _cuda().attn_small_q_supported(q, k):
        return _cuda().attn_small_q(q, k, v, None, scale, kv_len)
    B, _, H, D = q.shape
    cap, HK = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    kf = k.float().repeat_interleave(H // HK, dim=2)
    vf = v.float().repeat_interleave(H // HK, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * scale
    hidden = torch.arange(cap, device=q.device) >= kv_len.to(q.device)
    p = torch.softmax(s.masked_fill(hidden[None, None, None, :], float("-inf")), dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, vf).to(q.dtype)


def set_dual_attention_impl(impl: str) -> str:
    """``fused`` (default: one pass over K/V) or ``two_pass`` (two single-window calls, the reference's
    unpatched behaviour) — an A/B switch for benchmarks.  Returns the previous setting."""
    global _DUAL_IMPL
    if impl not in ("fused", "two_pass"):
        raise ValueError(f"unknown dual attention implementation {impl!r}")
    prev, _DUAL_IMPL = _DUAL_IMPL, impl
    return prev


def dual_window_attention(q, k, v, window_teacher, window_student, scale=None, cu_seqlens=None):
    """Teacher and student sliding-window outputs in one pass over K/V."""
    if _DUAL_IMPL == "two_pass":
        return (attention(q, k, v, window_teacher, scale, cu_seqlens), attention(q, k, v, window_student, scale, cu_seqlens))
    if _native.use_native(q):
        return _cuda().dual_window_attention(q, k, v, window_teacher, window_student, scale, cu_seqlens)
    return reference.dual_window_attention(q, k, v, window_teacher, window_student, scale, cu_seqlens)


def lse_dual_window_attention(q, k, v, window_teacher, window_student, scale=None):
    """Teacher and student outputs by LSE combination (the reference's ``lse_dual_window_attn``,
    profiling/lse_dual_attn.py:16-39): student = attention(w_S); the keys only the teacher sees,
    [i - w_T + 1, i - w_S], are attended by shifting the arrays by w_S (window w_T - w_S); the teacher is
    the LSE-weighted merge of the two.  A benchmark variant: the fused kernel does the same in one pass."""
    T = q.shape[1]
    o_s, lse_s = attention(q, k, v, window_student, scale, return_lse=True)
    if T <= window_student or window_teacher <= window_student:
        return o_s, o_s
    o_far, lse_far = attention(q[:, window_student:], k[:, :T - window_student], v[:, :T - window_student],
                               window_teacher - window_student, scale, return_lse=True)
    tail = lse_merge(o_s[:, window_student:], lse_s[..., window_student:], o_far, lse_far)
    return torch.cat([o_s[:, :window_student], tail], dim=1), o_s


def lse_merge(o_a, lse_a, o_b, lse_b):
    if _native.use_native(o_a):
        return _cuda().lse_merge(o_a, lse_a, o_b, lse_b)
    return reference.lse_merge(o_a, lse_a, o_b, lse_b)


# -- fast-weight scan ----------------------------------------------------------------------

def ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, *, lr, update_every, state_dtype=None,
             normalize_student=False, norm_proj_diff=False, post_proj=None, return_last_dw_norm=False, cp=None,
             proj_reduce=None, key=None):
    """``key``: identifies the calling layer (context parallel: names the peer buffers of its rank prefix)."""
    plain = not normalize_student and not norm_proj_diff and post_proj is None
    if _native.use_native(z_out) and plain and (state_dtype in (None, torch.bfloat16, torch.float32)):
        T, C = z_out.shape[1], z_out.shape[2]
        sharded = cp is not None and cp.size > 1
        fused_ok = ((not sharded or getattr(cp, "barrier", None) is not None) and proj_reduce is None and C >= 128
                    and z_out.shape[3] >= 128 and w_down.shape[0] >= 128 and z_out.shape[3] % 8 == 0
                    and w_down.shape[0] % 8 == 0)
        if fused_ok:
            # grouping by update_every only bounds the reference's memory; the prefix over chunks is the same sum:
            # batched GEMMs + one streaming prefix kernel (ops/cuda.py::_TTTScan); under context parallelism the
            # prefix over ranks runs over peer memory
            y, last = _cuda().ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, lr, cp if sharded else None, key)
            return (y, last) if return_last_dw_norm else y
        return reference.ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, lr=lr,
                                  update_every=update_every, state_dtype=torch.float32,
                                  return_last_dw_norm=return_last_dw_norm, matmul=_cuda().matmul, cp=cp, proj_reduce=proj_reduce)
    return reference.ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, lr=lr,
                              update_every=update_every, state_dtype=state_dtype,
                              normalize_student=normalize_student, norm_proj_diff=norm_proj_diff,
                              post_proj=post_proj, return_last_dw_norm=return_last_dw_norm, cp=cp, proj_reduce=proj_reduce)


# -- losses ------------------------------------------------------------------------------------

def cross_entropy(logits, labels, ignore_index: int = -100, label_smoothing: float = 0.0, z_loss: float = 0.0):
    if _native.use_native(logits) and logits.dim() == 2 and logits.shape[-1] % 8 == 0:
        return _cuda().cross_entropy(logits, labels, ignore_index, label_smoothing, z_loss)
    return reference.cross_entropy(logits, labels, ignore_index, label_smoothing, z_loss)


def linear_cross_entropy(hidden, labels, weight, bias=None, ignore_index: int = -100, num_chunks: int = 8,
                         l2_penalty: float = 0.0):
    """CE(hidden @ weight^T) without the full logits; ``l2_penalty`` > 0 adds the l2-warp gradient term (max logit
    * l2_penalty / valid tokens at each row's arg-max column) inside the same pass."""
    if _native.use_native(hidden) and bias is None:
        return _cuda().linear_cross_entropy(hidden, labels, weight, ignore_index, num_chunks, l2_penalty)
    return reference.linear_cross_entropy(hidden, labels, weight, bias, ignore_index, l2_penalty)


def newton_schulz(g, coeffs=reference.NS_COEFFS):
    if g.is_cuda and _native.available():
        return _cuda().newton_schulz(g, coeffs)
    return reference.newton_schulz(g, coeffs)


# chunk length of the (gated) delta rule (0: 256 for sequences of 1024 tokens and more, else 64).  The work inside a chunk
# is one batched triangular solve and a few batched GEMMs; the chain over chunks is a prefix scan of D x D maps, whose
# intermediates shrink with the number of chunks.
_DELTA_CHUNK = int(os.environ.get("TTCD_DELTA_CHUNK", "0"))
_DELTA_FUSED = os.environ.get("TTCD_DELTA_FUSED", "1") != "0"


def gated_delta_rule(q, k, v, g, beta, *, scale=None, l2norm: bool = True, cu_seqlens=None, initial_state=None,
                     output_final_state: bool = False, recurrent: bool = False):
    """(Gated) delta rule over q, k [B,T,H,Dk], v [B,T,H,Dv], log decay g and write strength beta [B,T,H]; ``g`` None is
    the plain delta rule.  ``recurrent`` takes the token-by-token form (short decode steps), otherwise the chunked
    form.  Returns (o, final state or None).

    On the GPU, for head sizes the kernels take, the chunked form is one op with a hand-written backward
    (``ops/delta_fused.py``: chunk-local kernels, chain kernels, batched products; its fp32 intermediates are kept for
    backward within a memory budget and rebuilt beyond it).  Elsewhere it is the PyTorch statement under activation
    recomputation: autograd keeps q, k, v, g, beta and rebuilds the per-chunk factors and states in backward."""
    if recurrent and cu_seqlens is None:
        return reference.gated_delta_rule_recurrent(q, k, v, g, beta, scale, l2norm, initial_state, output_final_state)
    if _DELTA_FUSED and not _DELTA_CHUNK and delta_fused.native_ok(q, v):
        # one op with a hand-written backward: chunk-local kernels, the chain kernels, batched products in between
        if cu_seqlens is None:
            return delta_fused.gated_delta_rule_fused(q, k, v, g, beta, scale, l2norm, initial_state, output_final_state)
        bounds = cu_seqlens.tolist()
        outs, finals = [], []
        for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):      # every packed sequence starts from its own state
            o, s = delta_fused.gated_delta_rule_fused(q[:, a:b], k[:, a:b], v[:, a:b], None if g is None else g[:, a:b],
                                                      beta[:, a:b], scale, l2norm,
                                                      None if initial_state is None else initial_state[i:i + 1], output_final_state)
            outs.append(o)
            finals.append(s)
        return torch.cat(outs, dim=1), (torch.cat(finals, dim=0) if output_final_state else None)
    # on the GPU the chain over chunks is one kernel per direction (64-row chunks, small per-chunk tensors); elsewhere
    # fewer, longer chunks keep the number of dependent steps down
    chain = q.is_cuda and _native.available() and _native.has("ttcd_delta_chain_fwd") \
        and q.shape[-1] in (32, 64, 128, 256) and v.shape[-1] % 32 == 0
    chunk = _DELTA_CHUNK or (64 if chain else (256 if q.shape[1] >= 1024 else 64))
    if chunk != 64:
        chain = False
    args = (q, k, v, g, beta, scale, l2norm, chunk, cu_seqlens, initial_state, output_final_state, True, chain)
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta))
    if needs_grad and not _keep_delta_intermediates(q, v, chunk):
        from torch.utils.checkpoint import checkpoint
        return checkpoint(reference.gated_delta_rule_chunked, *args, use_reentrant=False)
    return reference.gated_delta_rule_chunked(*args)


def _keep_delta_intermediates(q, v, chunk: int) -> bool:
    """Whether a call of the chunked rule keeps its fp32 intermediates for backward instead of recomputing them.
    Recomputation is the default: kept, the intermediates of a 24-layer model at 16 x 4096 tokens come to ~140 GB (for a
    5 % shorter step on `delta_net` 340M, and more than 180 GB on `gated_deltanet`).  ``TTCD_DELTA_KEEP=1`` keeps them."""
    return q.is_cuda and os.environ.get("TTCD_DELTA_KEEP", "0") == "1"
