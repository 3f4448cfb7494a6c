"""Plain-PyTorch statements of every op in the framework.

These are the numerical oracles for the CUDA kernels (tests compare a kernel
against the function here evaluated in fp32) and the execution path for CPU
tensors.  Nothing in this file launches a hand-written kernel.

Semantics follow the reference's layers: RMSNorm with fp32 statistics and an
optional fused residual add (fla/modules/layernorm.py:254-320), NeoX-style RoPE
(fla/modules/rotary.py:27-32), flash-attn window semantics
``window_size=(W-1, 0)`` with bottom-right alignment when ``Tq < Tk``
(test/test_fused_dual_attn.py:88-110), the per-chunk causal depthwise conv
(custom_models/ipttcd/modeling_ipttcdv9.py:203-211) and the grouped fast-weight
scan (custom_models/ipttcd/modeling_ipttcdv9_lowcopy_scanfuse.py:117-204).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

# ----------------------------------------------------------------------------
# normalisation / rotary / activation
# ----------------------------------------------------------------------------


def rmsnorm(x, weight, eps: float, residual=None, prenorm: bool = False):
    """y = rmsnorm(x + residual) * weight; optionally also return the summed residual."""
    out_dtype = x.dtype
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
    res_out = xf.to(residual.dtype if residual is not None else out_dtype)
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = xf * rstd
    if weight is not None:
        y = y * weight.float()
    y = y.to(out_dtype)
    return (y, res_out) if prenorm else y


def rmsnorm_dual(attn_teacher, attn_student, residual, weight, eps: float):
    """The TTT block's two mlp_norm calls sharing one residual.

    Returns (teacher_normed, student_normed, new_residual) with
    new_residual = residual + attn_teacher (the student sum is not kept).
    """
    x, res_out = rmsnorm(attn_teacher, weight, eps, residual=residual, prenorm=True)
    t = rmsnorm(attn_student, weight, eps, residual=residual, prenorm=False)
    return x, t, res_out


def rope_tables(head_dim: int, base: float, seqlen: int, device=None, dtype=torch.float32,
                inv_freq: torch.Tensor | None = None, attn_scale: float = 1.0):
    """cos/sin tables [seqlen, head_dim/2]: fp32 math, stored in ``dtype``."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seqlen, device=device, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq.to(device=device, dtype=torch.float32))
    cos, sin = torch.cos(freqs), torch.sin(freqs)
    if attn_scale != 1.0:
        cos, sin = cos * attn_scale, sin * attn_scale
    return cos.to(dtype), sin.to(dtype)


def yarn_inv_freq(head_dim: int, base: float, factor: float, original_max_position: int,
                  beta_fast: float = 32.0, beta_slow: float = 1.0, device=None) -> torch.Tensor:
    """YaRN inverse frequencies: blend of extrapolation and interpolation by a per-pair ramp."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    if factor <= 1.0:
        return inv_freq

    def correction_dim(n_rot: float) -> float:
        return head_dim * math.log(original_max_position / (2.0 * math.pi * n_rot)) / (2.0 * math.log(base))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), head_dim - 1)
    lo, hi = low / 2.0, high / 2.0
    if lo == hi:
        hi += 0.001
    idx = torch.arange(inv_freq.shape[0], device=device, dtype=torch.float32)
    ramp = ((idx - lo) / (hi - lo)).clamp(0.0, 1.0)
    return inv_freq * (1.0 - ramp) + (inv_freq / factor) * ramp


def llama3_inv_freq(head_dim: int, base: float, factor: float, original_max_position: int,
                    low_freq_factor: float = 1.0, high_freq_factor: float = 4.0, device=None) -> torch.Tensor:
    """Llama-3 rotary scaling: wavelengths longer than original/low_freq_factor are slowed by ``factor``, those
    shorter than original/high_freq_factor are kept, the band between is blended linearly in original/wavelength."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    wavelen = 2.0 * math.pi / inv_freq
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    smooth = ((original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)).clamp(0.0, 1.0)
    blended = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
    out = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    middle = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
    return torch.where(middle, blended, out)


def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    if factor <= 1.0:
        return 1.0
    return float(mscale) if mscale != 1.0 else 0.1 * math.log(factor) + 1.0


def rope(x, cos, sin, offset=0, positions=None, conjugate: bool = False):
    """NeoX (half-split) rotary on x[B,T,H,D] with tables [*, D/2].

    ``offset`` is an int or a per-batch tensor; ``positions`` (shape [B,T] or [T])
    overrides it (varlen packing, context-parallel shards).
    """
    B, T, H, D = x.shape
    half = cos.shape[-1]
    if positions is None:
        base = torch.arange(T, device=x.device)
        if isinstance(offset, torch.Tensor):
            positions = base[None, :] + offset.to(x.device).view(-1, 1)
        else:
            positions = (base + int(offset))[None, :]
    elif positions.dim() == 1:
        positions = positions[None, :]
    c = cos[positions].float().unsqueeze(2)  # [B|1, T, 1, half]
    s = sin[positions].float().unsqueeze(2)
    if conjugate:
        s = -s
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:2 * half]
    out = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, xf[..., 2 * half:]], dim=-1)
    return out.to(x.dtype)


def swiglu(gate, up):
    gf = gate.float()
    return (gf * torch.sigmoid(gf) * up.float()).to(gate.dtype)


# ----------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------


def window_mask(tq: int, tk: int, window: int | None, device=None) -> torch.Tensor:
    """Boolean [tq, tk] visibility mask, causal, bottom-right aligned, W keys incl. self."""
    qi = torch.arange(tq, device=device)[:, None] + (tk - tq)
    kj = torch.arange(tk, device=device)[None, :]
    mask = kj <= qi
    if window is not None and window > 0:
        mask &= kj > qi - window
    return mask


def _segment_mask(cu_seqlens: torch.Tensor, total: int, device) -> torch.Tensor:
    seg = torch.zeros(total, dtype=torch.long, device=device)
    bounds = cu_seqlens.to(device=device, dtype=torch.long)
    seg[bounds[1:-1]] = 1
    seg = seg.cumsum(0)
    return seg[:, None] == seg[None, :]


def attention(q, k, v, window: int | None = None, scale: float | None = None,
              cu_seqlens: torch.Tensor | None = None, return_lse: bool = False):
    """Causal (sliding-window) attention on q[B,Tq,H,D], k/v[B,Tk,HK,D]; fp32 softmax."""
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    rep = H // HK
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = window_mask(Tq, Tk, window, device=q.device)
    if cu_seqlens is not None:
        mask = mask & _segment_mask(cu_seqlens, Tk, q.device)[Tk - Tq:]
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    return (o, lse) if return_lse else o


def dual_window_attention(q, k, v, window_teacher: int | None, window_student: int,
                          scale: float | None = None, cu_seqlens=None):
    """Teacher (w_T) and student (w_S) outputs over shared Q/K/V."""
    o_t = attention(q, k, v, window_teacher, scale, cu_seqlens)
    o_s = attention(q, k, v, window_student, scale, cu_seqlens)
    return o_t, o_s


def l2_softmax_attention(q, k, v, scale: float | None = None, cu_seqlens=None, block: int = 1024):
    """Causal attention whose weights are the exponentials normalised by their L2 norm instead of their sum:
    p_ij = exp(s_ij - m_i) / sqrt(sum_j exp(2 (s_ij - m_i)))  (fla/ops/attn/parallel.py:71-165 with ``use_l2``; the
    reference applies no sliding window on this path, fla/layers/attn.py:246-279).  q [B,Tq,H,D], k/v [B,Tk,HK,D],
    bottom-right aligned when Tq < Tk; query rows are processed ``block`` at a time so that the score matrix stays
    small.  Differentiable through autograd."""
    if cu_seqlens is not None:
        bounds = cu_seqlens.tolist()
        return torch.cat([l2_softmax_attention(q[:, a:b], k[:, a:b], v[:, a:b], scale, None, block)
                          for a, b in zip(bounds[:-1], bounds[1:])], dim=1)
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    kf = k.float().repeat_interleave(H // HK, dim=2)
    vf = v.float().repeat_interleave(H // HK, dim=2)
    outs = []
    for r0 in range(0, Tq, block):
        r1 = min(Tq, r0 + block)
        hi = Tk - Tq + r1                                            # keys any row of this block may see
        s = torch.einsum("bqhd,bkhd->bhqk", q[:, r0:r1].float(), kf[:, :hi]) * scale
        rows = torch.arange(r0, r1, device=q.device)[:, None] + (Tk - Tq)
        s = s.masked_fill(torch.arange(hi, device=q.device)[None, :] > rows, float("-inf"))
        e = torch.exp(s - s.amax(dim=-1, keepdim=True))
        p = e / e.square().sum(-1, keepdim=True).sqrt()
        outs.append(torch.einsum("bhqk,bkhd->bqhd", p, vf[:, :hi]))
    return torch.cat(outs, dim=1).to(q.dtype)


def lse_merge(o_a, lse_a, o_b, lse_b):
    """Merge two partial softmax results (o[B,T,H,D], lse[B,H,T]) over disjoint key sets."""
    m = torch.maximum(lse_a, lse_b)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    wa = torch.exp(lse_a - m)
    wb = torch.exp(lse_b - m)
    denom = (wa + wb).clamp_min(1e-38)
    wa = (wa / denom).transpose(1, 2).unsqueeze(-1)
    wb = (wb / denom).transpose(1, 2).unsqueeze(-1)
    return (o_a.float() * wa + o_b.float() * wb).to(o_a.dtype)


# ----------------------------------------------------------------------------
# depthwise conv
# ----------------------------------------------------------------------------


def dwconv_chunked(x, weight, causal: bool = True):
    """Depthwise conv over the C axis of x[b,T,C,D] with zero context per chunk.

    weight: [D, K].  causal: y[c] = sum_j w[:, j] * x[c - (K-1) + j]; otherwise
    centred ('same' padding K//2).
    """
    b, T, C, D = x.shape
    K = weight.shape[-1]
    xf = x.float()
    wf = weight.float().reshape(D, K)
    left = K - 1 if causal else K // 2
    right = 0 if causal else K - 1 - left
    xp = F.pad(xf, (0, 0, left, right))
    y = torch.zeros_like(xf)
    for j in range(K):
        y = y + xp[:, :, j:j + C, :] * wf[:, j]
    return y.to(x.dtype)


def dwconv_sequence(x, weight, bias=None, activation: str | None = None, residual=None,
                    cu_seqlens=None):
    """Sequence-level causal depthwise conv on x[B,T,D] (no per-chunk reset), weight [D,K]."""
    B, T, D = x.shape
    if cu_seqlens is not None:
        outs = []
        bounds = cu_seqlens.tolist()
        for s, e in zip(bounds[:-1], bounds[1:]):
            outs.append(dwconv_chunked(x[:, s:e].unsqueeze(1), weight, True).squeeze(1))
        y = torch.cat(outs, dim=1)
    else:
        y = dwconv_chunked(x.unsqueeze(1), weight, True).squeeze(1)
    y = y.float()
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


# ----------------------------------------------------------------------------
# TTT fast-weight scan
# ----------------------------------------------------------------------------


def ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_update_t, *, lr: float, update_every: int,
             state_dtype: torch.dtype | None = None, normalize_student: bool = False,
             norm_proj_diff: bool = False, post_proj: torch.Tensor | None = None,
             return_last_dw_norm: bool = False, matmul=torch.matmul, cp=None, proj_reduce=None):
    """Grouped fast-weight scan.

    ``matmul`` is the batched-matmul primitive (torch.matmul, or the tensor-core
    kernel wrapper for CUDA bf16 inputs).

    z_out, z_tgt, z_hat: [b, T, C, d_i]; beta: [b, T, C, 1] or None;
    w_down: [d_h, d_i]; w_update_t: [d_i, d_h] (= W_down^T @ W_p when the
    projection is folded in, else W_down^T); post_proj: optional [d_h, d_h]
    applied after beta when the projection is not folded.

        P_j  = beta_j * ((z_tgt_j - z_hat_j) @ w_update_t)
        dW_j = P_j^T @ z_hat_j                      (j = 0..T-2)
        W_i  = w_down + lr * sum_{j<i} dW_j          (prefix kept in state_dtype, grouped)
        Y_i  = z_out_i @ W_i^T

    ``proj_reduce``: applied to the projected difference before beta (tensor parallelism shards d_i, so each
    rank holds a partial sum there; the caller passes an all-reduce that also all-reduces in backward).

    ``cp`` (context-parallel state with ``rank``/``size``): the T chunks are this rank's slice of a
    longer sequence; the scan then starts from ``w_down + lr * sum`` of every earlier rank's updates
    (exclusive prefix over ranks) and this rank's last chunk also produces an update for its successors.
    """
    b, T, C, d_i = z_out.shape
    compute_dtype = z_out.dtype
    state_dtype = compute_dtype if state_dtype is None else state_dtype
    w_cur = w_down.to(state_dtype).unsqueeze(0).expand(b, -1, -1)
    lr_t = w_cur.new_tensor(lr)
    group = max(1, min(T, update_every))

    def delta_w(lo: int, hi: int):
        diff = z_tgt[:, lo:hi] - z_hat[:, lo:hi]
        proj = matmul(diff, w_update_t.to(compute_dtype))
        if proj_reduce is not None:       # tensor parallel: d_i is sharded, the projection is a partial sum
            proj = proj_reduce(proj)
        if norm_proj_diff:
            proj = F.normalize(proj, p=2, dim=-1, eps=1e-6)
        zh = z_hat[:, lo:hi]
        if normalize_student:
            zh = F.normalize(zh, p=2, dim=-1, eps=1e-6)
        if beta is not None:
            proj = proj * beta[:, lo:hi]
        if post_proj is not None:
            proj = matmul(proj, post_proj.to(compute_dtype))
        return matmul(proj.transpose(-1, -2), zh)

    d_w_all = None
    if cp is not None and cp.size > 1:
        from ..parallel import context as _context
        n_upd = T if cp.rank < cp.size - 1 else T - 1     # globally, only the very last chunk never updates
        if n_upd > 0:
            d_w_all = delta_w(0, n_upd)
            local_sum = lr_t * d_w_all.to(state_dtype).sum(dim=1)
        else:
            local_sum = torch.zeros(b, w_down.shape[0], w_down.shape[1], dtype=state_dtype, device=z_out.device)
        w_cur = w_cur + _context.rank_prefix(local_sum)

    outs = []
    last_norm = None
    for gs in range(0, T, group):
        ge = min(gs + group, T)
        upd_end = min(ge, T - 1)
        k_upd = upd_end - gs
        cs = None
        if k_upd > 0:
            d_w = d_w_all[:, gs:upd_end] if d_w_all is not None else delta_w(gs, upd_end)
            if return_last_dw_norm:
                last_norm = d_w[:, -1].detach().float().norm()
            cs = lr_t * torch.cumsum(d_w.to(state_dtype), dim=1)
        for local in range(ge - gs):
            if local == 0 or k_upd == 0:
                w_step = w_cur
            else:
                w_step = w_cur + cs[:, min(local - 1, k_upd - 1)]
            outs.append(matmul(z_out[:, gs + local], w_step.to(compute_dtype).transpose(-1, -2)))
        if k_upd > 0:
            w_cur = w_cur + cs[:, -1]
    y = torch.stack(outs, dim=1)
    return (y, last_norm) if return_last_dw_norm else y


# ----------------------------------------------------------------------------
# losses
# ----------------------------------------------------------------------------


def cross_entropy(logits, labels, ignore_index: int = -100, label_smoothing: float = 0.0,
                  z_loss: float = 0.0):
    """Mean CE over non-ignored rows; fp32 math."""
    lf = logits.float()
    loss = F.cross_entropy(lf, labels, ignore_index=ignore_index, label_smoothing=label_smoothing,
                           reduction="sum")
    valid = labels.ne(ignore_index)
    if z_loss:
        lse = torch.logsumexp(lf, dim=-1)
        loss = loss + z_loss * (lse.pow(2) * valid).sum()
    return loss / valid.sum().clamp_min(1)


class _L2WarpRows(torch.autograd.Function):
    """Identity on the loss; adds max logit * factor at every row's arg-max column to the gradient of the logits
    (the l2-warp term of fla/modules/fused_linear_cross_entropy.py:250-283; every row, ignored labels included)."""

    @staticmethod
    def forward(ctx, loss, logits, factor):
        ctx.save_for_backward(logits)
        ctx.factor = factor
        return loss.view_as(loss)

    @staticmethod
    def backward(ctx, grad):
        (logits,) = ctx.saved_tensors
        mx, idx = logits.max(-1, keepdim=True)
        g = torch.zeros_like(logits).scatter_(-1, idx, mx * ctx.factor)
        return grad, g * grad, None


def linear_cross_entropy(hidden, labels, weight, bias=None, ignore_index: int = -100, l2_penalty: float = 0.0):
    """CE(hidden @ weight^T + bias, labels) with the logits GEMM in the activation dtype; ``l2_penalty`` > 0 adds the
    l2-warp gradient term scaled by 1 / (number of valid labels)."""
    logits = F.linear(hidden, weight.to(hidden.dtype), None if bias is None else bias.to(hidden.dtype))
    logits = logits.view(-1, logits.shape[-1])
    loss = cross_entropy(logits, labels.reshape(-1), ignore_index)
    if l2_penalty:
        total = labels.ne(ignore_index).sum().clamp_min(1)
        loss = _L2WarpRows.apply(loss, logits, l2_penalty / total)
    return loss


def l2_warp_grad(logits, loss_scale: float = 1e-4):
    """Gradient term of l2-warp: 1e-4/(B*T) * max logit at the argmax position."""
    B, T, V = logits.shape
    mx, idx = logits.max(-1, keepdim=True)
    g = torch.zeros_like(logits)
    g.scatter_(-1, idx, mx * (loss_scale / (B * T)))
    return g


# ----------------------------------------------------------------------------
# optimiser math
# ----------------------------------------------------------------------------

NS_COEFFS = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)


def newton_schulz(g: torch.Tensor, coeffs=NS_COEFFS, dtype=torch.bfloat16) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of a matrix or batch of matrices."""
    squeeze = g.dim() == 2
    x = (g.unsqueeze(0) if squeeze else g).to(dtype)
    transposed = x.size(1) > x.size(2)
    if transposed:
        x = x.transpose(1, 2)
    x = x / (x.float().norm(dim=(1, 2), keepdim=True).to(dtype) + 1e-7)
    for a, b, c in coeffs:
        A = x @ x.transpose(1, 2)
        Bm = b * A + c * (A @ A)
        x = a * x + Bm @ x
    if transposed:
        x = x.transpose(1, 2)
    return x.squeeze(0) if squeeze else x


def adamw_step(param, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale: float = 1.0):
    """One decoupled-weight-decay Adam update in fp32 (in place on param and moments)."""
    g = grad.float() * grad_scale
    param.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    param.addcdiv_(exp_avg, denom, value=-lr / bc1)
    return param


# ---------------------------------------------------------------------------------------------
# delta rule (DeltaNet baseline)
# ---------------------------------------------------------------------------------------------
def delta_rule_recurrent(q, k, v, beta, scale=None, l2norm: bool = True):
    """Token-by-token statement: S_t = S_{t-1} + k_t (beta_t (v_t - S_{t-1}^T k_t))^T, o_t = S_t^T (scale q_t).
    q, k, v: [B, T, H, D]; beta: [B, T, H].  The oracle for ``delta_rule_chunked``."""
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    if l2norm:
        qf, kf = F.normalize(qf, dim=-1, eps=1e-6), F.normalize(kf, dim=-1, eps=1e-6)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    B, T, H, D = qf.shape
    S = qf.new_zeros(B, H, D, vf.shape[-1])
    out = []
    for t in range(T):
        kt, vt, bt = kf[:, t], vf[:, t], bf[:, t].unsqueeze(-1)
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, bt * (vt - pred))
        out.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t] * scale))
    return torch.stack(out, dim=1).to(q.dtype)


def delta_rule_chunked(q, k, v, beta, scale=None, l2norm: bool = True, chunk: int = 64, cu_seqlens=None):
    """Chunk-parallel delta rule (WY representation): inside a chunk the updates are solved with one
    unit-lower-triangular system, the state is carried chunk to chunk (the computation of
    fla/ops/delta_rule/chunk.py with ``use_qk_l2norm_in_kernel``).  Differentiable through autograd."""
    if cu_seqlens is not None:
        bounds = cu_seqlens.tolist()
        return torch.cat([delta_rule_chunked(q[:, a:b], k[:, a:b], v[:, a:b], beta[:, a:b], scale, l2norm, chunk)
                          for a, b in zip(bounds[:-1], bounds[1:])], dim=1)
    dtype = q.dtype
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    if l2norm:
        qf, kf = F.normalize(qf, dim=-1, eps=1e-6), F.normalize(kf, dim=-1, eps=1e-6)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    B, T, H, D = qf.shape
    pad = (-T) % chunk
    if pad:
        qf, kf, vf = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (qf, kf, vf))
        bf = F.pad(bf, (0, 0, 0, pad))
    n = (T + pad) // chunk
    # [B, H, n, C, D]
    qc, kc, vc = (x.view(B, n, chunk, H, -1).permute(0, 3, 1, 2, 4) for x in (qf * scale, kf, vf))
    bc = bf.view(B, n, chunk, H).permute(0, 3, 1, 2).unsqueeze(-1)
    kb, vb = kc * bc, vc * bc
    eye = torch.eye(chunk, device=q.device)
    lower = torch.tril(kb @ kc.transpose(-1, -2), -1)
    t_inv = torch.linalg.solve_triangular(eye + lower, eye.expand_as(lower), upper=False)
    w, u = t_inv @ kb, t_inv @ vb
    qk = torch.tril(qc @ kc.transpose(-1, -2))
    S = qf.new_zeros(B, H, D, vf.shape[-1])
    outs = []
    for i in range(n):
        u_i = u[:, :, i] - w[:, :, i] @ S
        outs.append(qc[:, :, i] @ S + qk[:, :, i] @ u_i)
        S = S + kc[:, :, i].transpose(-1, -2) @ u_i
    o = torch.stack(outs, dim=2)                           # [B, H, n, C, Dv]
    o = o.permute(0, 2, 3, 1, 4).reshape(B, n * chunk, H, -1)[:, :T]
    return o.to(dtype)


def gated_delta_rule_recurrent(q, k, v, g, beta, scale=None, l2norm: bool = True, initial_state=None,
                               output_final_state: bool = False):
    """Token-by-token gated delta rule (the statement of fla/ops/gated_delta_rule/fused_recurrent.py):
    S' = exp(g_t) S_{t-1};  u_t = beta_t (v_t - S'^T k_t);  S_t = S' + k_t u_t^T;  o_t = S_t^T (scale q_t).
    q, k: [B, T, H, Dk]; v: [B, T, H, Dv]; g (log decay, <= 0) and beta: [B, T, H]; ``g`` None means no decay (the
    plain delta rule).  The state is [B, H, Dk, Dv] in fp32.  Returns (o, final state or None).  The oracle of
    ``gated_delta_rule_chunked`` and the path single-token decoding takes."""
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    if l2norm:
        qf, kf = F.normalize(qf, dim=-1, eps=1e-6), F.normalize(kf, dim=-1, eps=1e-6)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    B, T, H, D = qf.shape
    S = qf.new_zeros(B, H, D, vf.shape[-1]) if initial_state is None else initial_state.float()
    out = []
    for t in range(T):
        kt, bt = kf[:, t], bf[:, t].unsqueeze(-1)
        if g is not None:
            S = S * g[:, t].float().exp()[..., None, None]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, bt * (vf[:, t] - pred))
        out.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t] * scale))
    return torch.stack(out, dim=1).to(q.dtype), (S if output_final_state else None)


class _full_fp32:
    """Inside the block fp32 products stay fp32 (the triangular solve of the chunk factors)."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        return self

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


class _tf32_matmuls:
    """On CUDA, let fp32 matrix products use the tensor cores' TF32 mode inside the block (10-bit mantissa operands,
    fp32 accumulation: finer than the bf16 operands the reference's Triton kernels multiply); restores the setting."""

    def __init__(self, enabled: bool):
        self.enabled = enabled

    def __enter__(self):
        if self.enabled:
            self.prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
        return self

    def __exit__(self, *exc):
        if self.enabled:
            torch.backends.cuda.matmul.allow_tf32 = self.prev


def gated_delta_rule_chunked(q, k, v, g, beta, scale=None, l2norm: bool = True, chunk: int = 64, cu_seqlens=None,
                             initial_state=None, output_final_state: bool = False, scan: bool = True, chain: bool = False):
    with _tf32_matmuls(q.is_cuda):
        return _gated_delta_rule_chunked(q, k, v, g, beta, scale, l2norm, chunk, cu_seqlens, initial_state,
                                         output_final_state, scan, chain)


def _gated_delta_rule_chunked(q, k, v, g, beta, scale=None, l2norm: bool = True, chunk: int = 64, cu_seqlens=None,
                              initial_state=None, output_final_state: bool = False, scan: bool = True, chain: bool = False):
    """Chunk-parallel gated delta rule (the computation of fla/ops/gated_delta_rule/chunk.py and, with ``g`` None, of
    fla/ops/delta_rule/chunk.py).  With G the running sum of g inside a chunk and S_0 the state entering it, the
    updates u solve the unit-lower-triangular system (I + L) U = beta V - (beta e^G K) S_0 with
    L_ij = beta_i e^{G_i - G_j} (k_i . k_j) for j < i; every exponent is a difference G_i - G_j with i >= j, so
    nothing overflows.  The chunk-to-chunk chain is one op with a hand-written backward (``chain``: ops/delta_chain.py,
    a CUDA kernel per direction), or, being affine in the state, a prefix scan of D x D maps (``scan``), or the plain
    loop over chunks.  Differentiable through autograd; shapes as in ``gated_delta_rule_recurrent``.  With
    ``cu_seqlens`` (batch 1) each packed sequence starts from a zero state (``initial_state`` then has one entry per
    sequence)."""
    if cu_seqlens is not None:
        bounds = cu_seqlens.tolist()
        outs, finals = [], []
        for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
            init = None if initial_state is None else initial_state[i:i + 1]
            o, s = gated_delta_rule_chunked(q[:, a:b], k[:, a:b], v[:, a:b], None if g is None else g[:, a:b], beta[:, a:b],
                                            scale, l2norm, chunk, None, init, output_final_state, scan, chain)
            outs.append(o)
            finals.append(s)
        return torch.cat(outs, dim=1), (torch.cat(finals, dim=0) if output_final_state else None)
    dtype = q.dtype
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    if l2norm:
        qf, kf = F.normalize(qf, dim=-1, eps=1e-6), F.normalize(kf, dim=-1, eps=1e-6)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    B, T, H, D = qf.shape
    gf = qf.new_zeros(B, T, H) if g is None else g.float()
    pad = (-T) % chunk
    if pad:                     # padded steps: beta = 0 (no update) and g = 0 (no decay) leave the state untouched
        qf, kf, vf = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (qf, kf, vf))
        bf, gf = F.pad(bf, (0, 0, 0, pad)), F.pad(gf, (0, 0, 0, pad))
    n = (T + pad) // chunk
    # [B, H, n, C, D], made contiguous once (every batched product would otherwise copy its strided operand)
    qc, kc, vc = (x.view(B, n, chunk, H, -1).permute(0, 3, 1, 2, 4).contiguous() for x in (qf * scale, kf, vf))
    bc = bf.view(B, n, chunk, H).permute(0, 3, 1, 2).unsqueeze(-1)
    G = gf.view(B, n, chunk, H).permute(0, 3, 1, 2).cumsum(-1)                                         # [B, H, n, C]
    tril = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    decay = (G.unsqueeze(-1) - G.unsqueeze(-2)).masked_fill(~tril, float("-inf")).exp()                # e^{G_i - G_j}, i >= j
    eg = G.exp().unsqueeze(-1)                                                                         # e^{G_i}
    to_end = (G[..., -1:] - G).exp().unsqueeze(-1)                                                     # e^{G_C - G_j}
    kb, vb = kc * bc, vc * bc
    eye = torch.eye(chunk, device=q.device)
    lower = torch.tril(kb @ kc.transpose(-1, -2) * decay, -1)
    with _tf32_matmuls(False) if not q.is_cuda else _full_fp32():
        t_inv = torch.linalg.solve_triangular(eye + lower, eye.expand_as(lower), upper=False)
    w, u = t_inv @ (kb * eg), t_inv @ vb
    qk = (qc @ kc.transpose(-1, -2)) * decay
    q_in, k_out = qc * eg, kc * to_end
    S0 = qf.new_zeros(B, H, D, vf.shape[-1]) if initial_state is None else initial_state.float()
    if chain:
        # the chain over chunks as ONE op (a CUDA kernel per direction on the GPU): ops/delta_chain.py
        from .delta_chain import delta_chain
        Dv = vf.shape[-1]
        flat = lambda t: t.reshape(B * H, n, *t.shape[3:])  # noqa: E731
        vn, states, S = delta_chain(flat(w), flat(u), flat(k_out), eg[:, :, :, -1, 0].reshape(B * H, n), S0.reshape(B * H, D, Dv))
        vn, states, S = vn.view(B, H, n, chunk, Dv), states.view(B, H, n, D, Dv), S.view(B, H, D, Dv)
        o = q_in @ states + qk @ vn
    elif n > 4 and scan and D <= 128:        # (for wider heads the D x D x D products of the scan cost more than the loop)
        # The state entering chunk i+1 is linear in the one entering chunk i:  S_{i+1} = M_i S_i + N_i  with
        # M_i = e^{G_C} I - k_out_i^T w_i  (D x D) and N_i = k_out_i^T u_i.  The chain over the n chunks is a prefix
        # composition of these affine maps, done in log2(n) rounds of batched products instead of n dependent steps.
        kt = k_out.transpose(-1, -2)                                             # [B, H, n, D, C]
        M = torch.diag_embed(eg[:, :, :, -1, :].expand(B, H, n, D)) - kt @ w     # [B, H, n, D, D]
        N = kt @ u                                                               # [B, H, n, D, Dv]
        d = 1
        while d < n:                                                             # inclusive prefix: (M, N)_i := map_i o ... o map_0
            M_lo, N_lo = M[:, :, :-d], N[:, :, :-d]
            N = torch.cat([N[:, :, :d], M[:, :, d:] @ N_lo + N[:, :, d:]], dim=2)
            M = torch.cat([M[:, :, :d], M[:, :, d:] @ M_lo], dim=2)
            d *= 2
        after = M @ S0.unsqueeze(2) + N                                          # state after chunk i
        states = torch.cat([S0.unsqueeze(2), after[:, :, :-1]], dim=2)           # state entering chunk i
        u_all = u - w @ states
        o = q_in @ states + qk @ u_all
        S = after[:, :, -1]
    else:
        S = S0
        outs = []
        for i in range(n):
            u_i = u[:, :, i] - w[:, :, i] @ S
            outs.append(q_in[:, :, i] @ S + qk[:, :, i] @ u_i)
            S = S * eg[:, :, i, -1:, :] + k_out[:, :, i].transpose(-1, -2) @ u_i
        o = torch.stack(outs, dim=2)
    o = o.permute(0, 2, 3, 1, 4).reshape(B, n * chunk, H, -1)[:, :T]
    return o.to(dtype), (S if output_final_state else None)


def dual_window_attention_backward_combined(q, k, v, d_o_t, d_o_s, window_teacher, window_student, scale=None):
    """Gradients of ``dual_window_attention`` through ONE softmax (the statement the combined backward kernels
    implement).  Inside the student window P_S = r * P_T with the per-row ratio r = exp(lse_T - lse_S), so the two
    incoming gradient streams collapse into dO' = dO_T + r dO_S and delta' = delta_T + r delta_S there; outside it
    only the teacher stream exists.  q [B,T,H,D], k/v [B,T,HK,D]; returns (dq, dk, dv) in fp32."""
    B, T, H, D = q.shape
    HK = k.shape[2]
    g = H // HK
    scale = D ** -0.5 if scale is None else scale
    qf, kf, vf = q.float(), k.float().repeat_interleave(g, dim=2), v.float().repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    in_t = (j <= i) & (j > i - window_teacher)
    in_s = (j <= i) & (j > i - window_student)
    lse_t = torch.logsumexp(s.masked_fill(~in_t, float("-inf")), -1)
    lse_s = torch.logsumexp(s.masked_fill(~in_s, float("-inf")), -1)
    p_t = torch.exp(s - lse_t[..., None]).masked_fill(~in_t, 0.0)
    o_t = torch.einsum("bhqk,bkhd->bqhd", p_t, vf)
    o_s = torch.einsum("bhqk,bkhd->bqhd", torch.exp(s - lse_s[..., None]).masked_fill(~in_s, 0.0), vf)
    r = torch.exp(lse_t - lse_s)                                            # [B, H, T]
    do_t, do_s = d_o_t.float(), d_o_s.float()
    do_c = do_t + r.transpose(1, 2).unsqueeze(-1) * do_s
    delta_t = (do_t * o_t).sum(-1).transpose(1, 2)
    delta_c = delta_t + r * (do_s * o_s).sum(-1).transpose(1, 2)
    dp_t = torch.einsum("bqhd,bkhd->bhqk", do_t, vf)
    dp_c = torch.einsum("bqhd,bkhd->bhqk", do_c, vf)
    only_t = in_t & ~in_s
    ds = p_t * (torch.where(in_s, dp_c - delta_c[..., None], torch.zeros_like(dp_c))
                + torch.where(only_t, dp_t - delta_t[..., None], torch.zeros_like(dp_t))) * scale
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf)
    dk = torch.einsum("bhqk,bqhd->bkhd", ds, qf).view(B, T, HK, g, D).sum(3)
    dv = (torch.einsum("bhqk,bqhd->bkhd", p_t * in_s, do_c) + torch.einsum("bhqk,bqhd->bkhd", p_t * only_t, do_t))
    return dq, dk, dv.view(B, T, HK, g, D).sum(3)
