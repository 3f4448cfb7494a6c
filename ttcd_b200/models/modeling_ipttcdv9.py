"""IP-TTCD v9 (model_type ``ipttcdv9``).

On the designated TTT layers attention runs over shared Q/K/V with two windows — teacher
``w_T = window_size`` and student ``w_S = ttt_visible_chunks * ttt_chunk`` — and the chunk-wise
discrepancy between teacher and student MLP features is written into fast weights on
``down_proj`` (custom_models/ipttcd/modeling_ipttcdv9.py:626-714 for the block,
modeling_ipttcdv9_lowcopy_scanfuse.py:36-219 for the grouped scan):

    r = x_in ; h = rmsnorm(x_in)
    q,k,v = heads(Wq h, Wk h, Wv h) ; q,k = headnorm ; q,k = rope
    o_T, o_S = dual_window_attention(q,k,v, w_T, w_S)          one pass over K/V
    a_T, a_S = Wo o_T, Wo o_S
    x, t, r  = rmsnorm(r + a_T), rmsnorm(r + a_S), r + a_T      one fused norm kernel
    z   = swiglu(Wg x, Wu x)        z_hat = conv_S(swiglu(Wg t, Wu t))     z_tgt = conv_T(z)
    P_j = beta_j * ((z_tgt_j - z_hat_j) @ (W_down^T W_p))        beta = sigmoid(t . b_proj)
    W_i = W_down + lr * sum_{j<i} P_j^T z_hat_j ;   y_i = z_out_i W_i^T ;   out = r + y

Unlike the reference, teacher and student rows are stacked so the o_proj and gate/up GEMMs run
once over 2x the rows, and the two attentions are one kernel.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.profiler import record_function

from .. import ops
from .base import DecoderForCausalLM, DecoderModel
from .configuration import IPTTCDv9Config
from .layers import GatedMLP, RMSNorm, WindowKVCache, _cp_state, _tp_state
from .modeling_ipttt import make_depthwise_conv, pad_to_chunks
from .modeling_transformer import build_attention

_STATE_DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32}


class IPTTCDMLP(GatedMLP):
    """SwiGLU MLP whose ``down_proj`` receives chunk-wise fast-weight updates on TTT layers."""

    def __init__(self, config: IPTTCDv9Config, layer_idx: int):
        super().__init__(config.hidden_size, config.resolved_intermediate_size)
        if config.hidden_act != "swish":
            raise ValueError(f"Unsupported hidden_act: {config.hidden_act}")
        self.layer_idx = layer_idx
        self.is_ttt_layer = bool(config.ttt_mode and layer_idx in set(config.ttt_layers))
        self._last_ttt_norm_metrics: dict = {}
        if not self.is_ttt_layer:
            return
        g = lambda name, default: getattr(config, name, default)  # noqa: E731
        self.ttt_chunk = config.ttt_chunk
        self.ttt_lr = float(config.ttt_lr)
        self.ttt_update_every = max(1, int(g("ttt_update_every", 1)))
        self.ttt_weight_renorm = bool(g("ttt_weight_renorm", False))
        self.ttt_norm_log_freq = max(1, int(g("ttt_norm_log_freq", 50)))
        self.ttt_conv_kernel_size = int(g("ttt_conv_kernel_size", 5))
        self.ttt_conv_causal = bool(g("ttt_conv_causal", True))
        self.ttt_output_use_teacher_conv = bool(g("ttt_output_use_teacher_conv", True))
        self.ttt_output_source = str(g("ttt_output_source", "teacher")).lower()
        self.dynamic_lr = bool(config.dynamic_lr)
        self.use_muon = bool(config.use_muon)
        self.ttt_norm_proj_diff = bool(g("ttt_norm_proj_diff", False))
        self.ttt_normalize_student_features = bool(g("ttt_normalize_student_features", True))
        self.ttt_fuse_proj_into_update = bool(g("ttt_fuse_proj_into_update", True))
        self.ttt_force_grouped_scan = bool(g("ttt_force_grouped_scan", False))
        self.ttt_scan_group_size = max(1, int(g("ttt_scan_group_size", 4)))
        self.ttt_scan_state_dtype = str(g("ttt_scan_state_dtype", "compute")).lower()

        self.ttt_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False) if config.ttt_proj else None
        if self.ttt_proj is not None:
            self.ttt_proj._is_ttt_proj = True
        k, causal = self.ttt_conv_kernel_size, self.ttt_conv_causal
        self.ttt_teacher_conv = make_depthwise_conv(self.intermediate_size, k, causal) if g("ttt_teacher_conv", False) else None
        self.ttt_student_conv = make_depthwise_conv(self.intermediate_size, k, causal) if g("ttt_student_conv", False) else None
        if self.ttt_teacher_conv is not None:
            self.ttt_teacher_conv._ttt_conv_role = "teacher"
        if self.ttt_student_conv is not None:
            self.ttt_student_conv._ttt_conv_role = "student"
        if self.dynamic_lr:
            # 1-D so that it shards evenly along dim 0 (a [1, d_h] Linear would not).
            self.b_proj = nn.Parameter(torch.empty(self.hidden_size))

    # ----------------------------------------------------------------------------------
    def _conv(self, x, conv):
        return x if conv is None else ops.dwconv_chunked(x, conv.weight, self.ttt_conv_causal)

    def _state_dtype(self, compute_dtype):
        return _STATE_DTYPES.get(self.ttt_scan_state_dtype, compute_dtype)

    def forward(self, x, t=None, **_):
        """x: teacher-side MLP input [b,S,d_h]; t: student-side input or None (plain MLP)."""
        if t is None or not self.is_ttt_layer:
            return super().forward(x)
        tag = f"ipttcdv9_scanfuse.mlp.{{}}.layer{self.layer_idx}"
        tp = _tp_state()
        b, seq_len, _ = x.shape
        if tp is not None:
            # token-sharded inputs: each stream is all-gathered inside its own gate/up GEMM
            if self.ttt_normalize_student_features or self.ttt_norm_proj_diff or self.ttt_weight_renorm or self.use_muon:
                raise NotImplementedError("tensor parallelism: feature normalisation / renorm over the sharded d_i")
            z, z_hat = self.features(x), self.features(t)
            seq_len = z.shape[1]
            if seq_len % self.ttt_chunk:
                raise ValueError("tensor parallelism needs the sequence length to be a multiple of ttt_chunk")
        else:
            with record_function(tag.format("teacher_gateup")):
                # teacher and student rows share the gate/up weights: one GEMM over 2x rows
                feats = self.features(torch.cat([x, t], dim=0))
            z, z_hat = feats[:b], feats[b:]
        with record_function(tag.format("teacher_ttt_prepare")):
            z_p = pad_to_chunks(z, self.ttt_chunk)
            z_tgt = self._conv(z_p, self.ttt_teacher_conv)
            teacher_out = z_tgt if self.ttt_output_use_teacher_conv else z_p
        with record_function(tag.format("student_gateup")):
            z_hat_p = self._conv(pad_to_chunks(z_hat, self.ttt_chunk), self.ttt_student_conv)
        z_out = teacher_out if self.ttt_output_source == "teacher" else z_hat_p
        T, C = z_p.shape[1], z_p.shape[2]
        beta = None
        if self.dynamic_lr:
            with record_function(tag.format("student_beta")):
                if tp is not None:
                    from ..parallel.tensor import gather_rows
                    gate = gather_rows(torch.sigmoid(t[0] @ self.b_proj.to(t.dtype)), tp)        # [S]
                    beta = gate.view(1, T, C, 1)
                else:
                    beta = torch.sigmoid(pad_to_chunks(t, self.ttt_chunk) @ self.b_proj.to(t.dtype)).unsqueeze(-1)

        compute_dtype = z_p.dtype
        w_down = self.down_proj.weight
        fold = self.ttt_fuse_proj_into_update and self.ttt_proj is not None and not self.ttt_norm_proj_diff
        with record_function(tag.format("fuse_base_proj")):
            w_down_t = w_down.to(compute_dtype).transpose(0, 1)
            w_update_t = ops.matmul(w_down_t, self.ttt_proj.weight.to(compute_dtype)) if fold else w_down_t
        post = None if (fold or self.ttt_proj is None) else self.ttt_proj.weight

        if self.ttt_weight_renorm or self.use_muon:
            y = self._scan_general(z_out, z_tgt, z_hat_p, beta, w_down, w_update_t, post)
        else:
            with record_function(tag.format("scanfused_output")):
                y, last = ops.ttt_scan(
                    z_out, z_tgt, z_hat_p, beta, w_down, w_update_t, lr=self.ttt_lr,
                    update_every=min(T, self.ttt_update_every), state_dtype=self._state_dtype(compute_dtype),
                    normalize_student=self.ttt_normalize_student_features, norm_proj_diff=self.ttt_norm_proj_diff,
                    post_proj=post, return_last_dw_norm=True, cp=_cp_state() if self.training else None,
                    proj_reduce=None if tp is None else (lambda v: _tp_sum(v, tp)), key=("ttt_scan", self.layer_idx))
            if self.training and last is not None:
                self._last_delta_w_norm_t = last  # device scalar; read lazily, no host sync here
        y = y.reshape(b, T * C, -1)[:, :seq_len]
        if tp is not None:
            from ..parallel.tensor import scatter_rows_sum
            return scatter_rows_sum(y[0], tp).unsqueeze(0)       # partial sums over d_i shards -> token shard
        return y

    @property
    def _last_delta_w_norm(self):
        v = getattr(self, "_last_delta_w_norm_t", None)
        return None if v is None else float(v)

    def _scan_general(self, z_out, z_tgt, z_hat, beta, w_down, w_update_t, post):
        """Grouped scan with the optional per-update Newton-Schulz and Frobenius renorm
        (custom_models/ipttcd/modeling_ipttcdv9.py:443-527); fp32 state, PyTorch ops."""
        b, T, C, _ = z_out.shape
        cd = z_out.dtype
        w_base = w_down.float().unsqueeze(0).expand(b, -1, -1)
        target_norm = w_base.flatten(1).norm(dim=-1).view(b, 1, 1)

        def renorm(w):
            cur = w.flatten(-2).norm(dim=-1, keepdim=True).unsqueeze(-1).clamp_min(1e-6)
            return w * (target_norm.view(b, *([1] * (w.dim() - 1))) / cur)

        w_cur = w_base
        group = min(T, self.ttt_update_every)
        outs = []
        for gs in range(0, T, group):
            ge = min(gs + group, T)
            upd_end = min(ge, T - 1)
            k_upd = upd_end - gs
            kg = ge - gs
            w_run = w_cur.unsqueeze(1).expand(-1, kg, -1, -1).clone()
            if k_upd > 0:
                zh = z_hat[:, gs:upd_end]
                proj = torch.matmul(z_tgt[:, gs:upd_end] - zh, w_update_t.to(cd))
                if self.ttt_norm_proj_diff:
                    proj = F.normalize(proj, p=2, dim=-1, eps=1e-6)
                if self.ttt_normalize_student_features:
                    zh = F.normalize(zh, p=2, dim=-1, eps=1e-6)
                if beta is not None:
                    proj = proj * beta[:, gs:upd_end]
                if post is not None:
                    proj = torch.matmul(proj, post.to(cd))
                d_w = torch.matmul(proj.float().transpose(-1, -2), zh.float())
                if self.use_muon:
                    shp = d_w.shape
                    d_w = ops.newton_schulz(d_w.reshape(-1, shp[-2], shp[-1])).reshape(shp).float()
                cs = self.ttt_lr * torch.cumsum(d_w, dim=1)
                fill = min(kg, k_upd + 1)
                if fill > 1:
                    w_run[:, 1:fill] = w_run[:, 1:fill] + cs[:, :fill - 1]
                if fill < kg:
                    w_run[:, fill:] = w_run[:, fill:] + cs[:, -1:]
                if self.ttt_weight_renorm:
                    w_run = renorm(w_run)
                    w_cur = renorm(w_cur + cs[:, -1])
                else:
                    w_cur = w_cur + cs[:, -1]
            outs.append(torch.matmul(z_out[:, gs:ge], w_run.to(cd).transpose(-1, -2)))
        return torch.cat(outs, dim=1)


def _tp_sum(v, tp):
    from ..parallel.tensor import sum_over_group
    return sum_over_group(v, tp)


def _fast_prefill_ok(block, hidden_states, attention_mask, kwargs) -> bool:
    if os.environ.get("IPTTCD_DISABLE_FAST_PREFILL") == "1":
        return False
    if hidden_states.shape[1] < block.ttt_chunk or kwargs.get("cu_seqlens") is not None:
        return False
    return attention_mask is None or bool(attention_mask.all())


class IPTTCDBlock(nn.Module):
    def __init__(self, config: IPTTCDv9Config, layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.is_ttt_layer = bool(config.ttt_mode and layer_idx in set(config.ttt_layers))
        if self.is_ttt_layer:
            self.ttt_chunk = config.ttt_chunk
            self.ttt_visible_chunks = config.ttt_visible_chunks
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        # rope_scaling is deliberately not forwarded (reference behaviour for this family).
        self.attn = build_attention(config, layer_idx, with_rope_scaling=False)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = IPTTCDMLP(config, layer_idx)

    @property
    def student_window(self) -> int:
        return self.ttt_visible_chunks * self.ttt_chunk

    def _dual_path(self, hidden_states, residual, past_key_values, kwargs):
        """Shared-QKV teacher+student attention; returns (teacher_attn_out, student_attn_out)."""
        attn = self.attn
        offset = 0
        cp = _cp_state() if past_key_values is None else None
        if cp is not None:
            offset = cp.position_offset(hidden_states.shape[1])
        if past_key_values is not None:
            offset = past_key_values.get_seq_length(attn.layer_idx)
        cu = kwargs.get("cu_seqlens")
        positions = kwargs.get("positions")
        q, k, v = attn.project_qkv(hidden_states, offset, positions=positions)
        if past_key_values is not None:
            had_content = offset > 0
            k_all, v_all = past_key_values.update(k, v, attn.layer_idx, attn.window_size)
            if had_content:
                k, v = k_all, v_all
        if cp is not None:
            from ..parallel import context as _context
            o_t, o_s = _context.dual_window_attention(q, k, v, attn.window_size, self.student_window, None, attn.layer_idx)
        else:
            o_t, o_s = ops.dual_window_attention(q, k, v, attn.window_size, self.student_window, cu_seqlens=cu)
        if _tp_state() is not None:     # row-parallel o_proj reduce-scatters over tokens: one stream per call
            return attn.finish(o_t, hidden_states), attn.finish(o_s, hidden_states)
        b = hidden_states.shape[0]
        both = attn.finish(torch.cat([o_t, o_s], dim=0), torch.cat([hidden_states, hidden_states], dim=0)
                           if attn.use_output_gate else hidden_states)
        return both[:b], both[b:]

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False, **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        student = None
        dual = self.is_ttt_layer and (
            self.training or _fast_prefill_ok(self, hidden_states, attention_mask, kwargs))
        if dual:
            a_t, a_s = self._dual_path(hidden_states, residual, None if self.training else past_key_values, kwargs)
            hidden_states, student, residual = ops.rmsnorm_dual(a_t, a_s, residual, self.mlp_norm.weight,
                                                                self.mlp_norm.eps)
        else:
            a_t, _ = self.attn(hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
                               use_cache=use_cache, **kwargs)
            if self.is_ttt_layer and hidden_states.shape[1] >= self.ttt_chunk:
                # padded / packed prefill: student attention computed separately, no cache
                q, k, v = self.attn.project_qkv(hidden_states, 0, positions=kwargs.get("positions"))
                o_s = ops.attention(q, k, v, window=self.student_window, cu_seqlens=kwargs.get("cu_seqlens"))
                a_s = self.attn.finish(o_s, hidden_states)
                student = self.mlp_norm(a_s, residual, False)
            hidden_states, residual = self.mlp_norm(a_t, residual, True)
        hidden_states = self.mlp(hidden_states, t=student if self.is_ttt_layer else None)
        return residual + hidden_states


class _IPTTCDInit:
    def _init_extra(self, module: nn.Module) -> None:
        cfg = self.config
        std = cfg.initializer_range
        if isinstance(module, nn.Linear) and getattr(module, "_is_ttt_proj", False):
            w = module.weight
            if w.device.type == "meta" or getattr(w, "_is_hf_initialized", False):
                return
            kind = getattr(cfg, "ttt_proj_init", "diagonal")
            n = min(w.shape)
            idx = torch.arange(n, device=w.device)
            if kind == "diagonal":
                w.zero_()
                w[idx, idx] = std
            elif kind == "diagonal_gaussian":
                w.zero_()
                w[idx, idx] = torch.randn(n, device=w.device, dtype=w.dtype) * std
            elif kind == "zero":
                w.zero_()
        if isinstance(module, nn.Conv1d) and getattr(module, "_is_ttt_conv", False):
            w = module.weight
            if w.device.type == "meta" or getattr(w, "_is_hf_initialized", False):
                return
            role = getattr(module, "_ttt_conv_role", "ttt")
            kind = getattr(cfg, f"ttt_{role}_conv_init", getattr(cfg, "ttt_conv_init", "zero"))
            if kind == "identity":
                tap = module.kernel_size[0] - 1 if module.padding[0] == 0 else module.kernel_size[0] // 2
                w.zero_()
                w[:, 0, tap] = 1.0
            elif kind == "zero":
                w.zero_()
            elif kind != "random":
                raise ValueError(f"Unsupported TTT conv init {kind!r} for role {role!r}")
        if isinstance(module, IPTTCDMLP) and module.is_ttt_layer and module.dynamic_lr:
            if module.b_proj.device.type != "meta" and not getattr(module.b_proj, "_is_hf_initialized", False):
                module.b_proj.normal_(mean=0.0, std=std)


class IPTTCDModel(_IPTTCDInit, DecoderModel):
    config_class = IPTTCDv9Config
    block_class = IPTTCDBlock
    _no_split_modules = ["IPTTCDBlock"]


class IPTTCDForCausalLM(_IPTTCDInit, DecoderForCausalLM):
    config_class = IPTTCDv9Config
    model_class = IPTTCDModel
    _no_split_modules = ["IPTTCDBlock"]

    def get_ttt_norm_metrics(self) -> dict:
        """Per-layer and aggregate ``ttt_norm/*`` metrics recorded by the last forward."""
        per_layer, rows = {}, []
        for layer in self.model.layers:
            m = getattr(layer.mlp, "_last_ttt_norm_metrics", None)
            if m:
                rows.append(m)
                for k, v in m.items():
                    per_layer[f"ttt_norm/layer_{layer.layer_idx}/{k}"] = v
        if not rows:
            return {}
        out = dict(per_layer)
        for key in ("z_hat_avg_norm", "proj_diff_avg_norm", "d_w_avg_norm"):
            vals = [m[key] for m in rows if key in m]
            if vals:
                out[f"ttt_norm/{key}"] = sum(vals) / len(vals)
        for key in ("z_hat_max_norm", "proj_diff_max_norm", "d_w_max_norm"):
            vals = [m[key] for m in rows if key in m]
            if vals:
                out[f"ttt_norm/{key}"] = max(vals)
        return out


IPTTCDv9Model = IPTTCDModel
IPTTCDv9ForCausalLM = IPTTCDForCausalLM
