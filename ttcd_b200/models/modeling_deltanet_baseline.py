"""SWA transformer with an extra DeltaNet sub-layer on ``ttt_layers`` during training (model_type
``deltanet_baseline``): the recurrent-memory baseline IP-TTCD is compared against
(custom_models/ipttcd/modeling_deltanet_baseline.py:30-190).

On the selected layers, in training mode only: ``dn_norm`` fuses the attention residual, q/k/v/beta are
projected from its output, the chunked delta rule (q, k L2-normalised) runs per head, ``dn_o_proj``
(zero-initialised, so the model starts as the plain transformer) maps back and ``mlp_norm`` fuses that
residual.  Outside training the sub-layer is skipped, as in the reference.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .base import DecoderForCausalLM, DecoderModel
from .configuration import DeltaNetBaselineConfig
from .layers import GatedMLP, RMSNorm
from .modeling_transformer import build_attention


class DeltaNetBaselineBlock(nn.Module):
    def __init__(self, config: DeltaNetBaselineConfig, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.is_deltanet_layer = bool(config.ttt_mode and layer_idx in set(config.ttt_layers))
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = build_attention(config, layer_idx, with_rope_scaling=False)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = GatedMLP(config.hidden_size, config.resolved_intermediate_size)
        if self.is_deltanet_layer:
            d = config.hidden_size
            self.dn_num_heads = config.num_heads
            self.dn_head_dim = d // config.num_heads
            self.dn_norm = RMSNorm(d, eps=config.norm_eps)
            self.dn_q_proj = nn.Linear(d, d, bias=False)
            self.dn_k_proj = nn.Linear(d, d, bias=False)
            self.dn_v_proj = nn.Linear(d, d, bias=False)
            self.dn_o_proj = nn.Linear(d, d, bias=False)
            self.dn_b_proj = nn.Linear(d, config.num_heads, bias=False)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False, **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        attn_out, _ = self.attn(hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
                                use_cache=use_cache, **kwargs)
        if self.is_deltanet_layer and self.training:
            dn_in, residual = self.dn_norm(attn_out, residual, True)
            b, t, _ = dn_in.shape
            shape = (b, t, self.dn_num_heads, self.dn_head_dim)
            q = ops.linear(dn_in, self.dn_q_proj.weight).view(shape)
            k = ops.linear(dn_in, self.dn_k_proj.weight).view(shape)
            v = ops.linear(dn_in, self.dn_v_proj.weight).view(shape)
            beta = torch.sigmoid(torch.nn.functional.linear(dn_in, self.dn_b_proj.weight))
            o, _ = ops.gated_delta_rule(q, k, v, None, beta, cu_seqlens=kwargs.get("cu_seqlens"))
            attn_out = ops.linear(o.reshape(b, t, -1), self.dn_o_proj.weight)
        hidden_states, residual = self.mlp_norm(attn_out, residual, True)
        return residual + self.mlp(hidden_states)


class _DeltaNetInit:
    def _init_extra(self, module: nn.Module) -> None:
        if isinstance(module, DeltaNetBaselineBlock) and module.is_deltanet_layer:
            w = module.dn_o_proj.weight
            if w.device.type != "meta" and not getattr(w, "_is_hf_initialized", False):
                w.zero_()


class DeltaNetBaselineModel(_DeltaNetInit, DecoderModel):
    config_class = DeltaNetBaselineConfig
    block_class = DeltaNetBaselineBlock
    _no_split_modules = ["DeltaNetBaselineBlock"]


class DeltaNetBaselineForCausalLM(_DeltaNetInit, DecoderForCausalLM):
    config_class = DeltaNetBaselineConfig
    model_class = DeltaNetBaselineModel
    _no_split_modules = ["DeltaNetBaselineBlock"]
