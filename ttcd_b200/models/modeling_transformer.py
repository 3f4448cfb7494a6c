"""Sliding-window transformer baseline (model_type ``transformer``).

Pre-norm blocks with the fused ``rmsnorm(x + residual)`` pattern and a SwiGLU MLP
(fla/models/transformer/modeling_transformer.py:43-122).  ``rope_scaling`` (YaRN)
is honoured here, as in the reference, and only here.
"""
from __future__ import annotations

import torch.nn as nn

from .base import DecoderForCausalLM, DecoderModel
from .configuration import TransformerConfig
from .layers import Attention, GatedMLP, RMSNorm


def build_attention(config, layer_idx: int, with_rope_scaling: bool) -> Attention:
    return Attention(
        hidden_size=config.hidden_size,
        num_heads=config.num_heads,
        num_kv_heads=config.num_kv_heads,
        head_dim=getattr(config, "head_dim", None),
        qkv_bias=config.qkv_bias,
        qk_norm=config.qk_norm,
        window_size=config.window_size,
        rope_theta=config.rope_theta,
        max_position_embeddings=config.max_position_embeddings,
        layer_idx=layer_idx,
        use_output_gate=config.use_output_gate,
        gate_fn=config.gate_fn,
        elementwise_affine=config.elementwise_affine,
        norm_eps=config.norm_eps,
        rope_scaling=getattr(config, "rope_scaling", None) if with_rope_scaling else None,
        use_l2_softmax=bool(getattr(config, "use_l2_softmax", False)),
    )


class TransformerBlock(nn.Module):
    def __init__(self, config: TransformerConfig, layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = build_attention(config, layer_idx, with_rope_scaling=True)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = GatedMLP(config.hidden_size, config.resolved_intermediate_size)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False, **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        hidden_states, _ = self.attn(hidden_states, attention_mask=attention_mask,
                                     past_key_values=past_key_values, use_cache=use_cache, **kwargs)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)
        hidden_states = self.mlp(hidden_states)
        return residual + hidden_states


class TransformerModel(DecoderModel):
    config_class = TransformerConfig
    block_class = TransformerBlock
    _no_split_modules = ["TransformerBlock"]


class TransformerForCausalLM(DecoderForCausalLM):
    config_class = TransformerConfig
    model_class = TransformerModel
    _no_split_modules = ["TransformerBlock"]
