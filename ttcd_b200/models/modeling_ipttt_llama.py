"""IP-TTT behind the HF-Llama interface: Llama configs, Llama parameter names, ``generate``.

The reference ships an inference-only port of IP-TTT written against ``LlamaForCausalLM`` (custom_models/ipttt/
inference.py: ``TTTDynamicCache`` :64-91, the chunk-wise fast-weight MLP :198-310, the decoder layer that carries the
unfinished chunk and the adapted ``down_proj`` across calls :470-545, ``generate`` that insists on that cache and on
batch 1 :1018-1036).  Here the same behaviour runs on this framework's IP-TTT model: a ``LlamaConfig`` (with the
``ttt_*`` extras) is translated to an ``IPTTTConfig``, Llama checkpoints load through a name map, and decoding
carries fast weights through ``FastWeightCache``.  What the port fixes and the training model leaves open:

* the fast-weight target of a block is the residual stream entering it (``ttt_target="layer_input"``);
* the target convolution is the centred 5-tap depthwise one with zero context per chunk, no activation convolution;
* attention is full causal (no window), rotary per the Llama config (plain, YaRN or Llama-3 scaling).
"""
from __future__ import annotations

import re
from typing import Any

import torch

from ..utils.convert import map_hf_key
from .configuration import IPTTTConfig
from .modeling_ipttt import FastWeightCache, IPTTTForCausalLM

_TTT_RULE = re.compile(r"^model\.layers\.(\d+)\.mlp\.(ttt_proj|ttt_conv)\.weight$")
_NATIVE_TO_LLAMA = [
    (re.compile(r"^model\.embeddings\.weight$"), "model.embed_tokens.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.attn\.([qkvo]_proj|[qk]_norm)\.(weight|bias)$"), r"model.layers.\1.self_attn.\2.\3"),
    (re.compile(r"^model\.layers\.(\d+)\.attn_norm\.weight$"), r"model.layers.\1.input_layernorm.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.mlp_norm\.weight$"), r"model.layers.\1.post_attention_layernorm.weight"),
]


class TTTDynamicCache(FastWeightCache):
    """The cache class name of the reference port; key/value windows plus per-layer (unfinished chunk inputs,
    unfinished chunk targets, adapted down_proj)."""


def llama_key_to_native(key: str) -> str | None:
    if _TTT_RULE.match(key):
        return key
    return map_hf_key(key)


def native_key_to_llama(key: str) -> str:
    for pattern, repl in _NATIVE_TO_LLAMA:
        if pattern.match(key):
            return pattern.sub(repl, key)
    return key


def ipttt_config_from_llama(llama_config: Any, **overrides) -> IPTTTConfig:
    """``LlamaConfig`` (object or dict, with optional ``ttt_mode / ttt_layers / ttt_chunk / ttt_lr / ttt_proj``)
    -> ``IPTTTConfig`` with the choices the inference port hard-codes."""
    get = (lambda k, d=None: llama_config.get(k, d)) if isinstance(llama_config, dict) else (
        lambda k, d=None: getattr(llama_config, k, d))
    if get("mlp_bias", False):
        raise NotImplementedError("mlp_bias=True has no counterpart here")
    if get("hidden_act", "silu") not in ("silu", "swish"):
        raise NotImplementedError(f"hidden_act {get('hidden_act')!r}")
    rope_scaling = get("rope_scaling")
    rope_theta = get("rope_theta")
    if rope_theta is None and isinstance(get("rope_parameters"), dict):       # transformers >= 5 layout
        rope_scaling = dict(get("rope_parameters"))
        rope_theta = rope_scaling.pop("rope_theta", 10000.0)
    kw = dict(
        hidden_size=get("hidden_size"), num_hidden_layers=get("num_hidden_layers"), num_heads=get("num_attention_heads"),
        num_kv_heads=get("num_key_value_heads") or get("num_attention_heads"), head_dim=get("head_dim"),
        intermediate_size=get("intermediate_size"), norm_eps=get("rms_norm_eps", 1e-6),
        rope_theta=float(rope_theta if rope_theta is not None else 10000.0), rope_scaling=rope_scaling,
        max_position_embeddings=get("max_position_embeddings", 2048), vocab_size=get("vocab_size"),
        qkv_bias=bool(get("attention_bias", False)), window_size=None,
        tie_word_embeddings=bool(get("tie_word_embeddings", False)), initializer_range=get("initializer_range", 0.02),
        pad_token_id=get("pad_token_id"), bos_token_id=get("bos_token_id", 1), eos_token_id=get("eos_token_id", 2),
        fuse_cross_entropy=False,
        ttt_mode=bool(get("ttt_mode", False)), ttt_layers=list(get("ttt_layers", []) or []),
        ttt_chunk=int(get("ttt_chunk", 8192)), ttt_lr=float(get("ttt_lr", 0.3)), ttt_proj=bool(get("ttt_proj", True)),
        ttt_target="layer_input", ttt_conv=True, ttt_conv_causal=False, ttt_conv_kernel_size=5, ttt_activation_conv=False,
    )
    kw.update(overrides)
    return IPTTTConfig(**kw)


class IPTTTLlamaForCausalLM(IPTTTForCausalLM):
    """``IPTTTForCausalLM`` that speaks Llama: built from a Llama config, loads and writes Llama-named state dicts,
    and generates with fast weights carried across decode steps (batch 1 while fast weights are on, as in the port)."""

    @classmethod
    def from_llama_config(cls, llama_config: Any, **overrides) -> "IPTTTLlamaForCausalLM":
        return cls(ipttt_config_from_llama(llama_config, **overrides))

    def load_llama_state_dict(self, state_dict: dict[str, torch.Tensor], strict: bool = True):
        mapped, unknown = {}, []
        for k, v in state_dict.items():
            if k.endswith("rotary_emb.inv_freq"):
                continue
            nk = llama_key_to_native(k)
            if nk is None:
                unknown.append(k)
            else:
                mapped[nk] = v
        if unknown and strict:
            raise KeyError(f"no counterpart for {unknown[:5]}{' ...' if len(unknown) > 5 else ''}")
        if self.config.tie_word_embeddings and "lm_head.weight" not in mapped and "model.embeddings.weight" in mapped:
            mapped["lm_head.weight"] = mapped["model.embeddings.weight"]
        return self.load_state_dict(mapped, strict=strict)

    def llama_state_dict(self) -> dict[str, torch.Tensor]:
        return {native_key_to_llama(k): v for k, v in self.state_dict().items()}

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor | None = None, past_key_values=None, **kwargs):
        if input_ids is None:
            raise ValueError("input_ids is required")
        if past_key_values is not None and not isinstance(past_key_values, FastWeightCache):
            raise TypeError("past_key_values must be a TTTDynamicCache")
        if self.config.ttt_mode and input_ids.shape[0] != 1:
            raise ValueError("fast-weight inference supports batch size 1 (as the reference port does)")
        kwargs.pop("use_graph", None)
        return super().generate(input_ids, use_graph=False, past_key_values=past_key_values, **kwargs)
