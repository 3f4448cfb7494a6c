"""Shared decoder scaffolding: weight init, the layer loop, the LM head with fused losses, decoding.

Mirrors the behaviour of the reference's model classes
(fla/models/transformer/modeling_transformer.py:124-389 and
custom_models/ipttcd/modeling_ipttcdv9.py:999-1273): labels are shifted inside the
model, ``logits_to_keep=0`` keeps every position, with ``fuse_linear_cross_entropy``
no logits tensor is produced, and tied embeddings share one parameter.
"""
from __future__ import annotations

import os

import math
from typing import Any

import torch
import torch.nn as nn
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast
from transformers.modeling_utils import PreTrainedModel

from .. import ops
from .layers import RMSNorm, WindowKVCache

IGNORE_INDEX = -100


# TTCD_NVTX=1: one NVTX range per block (forward) for timeline tools; off by default (a push/pop per layer).
_NVTX = os.environ.get("TTCD_NVTX", "0") == "1"

class FusedLinearCrossEntropyLoss(nn.Module):
    """criterion(hidden, labels, weight, bias): CE without materialising [tokens, vocab] logits."""

    ignore_index = IGNORE_INDEX

    def __init__(self, num_chunks: int = 8, use_l2warp: bool = False, l2_penalty_factor: float = 1e-4):
        super().__init__()
        self.num_chunks = num_chunks
        self.use_l2warp = use_l2warp
        self.l2_penalty_factor = l2_penalty_factor

    def forward(self, hidden, labels, weight, bias=None):
        return ops.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1), weight, bias,
                                        self.ignore_index, self.num_chunks,
                                        self.l2_penalty_factor if self.use_l2warp else 0.0)


class FusedCrossEntropyLoss(nn.Module):
    ignore_index = IGNORE_INDEX

    def __init__(self, label_smoothing: float = 0.0, lse_square_scale: float = 0.0, **_):
        super().__init__()
        self.label_smoothing = label_smoothing
        self.lse_square_scale = lse_square_scale

    def forward(self, logits, labels):
        return ops.cross_entropy(logits, labels, self.ignore_index, self.label_smoothing, self.lse_square_scale)


class _L2Warp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, loss, logits):
        ctx.save_for_backward(logits)
        return loss

    @staticmethod
    def backward(ctx, grad):
        (logits,) = ctx.saved_tensors
        return grad, ops.reference.l2_warp_grad(logits) * grad


class DecoderPreTrainedModel(PreTrainedModel):
    """Init rules: N(0, initializer_range) for Linear/Conv1d/Embedding, ones for norms."""

    base_model_prefix = "model"
    supports_gradient_checkpointing = True
    _skip_keys_device_placement = "past_key_values"

    def _init_weights(self, module: nn.Module, rescale_prenorm_residual: bool = False,
                      num_residuals_per_layer: int = 2):
        std = self.config.initializer_range

        def fresh(t) -> bool:
            """True for tensors that still need initialising (HF marks checkpoint-loaded tensors)."""
            return t is not None and t.device.type != "meta" and not getattr(t, "_is_hf_initialized", False)

        with torch.no_grad():
            if isinstance(module, (nn.Linear, nn.Conv1d)):
                if fresh(module.weight):
                    module.weight.normal_(mean=0.0, std=std)
                if fresh(module.bias):
                    module.bias.zero_()
            elif isinstance(module, nn.Embedding):
                if fresh(module.weight):
                    module.weight.normal_(mean=0.0, std=std)
            elif isinstance(module, RMSNorm):
                if fresh(module.weight):
                    module.weight.fill_(1.0)
            if rescale_prenorm_residual:
                for name in ("o_proj", "down_proj"):
                    p = getattr(module, name, None)
                    if isinstance(p, nn.Linear) and p.weight.device.type != "meta":
                        nn.init.kaiming_uniform_(p.weight, a=math.sqrt(5))
                        p.weight /= math.sqrt(num_residuals_per_layer * self.config.num_hidden_layers)
            self._init_extra(module)

    def _init_extra(self, module: nn.Module) -> None:  # family hooks
        pass

    def reinitialize(self) -> None:
        """Re-run every module's initialiser (used after materialising meta-device params)."""
        for m in self.modules():
            self._init_weights(m)
        self.tie_weights()


class DecoderModel(DecoderPreTrainedModel):
    """Embedding + block stack + final norm.  Subclasses set ``block_class``."""

    block_class: type[nn.Module] = None

    def __init__(self, config):
        super().__init__(config)
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList([self.block_class(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.gradient_checkpointing = False
        self.post_init()

    def get_input_embeddings(self):
        return self.embeddings

    def set_input_embeddings(self, value):
        self.embeddings = value

    def _block_kwargs(self, input_ids, inputs_embeds, kwargs) -> dict[str, Any]:
        return kwargs

    # which blocks are recomputed in backward: "full" (all), "everyN", "ttt" (fast-weight blocks only), "op" (all
    # blocks, but the GEMM / attention launches are not repeated: ops/selective.py)
    checkpoint_policy: str = "full"

    def _checkpoint_layer(self, layer) -> bool:
        policy = self.checkpoint_policy
        if policy in ("full", "op"):
            return True
        if policy == "ttt":
            return bool(getattr(layer, "is_ttt_layer", False))
        if policy.startswith("every"):
            n = max(1, int(policy[5:] or 1))
            return getattr(layer, "layer_idx", 0) % n == 0
        return False

    def forward(self, input_ids=None, attention_mask=None, past_key_values=None, inputs_embeds=None,
                use_cache=None, output_attentions=None, output_hidden_states=None, return_dict=None,
                **kwargs):
        cfg = self.config
        output_hidden_states = bool(output_hidden_states) if output_hidden_states is not None else bool(
            getattr(cfg, "output_hidden_states", False))
        use_cache = use_cache if use_cache is not None else (cfg.use_cache if not self.training else False)
        return_dict = True if return_dict is None else return_dict
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("Specify exactly one of input_ids / inputs_embeds")
        if use_cache and not isinstance(past_key_values, WindowKVCache):
            past_key_values = getattr(self, "cache_class", WindowKVCache)()
        if not use_cache:
            past_key_values = past_key_values if isinstance(past_key_values, WindowKVCache) else None
        if inputs_embeds is None:
            inputs_embeds = self.embeddings(input_ids)
        kwargs = self._block_kwargs(input_ids, inputs_embeds, kwargs)

        hidden_states = inputs_embeds
        all_hidden = () if output_hidden_states else None
        nvtx = _NVTX and hidden_states.is_cuda
        for i, layer in enumerate(self.layers):
            if output_hidden_states:
                all_hidden += (hidden_states,)
            if nvtx:
                torch.cuda.nvtx.range_push(f"layer{i}")
            if self.gradient_checkpointing and self.training and self._checkpoint_layer(layer):
                fn = layer
                if self.checkpoint_policy == "op":
                    from ..ops.selective import OpCache

                    def fn(*a, _layer=layer, _cache=OpCache(), **kw):
                        with _cache.scope():
                            return _layer(*a, **kw)
                hidden_states = torch.utils.checkpoint.checkpoint(
                    fn, hidden_states, attention_mask, None, False, use_reentrant=False, **kwargs)
            else:
                hidden_states = layer(hidden_states, attention_mask, past_key_values, use_cache, **kwargs)
            if nvtx:
                torch.cuda.nvtx.range_pop()
        hidden_states = self.norm(hidden_states)
        if output_hidden_states:
            all_hidden += (hidden_states,)
        next_cache = past_key_values if use_cache else None
        if not return_dict:
            return tuple(v for v in (hidden_states, next_cache, all_hidden) if v is not None)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=next_cache,
                                       hidden_states=all_hidden, attentions=None)


class DecoderForCausalLM(DecoderPreTrainedModel):
    """LM head + loss on top of a DecoderModel subclass (``model_class``)."""

    model_class: type[DecoderModel] = None
    _tied_weights_keys = {"lm_head.weight": "model.embeddings.weight"}

    def __init__(self, config):
        super().__init__(config)
        self.model = self.model_class(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.criterion = None
        self.post_init()

    # HF accessors
    def get_input_embeddings(self):
        return self.model.embeddings

    def set_input_embeddings(self, value):
        self.model.embeddings = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def get_decoder(self):
        return self.model

    def set_decoder(self, decoder):
        self.model = decoder

    def tie_weights(self, *args, **kwargs):
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embeddings.weight
        return None

    def _default_criterion(self):
        cfg = self.config
        if cfg.fuse_linear_cross_entropy:
            return FusedLinearCrossEntropyLoss(use_l2warp=cfg.use_l2warp)
        if cfg.fuse_cross_entropy:
            return FusedCrossEntropyLoss()
        return nn.CrossEntropyLoss()

    def forward(self, input_ids=None, attention_mask=None, past_key_values=None, inputs_embeds=None,
                labels=None, use_cache=None, output_attentions=None, output_hidden_states=None,
                return_dict=None, logits_to_keep: int | None = 0, **kwargs):
        return_dict = True if return_dict is None else return_dict
        kwargs.pop("num_logits_to_keep", None)
        shift_labels = kwargs.pop("shift_labels", True)   # False: the caller already aligned labels to positions
        outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, past_key_values=past_key_values,
                             inputs_embeds=inputs_embeds, use_cache=use_cache,
                             output_hidden_states=output_hidden_states, return_dict=True, **kwargs)
        hidden_states = outputs.last_hidden_state
        fuse_lce = bool(self.config.fuse_linear_cross_entropy) and labels is not None
        logits = None
        if not fuse_lce:
            keep = logits_to_keep or 0
            logits = ops.linear(hidden_states[:, -keep:], self.lm_head.weight, self.lm_head.bias)

        loss = None
        if labels is not None:
            criterion = self.criterion if getattr(self, "criterion", None) is not None else self._default_criterion()
            ignore = getattr(criterion, "ignore_index", IGNORE_INDEX)
            labels = labels.to(hidden_states.device)
            if shift_labels:
                labels = torch.cat((labels[..., 1:], torch.full_like(labels[:, :1], ignore)), dim=1)
            if fuse_lce:
                loss = criterion(hidden_states, labels, self.lm_head.weight, self.lm_head.bias)
            else:
                loss = criterion(logits.view(labels.numel(), -1), labels.view(-1))
                if self.config.use_l2warp:
                    loss = _L2Warp.apply(loss, logits)

        if not return_dict:
            out = (logits,) + tuple(v for v in (outputs.past_key_values, outputs.hidden_states) if v is not None)
            return ((loss,) + out) if loss is not None else out
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values,
                                      hidden_states=outputs.hidden_states, attentions=None)

    # -- decoding --------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, do_sample: bool = False,
                 temperature: float = 1.0, top_k: int | None = None, top_p: float | None = None,
                 eos_token_id: int | list[int] | None = None, attention_mask=None, use_graph: bool = True,
                 past_key_values=None, **_):
        """Prefill once (TTT layers run their dual path), then decode token by token from the cache.

        Mirrors the reference's behaviour: fast weights are built during prefill only and are not
        carried into single-token decode steps (custom_models/ipttcd/modeling_ipttcdv9.py:794-850).
        Greedy decoding on the native path replays one captured CUDA graph per token (models/decoding.py);
        ``use_graph=False`` keeps the eager loop.
        """
        eos = set(eos_token_id if isinstance(eos_token_id, (list, tuple)) else
                  ([eos_token_id] if eos_token_id is not None else []))
        cache = past_key_values if past_key_values is not None else getattr(self.model, "cache_class", WindowKVCache)()
        out = self(input_ids=input_ids, attention_mask=attention_mask, past_key_values=cache,
                   use_cache=True, logits_to_keep=1)
        tokens = input_ids
        finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        from . import decoding
        if (use_graph and max_new_tokens > 1 and not self.training and type(cache) is WindowKVCache
                and decoding.graph_decoding_supported(self, input_ids, attention_mask, do_sample)):
            # greedy decoding on the native path: the step is captured once and replayed per token
            first = out.logits[:, -1].float().argmax(-1, keepdim=True)
            if eos and bool(torch.isin(first.squeeze(1), torch.tensor(sorted(eos), device=first.device)).all()):
                return torch.cat([tokens, first], dim=1)
            rest = decoding.decoder_for(self, cache, max_new_tokens - 1).run(first, max_new_tokens - 1, eos)
            return torch.cat([tokens, first, rest], dim=1)
        for _step in range(max_new_tokens):
            logits = out.logits[:, -1].float()
            if do_sample:
                logits = logits / max(temperature, 1e-6)
                if top_k:
                    kth = torch.topk(logits, top_k).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                if top_p is not None and top_p < 1.0:
                    sorted_logits, idx = torch.sort(logits, descending=True)
                    cum = torch.softmax(sorted_logits, -1).cumsum(-1)
                    drop = cum - torch.softmax(sorted_logits, -1) > top_p
                    sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
                    logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, sorted_logits)
                nxt = torch.multinomial(torch.softmax(logits, -1), 1)
            else:
                nxt = logits.argmax(-1, keepdim=True)
            tokens = torch.cat([tokens, nxt], dim=1)
            if eos:
                finished |= torch.isin(nxt.squeeze(1), torch.tensor(sorted(eos), device=nxt.device))
                if bool(finished.all()):
                    break
            if attention_mask is not None:
                attention_mask = torch.cat([attention_mask, attention_mask.new_ones(attention_mask.shape[0], 1)], 1)
            out = self(input_ids=nxt, attention_mask=attention_mask, past_key_values=cache, use_cache=True,
                       logits_to_keep=1)
        return tokens
