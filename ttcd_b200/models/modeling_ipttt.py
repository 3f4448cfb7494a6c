"""IP-TTT (model_type ``ipttt``): single attention; the fast-weight update of ``down_proj`` is
driven by the MLP-input hidden state (or the input embedding) of each chunk.

Math (custom_models/ipttt/modeling_ipttt.py:137-180), per batch row with chunks j of C tokens:

    h    = swiglu(W_g x, W_u x)                       [T, C, d_i]  (optionally conv'd per chunk)
    tgt  = conv(t)                                    [T, C, d_h]
    dW_j = (tgt_j W_p)^T h_j                          [d_h, d_i]   j = 0..T-2  (W_p untransposed)
    W_i  = W_down + lr * sum_{j<i} dW_j
    y_i  = h_i W_i^T

which is the grouped fast-weight scan with P_j = tgt_j W_p, student features h and one group.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .base import DecoderForCausalLM, DecoderModel
from .configuration import IPTTTConfig
from .layers import WindowKVCache, GatedMLP, RMSNorm
from .modeling_transformer import build_attention


def pad_to_chunks(x: torch.Tensor, chunk: int) -> torch.Tensor:
    """[b, S, d] -> [b, T, chunk, d], zero padded at the end."""
    rem = x.shape[1] % chunk
    if rem:
        x = F.pad(x, (0, 0, 0, chunk - rem))
    return x.view(x.shape[0], -1, chunk, x.shape[-1])


def make_depthwise_conv(channels: int, kernel_size: int, causal: bool) -> nn.Conv1d:
    conv = nn.Conv1d(channels, channels, kernel_size=kernel_size, padding=0 if causal else kernel_size // 2,
                     groups=channels, bias=False)
    conv._is_ttt_conv = True
    return conv


class IPTTTMLP(GatedMLP):
    def __init__(self, config: IPTTTConfig, layer_idx: int):
        super().__init__(config.hidden_size, config.resolved_intermediate_size)
        self.layer_idx = layer_idx
        self.is_ttt_layer = bool(config.ttt_mode and layer_idx in set(config.ttt_layers))
        if not self.is_ttt_layer:
            return
        self.ttt_chunk = config.ttt_chunk
        self.ttt_lr = float(config.ttt_lr)
        self.ttt_conv_causal = bool(config.ttt_conv_causal)
        k = int(config.ttt_conv_kernel_size)
        self.ttt_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False) if config.ttt_proj else None
        if self.ttt_proj is not None:
            self.ttt_proj._is_ttt_proj = True
        self.ttt_conv = make_depthwise_conv(self.hidden_size, k, self.ttt_conv_causal) if config.ttt_conv else None
        self.ttt_activation_conv = (
            make_depthwise_conv(self.intermediate_size, k, self.ttt_conv_causal) if config.ttt_activation_conv else None
        )

    def forward(self, x, t=None, **_):
        if t is None or not self.is_ttt_layer:
            return super().forward(x)
        seq_len = x.shape[1]
        h = pad_to_chunks(self.features(x), self.ttt_chunk)
        tgt = pad_to_chunks(t, self.ttt_chunk)
        if self.ttt_conv is not None:
            tgt = ops.dwconv_chunked(tgt, self.ttt_conv.weight, self.ttt_conv_causal)
        if self.ttt_activation_conv is not None:
            h = ops.dwconv_chunked(h, self.ttt_activation_conv.weight, self.ttt_conv_causal)
        b, T, C, _ = h.shape
        if T == 1:
            y = ops.linear(h, self.down_proj.weight)
        else:
            p = tgt if self.ttt_proj is None else ops.matmul(tgt, self.ttt_proj.weight)
            y, last = _ipttt_scan(p, h, self.down_proj.weight, self.ttt_lr)
            if self.training:
                self._last_delta_w_norm_t = last
        return y.reshape(b, T * C, -1)[:, :seq_len]

    @property
    def _last_delta_w_norm(self):
        v = getattr(self, "_last_delta_w_norm_t", None)
        return None if v is None else float(v)

    def forward_online(self, x, t, past_w=None):
        """Incremental inference (custom_models/ipttt/inference.py:248-310): chunk by chunk, output with the
        current fast weight, then update it from every COMPLETE chunk.  Returns ``(y, present_w)`` with
        ``present_w`` [b, d_h, d_i] to carry into the next call."""
        b, seq_len, _ = x.shape
        h = self.features(x)
        w = self.down_proj.weight.to(h.dtype).expand(b, -1, -1) if past_w is None else past_w
        if t is None or not self.is_ttt_layer or seq_len < self.ttt_chunk:
            return torch.matmul(h, w.transpose(-1, -2)), w
        hp, tgt = pad_to_chunks(h, self.ttt_chunk), pad_to_chunks(t, self.ttt_chunk)
        if self.ttt_conv is not None:
            tgt = ops.dwconv_chunked(tgt, self.ttt_conv.weight, self.ttt_conv_causal)
        if self.ttt_activation_conv is not None:
            hp = ops.dwconv_chunked(hp, self.ttt_activation_conv.weight, self.ttt_conv_causal)
        p = tgt if self.ttt_proj is None else torch.matmul(tgt, self.ttt_proj.weight.to(tgt.dtype))
        n_chunks = hp.shape[1]
        complete = seq_len // self.ttt_chunk
        ys = []
        for i in range(n_chunks):
            ys.append(torch.matmul(hp[:, i], w.transpose(-1, -2)))
            if i < complete:
                w = w + self.ttt_lr * torch.matmul(p[:, i].transpose(-1, -2), hp[:, i])
        return torch.cat(ys, dim=1)[:, :seq_len], w


class FastWeightCache(WindowKVCache):
    """KV cache that also carries, per TTT layer, the adapted ``down_proj`` weight and the MLP inputs /
    targets of the last incomplete chunk (custom_models/ipttt/inference.py:64-79, 505-538), so fast weights
    persist across incremental ``forward`` calls and decode steps."""

    def __init__(self):
        super().__init__()
        self.ttt_states: dict[int, tuple] = {}

    def ttt_get(self, layer_idx: int):
        return self.ttt_states.get(layer_idx, (None, None, None))

    def ttt_update(self, state: tuple, layer_idx: int) -> None:
        self.ttt_states[layer_idx] = state

    def reorder(self, beam_idx: torch.Tensor):
        super().reorder(beam_idx)
        for i, (h, t, w) in self.ttt_states.items():
            sel = lambda v: None if v is None else v.index_select(0, beam_idx)  # noqa: E731
            self.ttt_states[i] = (sel(h), sel(t), sel(w))


def _ipttt_scan(p, h, w_down, lr):
    """Scan with externally supplied update vectors: dW_j = p_j^T h_j."""
    b, T, C, d_i = h.shape
    d_w = ops.matmul(p[:, :-1].transpose(-1, -2), h[:, :-1])              # [b, T-1, d_h, d_i]
    last = d_w.detach().float().norm()
    states = torch.cat([w_down.to(d_w.dtype).expand(b, 1, -1, -1), d_w * lr], dim=1).cumsum(dim=1)
    y = ops.matmul(h, states.transpose(-1, -2))
    return y, last


class IPTTTBlock(nn.Module):
    def __init__(self, config: IPTTTConfig, layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.is_ttt_layer = bool(config.ttt_mode and layer_idx in set(config.ttt_layers))
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = build_attention(config, layer_idx, with_rope_scaling=False)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = IPTTTMLP(config, layer_idx)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False,
                ttt_target_states=None, **kwargs):
        residual = layer_input = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        hidden_states, _ = self.attn(hidden_states, attention_mask=attention_mask,
                                     past_key_values=past_key_values, use_cache=use_cache, **kwargs)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)
        target = None
        if self.is_ttt_layer:
            kind = self.config.ttt_target
            target = ttt_target_states if kind == "embedding" else (layer_input if kind == "layer_input" else hidden_states)
        if self.is_ttt_layer and isinstance(past_key_values, FastWeightCache) and not self.training:
            return residual + self._online_mlp(hidden_states, target, past_key_values)
        hidden_states = self.mlp(hidden_states, t=target)
        return residual + hidden_states

    def _online_mlp(self, hidden_states, target, cache: "FastWeightCache"):
        """MLP with fast weights carried across calls: prepend the unfinished chunk kept in the cache, run the
        online scan from the cached weight, return the outputs of the new positions, keep the new remainder."""
        n_new = hidden_states.shape[1]
        past_h, past_t, past_w = cache.ttt_get(self.layer_idx)
        h_all = hidden_states if past_h is None else torch.cat([past_h, hidden_states], dim=1)
        t_all = target if past_t is None else torch.cat([past_t, target], dim=1)
        y, w = self.mlp.forward_online(h_all, t_all, past_w)
        rem = h_all.shape[1] % self.mlp.ttt_chunk
        tail_h, tail_t = (h_all[:, -rem:], t_all[:, -rem:]) if rem else (None, None)
        cache.ttt_update((tail_h, tail_t, w), self.layer_idx)
        return y[:, -n_new:]


class _IPTTTInit:
    def _init_extra(self, module: nn.Module) -> None:
        cfg = self.config
        if isinstance(module, nn.Linear) and getattr(module, "_is_ttt_proj", False):
            if module.weight.device.type == "meta" or getattr(module.weight, "_is_hf_initialized", False):
                return
            if cfg.ttt_proj_init in {"diagonal", "diagonal_gaussian"}:
                n = min(module.weight.shape)
                module.weight.zero_()
                idx = torch.arange(n, device=module.weight.device)
                module.weight[idx, idx] = torch.randn(n, device=module.weight.device,
                                                      dtype=module.weight.dtype) * cfg.initializer_range
            elif cfg.ttt_proj_init == "zero":
                module.weight.zero_()
        if isinstance(module, nn.Conv1d) and getattr(module, "_is_ttt_conv", False):
            if module.weight.device.type != "meta" and not getattr(module.weight, "_is_hf_initialized", False):
                module.weight.zero_()


class IPTTTModel(_IPTTTInit, DecoderModel):
    cache_class = FastWeightCache       # inference carries fast weights across calls
    config_class = IPTTTConfig
    block_class = IPTTTBlock
    _no_split_modules = ["IPTTTBlock"]

    def _block_kwargs(self, input_ids, inputs_embeds, kwargs):
        if self.config.ttt_target == "embedding":
            kwargs = dict(kwargs, ttt_target_states=inputs_embeds)
        return kwargs


class IPTTTForCausalLM(_IPTTTInit, DecoderForCausalLM):
    config_class = IPTTTConfig
    model_class = IPTTTModel
    _no_split_modules = ["IPTTTBlock"]
