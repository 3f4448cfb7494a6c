"""The linear-recurrent baseline families: ``delta_net`` and ``gated_deltanet``.

Both are pre-norm decoder stacks whose token mixer keeps a per-head matrix state instead of a key/value cache
(fla/models/delta_net/modeling_delta_net.py:35-110, fla/models/gated_deltanet/modeling_gated_deltanet.py; the mixers
are fla/layers/delta_net.py:50-300 and fla/layers/gated_deltanet.py:40-330):

* q, k, v are projected, passed through a causal depthwise convolution of ``conv_size`` taps with SiLU, and split into
  heads; q and k are L2-normalised per head.
* ``beta = sigmoid(b_proj(x))`` (doubled when negative eigenvalues are allowed) is the write strength; the gated
  variant adds the log decay ``g = -exp(A_log) * softplus(a_proj(x) + dt_bias)`` per value head.
* the (gated) delta rule turns these into outputs (``ops.gated_delta_rule``: chunked for sequences, token by token
  for short decode steps, state carried in the cache), a per-head RMSNorm (optionally gated by ``silu(g_proj(x))``)
  and ``o_proj`` finish the layer.

Parameter names follow the reference, so its checkpoints load unchanged.  Layers listed in ``config.attn['layers']``
are softmax attention instead (the hybrid layouts).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .base import DecoderForCausalLM, DecoderModel
from .configuration import DeltaNetConfig, GatedDeltaNetConfig
from .layers import Attention, GatedMLP, RMSNorm, WindowKVCache


class RecurrentCache(WindowKVCache):
    """Decoding state of the recurrent layers (matrix state + the last ``conv_size - 1`` inputs of each convolution)
    beside the key/value windows of hybrid attention layers."""

    def __init__(self):
        super().__init__()
        self.states: dict[int, dict] = {}

    def __len__(self) -> int:
        return max(len(self.layers), len(self.states))

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if layer_idx in self.states:
            return self.states[layer_idx]["seen"]
        return super().get_seq_length(layer_idx)

    def reorder(self, beam_idx: torch.Tensor):
        super().reorder(beam_idx)
        for st in self.states.values():
            st["recurrent"] = st["recurrent"].index_select(0, beam_idx)
            st["conv"] = tuple(None if c is None else c.index_select(0, beam_idx) for c in st["conv"])


class ShortConv(nn.Conv1d):
    """Causal depthwise convolution over time on [B, T, D] with optional SiLU, and a rolling input window for decoding
    (fla/modules/convolution.py ShortConvolution; the weight keeps the Conv1d layout [D, 1, K])."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: str | None = "silu"):
        super().__init__(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=bias, padding=kernel_size - 1)
        self.hidden_size, self.activation = hidden_size, activation

    def forward(self, x, cache=None, output_final_state: bool = False, cu_seqlens=None):
        taps = self.kernel_size[0] - 1
        if cache is not None:
            x_full = torch.cat([cache.to(x.dtype), x], dim=1)
            y = ops.dwconv_sequence(x_full, self.weight, self.bias, self.activation)[:, taps:]
        else:
            x_full = x
            y = ops.dwconv_sequence(x, self.weight, self.bias, self.activation, cu_seqlens=cu_seqlens)
        final = None
        if output_final_state:
            final = x_full[:, -taps:] if x_full.shape[1] >= taps else F.pad(x_full, (0, 0, taps - x_full.shape[1], 0))
        return y, final


def _qk_activation(name: str, x):
    if name == "relu":
        return x.relu()
    if name == "elu":
        return F.elu(x, 1.0, False) + 1.0
    if name in ("identity", "silu"):
        return x
    raise NotImplementedError(f"qk_activation {name!r}")


class _DeltaMixer(nn.Module):
    """What the two mixers share: the convolutions, the cache protocol, the rule call and the output stage."""

    gated = False

    def _build(self, hidden_size, key_dim, value_dim, head_k_dim, head_v_dim, rule_heads, use_short_conv, conv_size,
               use_gate, norm_eps, qk_act, layer_idx):
        self.hidden_size, self.key_dim, self.value_dim = hidden_size, key_dim, value_dim
        self.head_k_dim, self.head_v_dim, self.rule_heads = head_k_dim, head_v_dim, rule_heads
        self.use_short_conv, self.conv_size, self.use_gate, self.layer_idx = use_short_conv, conv_size, use_gate, layer_idx
        self.q_proj = nn.Linear(hidden_size, key_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, key_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, value_dim, bias=False)
        if use_short_conv:
            self.q_conv1d = ShortConv(key_dim, conv_size, activation=qk_act)
            self.k_conv1d = ShortConv(key_dim, conv_size, activation=qk_act)
            self.v_conv1d = ShortConv(value_dim, conv_size, activation="silu")
        if use_gate:
            self.g_proj = nn.Linear(hidden_size, value_dim, bias=False)
        self.o_norm = RMSNorm(head_v_dim, eps=norm_eps)
        self.o_proj = nn.Linear(value_dim, hidden_size, bias=False)

    # family hooks -----------------------------------------------------------------------------------------------
    def _strengths(self, x):
        """(g or None, beta) of shape [B, T, rule_heads]."""
        raise NotImplementedError

    def _shape_qk(self, q, k):
        return q, k

    qk_l2 = True

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache: bool = False,
                cu_seqlens=None, **_):
        B, T, _d = hidden_states.shape
        state = None
        if isinstance(past_key_values, RecurrentCache):
            state = past_key_values.states.get(self.layer_idx)
        packed = None
        if attention_mask is not None and not bool(attention_mask[:, -T:].all()):
            # padded batch: run the kept tokens as one packed row, every sample its own sequence
            if state is not None:
                raise NotImplementedError("a padded batch cannot continue a recurrent state; left-trim the prompts instead")
            keep = attention_mask[:, -T:].bool()
            lens = keep.sum(-1)
            cu_seqlens = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
            packed = keep.reshape(-1).nonzero().squeeze(-1)
            hidden_states = hidden_states.reshape(1, B * T, -1)[:, packed]
        x = hidden_states
        want_state = bool(use_cache and isinstance(past_key_values, RecurrentCache))
        convs = (None, None, None) if state is None else state["conv"]
        qp, kp, vp = (ops.linear(x, w) for w in (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
        if self.use_short_conv:
            q, cq = self.q_conv1d(qp, convs[0], want_state, cu_seqlens)
            k, ck = self.k_conv1d(kp, convs[1], want_state, cu_seqlens)
            v, cv = self.v_conv1d(vp, convs[2], want_state, cu_seqlens)
            if want_state and packed is not None:           # one input window per sample, not the packed row's tail
                cq, ck, cv = (self._window_per_sample(t, cu_seqlens) for t in (qp, kp, vp))
        else:
            cq = ck = cv = None
            q, k, v = self._no_conv_activation(qp, kp, vp)
        q = q.view(*q.shape[:2], -1, self.head_k_dim)
        k = k.view(*k.shape[:2], -1, self.head_k_dim)
        v = v.view(*v.shape[:2], -1, self.head_v_dim)
        q, k = self._shape_qk(q, k)
        g, beta = self._strengths(x)
        recurrent = x.shape[1] <= 64 and not self.training and cu_seqlens is None
        o, final = ops.gated_delta_rule(q, k, v, g, beta, l2norm=self.qk_l2, cu_seqlens=cu_seqlens,
                                        initial_state=None if state is None else state["recurrent"],
                                        output_final_state=want_state, recurrent=recurrent)
        if want_state:
            seen = (0 if state is None else state["seen"]) + T
            past_key_values.states[self.layer_idx] = dict(recurrent=final, conv=(cq, ck, cv), seen=seen)
        o = self.o_norm(o)
        if self.use_gate:
            gate = ops.linear(x, self.g_proj.weight).view_as(o)
            o = ops.swiglu(gate, o)
        o = ops.linear(o.reshape(*o.shape[:2], -1), self.o_proj.weight)
        if packed is not None:
            full = o.new_zeros(B * T, o.shape[-1])
            full[packed] = o[0]
            o = full.view(B, T, -1)
        return o, past_key_values

    def _window_per_sample(self, x, cu_seqlens):
        taps = self.conv_size - 1
        bounds = cu_seqlens.tolist()
        rows = []
        for a, b in zip(bounds[:-1], bounds[1:]):
            w = x[0, max(a, b - taps):b]
            rows.append(F.pad(w, (0, 0, taps - w.shape[0], 0)))
        return torch.stack(rows)

    def _no_conv_activation(self, q, k, v):
        return F.silu(q), F.silu(k), F.silu(v)


class DeltaNet(_DeltaMixer):
    """Delta-rule mixer (fla/layers/delta_net.py:50-300)."""

    def __init__(self, hidden_size=1024, expand_k=1.0, expand_v=1.0, num_heads=4, use_beta=True, use_gate=False,
                 use_short_conv=True, conv_size=4, allow_neg_eigval=False, layer_idx=None, qk_activation="silu",
                 qk_norm="l2", norm_eps=1e-5, mode="chunk", **_):
        super().__init__()
        if qk_activation not in ("silu", "relu", "elu", "identity") or qk_norm not in ("l2", "sum"):
            raise ValueError(f"qk_activation {qk_activation!r} / qk_norm {qk_norm!r}")
        if mode not in ("chunk", "fused_recurrent"):
            raise NotImplementedError(f"mode {mode!r}")
        key_dim, value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        if key_dim % num_heads or value_dim % num_heads:
            raise ValueError("key and value widths must divide by num_heads")
        self.num_heads, self.use_beta, self.allow_neg_eigval = num_heads, use_beta, allow_neg_eigval
        self.qk_activation, self.qk_norm, self.qk_l2 = qk_activation, qk_norm, qk_norm == "l2"
        self._build(hidden_size, key_dim, value_dim, key_dim // num_heads, value_dim // num_heads, num_heads,
                    use_short_conv, conv_size, use_gate, norm_eps, "silu" if qk_activation == "silu" else None, layer_idx)
        if use_beta:
            self.b_proj = nn.Linear(hidden_size, num_heads, bias=False)

    def _no_conv_activation(self, q, k, v):
        if self.qk_activation == "silu":
            q, k = F.silu(q), F.silu(k)
        return q, k, F.silu(v)

    def _shape_qk(self, q, k):
        q, k = _qk_activation(self.qk_activation, q), _qk_activation(self.qk_activation, k)
        if self.qk_norm == "sum":
            q, k = (q / q.sum(-1, keepdim=True)).to(q.dtype), (k / k.sum(-1, keepdim=True)).to(k.dtype)
        return q, k

    def _strengths(self, x):
        if self.use_beta:
            beta = torch.sigmoid(F.linear(x, self.b_proj.weight).float())
        else:
            beta = x.new_ones(*x.shape[:2], self.num_heads, dtype=torch.float32)
        return None, (beta * 2.0 if self.allow_neg_eigval else beta)


class GatedDeltaNet(_DeltaMixer):
    """Gated delta-rule mixer (fla/layers/gated_deltanet.py:40-330)."""

    gated = True

    def __init__(self, hidden_size=2048, expand_v=2.0, head_dim=256, num_heads=6, num_v_heads=None, use_gate=True,
                 use_short_conv=True, allow_neg_eigval=False, conv_size=4, layer_idx=None, norm_eps=1e-5, mode="chunk", **_):
        super().__init__()
        if mode not in ("chunk", "fused_recurrent"):
            raise NotImplementedError(f"mode {mode!r}")
        self.num_heads = num_heads
        self.num_v_heads = num_heads if num_v_heads is None else num_v_heads
        self.allow_neg_eigval = allow_neg_eigval
        head_v = head_dim * expand_v
        if not math.isclose(head_v, round(head_v), rel_tol=1e-5):
            raise ValueError(f"expand_v={expand_v} times head_dim={head_dim} is not an integer")
        if self.num_v_heads > num_heads and self.num_v_heads % num_heads:
            raise ValueError(f"num_v_heads={self.num_v_heads} must be a multiple of num_heads={num_heads}")
        head_v = int(round(head_v))
        self._build(hidden_size, num_heads * head_dim, self.num_v_heads * head_v, head_dim, head_v, self.num_v_heads,
                    use_short_conv, conv_size, use_gate, norm_eps, "silu", layer_idx)
        self.a_proj = nn.Linear(hidden_size, self.num_v_heads, bias=False)
        self.b_proj = nn.Linear(hidden_size, self.num_v_heads, bias=False)
        self.A_log = nn.Parameter(torch.empty(self.num_v_heads, dtype=torch.float32))
        self.dt_bias = nn.Parameter(torch.empty(self.num_v_heads, dtype=torch.float32))
        self.A_log._no_weight_decay = True
        self.dt_bias._no_weight_decay = True
        self.reset_decay_parameters()

    @torch.no_grad()
    def reset_decay_parameters(self, dt_min: float = 1e-3, dt_max: float = 0.1, dt_floor: float = 1e-4):
        """A ~ U(0, 16) stored as its log; dt log-uniform in [dt_min, dt_max], stored through the inverse softplus."""
        if self.A_log.device.type == "meta":
            return
        self.A_log.copy_(torch.log(torch.empty_like(self.A_log).uniform_(0, 16).clamp_min(1e-4)))
        dt = torch.exp(torch.rand_like(self.dt_bias) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = dt.clamp_min(dt_floor)
        self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))

    def _shape_qk(self, q, k):
        rep = self.num_v_heads // self.num_heads
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        return q, k

    def _strengths(self, x):
        beta = torch.sigmoid(F.linear(x, self.b_proj.weight).float())
        if self.allow_neg_eigval:
            beta = beta * 2.0
        g = -self.A_log.float().exp() * F.softplus(F.linear(x, self.a_proj.weight).float() + self.dt_bias.float())
        return g, beta


def _hybrid_attention(config, layer_idx):
    a = config.attn
    return Attention(hidden_size=config.hidden_size, num_heads=a["num_heads"], num_kv_heads=a["num_kv_heads"],
                     qkv_bias=a["qkv_bias"], window_size=a["window_size"], rope_theta=a["rope_theta"],
                     max_position_embeddings=config.max_position_embeddings, layer_idx=layer_idx)


class _RecurrentBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        if config.attn is not None and layer_idx in config.attn["layers"]:
            self.attn = _hybrid_attention(config, layer_idx)
        else:
            self.attn = self._mixer(config, layer_idx)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = GatedMLP(config.hidden_size, config.resolved_intermediate_size)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False, **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        hidden_states, _ = self.attn(hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
                                     use_cache=use_cache, **kwargs)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)
        return residual + self.mlp(hidden_states)


class DeltaNetBlock(_RecurrentBlock):
    @staticmethod
    def _mixer(c, layer_idx):
        return DeltaNet(hidden_size=c.hidden_size, expand_k=c.expand_k, expand_v=c.expand_v, num_heads=c.num_heads,
                        use_beta=c.use_beta, use_gate=c.use_gate, use_short_conv=c.use_short_conv, conv_size=c.conv_size,
                        qk_activation=c.qk_activation, qk_norm=c.qk_norm, norm_eps=c.norm_eps, mode=c.attn_mode,
                        layer_idx=layer_idx)


class GatedDeltaNetBlock(_RecurrentBlock):
    @staticmethod
    def _mixer(c, layer_idx):
        return GatedDeltaNet(hidden_size=c.hidden_size, expand_v=c.expand_v, head_dim=c.head_dim, num_heads=c.num_heads,
                             num_v_heads=c.num_v_heads, use_gate=c.use_gate, use_short_conv=c.use_short_conv,
                             allow_neg_eigval=c.allow_neg_eigval, conv_size=c.conv_size, norm_eps=c.norm_eps,
                             mode=c.attn_mode, layer_idx=layer_idx)


class _RecurrentInit:
    cache_class = RecurrentCache

    def _init_extra(self, module: nn.Module) -> None:
        if isinstance(module, GatedDeltaNet) and not getattr(module.A_log, "_is_hf_initialized", False):
            module.reset_decay_parameters()


class DeltaNetModel(_RecurrentInit, DecoderModel):
    config_class = DeltaNetConfig
    block_class = DeltaNetBlock
    _no_split_modules = ["DeltaNetBlock"]


class DeltaNetForCausalLM(_RecurrentInit, DecoderForCausalLM):
    config_class = DeltaNetConfig
    model_class = DeltaNetModel
    _no_split_modules = ["DeltaNetBlock"]


class GatedDeltaNetModel(_RecurrentInit, DecoderModel):
    config_class = GatedDeltaNetConfig
    block_class = GatedDeltaNetBlock
    _no_split_modules = ["GatedDeltaNetBlock"]


class GatedDeltaNetForCausalLM(_RecurrentInit, DecoderForCausalLM):
    config_class = GatedDeltaNetConfig
    model_class = GatedDeltaNetModel
    _no_split_modules = ["GatedDeltaNetBlock"]
