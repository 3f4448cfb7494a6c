"""Shared building blocks: RMSNorm, rotary tables, windowed KV cache, attention, gated MLP.

Parameter names match the reference's layers so checkpoints interchange:
``attn.{q,k,v,o}_proj``, ``attn.{q,k}_norm``, ``mlp.{gate,up,down}_proj``
(fla/layers/attn.py:64-168, fla/modules/mlp.py).  Behavioural notes reproduced
here: the per-head q/k norm uses eps 1e-5 regardless of ``config.norm_eps``
(fla/layers/attn.py:120-122); rotary tables are computed in fp32 and stored in
the activation dtype (fla/modules/rotary.py:475-525); the KV cache keeps only the
last ``window_size`` tokens (fla/models/utils.py:58-80).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref_ops


class RMSNorm(nn.Module):
    """y = x * rsqrt(mean(x^2) + eps) * weight, optionally fused with a residual add."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5):
        super().__init__()
        self.hidden_size = hidden_size
        self.eps = eps
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size))
        else:
            self.register_parameter("weight", None)

    def reset_parameters(self):
        if self.weight is not None:
            nn.init.ones_(self.weight)

    def forward(self, x, residual=None, prenorm: bool = False):
        return ops.rmsnorm(x, self.weight, self.eps, residual=residual, prenorm=prenorm)

    def extra_repr(self) -> str:
        return f"{self.hidden_size}, eps={self.eps}"


class RotaryEmbedding(nn.Module):
    """NeoX-style rotary tables with optional YaRN (mscale baked into cos/sin) or Llama-3 frequency rescaling."""

    def __init__(self, dim: int, base: float = 10000.0, rope_scaling: dict | None = None):
        super().__init__()
        self.dim = dim
        self.base = float(base)
        self.yarn = None
        self.attn_scale = 1.0
        kind = None if rope_scaling is None else (rope_scaling.get("type") or rope_scaling.get("rope_type"))
        if kind in (None, "default"):      # transformers >= 5 writes {"rope_type": "default"} for plain RoPE
            rope_scaling = None
        self.llama3 = None
        if rope_scaling is not None and kind == "llama3":
            self.llama3 = dict(
                factor=float(rope_scaling.get("factor", 1.0)),
                original_max_position=int(rope_scaling["original_max_position_embeddings"]),
                low_freq_factor=float(rope_scaling.get("low_freq_factor", 1.0)),
                high_freq_factor=float(rope_scaling.get("high_freq_factor", 4.0)),
            )
        elif rope_scaling is not None:
            if kind != "yarn":
                raise NotImplementedError(f"rope_scaling type {kind!r} is not supported (only 'yarn' and 'llama3')")
            factor = float(rope_scaling.get("factor", 1.0))
            self.yarn = dict(
                factor=factor,
                original_max_position=int(rope_scaling.get("original_max_position_embeddings", 0)),
                beta_fast=float(rope_scaling.get("beta_fast", 32.0)),
                beta_slow=float(rope_scaling.get("beta_slow", 1.0)),
            )
            if factor > 1.0 and not self.yarn["original_max_position"]:
                raise ValueError("yarn factor > 1 requires original_max_position_embeddings")
            self.attn_scale = ref_ops.yarn_mscale(factor, float(rope_scaling.get("mscale", 1.0)))
        self._cached = None  # (seqlen, device, dtype, cos, sin)

    def inv_freq(self, device=None) -> torch.Tensor:
        if self.yarn is not None and self.yarn["factor"] > 1.0:
            return ref_ops.yarn_inv_freq(self.dim, self.base, device=device, **self.yarn)
        if self.llama3 is not None:
            return ref_ops.llama3_inv_freq(self.dim, self.base, device=device, **self.llama3)
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device, dtype=torch.float32) / self.dim))

    def tables(self, seqlen: int, device, dtype):
        c = self._cached
        if c is None or c[0] < seqlen or c[1] != device or c[2] != dtype or (
            torch.is_grad_enabled() and c[3].is_inference()
        ):
            cos, sin = ref_ops.rope_tables(self.dim, self.base, seqlen, device=device, dtype=dtype,
                                           inv_freq=self.inv_freq(device), attn_scale=self.attn_scale)
            self._cached = (seqlen, device, dtype, cos, sin)
            c = self._cached
        return c[3], c[4]


class WindowKVCache:
    """Per-layer key/value cache that keeps at most ``window`` trailing tokens."""

    def __init__(self):
        self.layers: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.seen: dict[int, int] = {}

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.seen.get(layer_idx, 0)

    def __len__(self) -> int:
        return len(self.layers)

    def update(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int, window: int | None):
        """Append k/v [B,T,HK,D]; returns the tensors to attend over."""
        old = self.layers.get(layer_idx)
        self.seen[layer_idx] = self.seen.get(layer_idx, 0) + k.shape[1]
        if old is None:
            full_k, full_v = k, v
        else:
            full_k = torch.cat([old[0], k], dim=1)
            full_v = torch.cat([old[1], v], dim=1)
        if window is not None and full_k.shape[1] > window:
            keep_k, keep_v = full_k[:, -window:].contiguous(), full_v[:, -window:].contiguous()
        else:
            keep_k, keep_v = full_k, full_v
        self.layers[layer_idx] = (keep_k, keep_v)
        return full_k, full_v

    def reorder(self, beam_idx: torch.Tensor):
        for i, (k, v) in self.layers.items():
            self.layers[i] = (k.index_select(0, beam_idx), v.index_select(0, beam_idx))


class StaticWindowCache(WindowKVCache):
    """Decoding cache at fixed addresses: every layer keeps a ring buffer of ``window`` rows (layers without a window:
    the tokens seen plus ``max_new_tokens``, rounded up to 1024), the write slot, the fill count and the rotary
    position live in device tensors that ``advance()`` updates in place.  A decode step through this cache reads no
    value on the host and allocates nothing that outlives it, so it can be captured once as a CUDA graph and replayed
    per token.  The token of absolute index ``a`` sits in row ``a % capacity``; attention over a ring needs no mask
    beyond the fill count, because every row it holds is inside the window (keys carry their rotary phase already).
    One query token per step; prompts of unequal length (a padding mask) stay on the eager cache."""

    def __init__(self, source: WindowKVCache, windows: dict[int, int | None], max_new_tokens: int):
        super().__init__()
        seen = {source.seen[i] for i in source.layers}
        if len(seen) != 1:
            raise ValueError("the layers of the source cache have seen different numbers of tokens")
        self.start = seen.pop()
        self.max_position = self.start + max_new_tokens          # rotary table rows a decode run may touch
        first = next(iter(source.layers.values()))[0]
        dev = first.device
        self.capacity: dict[int, int] = {}
        for i, (k, v) in source.layers.items():
            w = windows.get(i)
            cap = int(w) if w is not None else -(-(self.start + max_new_tokens) // 1024) * 1024
            n = k.shape[1]
            if n > cap:
                raise ValueError(f"layer {i}: {n} cached rows do not fit a ring of {cap}")
            rk = k.new_zeros(k.shape[0], cap, *k.shape[2:])
            rv = v.new_zeros(v.shape[0], cap, *v.shape[2:])
            rows = torch.arange(self.start - n, self.start, device=dev) % cap
            rk.index_copy_(1, rows, k)
            rv.index_copy_(1, rows, v)
            self.layers[i] = (rk, rv)
            self.seen[i] = self.start
            self.capacity[i] = cap
        self.pos = torch.zeros(1, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(first.shape[0], 1, dtype=torch.int64, device=dev)
        self.positions._ttcd_bounded = True                      # never beyond max_position: no host check per step
        self.slot = {c: torch.zeros(1, dtype=torch.int64, device=dev) for c in set(self.capacity.values())}
        self.kv_len = {c: torch.zeros(1, dtype=torch.int32, device=dev) for c in set(self.capacity.values())}
        self.reset(self.start)

    def reset(self, position: int) -> None:
        """Point the device state at the token of absolute index ``position`` (the next one to be written)."""
        self.pos.fill_(position)
        self._derive()
        for i in self.seen:
            self.seen[i] = position

    def _derive(self) -> None:
        self.positions.copy_(self.pos.expand_as(self.positions))
        for c, slot in self.slot.items():
            torch.remainder(self.pos, c, out=slot)
            self.kv_len[c].copy_(torch.clamp(self.pos + 1, max=c))

    def advance(self) -> None:
        """Device side of moving on by one token (captured with the step)."""
        self.pos.add_(1)
        self._derive()

    def host_advance(self, n: int = 1) -> None:
        """Host mirror of ``advance`` for ``get_seq_length`` (a replayed graph runs no Python)."""
        for i in self.seen:
            self.seen[i] += n

    def append(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int):
        """Write this step's k/v [B,1,HK,D] into the ring; returns (ring k, ring v, fill count incl. this token)."""
        if k.shape[1] != 1:
            raise ValueError("the static cache takes one token per step")
        rk, rv = self.layers[layer_idx]
        c = self.capacity[layer_idx]
        rk.index_copy_(1, self.slot[c], k)
        rv.index_copy_(1, self.slot[c], v)
        return rk, rv, self.kv_len[c]

    def update(self, k, v, layer_idx, window):
        raise RuntimeError("StaticWindowCache is written through append()")


def _gate_activation(name: str):
    return {"sigmoid": torch.sigmoid, "swish": F.silu, "silu": F.silu, "relu": F.relu}[name]


class Attention(nn.Module):
    """GQA sliding-window attention with optional per-head q/k RMSNorm, RoPE/YaRN and output gate."""

    def __init__(self, hidden_size, num_heads, num_kv_heads=None, head_dim=None, qkv_bias=False,
                 qk_norm=False, window_size=None, rope_theta=10000.0, max_position_embeddings=None,
                 layer_idx=None, use_output_gate=False, gate_fn="sigmoid", elementwise_affine=True,
                 norm_eps=1e-5, rope_scaling=None, use_nope=False, use_l2_softmax=False):
        super().__init__()
        self.use_l2_softmax = use_l2_softmax
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        self.head_dim = head_dim if head_dim is not None else hidden_size // num_heads
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.qk_norm = qk_norm
        self.window_size = window_size
        self.max_position_embeddings = max_position_embeddings
        self.layer_idx = layer_idx
        self.use_nope = use_nope or rope_theta is None

        self.q_proj = nn.Linear(hidden_size, self.q_dim, bias=qkv_bias)
        self.k_proj = nn.Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.v_proj = nn.Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.o_proj = nn.Linear(self.q_dim, hidden_size, bias=False)
        if qk_norm:
            self.q_norm = RMSNorm(self.head_dim)  # eps 1e-5 by design, not config.norm_eps
            self.k_norm = RMSNorm(self.head_dim)
        if not self.use_nope:
            self.rotary = RotaryEmbedding(self.head_dim, rope_theta, rope_scaling)
        self.use_output_gate = use_output_gate
        if use_output_gate:
            self.g_proj = nn.Linear(hidden_size, self.kv_dim, bias=False)
            self.g_norm = RMSNorm(self.head_dim, elementwise_affine=elementwise_affine, eps=norm_eps)
            self.gate_fn = _gate_activation(gate_fn)

    # -- pieces shared with the TTT block ------------------------------------------------
    def project_qkv(self, hidden_states, seqlen_offset=0, max_seqlen=None, positions=None):
        """q/k/v projections, per-head norm and rotary.  Returns q[B,T,H,D], k, v[B,T,HK,D]."""
        B = hidden_states.shape[0]
        q, k, v = _fused_qkv(self, hidden_states)
        T = q.shape[1]                      # all tokens: under tensor parallelism the input is a token shard
        tags = [getattr(t, "_ttcd_grad_slab", None) for t in (q, k, v)]
        q = q.view(B, T, self.num_heads, self.head_dim)
        k = k.view(B, T, self.num_kv_heads, self.head_dim)
        v = v.view(B, T, self.num_kv_heads, self.head_dim)
        for t, tag in zip((q, k, v), tags):
            if tag is not None:
                t._ttcd_grad_slab = tag     # the views keep pointing at the shared gradient buffer
        cos = sin = None
        if not self.use_nope:
            if max_seqlen is None:
                base = seqlen_offset if isinstance(seqlen_offset, int) else int(seqlen_offset.max())
                max_seqlen = T + base
                if positions is not None:
                    max_seqlen = max(max_seqlen, int(positions.max()) + 1)
            if self.max_position_embeddings is not None:
                max_seqlen = max(max_seqlen, self.max_position_embeddings)
            cos, sin = self.rotary.tables(max_seqlen, hidden_states.device, hidden_states.dtype)
        qw = self.q_norm.weight if self.qk_norm else None
        kw = self.k_norm.weight if self.qk_norm else None
        eps = self.q_norm.eps if self.qk_norm else 0.0
        if self.qk_norm or cos is not None:
            q, k = ops.qkv_norm_rope(q, k, qw, kw, eps, cos, sin, seqlen_offset, positions)
        return q, k, v

    def finish(self, o, hidden_states):
        """Output gate (optional) and o_proj on o[B,T,H,D]."""
        B, T = o.shape[:2]
        if self.use_output_gate:
            g = ops.linear(hidden_states, self.g_proj.weight)
            o = self.g_norm(o).reshape(B, T, -1) * self.gate_fn(g)
        else:
            o = o.reshape(B, T, -1)
        tp = _tp_state()
        if tp is not None:
            from ..parallel.tensor import row_parallel_linear
            return row_parallel_linear(o.reshape(B * T, -1), self.o_proj.weight, tp).view(B, T // tp.world, -1)
        return ops.linear(o, self.o_proj.weight)

    # -- standard forward ---------------------------------------------------------------------
    def forward(self, hidden_states, attention_mask=None, past_key_values: WindowKVCache | None = None,
                use_cache: bool = False, cu_seqlens=None, positions=None, **_):
        B, T, _ = hidden_states.shape
        if isinstance(past_key_values, StaticWindowCache):          # one token, nothing read on the host (capturable)
            cache = past_key_values
            q, k, v = self.project_qkv(hidden_states, 0, max_seqlen=cache.max_position, positions=cache.positions)
            k_all, v_all, kv_len = cache.append(k, v, self.layer_idx)
            return self.finish(ops.decode_attention(q, k_all, v_all, kv_len), hidden_states), cache
        offset = 0
        cp = _cp_state() if past_key_values is None else None
        if cp is not None:
            offset = cp.position_offset(T)
        if past_key_values is not None:
            offset = past_key_values.get_seq_length(self.layer_idx)
            if attention_mask is not None:
                lens = attention_mask.sum(-1)
                offset = offset + lens - attention_mask.shape[-1]
        if cu_seqlens is not None and positions is None:
            positions = positions_from_cu_seqlens(cu_seqlens, T, hidden_states.device)
        q, k, v = self.project_qkv(hidden_states, offset, positions=positions)
        if past_key_values is not None:
            had_content = past_key_values.get_seq_length(self.layer_idx) > 0
            k_all, v_all = past_key_values.update(k, v, self.layer_idx, self.window_size)
            if had_content:
                k, v = k_all, v_all
        if self.use_l2_softmax:
            if cp is not None or (attention_mask is not None and not bool(attention_mask.all())):
                raise NotImplementedError("use_l2_softmax with context parallelism or a padding mask")
            o = ops.l2_softmax_attention(q, k, v, cu_seqlens=cu_seqlens)
        elif cp is not None:
            from ..parallel import context as _context
            o = _context.attention(q, k, v, self.window_size, None, self.layer_idx)
        elif attention_mask is not None and not bool(attention_mask.all()):
            o = _padded_attention(q, k, v, attention_mask, self.window_size)
        else:
            o = ops.attention(q, k, v, window=self.window_size, cu_seqlens=cu_seqlens)
        return self.finish(o, hidden_states), past_key_values


def _cp_state():
    """The active context-parallel state, if any (sequence shards + K/V halo from the previous rank)."""
    import sys
    mod = sys.modules.get("ttcd_b200.parallel.context")
    return mod.active() if mod is not None else None


def _tp_state():
    """The active tensor-parallel state, if any (token-sharded residual stream, head/row-sharded weights)."""
    import sys
    mod = sys.modules.get("ttcd_b200.parallel.tensor")
    return mod.current() if mod is not None else None


def positions_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int, device) -> torch.Tensor:
    """Position of each packed token inside its own sequence (restarts at every boundary)."""
    cu = cu_seqlens.to(device=device, dtype=torch.long)
    idx = torch.arange(total, device=device)
    seg = torch.searchsorted(cu, idx, right=True) - 1
    return idx - cu[seg]


def _padded_attention(q, k, v, attention_mask, window):
    """Left- or right-padded batches: every row attends over its own valid tokens only.

    Prefill (as many queries as keys): the valid tokens of all rows are packed into one row and run as ONE
    attention launch with per-sequence bounds, then scattered back (the unpad -> varlen -> pad sequence of
    fla/layers/attn.py:229-254).  Decode over a padded cache keeps one call per row."""
    B, Tq = q.shape[:2]
    Tk = k.shape[1]
    mask = attention_mask[:, -Tk:].bool()
    if Tq == Tk:
        flat = mask.reshape(-1)
        idx = flat.nonzero(as_tuple=False).squeeze(1)            # sizes the packed row (the one host sync of unpadding)
        lens = mask.sum(-1)
        cu = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
        pick = lambda t: t.reshape(1, B * Tq, *t.shape[2:])[:, idx]      # noqa: E731
        o = ops.attention(pick(q), pick(k), pick(v), window=window, cu_seqlens=cu)
        out = q.new_zeros(B * Tq, *q.shape[2:])
        out[idx] = o[0].to(out.dtype)
        return out.view(B, Tq, *q.shape[2:])
    outs = []
    for b in range(B):
        kb = k[b:b + 1, mask[b]]
        vb = v[b:b + 1, mask[b]]
        if Tq == 1:
            qb = q[b:b + 1]
            ob = ops.attention(qb, kb, vb, window=window)
        else:
            qmask = attention_mask[b, -Tq:].bool()
            qb = q[b:b + 1, qmask]
            ob_valid = ops.attention(qb, kb, vb, window=window)
            ob = q.new_zeros(1, Tq, *q.shape[2:])
            ob[:, qmask] = ob_valid
        outs.append(ob)
    return torch.cat(outs, dim=0)


def _slab_view(params: list[torch.Tensor]) -> torch.Tensor | None:
    """If the given 2-D weights sit back to back in memory, return them as one [sum(N), K] view."""
    first = params[0]
    if any(p.dim() != 2 or p.shape[1] != first.shape[1] or not p.is_contiguous() for p in params):
        return None
    expect = first.data_ptr()
    for p in params:
        if p.data_ptr() != expect or p.dtype != first.dtype or p.device != first.device:
            return None
        expect += p.numel() * p.element_size()
    rows = sum(p.shape[0] for p in params)
    try:
        return torch.as_strided(first.detach(), (rows, first.shape[1]), (first.shape[1], 1))
    except RuntimeError:
        return None


def _fused_qkv(attn: Attention, x):
    """One GEMM for q, k and v when their weights are laid out contiguously, else three."""
    ws = [attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight]
    tp = _tp_state()
    if tp is not None:
        from ..parallel.tensor import column_parallel_multi
        if x.shape[0] != 1:
            raise NotImplementedError("tensor parallelism shards the tokens of ONE sequence per step (batch 1)")
        return tuple(y.unsqueeze(0) for y in column_parallel_multi(x[0], ws, _slab_view(ws), tp))
    if attn.q_proj.bias is None and x.is_cuda:
        out = ops_fused_linear(x, ws)
        if out is not None:
            if torch.is_grad_enabled() and out[0].requires_grad:
                from ..ops import cuda
                cuda.GradSlab.tag(out, [w.shape[0] for w in ws])      # their gradients will meet in one buffer
            return out
    handle = getattr(attn.q_proj.weight, "_ttcd_gather", None)
    if handle is not None:              # sharded weights: no fused projection will gather the block, do it now
        attn.q_proj.weight._ttcd_gather = None
        handle.ensure()
    return (ops.linear(x, attn.q_proj.weight, attn.q_proj.bias),
            ops.linear(x, attn.k_proj.weight, attn.k_proj.bias),
            ops.linear(x, attn.v_proj.weight, attn.v_proj.bias))


def ops_fused_linear(x, weights: list[torch.Tensor]):
    """y_i = x @ W_i^T for several weights through one GEMM launch (native path only)."""
    from .. import _native
    if not _native.use_native(x):
        return None
    from ..ops import cuda
    return cuda.fused_linear(x, weights, _slab_view(weights))


class GatedMLP(nn.Module):
    """SwiGLU MLP: down(swish(gate(x)) * up(x))."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def features(self, x):
        """swiglu(gate(x), up(x)) with the two projections fused into one GEMM when possible."""
        tp = _tp_state()
        if tp is not None:
            from ..parallel.tensor import column_parallel_multi
            ws = [self.gate_proj.weight, self.up_proj.weight]
            flat = x.reshape(-1, x.shape[-1])
            g, u = column_parallel_multi(flat, ws, _slab_view(ws), tp)
            return ops.swiglu(g, u).view(*x.shape[:-2], x.shape[-2] * tp.world, -1)
        out = ops_fused_linear(x, [self.gate_proj.weight, self.up_proj.weight]) if x.is_cuda else None
        if out is not None:
            return ops.swiglu(out[0], out[1])
        return ops.swiglu(ops.linear(x, self.gate_proj.weight), ops.linear(x, self.up_proj.weight))

    def forward(self, x, **_):
        tp = _tp_state()
        if tp is not None:
            from ..parallel.tensor import row_parallel_linear
            feats = self.features(x)
            y = row_parallel_linear(feats.reshape(-1, feats.shape[-1]), self.down_proj.weight, tp)
            return y.view(*x.shape[:-1], -1)
        return ops.linear(self.features(x), self.down_proj.weight)
