"""Greedy decoding as one captured CUDA graph per token.

Eager decoding of a 28-layer model issues over a thousand small launches per token and is bound by the host; the
device work of a step (one pass over the weights and the key/value windows) is a fraction of a millisecond.  The
decode step therefore runs through ``StaticWindowCache`` (fixed addresses, positions and fill counts on the device),
is captured once per (batch, ring capacities) and replayed per token: the next token is chosen on the device and fed
back without the host seeing it; the host reads the tokens once at the end (or every few steps when it has to look
for an end-of-sequence token).

The reference decodes eagerly through HF ``generate`` (custom_models/ipttcd/modeling_ipttcdv9.py:794-850 for the
model side: fast weights are built during prefill only, a decode step is the plain windowed transformer step).
"""
from __future__ import annotations

import torch

from .layers import Attention, GatedMLP, StaticWindowCache, WindowKVCache


def pack_projection_weights(model) -> int:
    """Re-house q|k|v and gate|up weights of every block back to back in one buffer each, so that their projections
    run as ONE GEMM / GEMV without concatenating the weights per call.  Only touches weights that own their storage
    (a training runtime that keeps parameters as views of its flat buffers is left alone).  Returns how many groups
    were packed."""
    packed = 0
    for mod in model.modules():
        if isinstance(mod, Attention):
            group = [mod.q_proj, mod.k_proj, mod.v_proj]
        elif isinstance(mod, GatedMLP):
            group = [mod.gate_proj, mod.up_proj]
        else:
            continue
        ws = [lin.weight for lin in group]
        if any(lin.bias is not None for lin in group) or any(w.data._base is not None or not w.is_contiguous() for w in ws):
            continue
        if all(ws[i].data_ptr() + ws[i].numel() * ws[i].element_size() == ws[i + 1].data_ptr() for i in range(len(ws) - 1)):
            continue
        if len({(w.dtype, w.device, w.shape[1]) for w in ws}) != 1:
            continue
        slab = torch.cat([w.data for w in ws], dim=0)
        row = 0
        for w in ws:
            w.data = slab[row:row + w.shape[0]]
            row += w.shape[0]
        packed += 1
    return packed


def graph_decoding_supported(model, input_ids, attention_mask, do_sample: bool) -> bool:
    if do_sample or not input_ids.is_cuda or getattr(model.model, "cache_class", WindowKVCache) is not WindowKVCache:
        return False
    if attention_mask is not None and not bool(attention_mask.all()):
        return False
    if any(isinstance(m, Attention) and m.use_l2_softmax for m in model.modules()):
        return False
    from .. import _native
    return _native.available() and next(model.parameters()).dtype == torch.bfloat16


def _windows(model) -> dict[int, int | None]:
    return {m.layer_idx: m.window_size for m in model.modules() if isinstance(m, Attention)}


class GraphDecoder:
    """One captured decode step of ``model`` over a ``StaticWindowCache``; ``run`` replays it."""

    def __init__(self, model, source: WindowKVCache, max_new_tokens: int):
        self.model = model
        pack_projection_weights(model)
        self.cache = StaticWindowCache(source, _windows(model), max_new_tokens)
        batch = self.cache.positions.shape[0]
        dev = self.cache.pos.device
        self.token = torch.zeros(batch, 1, dtype=torch.long, device=dev)
        self.steps_capacity = max_new_tokens
        self.out = torch.zeros(batch, max_new_tokens, dtype=torch.long, device=dev)
        self.cursor = torch.zeros(1, dtype=torch.int64, device=dev)
        self.weights_at = self._weights_at()
        start = self.cache.start
        # warm-up on a side stream (allocator pools, rotary tables, lazily configured kernels), then rewind and capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._step()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.cache.reset(start)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step()
        self.load(source)                       # the warm-up step overwrote the oldest row of every ring
        self.tables = [m.rotary._cached for m in model.modules() if isinstance(m, Attention) and not m.use_nope]

    def _weights_at(self):
        return (self.model.lm_head.weight.data_ptr(), next(self.model.model.layers[0].parameters()).data_ptr())

    @torch.no_grad()
    def _step(self) -> None:
        logits = self.model(input_ids=self.token, past_key_values=self.cache, use_cache=True, logits_to_keep=1).logits
        self.last_logits = logits[:, -1]                 # (kept for inspection; lives in the graph's pool)
        nxt = self.last_logits.float().argmax(-1, keepdim=True)
        self.token.copy_(nxt)
        self.out.index_copy_(1, self.cursor, nxt)
        self.cursor.add_(1)
        self.cache.advance()

    def fits(self, source: WindowKVCache, max_new_tokens: int) -> bool:
        """Whether a new prompt's cache can reuse this capture (same shapes, rings large enough, same weights)."""
        if self._weights_at() != self.weights_at or max_new_tokens > self.steps_capacity:
            return False
        seen = {source.seen[i] for i in source.layers}
        if len(seen) != 1 or set(source.layers) != set(self.cache.layers):
            return False
        start = seen.pop()
        if start + max_new_tokens > self.cache.max_position:
            return False
        windows = _windows(self.model)
        for i, (k, _v) in source.layers.items():
            rk = self.cache.layers[i][0]
            if k.shape[0] != rk.shape[0] or k.shape[2:] != rk.shape[2:] or k.dtype != rk.dtype:
                return False
            cap = self.cache.capacity[i]
            if (windows.get(i) is not None and cap != windows[i]) or k.shape[1] > cap:
                return False
            if windows.get(i) is None and start + max_new_tokens > cap:
                return False
        return True

    def load(self, source: WindowKVCache) -> None:
        """Copy a new prompt's keys and values into the rings (addresses unchanged) and rewind the device state."""
        start = next(iter(source.seen.values()))
        for i, (k, v) in source.layers.items():
            rk, rv = self.cache.layers[i]
            n, cap = k.shape[1], self.cache.capacity[i]
            rows = torch.arange(start - n, start, device=k.device) % cap
            rk.index_copy_(1, rows, k)
            rv.index_copy_(1, rows, v)
        self.cache.start = start
        self.cache.reset(start)
        self.cursor.zero_()

    @torch.no_grad()
    def run(self, first_token: torch.Tensor, steps: int, eos: set[int], check_every: int = 16) -> torch.Tensor:
        """``first_token`` [B,1] (chosen from the prefill logits) is fed to the first replay; returns the ``steps``
        tokens that follow it, cut after the step at which every sample had produced an end-of-sequence token."""
        self.token.copy_(first_token)
        eos_t = torch.tensor(sorted(eos), device=self.token.device) if eos else None
        finished = torch.isin(first_token.squeeze(1), eos_t) if eos else None
        done = 0
        while done < steps:
            n = min(steps - done, check_every if eos else steps)
            for _ in range(n):
                self.graph.replay()
            self.cache.host_advance(n)
            done += n
            if eos:
                hit = torch.isin(self.out[:, :done], eos_t)
                hit[:, 0] |= finished
                all_done = hit.int().cummax(dim=1).values.bool().all(dim=0)          # per step: has every sample finished by now?
                if bool(all_done.any()):
                    done = int(all_done.float().argmax()) + 1
                    break
        return self.out[:, :done].clone()


def decoder_for(model, source: WindowKVCache, max_new_tokens: int) -> GraphDecoder:
    """The model's cached capture when the new prompt fits it, else a fresh one (kept for the next call)."""
    dec = getattr(model, "_graph_decoder", None)
    if dec is not None and dec.fits(source, max_new_tokens):
        dec.load(source)
        return dec
    model._graph_decoder = None                     # drop the old rings before allocating new ones
    dec = GraphDecoder(model, source, max_new_tokens)
    model._graph_decoder = dec
    return dec
