"""Selective activation checkpointing at the level of this library's ops.

The reference's ``--activation_checkpoint.mode selective --activation_checkpoint.selective_ac_option op`` saves the
outputs of the expensive ops (matmuls, attention) and recomputes the cheap ones in backward
(flame/models/parallelize_fla.py:313-371).  The ops here are autograd Functions around opaque kernel launches, so the
same policy is stated where the launches happen: a block runs under ``torch.utils.checkpoint`` (its saved tensors are
dropped and rebuilt by re-running the block in backward), and every Function that owns a tensor-core launch wraps it
in ``keep(...)``: the first run records the launch's outputs in the block's ``OpCache``; the re-run takes them from
there instead of launching again.  What is recomputed in backward is therefore only the norm / rotary / SwiGLU /
depthwise-conv / element-wise work; what stays resident between forward and backward is the GEMM and attention
outputs (about 64 % of a block's activations at the Qwen3-0.6B shape).
"""
from __future__ import annotations

import threading
from contextlib import contextmanager

import torch

_state = threading.local()


class OpCache:
    """Outputs of the kept launches of ONE checkpointed block call, in launch order."""

    def __init__(self):
        self.items: list = []
        self.pos = 0
        self.recorded = False

    @contextmanager
    def scope(self):
        """First entry records, every later entry (the recomputation in backward) replays."""
        prev = getattr(_state, "cache", None)
        self.pos = 0
        _state.cache = self
        try:
            yield self
        finally:
            _state.cache = prev
            if not self.recorded:
                self.recorded = True
            else:
                self.items = []          # replayed once: the recomputed graph owns the tensors now


def current() -> OpCache | None:
    return getattr(_state, "cache", None)


def _alias(x):
    if isinstance(x, torch.Tensor):
        return x.detach()
    if isinstance(x, (tuple, list)):
        return type(x)(_alias(v) for v in x)
    return x


def keep(compute):
    """Run ``compute()`` (a tensor-core launch returning a tensor or a tuple of tensors), or, inside the
    recomputation of a checkpointed block, return what its first run produced."""
    cache = current()
    if cache is None:
        return compute()
    if cache.recorded:
        if cache.pos >= len(cache.items):
            raise RuntimeError("selective recompute: the block launched more kept ops than its first run")
        out = cache.items[cache.pos]
        cache.items[cache.pos] = None
        cache.pos += 1
        return _alias(out)
    out = compute()
    cache.items.append(_alias(out))
    return out
