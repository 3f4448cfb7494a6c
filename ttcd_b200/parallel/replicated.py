"""Replicated data parallelism (DDP): every rank keeps the whole optimizer state, gradients are all-reduced.

The reference reaches this through ``replicate(model, bucket_cap_mb=100)`` when only the replicate degree
of the data-parallel mesh is used (flame/models/parallelize_fla.py:100-108, 500-516).  Here it is the same
flat-buffer runtime as the sharded path with a different collective: one flat gradient buffer per block acts
as the bucket, its all-reduce (NCCL, or gloo on CPU) is launched on a side stream as soon as the block's last
gradient is ready, and the optimizer step runs on the full buffers of every rank.  It is the non-fused
fallback; the sharded runtime with its peer-memory kernels is the default.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .sharded import ParamGroup, ShardedDataParallel


class ReplicatedDataParallel(ShardedDataParallel):
    def __init__(self, model, blocks=None, process_group=None, **kwargs):
        self.dp_pg = process_group
        self.dp_world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        kwargs.pop("comm", None)
        super().__init__(model, blocks, process_group=False, comm="nccl", **kwargs)     # local optimizer over full buffers
        if self.dp_world > 1:
            if self.device.type == "cuda":
                self.comm_stream = torch.cuda.Stream()
            self._install_hooks()

    def _reduce_group(self, g: ParamGroup):
        if self.dp_world == 1:
            g.reduce_event = True
            return
        if self.comm_stream is None:
            g.flat_grad.mul_(1.0 / self.dp_world)
            dist.all_reduce(g.flat_grad, group=self.dp_pg)
            g.reduce_event = True
            return
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            g.flat_grad.mul_(1.0 / self.dp_world)
            dist.all_reduce(g.flat_grad, group=self.dp_pg)
            g.reduce_event = torch.cuda.Event()
            g.reduce_event.record(self.comm_stream)

    @torch.no_grad()
    def step(self, lr=None):
        for g in self.groups:
            if g.reduce_event is None:
                self._reduce_group(g)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return super().step(lr)
