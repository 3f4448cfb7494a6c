"""Pipeline parallelism: manual stage split by layer name and a fill-drain micro-batch schedule over
point-to-point sends (the role of flame/models/pipeline_fla.py:30-162, which the reference ships but never
reaches: flame/train.py:234-237 raises).  Same status here: the trainer refuses
``--experimental.pipeline_parallel_degree > 1``; the pieces below are usable on their own and tested on CPU.

A stage owns a contiguous run of blocks; the first stage also owns the embedding, the last one the final
norm, the LM head and the loss.  Activations and their gradients travel with ``dist.send`` / ``dist.recv``
(NCCL p2p on GPUs, gloo on CPU).  Tied embeddings are not supported across stages (first and last stage
would both hold the matrix).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn


def stage_layer_ranges(num_layers: int, num_stages: int, split_points: list[str] | None = None) -> list[range]:
    """Block index ranges per stage.  ``split_points`` are names like ``layers.7``: a new stage starts there."""
    if split_points:
        starts = sorted(int(s.rsplit(".", 1)[1]) for s in split_points)
        if len(starts) != num_stages - 1 or any(not 0 < s < num_layers for s in starts):
            raise ValueError(f"{len(starts)} split points {starts} do not make {num_stages} stages of {num_layers} layers")
        edges = [0, *starts, num_layers]
    else:
        base, extra = divmod(num_layers, num_stages)
        edges = [0]
        for s in range(num_stages):
            edges.append(edges[-1] + base + (1 if s < extra else 0))
    return [range(a, b) for a, b in zip(edges[:-1], edges[1:])]


class PipelineStageModule(nn.Module):
    """The part of a causal-LM (``model.embeddings``, ``model.layers``, ``model.norm``, ``lm_head``) one stage runs."""

    def __init__(self, causal_lm: nn.Module, stage: int, num_stages: int, split_points: list[str] | None = None):
        super().__init__()
        inner = causal_lm.model
        if num_stages > 1 and getattr(causal_lm.config, "tie_word_embeddings", False):
            raise ValueError("tied embeddings cannot be split across pipeline stages")
        self.first, self.last = stage == 0, stage == num_stages - 1
        rng = stage_layer_ranges(len(inner.layers), num_stages, split_points)[stage]
        self.layer_ids = list(rng)
        self.layers = nn.ModuleList([inner.layers[i] for i in rng])
        self.embeddings = inner.embeddings if self.first else None
        self.norm = inner.norm if self.last else None
        self.lm_head = causal_lm.lm_head if self.last else None

    def forward(self, x: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        h = self.embeddings(x) if self.first else x
        for layer in self.layers:
            h = layer(h)
        if not self.last:
            return h
        logits = self.lm_head(self.norm(h))
        if labels is None:
            return logits
        return F.cross_entropy(logits[:, :-1].float().flatten(0, 1), labels[:, 1:].flatten(), ignore_index=-100)


class FillDrainSchedule:
    """All micro-batches forward, then all backward in reverse order (GPipe).  ``step`` returns the mean loss on
    the last stage (None elsewhere); parameter gradients accumulate in ``.grad`` scaled by 1/n_microbatches."""

    def __init__(self, stage: PipelineStageModule, stage_index: int, num_stages: int, group=None,
                 hidden_size: int | None = None, dtype: torch.dtype = torch.float32, device="cpu"):
        self.stage, self.idx, self.n, self.group = stage, stage_index, num_stages, group
        self.hidden, self.dtype, self.device = hidden_size, dtype, torch.device(device)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
        self.prev = ranks[stage_index - 1] if stage_index > 0 else None
        self.next = ranks[stage_index + 1] if stage_index < num_stages - 1 else None

    def step(self, input_ids: torch.Tensor, labels: torch.Tensor, n_microbatches: int):
        ids_mb, lab_mb = input_ids.chunk(n_microbatches), labels.chunk(n_microbatches)
        inputs, outputs, losses = [], [], []
        for ids, lab in zip(ids_mb, lab_mb):
            if self.stage.first:
                x = ids.to(self.device)
            else:
                x = torch.empty(ids.shape[0], ids.shape[1], self.hidden, dtype=self.dtype, device=self.device)
                dist.recv(x, src=self.prev, group=self.group)
                x.requires_grad_()
            out = self.stage(x, lab.to(self.device) if self.stage.last else None)
            if self.stage.last:
                losses.append(out.detach())
            else:
                dist.send(out.detach().contiguous(), dst=self.next, group=self.group)
            inputs.append(x)
            outputs.append(out)
        for x, out in zip(reversed(inputs), reversed(outputs)):
            if self.stage.last:
                (out / n_microbatches).backward()
            else:
                g = torch.empty_like(out)
                dist.recv(g, src=self.next, group=self.group)
                out.backward(g)
            if not self.stage.first:
                dist.send(x.grad.contiguous(), dst=self.prev, group=self.group)
        return torch.stack(losses).mean() if losses else None
