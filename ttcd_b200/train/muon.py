"""Muon for the flat-buffer sharded runtime: owner-compute Newton–Schulz with the gradient gather fused
into the reduction.

Behaviour follows the reference optimizer (custom_components/muon_v2.py:587-1310): Muon is applied to
parameters with ``ndim >= 2`` that are not embeddings, the LM head or the final norm (513-515), with
Nesterov momentum ``buf = g + mu*buf; g = g + mu*buf`` (904-912), five fixed-coefficient Newton–Schulz
iterations in bf16 (30-65), the update ``p *= 1 - lr*wd; p -= lr*0.2*sqrt(max(rows, cols)) * u`` (707-716,
914-919); everything else uses AdamW.  Ownership: parameters are sorted by Newton–Schulz cost and dealt
round-robin over the ranks (739-796).

Where the reference moves gradient shards to the owner with two ``all_to_all_single`` calls per chunk of
parameters and scatters the update back the same way, here the owner's reduction kernel *pulls* the
parameter's gradient from every peer's flat gradient buffer over NVLink while summing, casting and
scaling (one kernel, no staging), runs the orthogonalisation on the tcgen05 GEMM (A = XX^T, B = bA + cA^2,
X = aX + BX with alpha/beta epilogues), and stores the new bf16 weights straight into every peer's flat
parameter buffer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _native, ops

MUON_EXCLUDE = ("embeddings", "lm_head", "model.norm")


def default_is_muon(name: str, param: torch.Tensor) -> bool:
    return param.ndim >= 2 and not any(key in name for key in MUON_EXCLUDE)


def ns_cost(shape) -> int:
    rows, cols = int(shape[-2]), int(shape[-1])
    small, large = min(rows, cols), max(rows, cols)
    return int(math.prod(shape[:-2])) * small * small * large


@dataclass
class MuonParam:
    name: str
    param: torch.nn.Parameter
    group_index: int
    offset: int                 # element offset inside the group's flat buffers
    owner: int = 0
    master: torch.Tensor | None = None      # fp32, owner only
    momentum: torch.Tensor | None = None    # fp32, owner only
    grad32: torch.Tensor | None = None      # fp32 reduced gradient, owner only
    tp_dim: int | None = None               # tensor parallelism: the dimension along which ``param`` is a 1/tp slice


def assign_owners(params: list[MuonParam], world: int) -> None:
    order = sorted(range(len(params)), key=lambda i: -ns_cost(params[i].param.shape))
    for k, i in enumerate(order):
        params[i].owner = k % world


def orthogonalize(g: torch.Tensor) -> torch.Tensor:
    """Newton–Schulz on a 2-D gradient (3-D parameters are treated as a batch over the first dim)."""
    if g.dim() == 2:
        return ops.newton_schulz(g)
    g3 = g.reshape(-1, g.shape[-2], g.shape[-1])     # independent matrices over the leading dims (312-309, 820-826)
    if min(g3.shape[-2:]) < 64:
        # depthwise-conv taps and the like: a few scalars per matrix, not tensor-core work
        from ..ops import reference as ref_ops
        return ref_ops.newton_schulz(g3).reshape(g.shape)
    return ops.newton_schulz(g3).reshape(g.shape)


def muon_update(mp: MuonParam, lr: float, weight_decay: float, momentum: float, coef: torch.Tensor | None,
                nesterov: bool = True, skip: torch.Tensor | None = None) -> torch.Tensor:
    """Owner-side update of one parameter; returns the new fp32 master (in place).  ``skip``: device int
    scalar, non-zero when the step must leave momentum and weights untouched (non-finite gradient norm)."""
    muon_update_many([mp], lr, weight_decay, momentum, coef, nesterov, skip)
    return mp.master


def muon_update_many(params: list[MuonParam], lr: float, weight_decay: float, momentum: float,
                     coef: torch.Tensor | None, nesterov: bool = True, skip: torch.Tensor | None = None, tp=None) -> None:
    """Owner-side update of several parameters.  Parameters of one shape are orthogonalised as ONE batched
    Newton-Schulz call (15 GEMM launches for the whole group instead of 15 per matrix: the matrices of a 1024-wide
    model are a handful of tiles each, so per-matrix launches are pure latency); the reference batches the same way
    for its 3-D case (custom_components/muon_v2.py:68-110).

    ``tp`` (an object with ``group``, ``rank``, ``world``): under tensor parallelism a weight is a slice of its matrix
    along ``mp.tp_dim``.  Momentum is element-wise and stays on the slice; for the orthogonalisation the slices of
    the group's ranks are gathered into the whole matrix (every rank of the group then runs the same Newton-Schulz
    and keeps its slice of the result), and the update's scale uses the whole matrix's dimensions.  All ranks of a
    tensor-parallel group hold the same parameters in the same order, so they issue the same gathers."""
    if not params:
        return
    pre = []                          # (param, momentum after this step, Nesterov-combined gradient)
    for mp in params:
        g = mp.grad32 if coef is None else mp.grad32 * coef
        new_mom = mp.momentum * momentum + g
        g = g.add(new_mom, alpha=momentum) if nesterov else new_mom
        pre.append((mp, new_mom, g))

    def gathers(mp) -> bool:            # a slice of the matrix itself (not of a leading batch dimension)
        return tp is not None and tp.world > 1 and mp.tp_dim is not None and mp.tp_dim >= mp.param.dim() - 2

    def whole(x: torch.Tensor, dim: int) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(tp.world)]
        dist.all_gather(parts, x.contiguous(), group=tp.group)
        return torch.cat(parts, dim=dim)

    def mine(x: torch.Tensor, dim: int) -> torch.Tensor:
        per = x.shape[dim] // tp.world
        return x.narrow(dim, tp.rank * per, per)

    by_shape: dict[tuple, list[int]] = {}
    for i, (mp, _, _) in enumerate(pre):
        by_shape.setdefault((tuple(mp.param.shape), mp.tp_dim if gathers(mp) else None), []).append(i)
    updates: list[torch.Tensor | None] = [None] * len(pre)
    for (shape, dim), idx in by_shape.items():
        full_min = min(s_ * (tp.world if dim == k else 1) for k, s_ in enumerate(shape[-2:], start=len(shape) - 2)) \
            if dim is not None else min(shape[-2:])
        if len(shape) == 2 and full_min >= 64 and (len(idx) > 1 or dim is not None):
            stacked = torch.stack([pre[i][2].view(shape) for i in idx])            # [n, rows, cols]
            if dim is not None:
                u = mine(ops.newton_schulz(whole(stacked, dim + 1)).float(), dim + 1)
            else:
                u = ops.newton_schulz(stacked).float()
            for j, i in enumerate(idx):
                updates[i] = u[j].reshape(-1)
        else:
            for i in idx:
                g = pre[i][2].view(shape)
                if dim is not None:
                    updates[i] = mine(orthogonalize(whole(g, dim)).float(), dim).reshape(-1)
                else:
                    updates[i] = orthogonalize(g).float().reshape(-1)
    for (mp, new_mom, _), u in zip(pre, updates):
        rows, cols = mp.param.shape[-2], mp.param.shape[-1]      # last two dims also for >2-D parameters (707-716)
        if gathers(mp):
            rows, cols = (rows * tp.world, cols) if mp.tp_dim == mp.param.dim() - 2 else (rows, cols * tp.world)
        adj_lr = lr * 0.2 * math.sqrt(max(rows, cols))
        new_master = (mp.master * (1.0 - lr * weight_decay)).add_(u, alpha=-adj_lr)
        if skip is not None:
            keep = skip == 0
            new_mom = torch.where(keep, new_mom, mp.momentum)
            new_master = torch.where(keep, new_master, mp.master)
        mp.momentum.copy_(new_mom)
        mp.master.copy_(new_master)
