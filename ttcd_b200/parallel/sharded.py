"""Flat-buffer sharded data-parallel runtime (the FSDP role of the reference).

The reference wraps every block and the root in PyTorch FSDP2 (flame/models/parallelize_fla.py:436-497):
bf16 parameters are all-gathered before each use and freed after, gradients are reduce-scattered in
fp32, and AdamW runs on fp32 DTensor shards.  On a 180 GB B200 a 0.6 B-parameter model does not need
to free its bf16 weights between uses, so this runtime is organised around that:

* per group (one per block + one root group) a **flat bf16 parameter buffer** stays resident and the
  module parameters are views into it, laid out in registration order so that q/k/v and gate/up
  weights are contiguous slabs (one GEMM each);
* a **flat bf16 gradient buffer** per group receives autograd's accumulation in place;
* each rank owns a contiguous 1/world **fp32 master shard** with its Adam moments.  Default transport
  (``comm='peer'``): the flat buffers live in peer-addressable memory; after a group's backward a flag barrier
  and ONE kernel pull this rank's shard of the gradients from every peer over NVLink, fused with the bf16->fp32
  cast, the 1/world scale and the squared-norm partial (overlapped with the remaining backward on a side
  stream); the fused AdamW kernel then stores the new bf16 values straight into every peer's flat parameter
  buffer.  ``comm='nccl'`` is the baseline: cast/scale kernel + ``reduce_scatter_tensor``, AdamW, and
  ``all_gather_into_tensor`` of the updated slices;
* gradient clipping uses device-side squared norms and a device-side coefficient: no host sync;
* a peer wait that runs out (a rank more than the wait budget late) sets a device-side word that every rank's
  optimizer kernels of that step honour (the step is skipped everywhere, agreed through the gradient-norm
  all-reduce), and ``check_health()`` turns it into an exception at the next point that already synchronises;
* with gradient accumulation the reduction runs once, after the last micro-batch (``set_last_microbatch``);
* ``shard_weights=True`` (the reference's ZeRO-3 / ``fully_shard`` layout, flame/models/parallelize_fla.py:436-497):
  a block's bf16 parameters are stored 1/world per rank and exist in full only while the block runs.  The gather is
  fused into the block's first GEMM (``csrc/gemm_comm.cu::wgather_gemm``: the fused q|k|v projection pulls every
  rank's shard of the whole block into a pooled buffer while it multiplies, tile flags ordering the two); the buffer
  is handed back after the block's forward and gathered again for its backward.  The root group (embeddings, final
  norm, LM head) stays resident.

``world_size == 1`` degenerates to flat buffers + fused AdamW with no communication.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _native
from ..ops import reference as ref_ops


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclass
class ParamGroup:
    """One flat buffer: its parameters, their offsets, and this rank's optimizer shard."""

    name: str
    params: list[nn.Parameter]
    names: list[str]
    offsets: list[int] = field(default_factory=list)
    numel: int = 0             # padded to a multiple of 8 * world
    base: int = 0              # element offset of this group inside the symmetric gradient buffer
    pbase: int = 0             # element offset inside the symmetric (resident) parameter buffer
    total: int = 0             # numel (AdamW region) + the Muon-owned parameters laid out after it
    muon: list = field(default_factory=list)   # MuonParam entries of this group
    flat_param: torch.Tensor | None = None   # bf16 [numel]
    flat_grad: torch.Tensor | None = None    # bf16 [numel]
    master: torch.Tensor | None = None       # fp32 [numel / world]
    exp_avg: torch.Tensor | None = None
    exp_avg_sq: torch.Tensor | None = None
    grad_shard: torch.Tensor | None = None   # fp32 [numel / world] (world > 1)
    grad_full32: torch.Tensor | None = None  # fp32 [numel] staging for the reduce-scatter (world > 1)
    reduce_event: torch.cuda.Event | None = None
    pending_hooks: int = 0
    # sharded-weights mode (block groups only)
    sharded: bool = False
    shard_store: torch.Tensor | None = None  # bf16 [numel / world]: this rank's persistent shard of the parameters
    shard_base: int = 0                      # element offset of the shard inside the symmetric shard buffer
    head_elems: int = 0                      # leading elements that hold the < 2-D parameters (needed before the first GEMM)
    ready: torch.Tensor | None = None        # int32 [units]: flags of the fused gather
    epoch: int = 0
    pool_slot: int = -1                      # pooled full buffer currently holding the gathered parameters (-1: none)
    fixed_slot: int = 0                      # the pooled buffer this block always uses (block index % 2)
    gather: object = None                    # PendingGather while the block waits for its first GEMM
    in_backward: bool = False


class PendingGather:
    """A block whose sharded parameters are to be gathered by its first GEMM.

    ``linear(x, w)`` is called by the fused q|k|v projection: when the shapes fit the fused kernel it runs
    ``ttcd_wgather_gemm`` (the GEMM pulls every rank's shard of the whole block into the pooled buffer while it
    multiplies); otherwise it gathers with the stand-alone kernel and returns None so that the caller runs its
    ordinary GEMM.  Either way the block's parameters are complete, by stream order, for every later kernel."""

    def __init__(self, sdp, group, flat, shard_ptrs, shard_elems):
        self.sdp, self.group, self.flat, self.ptrs, self.shard = sdp, group, flat, shard_ptrs, shard_elems
        self.pending = True

    def ensure(self) -> None:
        if self.pending:
            self.pending = False
            _native.call("ttcd_peer_gather", _native.ptr(self.flat), self.ptrs, _native.i32(self.sdp.world),
                         _native.i64(self.shard), _native.stream_ptr())

    def linear(self, x2: torch.Tensor, w: torch.Tensor):
        """y = x2 @ w^T with ``w`` [N, K] a contiguous slice of the block's flat buffer; None if the shapes do not fit."""
        if not self.pending:
            return None
        M, K = x2.shape
        N = w.shape[0]
        off = (w.data_ptr() - self.flat.data_ptr()) // 2
        fits = (M % 128 == 0 and N % 256 == 0 and K % 64 == 0 and x2.stride(1) == 1 and x2.stride(0) % 8 == 0
                and w.is_contiguous() and 0 <= off and off + N * K <= self.flat.numel() and off % 8 == 0
                and x2.data_ptr() % 16 == 0)
        if not fits:
            self.ensure()
            return None
        self.pending = False
        g = self.group
        y = torch.empty(M, N, dtype=x2.dtype, device=x2.device)
        _native.call("ttcd_wgather_gemm", _native.ptr(x2), _native.ptr(y), _native.ptr(self.flat), self.ptrs, _native.ptr(g.ready),
                     _native.i32(self.sdp.rank), _native.i32(self.sdp.world), _native.i64(M), _native.i64(N), _native.i64(K),
                     _native.i64(x2.stride(0)), _native.i64(N), _native.i64(off), _native.i64(self.shard), _native.i32(0),
                     _native.i32(g.epoch), _native.i64(self.sdp.peer_wait_ns), _native.stream_ptr())
        return y


class ShardedDataParallel:
    """Owns the flat buffers of ``model`` and performs the sharded optimizer step."""

    def __init__(self, model: nn.Module, blocks: list[nn.Module] | None = None,
                 process_group: dist.ProcessGroup | None = None, *, lr: float = 1e-4, betas=(0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.1, max_norm: float | None = 1.0,
                 param_dtype: torch.dtype = torch.bfloat16, overlap: bool = True, comm: str | None = None,
                 muon: bool = False, muon_momentum: float = 0.95, muon_filter=None, peer_wait_ns: int = 0,
                 replicate_group: dist.ProcessGroup | None = None, shard_weights: bool = False, tensor_parallel=None):
        """``comm``: 'peer' = fused peer-memory kernels over NVLink (default on CUDA with the native
        library), 'nccl' = the NCCL reduce-scatter / all-gather baseline (also TTCD_COMM=nccl).
        ``peer_wait_ns``: budget of one peer-flag wait (0: the library default of 10 s).
        ``replicate_group``: hybrid sharding (the reference's HSDP mesh, flame/models/parallelize_fla.py:75-78):
        ``process_group`` shards the optimizer state, and the ranks of ``replicate_group`` (one per shard group,
        holding the same shard) average their reduced gradient shards with an all-reduce before the update.
        ``tensor_parallel``: the tensor-parallel state (``group``, ``rank``, ``world``) when the model's weights are
        1/tp slices; Muon then orthogonalises the whole matrices (train/muon.py)."""
        import os
        self.tensor_parallel = tensor_parallel
        self.shard_weights = bool(shard_weights)
        self.replicate_pg = replicate_group
        self.replicate_world = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.peer_wait_ns = int(peer_wait_ns or os.environ.get("TTCD_PEER_WAIT_NS", "0"))
        self.model = model
        self.comm = comm or os.environ.get("TTCD_COMM", "peer")
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_initialized() and process_group is not False) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.lr, self.betas, self.eps, self.weight_decay, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.param_dtype = param_dtype
        self.step_count = 0
        self.overlap = overlap
        first = next(model.parameters())
        self.device = first.device
        self.use_native = self.device.type == "cuda" and param_dtype == torch.bfloat16 and _native.available()
        if self.device.type == "cuda" and param_dtype == torch.bfloat16 and not self.use_native:
            _native.load(required=not _native.torch_fallback_allowed())
        self.peer = self.world > 1 and self.use_native and self.comm == "peer"
        self.muon_enabled, self.muon_momentum, self.muon_filter = muon, muon_momentum, muon_filter
        self.norm_sq_hook = None
        self.muon_params: list = []
        self.sym_params = self.sym_grads = self.barrier = None
        # [sum of squared gradients, "a peer wait ran out" (set by the barrier kernel)]: all-reduced together
        self._stats = torch.zeros(2, dtype=torch.float32, device=self.device)
        self.groups: list[ParamGroup] = []
        self._build_groups(blocks)
        self.comm_stream = torch.cuda.Stream() if (self.device.type == "cuda" and self.world > 1) else None
        self._norm_sq = self._stats[0:1]
        self._fail = self._stats[1:2]
        self._last_microbatch = True
        self._failed_steps = torch.zeros(1, dtype=torch.float32, device=self.device)   # steps skipped after a wait ran out
        self._coef = torch.ones(1, dtype=torch.float32, device=self.device)
        self._skip = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.last_grad_norm: torch.Tensor | None = None
        self.skip_nan_inf = False
        if self.world > 1:
            self._install_hooks()
        if self.shard_weights and self.world > 1:
            self._install_shard_hooks(blocks)

    # ---------------------------------------------------------------------------------- layout
    def _build_groups(self, blocks):
        seen: set[int] = set()
        groups: list[ParamGroup] = []
        blocks = list(blocks) if blocks is not None else []
        for i, blk in enumerate(blocks):
            ps, ns = [], []
            for n, p in blk.named_parameters():
                if id(p) not in seen:
                    seen.add(id(p)); ps.append(p); ns.append(n)
            if ps:
                groups.append(ParamGroup(f"block{i}", ps, ns))
        ps, ns = [], []
        for n, p in self.model.named_parameters():
            if id(p) not in seen:
                seen.add(id(p)); ps.append(p); ns.append(n)
        if ps:
            groups.append(ParamGroup("root", ps, ns))
        global_names = {id(p): n for n, p in self.model.named_parameters()}
        from ..train.muon import MuonParam, assign_owners, default_is_muon
        is_muon = self.muon_filter or default_is_muon
        for gi, g in enumerate(groups):
            pairs = list(zip(g.params, g.names))
            chosen = [(p, n) for p, n in pairs if self.muon_enabled and p.requires_grad and is_muon(global_names[id(p)], p)
                      and p.numel() % 8 == 0]      # 16-byte granules for the vectorised pull/push kernels
            chosen_ids = {id(p) for p, _ in chosen}
            adam = [(p, n) for p, n in pairs if id(p) not in chosen_ids]
            g.sharded = self.shard_weights and self.world > 1 and g.name != "root"
            if g.sharded:
                if chosen:
                    raise NotImplementedError("sharded weights are not combined with Muon (it needs whole matrices)")
                adam.sort(key=lambda pn: 0 if pn[0].dim() < 2 else 1)     # norm weights etc. first: needed before the first GEMM
            off = 0
            for p, _ in adam:
                g.offsets.append(off)
                off += _align(p.numel(), 8)          # 16-byte aligned starts (TMA / vector loads)
            if g.sharded:
                g.head_elems = sum(_align(p.numel(), 8) for p, _ in adam if p.dim() < 2)
                g.numel = _align(off, 32768 * self.world)      # 64 KB units per shard: flag granularity of the fused gather
            else:
                g.numel = _align(off, 8 * self.world)    # AdamW region: sharded 1/world by flat position
            off = g.numel
            for p, n in chosen:                      # Muon region: whole parameters, owned by one rank each
                g.offsets.append(off)
                mp = MuonParam(global_names[id(p)], p, gi, off)
                spec = getattr(p, "_tp_shard", None)
                mp.tp_dim = None if spec is None else int(spec[0])
                g.muon.append(mp)
                self.muon_params.append(mp)
                off += _align(p.numel(), 8)
            g.total = _align(off, 8)
            g.params = [p for p, _ in adam] + [p for p, _ in chosen]
            g.names = [n for _, n in adam] + [n for _, n in chosen]
        assign_owners(self.muon_params, self.world)
        total = sum(g.total for g in groups)
        shard_total = sum(g.numel // self.world for g in groups if g.sharded)
        self.sym_shards = None
        if shard_total:
            esz = torch.empty((), dtype=self.param_dtype).element_size()
            if self.peer:
                from ..comm.symmetric import SymmetricBuffer
                self.sym_shards = SymmetricBuffer(shard_total * esz, self.pg, self.device)
                shard_flat = self.sym_shards.view(self.param_dtype, shard_total, 0)
            else:
                shard_flat = torch.zeros(shard_total, dtype=self.param_dtype, device=self.device)
            pool_numel = max(g.total for g in groups if g.sharded)
            self._pool = [torch.empty(pool_numel, dtype=self.param_dtype, device=self.device) for _ in range(2)]
            self._pool_owner: list = [None, None]
        if self.peer:
            # flat parameters and gradients live in peer-addressable memory: the fused kernels read every
            # rank's gradients and write every rank's parameters directly over NVLink
            from ..comm.symmetric import PeerBarrier, SymmetricBuffer
            esize = torch.empty((), dtype=self.param_dtype).element_size()
            resident = sum(g.total for g in groups if not g.sharded)
            self.sym_params = SymmetricBuffer(max(resident, 8) * esize, self.pg, self.device)
            self.sym_grads = SymmetricBuffer(total * esize, self.pg, self.device)
            self.barrier = PeerBarrier(self.pg, slots=4, wait_ns=self.peer_wait_ns, fail=self._stats[1:2])
        base = 0
        pbase = 0
        sbase = 0
        for g in groups:
            g.base = base
            g.pbase = pbase
            if self.peer:
                if g.sharded:       # a temporary full copy, only to lay the parameters out
                    g.flat_param = torch.zeros(g.total, dtype=self.param_dtype, device=self.device)
                else:
                    g.flat_param = self.sym_params.view(self.param_dtype, g.total, pbase * esize)
                    pbase += g.total
                g.flat_grad = self.sym_grads.view(self.param_dtype, g.total, base * esize)
            else:
                g.flat_param = torch.zeros(g.total, dtype=self.param_dtype, device=self.device)
                g.flat_grad = torch.zeros(g.total, dtype=self.param_dtype, device=self.device)
            base += g.total
            if g.sharded:
                g.shard_base = sbase
                g.shard_store = shard_flat[sbase:sbase + g.numel // self.world]
                sbase += g.numel // self.world
                if self.peer:
                    g.ready = torch.zeros(g.numel * 2 // 65536, dtype=torch.int32, device=self.device)
            for p, o in zip(g.params, g.offsets):
                view = g.flat_param[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = g.flat_grad[o:o + p.numel()].view(p.shape)
            shard = g.numel // self.world
            lo = self.rank * shard
            g.master = g.flat_param[lo:lo + shard].float()
            if g.sharded:
                g.shard_store.copy_(g.flat_param[lo:lo + shard])
            g.exp_avg = torch.zeros(shard, dtype=torch.float32, device=self.device)
            g.exp_avg_sq = torch.zeros(shard, dtype=torch.float32, device=self.device)
            if self.world > 1:
                g.grad_shard = torch.zeros(shard, dtype=torch.float32, device=self.device)
                if not self.peer:
                    g.grad_full32 = torch.empty(g.numel, dtype=torch.float32, device=self.device)
            for mp in g.muon:
                if mp.owner == self.rank:
                    n = mp.param.numel()
                    mp.master = g.flat_param[mp.offset:mp.offset + n].float()
                    mp.momentum = torch.zeros(n, dtype=torch.float32, device=self.device)
                    mp.grad32 = torch.zeros(_align(n, 8), dtype=torch.float32, device=self.device)
        self.groups = groups
        if shard_total:
            # the full copies of the sharded groups were only needed to lay the parameters out: the symmetric parameter
            # buffer keeps the root group, the blocks' parameters now live in the shards and, while a block runs, in a
            # pooled buffer
            for g in groups:
                if g.sharded:
                    g.flat_param = None
                    self._point_params(g, self._pool[0])

    def _own_slice(self, g: ParamGroup) -> torch.Tensor:
        """This rank's 1/world of the group's bf16 parameters (a slice of the resident flat buffer, the persistent
        shard, or, inside ``full_parameters()``, a slice of the temporary full copy)."""
        shard = g.numel // self.world
        if g.sharded and g.flat_param is None:
            return g.shard_store
        return g.flat_param[self.rank * shard:(self.rank + 1) * shard]

    def resync_master(self) -> None:
        """Re-derive the fp32 master shards from the current bf16 parameters (after a weight load)."""
        for g in self.groups:
            g.master.copy_(self._own_slice(g).float())
            for mp in g.muon:
                if mp.master is not None:
                    mp.master.copy_(g.flat_param[mp.offset:mp.offset + mp.param.numel()].float())

    def load_full_master(self, full: dict[int, torch.Tensor]) -> None:
        """Take full-precision parameter values (``{param.data_ptr(): fp32 tensor of the parameter's shape}``, e.g. as
        read from a checkpoint) into this rank's fp32 master shards; entries that are missing or not fp32 keep the
        value derived from the bf16 parameter."""
        for g in self.groups:
            shard = g.numel // self.world
            lo, hi = self.rank * shard, (self.rank + 1) * shard
            muon = {id(mp.param): mp for mp in g.muon}
            for p, o in zip(g.params, g.offsets):
                src = full.get(p.data_ptr())
                if src is None or src.dtype != torch.float32 or src.numel() != p.numel():
                    continue
                src = src.reshape(-1)
                mp = muon.get(id(p))
                if mp is not None:
                    if mp.master is not None:
                        mp.master.copy_(src)
                    continue
                a, b = max(o, lo), min(o + p.numel(), hi)
                if a < b:
                    g.master[a - lo:b - lo].copy_(src[a - o:b - o])

    # ---------------------------------------------------------------------------------- sharded weights
    def _point_params(self, g: ParamGroup, flat: torch.Tensor) -> None:
        for p, o in zip(g.params, g.offsets):
            p.data = flat[o:o + p.numel()].view(p.shape)

    def _install_shard_hooks(self, blocks) -> None:
        by_name = {g.name: g for g in self.groups}
        inner = getattr(self.model, "model", None)
        for i, blk in enumerate(blocks or []):
            g = by_name.get(f"block{i}")
            if g is None or not g.sharded:
                continue

            def pre_fwd(module, args, g=g):
                # first forward, or the recomputation inside backward: the block's first GEMM gathers (fused)
                self._prepare_group(g, fused=True, module=module)

            def post_fwd(module, args, out, g=g):
                if not g.in_backward:
                    self._release_group(g)

            def pre_bwd(module, grad_out, g=g, blk=blk):
                g.in_backward = True
                recompute = bool(inner is not None and inner.gradient_checkpointing and inner._checkpoint_layer(blk))
                if not recompute:           # the backward kernels are the first consumers: gather up front
                    self._prepare_group(g, fused=False, module=module)

            def post_bwd(module, grad_in, grad_out, g=g):
                g.in_backward = False
                self._release_group(g)

            g.fixed_slot = i % 2
            blk.register_forward_pre_hook(pre_fwd)
            blk.register_forward_hook(post_fwd)
            blk.register_full_backward_pre_hook(pre_bwd)
            blk.register_full_backward_hook(post_bwd)

    def _prepare_group(self, g: ParamGroup, fused: bool, module=None) -> None:
        """Make the group's parameters addressable in full: take a pooled buffer, point the parameters at it and
        fill it, either at once (``fused=False``: one gather kernel / all-gather) or, for everything past the small
        1-D parameters, inside the block's first GEMM (``fused=True``; see ``PendingGather``)."""
        if g.pool_slot >= 0:
            return
        # a block always lands in the same pooled buffer: tensors that autograd saved in the forward (weights are saved
        # as views) must find the re-gathered values at the same addresses in the backward
        slot = g.fixed_slot
        if self._pool_owner[slot] is not None:
            raise RuntimeError(f"sharded weights: pooled buffer {slot} is still held by {self._pool_owner[slot].name} "
                               f"when {g.name} needs it (blocks must run one after the other)")
        self._pool_owner[slot] = g
        g.pool_slot = slot
        flat = self._pool[slot][:g.total]
        self._point_params(g, flat)
        shard = g.numel // self.world
        if not self.peer:
            dist.all_gather_into_tensor(flat[:g.numel], g.shard_store, group=self.pg)      # NCCL / gloo statement
            return
        ptrs = self.sym_shards.ptr_array(g.shard_base * 2)
        attn = getattr(module, "attn", None)
        if fused and attn is not None and hasattr(attn, "q_proj"):
            # the 1-D parameters (norm weights ...) are read before the first GEMM: they sit at the head of rank 0's shard
            if g.head_elems:
                _native.call("ttcd_peer_add", _native.ptr(flat), _native.i64(self.sym_shards.peer_ptrs[0] + g.shard_base * 2),
                             _native.i64(g.head_elems), _native.i32(0), _native.stream_ptr())
            g.epoch += 1
            g.gather = PendingGather(self, g, flat, ptrs, shard)
            attn.q_proj.weight._ttcd_gather = g.gather
            return
        _native.call("ttcd_peer_gather", _native.ptr(flat), ptrs, _native.i32(self.world), _native.i64(shard), _native.stream_ptr())

    def _release_group(self, g: ParamGroup) -> None:
        if g.pool_slot < 0:
            return
        if g.gather is not None:
            g.gather.pending = False
        g.gather = None
        self._pool_owner[g.pool_slot] = None
        g.pool_slot = -1

    def full_parameters(self):
        """Context manager: every sharded group's parameters materialised in full (checkpoint save / load,
        evaluation).  On exit this rank's slices are written back to its shards and the full copies dropped."""
        from contextlib import contextmanager

        @contextmanager
        def ctx():
            held = []
            for g in self.groups:
                if not g.sharded:
                    continue
                self._release_group(g)
                full = torch.empty(g.total, dtype=self.param_dtype, device=self.device)
                shard = g.numel // self.world
                if self.peer:
                    _native.call("ttcd_peer_gather", _native.ptr(full), self.sym_shards.ptr_array(g.shard_base * 2),
                                 _native.i32(self.world), _native.i64(shard), _native.stream_ptr())
                else:
                    dist.all_gather_into_tensor(full[:g.numel], g.shard_store, group=self.pg)
                g.flat_param = full
                self._point_params(g, full)
                held.append(g)
            try:
                yield self
            finally:
                for g in held:
                    shard = g.numel // self.world
                    g.shard_store.copy_(g.flat_param[self.rank * shard:(self.rank + 1) * shard])
                    g.flat_param = None
                    self._point_params(g, self._pool[0])
                if held and self.world > 1:
                    if self.device.type == "cuda":
                        torch.cuda.synchronize(self.device)
                    dist.barrier(group=self.pg)          # every rank's shard is written before anyone gathers again
        return ctx()

    # ---------------------------------------------------------------------------------- reduce-scatter
    def _install_hooks(self):
        """Launch a group's gradient reduce-scatter as soon as its last parameter gradient is ready."""
        for g in self.groups:
            for p in g.params:
                if p.requires_grad:
                    p.register_post_accumulate_grad_hook(self._make_hook(g))

    def _make_hook(self, g: ParamGroup):
        n_params = sum(1 for p in g.params if p.requires_grad)

        def hook(_param):
            g.pending_hooks += 1
            if g.pending_hooks == n_params:
                g.pending_hooks = 0
                if self.overlap and self._last_microbatch:
                    self._reduce_group(g)
        return hook

    def set_last_microbatch(self, last: bool) -> None:
        """Gradient accumulation: call with False before every micro-batch but the last one.  The flat gradient
        buffers accumulate locally and the reduction (which also takes the gradient norm) runs once, from the
        hooks of the last micro-batch or from ``step``."""
        self._last_microbatch = bool(last)

    def _reduce_group(self, g: ParamGroup):
        """Gradient reduce-scatter of one group into this rank's fp32 shard, on the side stream.

        peer mode: flag barrier (every rank's gradients of this group are complete), then ONE kernel pulls
        this rank's shard from every peer over NVLink and fuses the bf16->fp32 cast, the 1/world scale and
        the squared-norm partial.  nccl mode: cast/scale kernel + ``reduce_scatter_tensor``."""
        if self.comm_stream is None:
            # host tensors (gloo): all-reduce in fp32 and keep this rank's slice
            shard = g.numel // self.world
            g.grad_full32.copy_(g.flat_grad[:g.numel])
            g.grad_full32.mul_(1.0 / self.world)
            dist.all_reduce(g.grad_full32, group=self.pg)
            g.grad_shard.copy_(g.grad_full32[self.rank * shard:(self.rank + 1) * shard])
            self._reduce_muon_baseline(g)
            g.reduce_event = True
            return
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            if self.peer:
                from ..ops import cuda  # noqa: F401
                shard = g.numel // self.world
                self.barrier.sync(slot=0, stream=self.comm_stream)
                _native.call("ttcd_rs_cast_scale_norm", self.sym_grads.ptr_array(), _native.i32(self.world),
                             _native.i64(g.base + self.rank * shard), _native.i64(shard), _native.f32(1.0 / self.world),
                             _native.ptr(g.grad_shard), _native.ptr(self._norm_sq), _native.stream_ptr())
                for mp in g.muon:
                    # Muon: the owner pulls the WHOLE parameter's gradient from every peer while reducing
                    if mp.owner == self.rank:
                        _native.call("ttcd_rs_cast_scale_norm", self.sym_grads.ptr_array(), _native.i32(self.world),
                                     _native.i64(g.base + mp.offset), _native.i64(mp.grad32.numel()),
                                     _native.f32(1.0 / self.world), _native.ptr(mp.grad32), _native.ptr(self._norm_sq),
                                     _native.stream_ptr())
            else:
                if self.use_native:
                    from ..ops import cuda
                    cuda.cast_scale(g.flat_grad[:g.numel], g.grad_full32, 1.0 / self.world)
                else:
                    g.grad_full32.copy_(g.flat_grad[:g.numel])
                    g.grad_full32.mul_(1.0 / self.world)
                dist.reduce_scatter_tensor(g.grad_shard, g.grad_full32, group=self.pg)
                self._reduce_muon_baseline(g)
            g.reduce_event = torch.cuda.Event()
            g.reduce_event.record(self.comm_stream)

    def _reduce_muon_baseline(self, g: ParamGroup):
        """NCCL / gloo statement of the owner reduction: ``dist.reduce`` of each Muon parameter's gradient."""
        for mp in g.muon:
            n = mp.param.numel()
            buf = g.flat_grad[mp.offset:mp.offset + n].float().mul_(1.0 / self.world)
            dist.reduce(buf, dst=dist.get_global_rank(self.pg, mp.owner) if self.pg is not None else mp.owner, group=self.pg)
            if mp.owner == self.rank:
                mp.grad32[:n].copy_(buf)

    # ---------------------------------------------------------------------------------- step
    def zero_grad(self):
        self._last_microbatch = True
        if self.peer:
            self._norm_sq.zero_()       # the reduce kernels add into it; the fail word next to it is cleared in step()
        for g in self.groups:
            g.flat_grad.zero_()
            g.reduce_event = None
            g.pending_hooks = 0
            for p, o in zip(g.params, g.offsets):
                if p.grad is None or p.grad.data_ptr() != g.flat_grad.data_ptr() + o * g.flat_grad.element_size():
                    p.grad = g.flat_grad[o:o + p.numel()].view(p.shape)

    def _local_grad(self, g: ParamGroup) -> torch.Tensor:
        return g.grad_shard if self.world > 1 else g.flat_grad[:g.numel]

    def local_grad_slices(self, params) -> list[torch.Tensor]:
        """Views of this rank's (reduced) gradient shard that belong to ``params``, in group order.  Ranks with the
        same position in different data-parallel groups get slices of the same elements."""
        wanted = {id(p) for p in params}
        out = []
        for g in self.groups:
            shard = g.numel // self.world
            lo = self.rank * shard if self.world > 1 else 0
            hi = lo + shard
            grad = self._local_grad(g)
            muon = {id(mp.param): mp for mp in g.muon}
            for p, off in zip(g.params, g.offsets):
                if id(p) not in wanted:
                    continue
                if id(p) in muon:                       # whole parameter at its owner, nothing elsewhere
                    mp = muon[id(p)]
                    if mp.owner == self.rank and mp.grad32 is not None:
                        out.append(mp.grad32[:p.numel()])
                    continue
                a, b = max(off, lo), min(off + p.numel(), hi)
                if a < b:
                    out.append(grad[a - lo:b - lo])
        return out

    @torch.no_grad()
    def step(self, lr: float | None = None) -> torch.Tensor:
        """Clip (global norm), AdamW on the local shards, publish bf16 params.  Returns the grad norm
        as a device scalar (read it lazily; nothing here synchronises with the host)."""
        lr = self.lr if lr is None else lr
        self.step_count += 1
        cur = torch.cuda.current_stream() if self.device.type == "cuda" else None
        if self.world > 1:
            for g in self.groups:
                if g.reduce_event is None:
                    self._reduce_group(g)
            if self.comm_stream is not None:
                cur.wait_stream(self.comm_stream)
        if self.world == 1:
            for mp in self.muon_params:
                n = mp.param.numel()
                mp.grad32[:n].copy_(self.groups[mp.group_index].flat_grad[mp.offset:mp.offset + n])
        owned = [mp for mp in self.muon_params if mp.owner == self.rank]
        hybrid = self.replicate_world > 1
        if hybrid:
            # hybrid sharding: the ranks that hold the same shard in different shard groups average it
            for g in self.groups:
                grad = self._local_grad(g)
                dist.all_reduce(grad, group=self.replicate_pg)
                grad.mul_(1.0 / self.replicate_world)
            for mp in owned:
                dist.all_reduce(mp.grad32, group=self.replicate_pg)
                mp.grad32.mul_(1.0 / self.replicate_world)
        # ---- global grad norm (device side); in peer mode the reduce kernels already accumulated it
        if self.peer and not hybrid:
            pass
        elif self.use_native:
            self._norm_sq.zero_()
            from ..ops import cuda
            for g in self.groups:
                cuda.sumsq(self._local_grad(g), self._norm_sq)
            for mp in owned:
                cuda.sumsq(mp.grad32, self._norm_sq)
        else:
            self._norm_sq.zero_()
            for g in self.groups:
                self._norm_sq += self._local_grad(g).float().pow(2).sum()
            for mp in owned:
                self._norm_sq += mp.grad32.pow(2).sum()
        if self.world > 1:
            # the "a wait ran out" word travels with the norm, so that every rank takes the same decision
            dist.all_reduce(self._stats if self.peer else self._norm_sq, group=self.pg)
        if self.norm_sq_hook is not None:      # e.g. tensor parallelism: add the other ranks' weight shards
            self.norm_sq_hook(self._norm_sq)
        norm = self._norm_sq.sqrt()
        self.last_grad_norm = norm
        if self.max_norm is not None:
            torch.clamp(self.max_norm / (norm + 1e-6), max=1.0, out=self._coef)
        else:
            self._coef.fill_(1.0)
        if self.peer:
            failed = self._fail > 0
            self._failed_steps += failed.to(torch.float32)
            bad = failed | ~torch.isfinite(norm) if self.skip_nan_inf else failed
            self._skip.copy_(bad.to(torch.int32))
            self._fail.zero_()          # from here on the word collects the waits of the step's closing barrier
        elif self.skip_nan_inf:
            self._skip.copy_((~torch.isfinite(norm)).to(torch.int32))
        b1, b2 = self.betas
        for g in self.groups:
            shard = g.numel // self.world
            lo = self.rank * shard
            if g.sharded:
                # sharded weights: the update stays in this rank's shard; the next use gathers it
                if self.use_native:
                    from ..ops import cuda
                    cuda.adamw_step(g.master, g.grad_shard, g.exp_avg, g.exp_avg_sq, g.shard_store, lr=lr, beta1=b1, beta2=b2,
                                    eps=self.eps, weight_decay=self.weight_decay, step=self.step_count, coef=self._coef,
                                    skip=self._skip if (self.skip_nan_inf or self.peer) else None)
                elif not (self.skip_nan_inf and bool(self._skip)):
                    ref_ops.adamw_step(g.master, g.grad_shard.float() * self._coef, g.exp_avg, g.exp_avg_sq, lr=lr, beta1=b1,
                                       beta2=b2, eps=self.eps, weight_decay=self.weight_decay, step=self.step_count)
                    g.shard_store.copy_(g.master)
                continue
            out_slice = g.flat_param[lo:lo + shard]
            if self.peer:
                bc1 = 1.0 - b1 ** self.step_count
                bc2_sqrt = math.sqrt(1.0 - b2 ** self.step_count)
                _native.call("ttcd_adamw_push", _native.ptr(g.master), _native.ptr(g.grad_shard), _native.ptr(g.exp_avg),
                             _native.ptr(g.exp_avg_sq), self.sym_params.ptr_array(), _native.i32(self.world),
                             _native.i64(g.pbase + lo), _native.i64(shard), _native.f32(lr), _native.f32(b1), _native.f32(b2),
                             _native.f32(self.eps), _native.f32(self.weight_decay), _native.f32(bc1), _native.f32(bc2_sqrt),
                             _native.ptr(self._coef), _native.ptr(self._skip), _native.stream_ptr())
                continue
            if self.use_native:
                from ..ops import cuda
                cuda.adamw_step(g.master, self._local_grad(g) if self.world > 1 else g.flat_grad[lo:lo + shard],
                                g.exp_avg, g.exp_avg_sq, out_slice, lr=lr, beta1=b1, beta2=b2, eps=self.eps,
                                weight_decay=self.weight_decay, step=self.step_count, coef=self._coef,
                                skip=self._skip if self.skip_nan_inf else None)
            elif self.skip_nan_inf and bool(self._skip):
                pass          # PyTorch statement of the step (CPU): the host may look at the flag
            else:
                grad = (self._local_grad(g) if self.world > 1 else g.flat_grad[lo:lo + shard]).float() * self._coef
                ref_ops.adamw_step(g.master, grad, g.exp_avg, g.exp_avg_sq, lr=lr, beta1=b1, beta2=b2, eps=self.eps,
                                   weight_decay=self.weight_decay, step=self.step_count)
                out_slice.copy_(g.master)
            if self.world > 1 and self.comm_stream is None:
                dist.all_gather_into_tensor(g.flat_param[:g.numel], out_slice.clone(), group=self.pg)
            elif self.world > 1:
                # publish: every rank contributes its updated slice; overlaps the next group's AdamW
                self.comm_stream.wait_stream(cur)
                with torch.cuda.stream(self.comm_stream):
                    dist.all_gather_into_tensor(g.flat_param[:g.numel], out_slice, group=self.pg)
        if self.muon_params:
            self._step_muon(lr, cur)
        if self.peer:
            # every rank's pushes have landed everywhere (and nobody still reads this rank's gradients)
            self.barrier.sync(slot=1)
        elif self.world > 1 and self.comm_stream is not None:
            cur.wait_stream(self.comm_stream)
        return norm

    def _step_muon(self, lr: float, cur) -> None:
        """Owner-side Muon updates (same-shape matrices orthogonalised as one batch), then publication of the new
        bf16 weights to every rank."""
        from ..train.muon import muon_update_many
        coef = self._coef if self.max_norm is not None else None
        owned = [mp for mp in self.muon_params if mp.owner == self.rank]
        saved = {}
        for mp in owned:
            saved[id(mp)] = mp.grad32
            mp.grad32 = mp.grad32[:mp.param.numel()]
        muon_update_many(owned, lr, self.weight_decay, self.muon_momentum, coef,
                         skip=self._skip if (self.skip_nan_inf or self.peer) else None, tp=self.tensor_parallel)
        for mp in owned:
            mp.grad32 = saved[id(mp)]
        for mp in self.muon_params:
            g = self.groups[mp.group_index]
            n = mp.param.numel()
            dst = g.flat_param[mp.offset:mp.offset + n]
            if mp.owner == self.rank:
                if self.peer:
                    n8 = n // 8 * 8
                    _native.call("ttcd_push_cast", _native.ptr(mp.master), self.sym_params.ptr_array(), _native.i32(self.world),
                                 _native.i64(g.pbase + mp.offset), _native.i64(n8), _native.stream_ptr())
                    if n8 != n:
                        dst[n8:].copy_(mp.master[n8:])
                else:
                    dst.copy_(mp.master)
            if self.world > 1 and not self.peer:
                src = dist.get_global_rank(self.pg, mp.owner) if self.pg is not None else mp.owner
                dist.broadcast(dst, src=src, group=self.pg)

    def close(self) -> None:
        """Give the device memory back: the symmetric buffers (peer mappings first, then this rank's allocation, after
        every rank has stopped using them), the optimizer state and the pooled weight buffers.  The model's parameters
        and gradients are views of those buffers, so the model is unusable afterwards."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.pg)
        for p in self.model.parameters():
            p.grad = None
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        for buf in (self.sym_params, self.sym_grads, getattr(self, "sym_shards", None),
                    None if self.barrier is None else self.barrier.buf):
            if buf is not None:
                buf.close()
        self.sym_params = self.sym_grads = self.sym_shards = self.barrier = None
        self._pool = []
        for g in self.groups:
            g.master = g.exp_avg = g.exp_avg_sq = g.flat_param = g.flat_grad = g.shard_store = None
            g.grad_shard = g.grad_full32 = None
        for mp in self.muon_params:
            mp.master = mp.momentum = mp.grad32 = None
        self.groups, self.muon_params = [], []
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def check_health(self) -> None:
        """Raise if a bounded device-side wait ran out since the last check (a peer was later than the wait budget,
        or a kernel's own pipeline stalled).  Synchronises the device: call it where the host already waits (a
        logging step, before a checkpoint).  The steps in question were skipped on every rank, so the weights
        are still consistent when this raises."""
        if self.device.type != "cuda" or not self.use_native:
            return
        torch.cuda.synchronize(self.device)
        code = _native.device_status()
        skipped = int(self._failed_steps.item())
        pending = float(self._fail.item()) > 0
        if code or skipped or pending:
            self._failed_steps.zero_()
            who = f"peer rank {code - 500} never arrived" if 500 <= code < 500 + 64 else f"code {code}"
            raise RuntimeError(f"rank {self.rank}: a bounded device wait ran out ({who}); {skipped} optimizer step(s) were "
                               "skipped on every rank, the weights are unchanged by them")

    # ---------------------------------------------------------------------------------- state
    def optimizer_state_dict(self) -> dict:
        return {
            "step": self.step_count,
            "groups": {g.name: {"master": g.master, "exp_avg": g.exp_avg, "exp_avg_sq": g.exp_avg_sq} for g in self.groups},
            "world": self.world, "rank": self.rank,
        }

    def load_optimizer_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step"])
        for g in self.groups:
            s = state["groups"][g.name]
            g.master.copy_(s["master"]); g.exp_avg.copy_(s["exp_avg"]); g.exp_avg_sq.copy_(s["exp_avg_sq"])
            self._own_slice(g).copy_(g.master)
        if self.world > 1:
            for g in self.groups:
                if g.sharded:
                    continue
                shard = g.numel // self.world
                dist.all_gather_into_tensor(g.flat_param, g.flat_param[self.rank * shard:(self.rank + 1) * shard].clone(),
                                            group=self.pg)

    # ---------------------------------------------------------------------------------- full (unsharded) views
    def _gather_flat(self, g: ParamGroup, which: str) -> torch.Tensor:
        shard = getattr(g, which)
        if self.world == 1:
            return shard
        full = torch.empty(g.numel, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.pg)
        return full

    def _global_names(self) -> dict[int, str]:
        return {id(p): n for n, p in self.model.named_parameters()}

    def gather_full(self, which: str = "master") -> dict[int, torch.Tensor]:
        """{param.data_ptr(): full fp32 tensor} rebuilt from every rank's shard of ``which``."""
        out = {}
        for g in self.groups:
            flat = self._gather_flat(g, which)
            muon_ids = {id(mp.param) for mp in g.muon}
            for p, o in zip(g.params, g.offsets):
                if id(p) in muon_ids:      # Muon-owned: the owner's fp32 master (the moments are not per element)
                    mp = next(m for m in g.muon if m.param is p)
                    if which != "master":
                        out[p.data_ptr()] = p.detach().float()
                        continue
                    buf = torch.zeros(p.shape, dtype=torch.float32, device=self.device)
                    if mp.owner == self.rank:
                        buf.copy_(mp.master.view(p.shape))
                    if self.world > 1:
                        dist.all_reduce(buf, group=self.pg)
                    out[p.data_ptr()] = buf
                else:
                    out[p.data_ptr()] = flat[o:o + p.numel()].view(p.shape)
        return out

    def full_optimizer_state(self, template: bool = False) -> dict[str, torch.Tensor]:
        """Per-parameter fp32 Adam moments (gathered), keyed by the global parameter name."""
        names = self._global_names()
        sd: dict[str, torch.Tensor] = {"step": torch.tensor(self.step_count, dtype=torch.int64)}
        for g in self.groups:
            flats = {}
            for which in ("exp_avg", "exp_avg_sq"):
                flats[which] = None if template else self._gather_flat(g, which)
            muon_ids = {id(mp.param) for mp in g.muon}
            for mp in g.muon:
                key = f"{mp.name}.momentum_buffer"
                buf = torch.zeros(mp.param.shape, dtype=torch.float32, device="cpu" if template else self.device)
                if not template:
                    if mp.owner == self.rank:
                        buf.copy_(mp.momentum.view(mp.param.shape))
                    if self.world > 1:
                        dist.all_reduce(buf, group=self.pg)
                sd[key] = buf
            for p, o in zip(g.params, g.offsets):
                if id(p) in muon_ids:
                    continue
                for which in ("exp_avg", "exp_avg_sq"):
                    key = f"{names[id(p)]}.{which}"
                    if template:
                        sd[key] = torch.empty(p.shape, dtype=torch.float32, device="cpu")
                    else:
                        sd[key] = flats[which][o:o + p.numel()].view(p.shape)
        return sd

    def load_full_optimizer_state(self, sd: dict[str, torch.Tensor]) -> None:
        names = self._global_names()
        self.step_count = int(sd["step"])
        for g in self.groups:
            shard = g.numel // self.world
            lo, hi = self.rank * shard, (self.rank + 1) * shard
            muon_ids = {id(mp.param) for mp in g.muon}
            for mp in g.muon:
                if mp.owner == self.rank and f"{mp.name}.momentum_buffer" in sd:
                    mp.momentum.copy_(sd[f"{mp.name}.momentum_buffer"].reshape(-1))
            for which in ("exp_avg", "exp_avg_sq"):
                dst = getattr(g, which)
                for p, o in zip(g.params, g.offsets):
                    if id(p) in muon_ids:
                        continue
                    src = sd[f"{names[id(p)]}.{which}"].reshape(-1)
                    a, b = max(o, lo), min(o + p.numel(), hi)
                    if a < b:
                        dst[a - lo:b - lo].copy_(src[a - o:b - o])

    def num_params(self) -> int:
        return sum(p.numel() for g in self.groups for p in g.params)
