"""Training engine: model + sharded runtime + one-call train step.

This is the object the trainer entry point (``python -m flame.train``) and ``bench.py`` drive; it
plays the role of the reference's model-build / parallelize / optimizer section of
flame/train.py:299-470 and its hot loop body (563-700): forward, backward, gradient clipping,
optimizer step, with full or no activation checkpointing.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from ..models import IPTTCDv9Config, IPTTTConfig, TransformerConfig  # noqa: F401  (registers Auto classes)
from ..parallel.sharded import ShardedDataParallel


@dataclass
class EngineConfig:
    lr: float = 1e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-15
    weight_decay: float = 0.1
    max_norm: float | None = 1.0
    replicate: bool = False                   # DDP-style replicated optimizer state + gradient all-reduce (fallback path)
    replicate_degree: int = 1                 # hybrid sharding: this many shard groups, gradients averaged across them
    shard_weights: bool = False               # ZeRO-3: block parameters stored 1/world per rank, gathered inside the first GEMM
    activation_offload: bool = False          # saved activations -> pinned host memory on a side stream
    activation_checkpoint: str = "full"       # full | none | everyN (every Nth block) | ttt (TTT blocks only) | op (cheap ops only)
    dtype: torch.dtype = torch.bfloat16
    skip_nan_inf: bool = False
    seed: int = 42
    enable_muon: bool = False
    muon_momentum: float = 0.95
    tensor_parallel: int = 1
    context_parallel: int = 1


def load_model_config(path_or_cfg, **overrides):
    from transformers import AutoConfig
    if isinstance(path_or_cfg, (str, Path)):
        data = json.loads(Path(path_or_cfg).read_text())
        data.update(overrides)
        if "num_hidden_layers" in overrides and "ttt_layers" in data:
            data["ttt_layers"] = [i for i in data["ttt_layers"] if i < overrides["num_hidden_layers"]]
        model_type = data.pop("model_type")
        from ..models import MODEL_CLASSES
        if model_type in MODEL_CLASSES:
            return MODEL_CLASSES[model_type][0](**data)
        return AutoConfig.for_model(model_type, **data)
    for k, v in overrides.items():
        setattr(path_or_cfg, k, v)
    return path_or_cfg


def build_model(config, device, dtype, seed: int = 42):
    """Random-init model built directly on ``device`` in ``dtype`` (same seed on every rank)."""
    from transformers import AutoModelForCausalLM
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        from ..models import MODEL_CLASSES
        own = MODEL_CLASSES.get(getattr(config, "model_type", None))
        with torch.device(device):
            if own is not None and isinstance(config, own[0]):
                model = own[1](config)
            else:
                model = AutoModelForCausalLM.from_config(config)
    finally:
        torch.set_default_dtype(prev)
    model.to(device=device, dtype=dtype)
    model.tie_weights()
    return model


class TrainEngine:
    """``engine.train_step(input_ids, labels)`` runs one optimizer step and returns the loss."""

    def __init__(self, model_config, engine_config: EngineConfig | None = None, device=None,
                 process_group=None, model=None):
        self.cfg = engine_config or EngineConfig()
        self.device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.model_config = model_config
        self.model = model if model is not None else build_model(model_config, self.device, self.cfg.dtype, self.cfg.seed)
        self.model.train()
        self.set_activation_checkpointing(self.cfg.activation_checkpoint)
        if self.cfg.tensor_parallel > 1 or self.cfg.context_parallel > 1:
            from ..parallel import context as _ctx
            _ctx.configure(self, tensor_parallel=self.cfg.tensor_parallel, context_parallel=self.cfg.context_parallel)
        self.tp = getattr(self, "tp", None)
        self._tp_dp = False
        if self.tp is not None:
            world, rank = dist.get_world_size(), dist.get_rank()
            process_group = False           # every rank optimises its own weight shards
            if self.tp.world != world:
                # data parallel x tensor parallel: consecutive ranks form a tensor-parallel group, ranks with the
                # same position in their group hold the same weight shards and form a sharded data-parallel group
                for t in range(self.tp.world):
                    g = dist.new_group(list(range(t, world, self.tp.world)))
                    if rank % self.tp.world == t:
                        process_group = g
                self._tp_dp = True
        extra = {}
        if self.tp is not None and self.cfg.enable_muon:
            extra["tensor_parallel"] = self.tp          # Muon gathers the weight slices into whole matrices
        if self.cfg.shard_weights:
            if self.tp is not None or getattr(self, "cp", None) is not None or self.cfg.replicate:
                raise NotImplementedError("sharded weights are combined with plain sharded data parallelism only")
            extra["shard_weights"] = True
        if self.cfg.replicate_degree > 1 and not self.cfg.replicate:
            # hybrid sharding (replicate x shard): rank = r * S + s; a shard group holds the ranks with the same r,
            # a replicate group the ranks with the same s
            if self.tp is not None or getattr(self, "cp", None) is not None:
                raise NotImplementedError("hybrid sharding is not combined with tensor or context parallelism")
            world, rank = dist.get_world_size(), dist.get_rank()
            R = self.cfg.replicate_degree
            if world % R:
                raise ValueError(f"world size {world} is not divisible by the replicate degree {R}")
            S = world // R
            for r in range(R):
                g = dist.new_group(list(range(r * S, (r + 1) * S)))
                if rank // S == r:
                    process_group = g
            for s_ in range(S):
                g = dist.new_group(list(range(s_, world, S)))
                if rank % S == s_:
                    extra["replicate_group"] = g
        multi = process_group is not False and dist.is_initialized() and dist.get_world_size(process_group) > 1
        runtime = ShardedDataParallel
        if self.cfg.replicate and multi:
            from ..parallel.replicated import ReplicatedDataParallel as runtime
        self.sdp = runtime(
            self.model, blocks=list(self.model.model.layers), process_group=process_group if multi else False,
            lr=self.cfg.lr, betas=self.cfg.betas, eps=self.cfg.eps, weight_decay=self.cfg.weight_decay,
            max_norm=self.cfg.max_norm, param_dtype=self.cfg.dtype, muon=self.cfg.enable_muon,
            muon_momentum=self.cfg.muon_momentum, **extra)
        self.sdp.skip_nan_inf = self.cfg.skip_nan_inf
        if self.tp is not None:
            self.sdp.norm_sq_hook = self._tp_norm_sq
        self.world = self.sdp.world
        self._dev_ids = None
        self.last_loss: torch.Tensor | None = None
        self.last_logits: torch.Tensor | None = None      # detached logits of the last micro-batch, when the model makes them
        self.last_labels: torch.Tensor | None = None
        self.tokens_seen = 0

    # ------------------------------------------------------------------------------------------
    def set_activation_checkpointing(self, mode: str) -> None:
        """'full' recomputes every block in backward (the reference recipe, sized for 80 GB GPUs);
        'ttt' recomputes only the fast-weight blocks; 'everyN' every Nth block; 'op' recomputes the norm / rotary /
        SwiGLU / conv work of every block but keeps its GEMM and attention outputs; 'none' keeps all
        activations resident (fits at 64K tokens on a 180 GB B200)."""
        inner = self.model.model
        inner.gradient_checkpointing = mode != "none"
        inner.checkpoint_policy = mode if mode != "none" else "full"
        self.cfg.activation_checkpoint = mode

    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def forward_backward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, scale: float = 1.0,
                         **model_kwargs) -> torch.Tensor:
        ids = self._to_device(input_ids)
        lab = ids if labels is None else self._to_device(labels)
        cp = getattr(self, "cp", None)
        if cp is not None:
            return self._forward_backward_cp(ids, lab, scale, cp, **model_kwargs)
        if self.tp is not None:
            return self._forward_backward_tp(ids, lab, scale, **model_kwargs)
        from .activation_offload import get_act_offloading_ctx_manager
        with get_act_offloading_ctx_manager(self.cfg.activation_offload and self.device.type == "cuda"):
            out = self.model(input_ids=ids, labels=lab, **model_kwargs)
            loss = out.loss
        logits = getattr(out, "logits", None)
        self.last_logits = None if logits is None else logits.detach()
        self.last_labels = lab if logits is not None else None
        (loss * scale if scale != 1.0 else loss).backward()
        self.tokens_seen += ids.numel()
        return loss.detach()

    def _forward_backward_cp(self, ids, lab, scale, cp, **model_kwargs):
        """Context-parallel step: every rank of the group receives the same full sequences, shifts the
        labels globally, keeps its contiguous shard and weights its mean loss by its share of the valid
        tokens, so that averaging gradients over all ranks yields the gradient of the global mean loss."""
        B, S = ids.shape
        if S % cp.size:
            raise ValueError(f"sequence length {S} is not divisible by the context-parallel degree {cp.size}")
        s_l = S // cp.size
        shifted = torch.cat((lab[:, 1:], torch.full_like(lab[:, :1], -100)), dim=1)
        lo = cp.rank * s_l
        ids_l, lab_l = ids[:, lo:lo + s_l].contiguous(), shifted[:, lo:lo + s_l].contiguous()
        out = self.model(input_ids=ids_l, labels=lab_l, shift_labels=False, **model_kwargs)
        n_local = lab_l.ne(-100).sum().float()
        n_total = n_local.clone()
        dist.all_reduce(n_total, group=cp.group)
        weight = n_local * cp.size / n_total.clamp_min(1.0)
        (out.loss * (weight * scale)).backward()
        global_loss = (out.loss.detach() * n_local)
        dist.all_reduce(global_loss, group=cp.group)
        self.tokens_seen += ids.numel() // cp.size
        return global_loss / n_total.clamp_min(1.0)

    def _forward_backward_tp(self, ids, lab, scale, **model_kwargs):
        """Tensor + sequence parallel step: every rank receives the same sequence, embeds and scores its own
        token shard (labels shifted globally first); the blocks gather / scatter tokens inside their fused
        GEMM+collective kernels.  Each rank back-propagates its share ``n_local / n_total`` of the mean loss;
        gradients of replicated parameters are then summed over the group."""
        from ..parallel.tensor import all_reduce_replicated_grads
        tp = self.tp
        B, S = ids.shape
        if B != 1 or S % tp.world:
            raise ValueError("tensor parallelism takes one sequence per step, length divisible by the degree")
        s_l = S // tp.world
        shifted = torch.cat((lab[:, 1:], torch.full_like(lab[:, :1], -100)), dim=1)
        lo = tp.rank * s_l
        ids_l, lab_l = ids[:, lo:lo + s_l].contiguous(), shifted[:, lo:lo + s_l].contiguous()
        out = self.model(input_ids=ids_l, labels=lab_l, shift_labels=False, **model_kwargs)
        n_local = lab_l.ne(-100).sum().float()
        n_total = n_local.clone()
        dist.all_reduce(n_total, group=tp.group)
        share = n_local / n_total.clamp_min(1.0)
        (out.loss * (share * scale)).backward()
        if not self._tp_dp:                 # with data parallelism the reduced shards are summed instead (_tp_norm_sq)
            all_reduce_replicated_grads(self.model, tp)
        global_loss = out.loss.detach() * share
        dist.all_reduce(global_loss, group=tp.group)
        self.tokens_seen += ids.numel()
        return global_loss

    def _tp_norm_sq(self, norm_sq: torch.Tensor) -> None:
        """Global gradient norm under tensor parallelism: sharded weights contribute from every rank,
        replicated ones (identical after their all-reduce) once.

        Combined with data parallelism the gradients have already been reduce-scattered over the data-parallel
        group when this runs, so the sum of the replicated parameters' gradients over the tensor-parallel group is
        taken here, on this rank's slice of the reduced gradient (1/dp of the bytes), before the optimizer reads it."""
        from ..parallel.tensor import replicated_parameters
        rep_params = replicated_parameters(self.model)
        if not self._tp_dp:
            rep = torch.zeros_like(norm_sq)
            for p in rep_params:
                if p.grad is not None:
                    rep += p.grad.float().pow(2).sum()
            sharded = norm_sq - rep
            dist.all_reduce(sharded, group=self.tp.group)
            norm_sq.copy_(sharded + rep)
            return
        pieces = self.sdp.local_grad_slices(rep_params)
        flat = torch.cat([x.reshape(-1) for x in pieces]) if pieces else norm_sq.new_zeros(0)
        stats = torch.zeros(2, dtype=torch.float32, device=norm_sq.device)
        stats[0] = flat.float().pow(2).sum()
        dist.all_reduce(flat, group=self.tp.group)
        stats[1] = flat.float().pow(2).sum()
        off = 0
        for x in pieces:
            x.copy_(flat[off:off + x.numel()].view_as(x))
            off += x.numel()
        if self.sdp.world > 1:
            dist.all_reduce(stats, group=self.sdp.pg)
        sharded = norm_sq - stats[0]
        dist.all_reduce(sharded, group=self.tp.group)
        norm_sq.copy_(sharded + stats[1])

    def train_step(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, lr: float | None = None,
                   return_loss_on_host: bool = True, **model_kwargs):
        """One full step: (H2D copy if the tensors live on the host) forward, backward, clip, AdamW.

        Returns the loss as a Python float (device->host read) or, with ``return_loss_on_host=False``,
        as a device scalar so that nothing synchronises.
        """
        self.sdp.zero_grad()
        loss = self.forward_backward(input_ids, labels, **model_kwargs)
        self.sdp.step(lr)
        self.last_loss = loss
        return float(loss.item()) if return_loss_on_host else loss

    def close(self) -> None:
        """Release the device memory of the runtime (flat buffers, optimizer state, peer mappings); the engine and its
        model cannot be used afterwards."""
        for part in (getattr(self, "tp", None), getattr(self, "cp", None)):
            if part is not None and hasattr(part, "close"):
                part.close()
        if hasattr(self.sdp, "close"):
            self.sdp.close()

    @property
    def grad_norm(self):
        return self.sdp.last_grad_norm
