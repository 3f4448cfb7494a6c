"""Tensor + sequence parallelism on fused GEMM/collective kernels.

Layout (the reference's plan, flame/models/parallelize_fla.py:118-208): between blocks the residual stream
is sharded over tokens (``SequenceParallel`` norms); q/k/v and gate/up are column parallel (all-gather of the
token shards feeding the GEMM), o_proj and down_proj are row parallel (GEMM feeding a reduce-scatter back
to token shards).  Where the reference composes DTensor redistributes with cuBLAS (or torch's async-TP
micro-pipelining, 283-287), each of the two patterns is ONE kernel here (``csrc/gemm_comm.cu``):

* ``ag_linear``  : all-gather -> GEMM.  Peers' row blocks are pulled into a local gathered buffer by bulk
  async copies inside the GEMM kernel; tiles start on the rank's own rows and follow the flags.
* ``rs_linear``  : GEMM -> reduce-scatter.  Other ranks' row blocks are computed first and each finished tile
  is pushed (coalesced bf16 stores over NVLink) into its owner's receive buffer and flagged there; the rank's
  own rows are computed last and their epilogue adds the tiles the peers pushed, in a fixed order.

Backward uses the same two kernels with the weight read MN-major (dX of a column-parallel layer is a
GEMM -> reduce-scatter, dX of a row-parallel layer an all-gather -> GEMM) and the plain GEMM for dW on the
gathered operand the forward kernel left behind.  CPU / gloo: the same functions run as
``all_gather`` / ``reduce_scatter`` + matmul so the layer logic is testable without GPUs.

Buffers are double buffered and every fused call is preceded by one flag barrier: a buffer is rewritten two
calls after peers read it, and every peer has passed the barrier in between.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native as nv

_CTX: "TensorParallel | None" = None


def current() -> "TensorParallel | None":
    return _CTX


class TensorParallel:
    """Per-process state of one tensor-parallel group: symmetric staging buffers, flags, barrier."""

    BM, BN = 128, 256

    def __init__(self, group=None, device=None, max_rows_per_rank: int = 8192, max_features: int = 6144,
                 wait_ns: int = 0, fused: bool | None = None):
        global _CTX
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device if device is not None else "cpu")
        self.fused = (self.device.type == "cuda" and nv.available()) if fused is None else fused
        self.wait_ns = wait_ns
        self._warned: set = set()
        self.rs_lag = 32              # gemm_rs schedule: own row blocks trail the pushes by 32 rounds (csrc/gemm_comm.cu::gc_tile)
        self.epoch = 0
        self.calls = 0
        if self.fused:
            from ..comm.symmetric import PeerBarrier, SymmetricBuffer
            rows, feat, w = max_rows_per_rank, max_features, self.world
            self.max_rows, self.max_feat = rows, feat
            self.x_sym = [SymmetricBuffer(rows * feat * 2, group, self.device) for _ in range(2)]
            self.part_sym = [SymmetricBuffer(rows * w * feat * 2, group, self.device) for _ in range(2)]
            nflags = (rows // self.BM) * w * (feat // self.BN)
            self.flag_sym = [SymmetricBuffer(nflags * 4, group, self.device) for _ in range(2)]
            self.gathered = torch.empty(rows * w * feat, dtype=torch.bfloat16, device=self.device)
            self.ready = torch.zeros((rows // self.BM) * w, dtype=torch.int32, device=self.device)
            self.barrier = PeerBarrier(group, slots=2, wait_ns=wait_ns)
        _CTX = self

    def close(self):
        global _CTX
        if self.fused:
            torch.cuda.synchronize()
            for b in self.x_sym + self.part_sym + self.flag_sym + [self.barrier.buf]:
                b.close()
        if _CTX is self:
            _CTX = None

    # ------------------------------------------------------------------------------- raw collectives+GEMM
    def _fits(self, m_shard: int, n: int, k: int) -> bool:
        ok = (self.fused and m_shard % self.BM == 0 and n % self.BN == 0 and k % 64 == 0 and m_shard <= self.max_rows
              and max(n, k) <= self.max_feat and (self.BM * k * 2) % 16384 == 0)
        if not ok and self.fused and (m_shard, n, k) not in self._warned:
            # said once per shape: the layer then runs NCCL + the plain GEMM instead of the fused kernel
            self._warned.add((m_shard, n, k))
            import logging
            logging.getLogger("ttcd_b200").warning(
                "tensor parallel: shape rows/rank=%d N=%d K=%d does not fit the fused GEMM+collective kernels "
                "(rows %% 128, N %% 256, K %% 64, buffer sizes): using NCCL + GEMM for it", m_shard, n, k)
        return ok

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, w_is_kn: bool = False):
        """``(all_gather_rows(x_shard) @ W^T, gathered)``.  ``w``: [N, K], or [K, N] when ``w_is_kn``."""
        m, k = x_shard.shape
        n = w.shape[1] if w_is_kn else w.shape[0]
        if not self._fits(m, n, k):
            return self._ag_gemm_baseline(x_shard, w, w_is_kn)
        self.calls += 1
        self.epoch += 1
        b = self.calls & 1
        xs = self.x_sym[b]
        xs.view(torch.bfloat16, m * k).view(m, k).copy_(x_shard)
        self.barrier.sync(slot=0)
        out = torch.empty(m * self.world, n, dtype=torch.bfloat16, device=self.device)
        w = w if w.stride(-1) == 1 else w.contiguous()
        nv.call("ttcd_ag_gemm", xs.ptr_array(), nv.ptr(w), nv.ptr(out), nv.ptr(self.gathered), nv.ptr(self.ready),
                nv.i32(self.rank), nv.i32(self.world), nv.i64(m), nv.i64(n), nv.i64(k), nv.i64(w.stride(0)), nv.i64(n),
                nv.i32(1 if w_is_kn else 0), nv.i32(self.epoch), nv.i64(self.wait_ns), nv.stream_ptr())
        full = self.gathered[:m * self.world * k].view(m * self.world, k)
        full[self.rank * m:(self.rank + 1) * m].copy_(x_shard)       # the kernel read the own rows in place
        return out, full

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, w_is_kn: bool = False, lag: int | None = None) -> torch.Tensor:
        """Rows of this rank of ``sum_ranks(x_r @ W_r^T)``.  ``x``: [world*m_shard, K_local].  ``lag``: rounds by which
        the rank's own row blocks trail the pushes to the peers (default ``self.rs_lag``; 0 = all own blocks last)."""
        mt, k = x.shape
        m = mt // self.world
        n = w.shape[1] if w_is_kn else w.shape[0]
        if mt % self.world or not self._fits(m, n, k):
            return self._gemm_rs_baseline(x, w, w_is_kn)
        self.calls += 1
        self.epoch += 1
        b = self.calls & 1
        self.barrier.sync(slot=0)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        x = x if x.stride(-1) == 1 else x.contiguous()
        w = w if w.stride(-1) == 1 else w.contiguous()
        nv.call("ttcd_gemm_rs", nv.ptr(x), nv.ptr(w), nv.ptr(out), self.part_sym[b].ptr_array(), self.flag_sym[b].ptr_array(),
                nv.i32(self.rank), nv.i32(self.world), nv.i64(m), nv.i64(n), nv.i64(k), nv.i64(x.stride(0)),
                nv.i64(w.stride(0)), nv.i64(n), nv.i32(1 if w_is_kn else 0), nv.i32(self.epoch), nv.i64(self.wait_ns),
                nv.i32(self.rs_lag if lag is None else lag), nv.stream_ptr())
        return out

    # NCCL / gloo statement of the same two operations (baseline and CPU path)
    def _ag_gemm_baseline(self, x_shard, w, w_is_kn):
        full = torch.empty(x_shard.shape[0] * self.world, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        from .. import ops
        return (ops.matmul(full, w) if w_is_kn else ops.linear(full, w)), full

    def _gemm_rs_baseline(self, x, w, w_is_kn):
        from .. import ops
        y = ops.matmul(x, w) if w_is_kn else ops.linear(x, w)
        out = torch.empty(y.shape[0] // self.world, y.shape[1], dtype=y.dtype, device=y.device)
        if y.device.type == "cpu":          # gloo has no reduce_scatter
            dist.all_reduce(y, group=self.group)
            out.copy_(y[self.rank * out.shape[0]:(self.rank + 1) * out.shape[0]])
        else:
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.group)
        return out

    def check(self) -> None:
        """Raise if any bounded wait of a fused kernel expired."""
        if self.fused:
            torch.cuda.synchronize()
            code = nv.device_status()
            if code:
                raise RuntimeError(f"tensor-parallel kernel wait expired (status {code})")


# ----------------------------------------------------------------------------------------- autograd
class _ColumnParallel(torch.autograd.Function):
    """y[all tokens, N_local] = all_gather(x_shard) @ W_local^T."""

    @staticmethod
    def forward(ctx, x_shard, weight, tp: TensorParallel):
        y, full = tp.ag_gemm(x_shard, weight)
        ctx.save_for_backward(full.clone() if tp.fused else full, weight)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        from .. import ops
        full, weight = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx_shard = tp.gemm_rs(dy, weight, w_is_kn=True)            # dX = dY @ W, reduce-scattered over tokens
        dw = ops.matmul(dy.t(), full).to(weight.dtype)               # [N_local, K]
        return dx_shard, dw, None


class _RowParallel(torch.autograd.Function):
    """y_shard[my tokens, N] = reduce_scatter(x[all tokens, K_local] @ W_local^T)."""

    @staticmethod
    def forward(ctx, x, weight, tp: TensorParallel):
        ctx.save_for_backward(x, weight)
        ctx.tp = tp
        return tp.gemm_rs(x, weight)

    @staticmethod
    def backward(ctx, dy_shard):
        from .. import ops
        x, weight = ctx.saved_tensors
        tp = ctx.tp
        dx, dy_full = tp.ag_gemm(dy_shard.contiguous(), weight, w_is_kn=True)   # dX = all_gather(dY) @ W
        dw = ops.matmul(dy_full.t(), x).to(weight.dtype)                          # [N, K_local]
        return dx, dw, None


def column_parallel_linear(x_shard: torch.Tensor, weight: torch.Tensor, tp: TensorParallel | None = None) -> torch.Tensor:
    return _ColumnParallel.apply(x_shard, weight, tp or _CTX)


def row_parallel_linear(x: torch.Tensor, weight: torch.Tensor, tp: TensorParallel | None = None) -> torch.Tensor:
    return _RowParallel.apply(x, weight, tp or _CTX)


# ----------------------------------------------------------------------------------------- model wiring
class _ColumnParallelSlab(torch.autograd.Function):
    """Several column-parallel projections of the same token-sharded input through ONE all-gather -> GEMM:
    the weights are adjacent rows of one slab (the flat parameter buffer lays q/k/v and gate/up back to
    back); outputs are column slices of the product."""

    @staticmethod
    def forward(ctx, x_shard, tp, slab, *weights):
        w_all = slab if slab is not None else torch.cat([w.detach() for w in weights], dim=0)
        y, full = tp.ag_gemm(x_shard, w_all)
        ctx.save_for_backward(full.clone() if tp.fused else full, w_all)
        ctx.tp, ctx.sizes = tp, [w.shape[0] for w in weights]
        return tuple(y.split(ctx.sizes, dim=1))

    @staticmethod
    def backward(ctx, *dys):
        from .. import ops
        full, w_all = ctx.saved_tensors
        dy = torch.cat([d.to(w_all.dtype) for d in dys], dim=1)
        dx_shard = ctx.tp.gemm_rs(dy, w_all, w_is_kn=True)
        dw = ops.matmul(dy.t(), full)
        return (dx_shard, None, None) + tuple(dw.split(ctx.sizes, dim=0))


class _SumOverGroup(torch.autograd.Function):
    """Sum of per-rank partial results whose consumers are again rank-local shards: all-reduce in forward
    (leaving one parallel region) and in backward (entering the next)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _GatherRows(torch.autograd.Function):
    """all_gather along dim 0 (backward: reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        out = torch.empty(x.shape[0] * tp.world, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=tp.group)
        return out

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        g = g.contiguous()
        n = g.shape[0] // tp.world
        if g.device.type == "cpu":
            g = g.clone()
            dist.all_reduce(g, group=tp.group)
            return g[tp.rank * n:(tp.rank + 1) * n], None
        out = torch.empty(n, *g.shape[1:], dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=tp.group)
        return out, None


class _ScatterRowsSum(torch.autograd.Function):
    """reduce-scatter along dim 0 of per-rank partial sums (backward: all-gather)."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        n = x.shape[0] // tp.world
        if x.device.type == "cpu":
            y = x.contiguous().clone()
            dist.all_reduce(y, group=tp.group)
            return y[tp.rank * n:(tp.rank + 1) * n].clone()
        out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=tp.group)
        return out

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        out = torch.empty(g.shape[0] * tp.world, *g.shape[1:], dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=tp.group)
        return out, None


def column_parallel_multi(x_shard, weights, slab=None, tp: TensorParallel | None = None):
    return _ColumnParallelSlab.apply(x_shard, tp or _CTX, slab, *weights)


def sum_over_group(x, tp: TensorParallel | None = None):
    tp = tp or _CTX
    return _SumOverGroup.apply(x, tp.group)


def gather_rows(x, tp: TensorParallel | None = None):
    return _GatherRows.apply(x, tp or _CTX)


def scatter_rows_sum(x, tp: TensorParallel | None = None):
    return _ScatterRowsSum.apply(x, tp or _CTX)


def _slice_param(module, name: str, dim: int, rank: int, world: int, block: int = 1) -> None:
    """Replace ``module.<name>`` by this rank's 1/world slice along ``dim`` (in units of ``block``)."""
    p = getattr(module, name)
    units = p.shape[dim] // block
    if units % world:
        raise ValueError(f"{name}: {units} units of {block} along dim {dim} do not divide by tp={world}")
    per = units // world * block
    new = torch.nn.Parameter(p.detach().narrow(dim, rank * per, per).clone(), requires_grad=p.requires_grad)
    new._tp_shard = (dim, world)
    setattr(module, name, new)


def shard_model(model, tp: TensorParallel) -> None:
    """Megatron-style sharding of every block in place: q/k/v by heads and gate/up by rows (column
    parallel), o_proj/down_proj by columns (row parallel), depthwise conv channels with the intermediate
    dimension.  Norm weights, ``ttt_proj``, ``b_proj``, embeddings and the LM head stay replicated."""
    r, w = tp.rank, tp.world
    for layer in model.model.layers:
        attn = layer.attn
        if attn.num_heads % w or attn.num_kv_heads % w:
            raise ValueError(f"heads ({attn.num_heads}, kv {attn.num_kv_heads}) do not divide by tp={w}")
        if attn.use_output_gate or attn.q_proj.bias is not None:
            raise NotImplementedError("tensor parallelism: output gate / qkv bias are not supported")
        D = attn.head_dim
        _slice_param(attn.q_proj, "weight", 0, r, w, D)
        _slice_param(attn.k_proj, "weight", 0, r, w, D)
        _slice_param(attn.v_proj, "weight", 0, r, w, D)
        _slice_param(attn.o_proj, "weight", 1, r, w, D)
        attn.num_heads //= w
        attn.num_kv_heads //= w
        attn.q_dim, attn.kv_dim = attn.num_heads * D, attn.num_kv_heads * D
        mlp = layer.mlp
        _slice_param(mlp.gate_proj, "weight", 0, r, w)
        _slice_param(mlp.up_proj, "weight", 0, r, w)
        _slice_param(mlp.down_proj, "weight", 1, r, w)
        mlp.intermediate_size //= w
        for name in ("ttt_teacher_conv", "ttt_student_conv", "ttt_activation_conv"):
            conv = getattr(mlp, name, None)
            if conv is not None:
                _slice_param(conv, "weight", 0, r, w)
    model._tp = tp


def replicated_parameters(model):
    return [p for p in model.parameters() if not hasattr(p, "_tp_shard")]


def all_reduce_replicated_grads(model, tp: TensorParallel) -> None:
    """Replicated parameters see only this rank's token shard (or heads): sum their gradients over the group."""
    for p in replicated_parameters(model):
        if p.grad is not None:
            dist.all_reduce(p.grad, group=tp.group)


def gather_full_state_dict(model, tp: TensorParallel) -> dict:
    """State dict with every sharded tensor all-gathered back to its full shape (for checkpoints)."""
    out = {}
    for name, p in model.state_dict().items():
        src = dict(model.named_parameters()).get(name)
        shard = getattr(src, "_tp_shard", None) if src is not None else None
        if shard is None:
            out[name] = p.detach()
            continue
        dim = shard[0]
        parts = [torch.empty_like(p) for _ in range(tp.world)]
        dist.all_gather(parts, p.detach().contiguous(), group=tp.group)
        out[name] = torch.cat(parts, dim=dim)
    return out


def load_full_state_dict(model, full: dict, tp: TensorParallel) -> None:
    """Inverse of ``gather_full_state_dict``: every rank keeps its slice of the sharded tensors."""
    params = dict(model.named_parameters())
    with torch.no_grad():
        for name, value in full.items():
            p = params.get(name)
            if p is None:
                continue
            shard = getattr(p, "_tp_shard", None)
            if shard is not None:
                per = value.shape[shard[0]] // tp.world
                value = value.narrow(shard[0], tp.rank * per, per)
            p.copy_(value.to(p.dtype))


def _shard_spec(model, key: str):
    """``(dim, world)`` of the sharded parameter a state key belongs to (``name`` or ``name.<state>``)."""
    params = dict(model.named_parameters())
    p = params.get(key)
    if p is None and "." in key:
        p = params.get(key.rsplit(".", 1)[0])
    return getattr(p, "_tp_shard", None) if p is not None else None


def gather_named(model, tp: TensorParallel, tensors: dict) -> dict:
    """All-gather every entry that belongs to a sharded parameter (weights or per-parameter optimizer state)."""
    out = {}
    for key, t in tensors.items():
        spec = _shard_spec(model, key) if isinstance(t, torch.Tensor) and t.dim() > 0 else None
        if spec is None:
            out[key] = t
            continue
        parts = [torch.empty_like(t) for _ in range(tp.world)]
        dist.all_gather(parts, t.contiguous(), group=tp.group)
        out[key] = torch.cat(parts, dim=spec[0])
    return out


def slice_named(model, tp: TensorParallel, tensors: dict) -> dict:
    """Inverse of ``gather_named``: keep this rank's slice of every entry of a sharded parameter."""
    out = {}
    for key, t in tensors.items():
        spec = _shard_spec(model, key) if isinstance(t, torch.Tensor) and t.dim() > 0 else None
        if spec is None:
            out[key] = t
        else:
            per = t.shape[spec[0]] // tp.world
            out[key] = t.narrow(spec[0], tp.rank * per, per).contiguous()
    return out


def full_shape(p: torch.Tensor) -> tuple:
    spec = getattr(p, "_tp_shard", None)
    shape = list(p.shape)
    if spec is not None:
        shape[spec[0]] *= spec[1]
    return tuple(shape)


def configure(engine, degree: int) -> None:
    """Called by the engine: build the tensor-parallel group of ``degree`` consecutive ranks, shard the
    model and switch its layers to the parallel paths."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % degree:
        raise ValueError("world size must be a multiple of the tensor-parallel degree")
    group = None
    for start in range(0, world, degree):
        ranks = list(range(start, start + degree))
        g = dist.new_group(ranks)
        if rank in ranks:
            group = g
    cfg = engine.model_config
    feat = max(getattr(cfg, "resolved_intermediate_size", cfg.hidden_size), cfg.hidden_size)
    rows = max(128, int(getattr(engine.cfg, "tp_max_tokens", 65536)) // degree)
    tp = TensorParallel(group, engine.device, max_rows_per_rank=rows, max_features=max(feat, 1024))
    shard_model(engine.model, tp)
    engine.tp = tp


# ----------------------------------------------------------------------------------------- loss parallel
class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over logits whose vocabulary dimension is sharded across the group (the reference's
    vocab-parallel path, fla/modules/fused_cross_entropy.py:205-212): every rank reduces its shard to a row
    maximum / sum-exp and its share of the target logit; two small all-reduces combine them.  The default
    tensor-parallel layout here keeps the LM head replicated and shards the tokens instead, so this is only
    needed for column-parallel heads."""

    @staticmethod
    def forward(ctx, logits, labels, group, vocab_start, ignore_index):
        lf = logits.float()
        local_max = lf.max(dim=-1).values
        gmax = local_max.clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lf - gmax[:, None])
        sumexp = ex.sum(-1)
        dist.all_reduce(sumexp, group=group)
        local = labels - vocab_start
        mine = (local >= 0) & (local < logits.shape[-1]) & labels.ne(ignore_index)
        tgt = torch.where(mine, lf.gather(-1, local.clamp(0, logits.shape[-1] - 1)[:, None]).squeeze(-1), torch.zeros_like(gmax))
        dist.all_reduce(tgt, group=group)
        valid = labels.ne(ignore_index)
        n = valid.sum().clamp_min(1)
        loss = ((torch.log(sumexp) + gmax - tgt) * valid).sum() / n
        ctx.save_for_backward(ex / sumexp[:, None], local, mine, valid, n)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        probs, local, mine, valid, n = ctx.saved_tensors
        grad = probs.clone()
        rows = torch.nonzero(mine).squeeze(-1)
        grad[rows, local[rows]] -= 1.0
        grad = grad * (valid[:, None] * (g / n))
        return grad.to(ctx.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits_shard: torch.Tensor, labels: torch.Tensor, tp: TensorParallel | None = None,
                                 ignore_index: int = -100) -> torch.Tensor:
    """Mean CE of ``[rows, vocab / world]`` logit shards (rank r holds columns [r*V_l, (r+1)*V_l))."""
    tp = tp or _CTX
    return _VocabParallelCE.apply(logits_shard, labels, tp.group, tp.rank * logits_shard.shape[-1], ignore_index)
