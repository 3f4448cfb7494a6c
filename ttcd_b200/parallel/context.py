"""Context parallelism: contiguous sequence shards + a one-sided K/V halo for sliding-window layers, head-parallel
(all-to-all) attention where a halo does not do (full-attention teachers, windows longer than a shard).

Rank r of a context-parallel group holds tokens [r*S_l, (r+1)*S_l).  Because every layer is windowed,
the only remote data attention needs is the tail of the PREVIOUS rank's K/V (the last ``w_T - 1`` keys,
rounded up to 128): those rows are pulled once per layer over NVLink into local memory by a plain-load
kernel right before the attention kernel, whose TMA loads then treat them as key blocks in front of the shard
(``TTCD_CP_HALO=direct`` lets the kernels' TMA loads address the previous rank's buffer themselves: no copy, but
each query tile near the boundary then fetches its halo blocks across the link again, 2 GB instead of 33 MB per
layer at 64K / 2 ranks); in backward the halo part of dK/dV is handed back to its owner through peer memory.  RoPE uses position offset r*S_l.  The
fast-weight scan needs the exclusive prefix over ranks of each rank's summed update; labels are shifted
before sharding so the shard boundary is handled by the data layout.

The reference accepts ``--experimental.context_parallel_degree`` but its mechanism (torchtitan's SDPA
context manager) does nothing for flash-attn models (flame/train.py:612-624); this is new capability.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import _native as nv

_ACTIVE: "ContextParallel | None" = None


def active() -> "ContextParallel | None":
    return _ACTIVE


@dataclass
class _LayerBuffers:
    kv: object            # SymmetricBuffer: K then V, each [B, S_l, HK, D] bf16
    dkv: object           # SymmetricBuffer: halo dK then dV, each [B, halo, HK, D] bf16
    shape: tuple
    halo_local: object = None   # [2, B, S, HK, D] bf16: local copy of the previous rank's K/V tail (tail rows only)
    halo_ptrs: tuple = (0, 0)   # where the kernels find the halo keys / values (local copy, or the peer's buffer)


class ContextParallel:
    """Per-process context-parallel state (rank, peers, per-layer symmetric K/V buffers, barriers)."""

    def __init__(self, group, window: int | None):
        from ..comm.symmetric import PeerBarrier
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.window = window
        self.barrier = PeerBarrier(group, slots=4) if (torch.cuda.is_available() and nv.available()) else None
        self.layers: dict[int, _LayerBuffers] = {}
        self._sum_bufs: dict = {}

    @staticmethod
    def by_heads(s_local: int, window: int | None, tiles: bool) -> bool:
        """Whether attention runs head-parallel (all-to-all) instead of with a halo: a full-attention layer needs every
        earlier rank's keys, and a window longer than the shard needs more than the previous rank's (``tiles``: the
        kernels take the halo in whole 128-key blocks)."""
        if window is None:
            return True
        need = (window - 1 + 127) // 128 * 128 if tiles else window - 1
        return need > s_local

    def halo_len(self, s_local: int) -> int:
        if self.rank == 0:
            return 0
        need = (self.window - 1 + 127) // 128 * 128
        if need > s_local:
            raise NotImplementedError(
                f"context-parallel shard of {s_local} tokens is shorter than the {need}-key halo; "
                "use fewer context-parallel ranks or a longer sequence")
        return need

    def buffers(self, layer_idx: int, B: int, S: int, HK: int, D: int) -> _LayerBuffers:
        from ..comm.symmetric import SymmetricBuffer
        lb = self.layers.get(layer_idx)
        shape = (B, S, HK, D)
        if lb is None or lb.shape != shape:
            n = B * S * HK * D * 2
            halo = (self.window - 1 + 127) // 128 * 128
            nh = B * min(halo, S) * HK * D * 2
            lb = _LayerBuffers(SymmetricBuffer(2 * n, self.group), SymmetricBuffer(2 * nh, self.group), shape)
            self.layers[layer_idx] = lb
        return lb

    def position_offset(self, s_local: int) -> int:
        return self.rank * s_local

    def exclusive_sum(self, x: torch.Tensor, key, before: bool) -> torch.Tensor:
        """Sum of ``x`` (fp32, same shape on every rank) over the ranks before (``before=True``) or after this one,
        read straight from the peers' memory by one kernel (fixed order: deterministic); zeros where there is no
        such rank.  ``key`` names the calling layer: each (key, direction) has its own peer buffer, and the flag
        barriers around the read make it reusable every step."""
        from ..comm.symmetric import SymmetricBuffer
        n = x.numel()
        slot_key = (key, before, n)
        buf = self._sum_bufs.get(slot_key)
        if buf is None:
            buf = SymmetricBuffer(n * 4, self.group)
            self._sum_bufs[slot_key] = buf
        buf.view(torch.float32, n).copy_(x.reshape(-1))
        self.barrier.sync(slot=3)                    # every rank's contribution is in place
        out = torch.empty_like(x, dtype=torch.float32)
        first, count = (0, self.rank) if before else (self.rank + 1, self.size - 1 - self.rank)
        if count > 0:
            nv.call("ttcd_peer_sum_f32", nv.ptr(out), buf.ptr_array(), nv.i32(self.size), nv.i64(n), nv.i32(first),
                    nv.i32(count), nv.stream_ptr())
        else:
            out.zero_()
        self.barrier.sync(slot=3)                    # peers are done reading before the buffer is written again
        return out


import os as _os

_HALO_MODE = _os.environ.get("TTCD_CP_HALO", "pull")      # pull (default) | direct


def _pull_halo(lb: _LayerBuffers, cp: "ContextParallel", halo: int, B: int, S: int, HK: int, D: int, device):
    """Copy the last ``halo`` keys/values of the previous rank's shard into local memory (one pass over NVLink,
    plain peer loads) and return the local pointers.  Every query tile whose window reaches back over the
    shard boundary reads them many times over; from local memory (and L2) instead of across the link."""
    if not halo:
        return 0, 0
    if _HALO_MODE == "direct":
        # the attention kernels' TMA loads address the previous rank's buffer themselves: no copy, but every
        # query tile near the shard boundary fetches its halo blocks over the link again
        n = B * S * HK * D
        prev = cp.rank - 1
        lb.halo_ptrs = (lb.kv.peer_ptrs[prev], lb.kv.peer_ptrs[prev] + n * 2)
        return lb.halo_ptrs
    if lb.halo_local is None:
        lb.halo_local = torch.empty(2, B, S, HK, D, dtype=torch.bfloat16, device=device)
    n = B * S * HK * D
    prev = cp.rank - 1
    cnt = halo * HK * D
    for which in range(2):
        for b in range(B):
            off = (b * S + (S - halo)) * HK * D
            nv.call("ttcd_peer_add", nv.i64(lb.halo_local[which].data_ptr() + off * 2),
                    nv.i64(lb.kv.peer_ptrs[prev] + which * n * 2 + off * 2), nv.i64(cnt), nv.i32(0), nv.stream_ptr())
    lb.halo_ptrs = (lb.halo_local[0].data_ptr(), lb.halo_local[1].data_ptr())
    return lb.halo_ptrs


class _CPAttention(torch.autograd.Function):
    """Sliding-window (dual) attention over a sequence shard with the halo read from the previous rank."""

    @staticmethod
    def forward(ctx, q, k, v, window_t, window_s, scale, dual, cp: ContextParallel, layer_idx: int):
        B, S, H, D = q.shape
        HK = k.shape[2]
        lb = cp.buffers(layer_idx, B, S, HK, D)
        n = B * S * HK * D
        k_sym = lb.kv.view(torch.bfloat16, n, 0).view(B, S, HK, D)
        v_sym = lb.kv.view(torch.bfloat16, n, n * 2).view(B, S, HK, D)
        k_sym.copy_(k)
        v_sym.copy_(v)
        cp.barrier.sync(slot=0)                      # every rank's K/V of this layer is in place
        halo = cp.halo_len(S)
        kh, vh = _pull_halo(lb, cp, halo, B, S, HK, D, q.device)
        qc = q.contiguous()
        o_t = torch.empty(B, S, H, D, dtype=torch.bfloat16, device=q.device)
        lse_t = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
        o_s = torch.empty_like(o_t) if dual else None
        lse_s = torch.empty_like(lse_t) if dual else None
        ld, sb = HK * D, S * HK * D
        nv.call("ttcd_attn_fwd_cp", nv.ptr(qc), nv.ptr(k_sym), nv.ptr(v_sym), nv.i64(kh), nv.i64(vh), nv.ptr(o_t), nv.ptr(o_s),
                nv.ptr(lse_t), nv.ptr(lse_s), nv.i32(B), nv.i32(S), nv.i32(S), nv.i32(H), nv.i32(HK), nv.i32(D),
                nv.i64(H * D), nv.i64(ld), nv.i64(ld), nv.i64(S * H * D), nv.i64(sb), nv.i64(sb), nv.i32(halo), nv.i32(S),
                nv.i32(window_t or 0), nv.i32(window_s or 0), nv.f32(scale), nv.ptr(None), nv.stream_ptr())
        ctx.save_for_backward(qc, o_t, o_s, lse_t, lse_s)
        ctx.cfg = (window_t, window_s, scale, dual, cp, layer_idx, halo)
        ctx.mark_non_differentiable(lse_t)
        if dual:
            ctx.mark_non_differentiable(lse_s)
            return o_t, o_s, lse_t, lse_s
        return o_t, lse_t

    @staticmethod
    def backward(ctx, *grads):
        qc, o_t, o_s, lse_t, lse_s = ctx.saved_tensors
        window_t, window_s, scale, dual, cp, layer_idx, halo = ctx.cfg
        B, S, H, D = qc.shape
        lb = cp.layers[layer_idx]
        HK = lb.shape[2]
        n = B * S * HK * D
        k_sym = lb.kv.view(torch.bfloat16, n, 0)
        v_sym = lb.kv.view(torch.bfloat16, n, n * 2)
        do_t = (grads[0] if grads[0] is not None else torch.zeros_like(o_t)).contiguous()
        do_s = None
        if dual:
            do_s = (grads[1] if grads[1] is not None else torch.zeros_like(o_s)).contiguous()

        from ..ops import cuda as _cuda
        # row statistics; dual window: delta_T, delta' and dO' from one kernel (see ops.cuda.attn_backward_streams)
        delta_t, do_c, delta_c = _cuda.attn_backward_streams(o_t, o_s, lse_t, lse_s, do_t, do_s)
        # the halo keys/values were copied into local memory by the forward pass
        kh, vh = lb.halo_ptrs if halo else (0, 0)
        dq = torch.empty_like(qc)
        dk_ext = torch.empty(B, halo + S, HK, D, dtype=torch.bfloat16, device=qc.device)
        dv_ext = torch.empty_like(dk_ext)
        ld, sb = HK * D, S * HK * D
        nv.call("ttcd_attn_bwd_cp", nv.ptr(qc), nv.ptr(k_sym), nv.ptr(v_sym), nv.i64(kh), nv.i64(vh), nv.ptr(do_t), nv.ptr(do_c),
                nv.ptr(lse_t), nv.ptr(delta_t), nv.ptr(delta_c), nv.ptr(dq), nv.ptr(dk_ext), nv.ptr(dv_ext),
                nv.i32(B), nv.i32(S), nv.i32(S), nv.i32(H), nv.i32(HK), nv.i32(D), nv.i64(H * D), nv.i64(ld), nv.i64(ld),
                nv.i64(S * H * D), nv.i64(sb), nv.i64(sb), nv.i64(0), nv.i64(0), nv.i32(halo), nv.i32(S),
                nv.i32(window_t or 0), nv.i32(window_s or 0), nv.f32(scale), nv.ptr(None), nv.ptr(None), nv.i32(0),
                nv.stream_ptr())
        dk = dk_ext[:, halo:].contiguous()
        dv = dv_ext[:, halo:].contiguous()
        # hand the halo part back to its owner: publish it, then every rank pulls from its successor
        hmax = min((cp.window - 1 + 127) // 128 * 128, S)
        nh = B * hmax * HK * D
        if halo:
            lb.dkv.view(torch.bfloat16, nh, 0).view(B, hmax, HK, D).copy_(dk_ext[:, :halo])
            lb.dkv.view(torch.bfloat16, nh, nh * 2).view(B, hmax, HK, D).copy_(dv_ext[:, :halo])
        cp.barrier.sync(slot=1)
        if cp.rank + 1 < cp.size:
            nxt = cp.rank + 1
            recv_k = torch.empty(B, hmax, HK, D, dtype=torch.bfloat16, device=qc.device)
            recv_v = torch.empty_like(recv_k)
            nv.call("ttcd_peer_add", nv.ptr(recv_k), nv.i64(lb.dkv.peer_ptrs[nxt]), nv.i64(nh), nv.i32(0), nv.stream_ptr())
            nv.call("ttcd_peer_add", nv.ptr(recv_v), nv.i64(lb.dkv.peer_ptrs[nxt] + nh * 2), nv.i64(nh), nv.i32(0),
                    nv.stream_ptr())
            dk[:, S - hmax:] += recv_k
            dv[:, S - hmax:] += recv_v
        cp.barrier.sync(slot=2)                      # peers are done reading before the buffer is reused
        return dq, dk, dv, None, None, None, None, None, None


class _GatherPrefix(torch.autograd.Function):
    """cat of ranks 0..mine of x along dim 1 (differentiable; gradients of a rank's slice are summed over
    the ranks that used it)."""

    @staticmethod
    def forward(ctx, x, cp):
        ctx.cp = cp
        ctx.n = x.shape[1]
        parts = [torch.empty_like(x) for _ in range(cp.size)]
        dist.all_gather(parts, x.contiguous(), group=cp.group)
        return torch.cat(parts[:cp.rank + 1], dim=1)

    @staticmethod
    def backward(ctx, g):
        cp, n = ctx.cp, ctx.n
        full = g.new_zeros(g.shape[0], cp.size * n, *g.shape[2:])
        full[:, :g.shape[1]] = g
        dist.all_reduce(full, group=cp.group)
        return full[:, cp.rank * n:(cp.rank + 1) * n].contiguous(), None


def _gathered_kv(k, v, cp):
    """CPU / fp32 statement of the halo exchange: differentiable all-gather, keep ranks <= mine."""
    return _GatherPrefix.apply(k, cp), _GatherPrefix.apply(v, cp)


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, group) -> None:
    """out[i] = the block that rank i addressed to this rank (inp[j] goes to rank j); blocks along dim 0."""
    if dist.get_backend(group) == "gloo":            # no all-to-all there: gather everything, keep this rank's column
        parts = [torch.empty_like(inp) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, inp, group=group)
        me = dist.get_rank(group)
        for i, part in enumerate(parts):
            out[i].copy_(part[me])
        return
    dist.all_to_all_single(out, inp, group=group)


class _SeqToHeads(torch.autograd.Function):
    """[B, S_l, H, D] (this rank's tokens, all heads) -> [B, S_l * size, H / size, D] (all tokens, this rank's heads),
    and back in backward.  ``inverse`` swaps the two directions."""

    @staticmethod
    def forward(ctx, x, cp, inverse: bool):
        ctx.cp, ctx.inverse = cp, inverse
        return _SeqToHeads._run(x, cp, inverse)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads._run(g, ctx.cp, not ctx.inverse), None, None

    @staticmethod
    def _run(x, cp, inverse):
        n = cp.size
        if not inverse:
            B, S, H, D = x.shape
            h = H // n
            inp = x.reshape(B, S, n, h, D).permute(2, 0, 1, 3, 4).contiguous()        # [to rank, B, S_l, h, D]
            out = torch.empty_like(inp)
            _all_to_all(out, inp, cp.group)                                          # [from rank, B, S_l, h, D]
            return out.permute(1, 0, 2, 3, 4).reshape(B, n * S, h, D)
        B, T, h, D = x.shape
        S = T // n
        inp = x.reshape(B, n, S, h, D).permute(1, 0, 2, 3, 4).contiguous()            # [to rank (its tokens), B, S_l, h, D]
        out = torch.empty_like(inp)
        _all_to_all(out, inp, cp.group)                                              # [from rank (its heads), B, S_l, h, D]
        return out.permute(1, 2, 0, 3, 4).reshape(B, S, n * h, D)


def _attention_by_heads(q, k, v, window_t, window_s, scale, dual, cp):
    """Head-parallel attention: one all-to-all turns the token shards of all heads into all tokens of H / size heads,
    the single-GPU kernels (any window, dual or not) run on those heads, a second all-to-all returns the outputs to
    the token shards.  Used when a halo does not do: full-attention teachers, windows longer than a shard."""
    from .. import ops
    if q.shape[2] % cp.size or k.shape[2] % cp.size:
        raise NotImplementedError(
            f"head-parallel attention needs the head counts ({q.shape[2]} query, {k.shape[2]} key/value) to divide by the "
            f"context-parallel degree {cp.size}")
    qh, kh, vh = (_SeqToHeads.apply(t, cp, False) for t in (q, k, v))
    if dual:
        o_t, o_s = ops.dual_window_attention(qh, kh, vh, window_t, window_s, scale)
        return _SeqToHeads.apply(o_t, cp, True), _SeqToHeads.apply(o_s, cp, True)
    return _SeqToHeads.apply(ops.attention(qh, kh, vh, window=window_t, scale=scale), cp, True)


def attention(q, k, v, window, scale, layer_idx):
    cp = _ACTIVE
    if cp.by_heads(q.shape[1], window, nv.use_native(q)):
        return _attention_by_heads(q, k, v, window, window, scale, False, cp)
    if not nv.use_native(q):
        from ..ops import reference
        k_all, v_all = _gathered_kv(k, v, cp)
        return reference.attention(q, k_all, v_all, window, scale)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    o, _ = _CPAttention.apply(q, k, v, window, window, scale, False, cp, layer_idx)
    return o


def dual_window_attention(q, k, v, window_t, window_s, scale, layer_idx):
    cp = _ACTIVE
    if cp.by_heads(q.shape[1], window_t, nv.use_native(q)):
        return _attention_by_heads(q, k, v, window_t, window_s, scale, True, cp)
    if not nv.use_native(q):
        from ..ops import reference
        k_all, v_all = _gathered_kv(k, v, cp)
        return reference.dual_window_attention(q, k_all, v_all, window_t, window_s, scale)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    o_t, o_s, _, _ = _CPAttention.apply(q, k, v, window_t, window_s, scale, True, cp, layer_idx)
    return o_t, o_s


class _RankPrefix(torch.autograd.Function):
    """Exclusive prefix sum over context-parallel ranks of a per-rank tensor (fast-weight update sums).

    forward:  out_r = sum_{r' < r} x_{r'}        backward:  dx_r = sum_{r' > r} dout_{r'}
    Implemented with an all-gather over the group (the tensors are a few MiB)."""

    @staticmethod
    def forward(ctx, x, cp: ContextParallel):
        ctx.cp = cp
        parts = [torch.empty_like(x) for _ in range(cp.size)]
        dist.all_gather(parts, x.contiguous(), group=cp.group)
        out = torch.zeros_like(x)
        for r in range(cp.rank):
            out += parts[r]
        return out

    @staticmethod
    def backward(ctx, g):
        cp = ctx.cp
        parts = [torch.empty_like(g) for _ in range(cp.size)]
        dist.all_gather(parts, g.contiguous(), group=cp.group)
        out = torch.zeros_like(g)
        for r in range(cp.rank + 1, cp.size):
            out += parts[r]
        return out, None


def rank_prefix(x: torch.Tensor) -> torch.Tensor:
    return _RankPrefix.apply(x, _ACTIVE)


def configure(engine, tensor_parallel: int = 1, context_parallel: int = 1) -> None:
    """Attach context-parallel state to an engine (called by TrainEngine)."""
    global _ACTIVE
    if tensor_parallel > 1:
        from . import tensor as _tp
        _tp.configure(engine, tensor_parallel)
    if context_parallel > 1:
        world = dist.get_world_size()
        rank = dist.get_rank()
        if world % context_parallel:
            raise ValueError("world size must be a multiple of the context-parallel degree")
        group = None
        for start in range(0, world, context_parallel):
            ranks = list(range(start, start + context_parallel))
            g = dist.new_group(ranks)
            if rank in ranks:
                group = g
        _ACTIVE = ContextParallel(group, getattr(engine.model_config, "window_size", None))
        engine.cp = _ACTIVE


def shutdown() -> None:
    global _ACTIVE
    _ACTIVE = None
