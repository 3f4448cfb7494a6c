"""Activation offloading to pinned host memory (the role of flame/models/activation_offloading.py:139-356).

``OffloadActivations`` is a ``saved_tensors_hooks`` context: tensors saved for backward that are large enough
are copied to pinned host buffers on a side stream while the forward continues (at most ``max_fwd_stash``
device copies are kept alive waiting for their transfer), and brought back on the same side stream in
backward, the consumer stream waiting on the copy's event.  Parameters, tiny tensors and non-CUDA tensors
stay where they are.  With 180 GB per GPU the flagship recipe does not need it; it is for longer sequences
(the 512K config) and smaller parts.  Host buffers are recycled by size, so steady-state steps allocate
nothing on the host.
"""
from __future__ import annotations

import contextlib
from collections import deque

import torch


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    def __init__(self, min_offload_bytes: int = 1 << 20, max_fwd_stash: int = 5, use_pin_memory: bool = True):
        self.min_bytes, self.max_stash, self.pin = int(min_offload_bytes), int(max_fwd_stash), use_pin_memory
        self.stream: torch.cuda.Stream | None = None
        self.next_id = 0
        self.host: dict[int, tuple] = {}
        self.stash: deque[tuple[torch.Tensor, torch.cuda.Event]] = deque()
        self.pool: dict[tuple, list[torch.Tensor]] = {}
        self.bytes_offloaded = 0
        super().__init__(self._pack, self._unpack)

    # -------------------------------------------------------------------------------- helpers
    def _side(self) -> torch.cuda.Stream:
        if self.stream is None:
            self.stream = torch.cuda.Stream()
        return self.stream

    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        key = (t.dtype, t.numel())
        free = self.pool.get(key)
        if free:
            return free.pop()
        return torch.empty(t.numel(), dtype=t.dtype, device="cpu", pin_memory=self.pin and torch.cuda.is_available())

    def _eligible(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.is_contiguous() and not isinstance(t, torch.nn.Parameter)
                and t.numel() * t.element_size() >= self.min_bytes)

    # -------------------------------------------------------------------------------- hooks
    def _pack(self, t: torch.Tensor):
        if not self._eligible(t):
            return t
        side, cur = self._side(), torch.cuda.current_stream()
        buf = self._host_buffer(t)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            buf.copy_(t.detach().reshape(-1), non_blocking=True)
            done = torch.cuda.Event()
            done.record(side)
        self.stash.append((t, done))                 # keeps the device copy alive until the transfer ran
        while len(self.stash) > self.max_stash:
            _, ev = self.stash.popleft()
            ev.synchronize()
        key = self.next_id
        self.next_id += 1
        self.host[key] = (buf, t.device, done, tuple(t.shape))
        self.bytes_offloaded += t.numel() * t.element_size()
        return ("offloaded", key)

    def _unpack(self, handle):
        if isinstance(handle, torch.Tensor):
            return handle
        _, key = handle
        buf, device, done, shape = self.host.pop(key)
        self.stash.clear()                            # backward has begun: forward transfers are long done or waited below
        side, cur = self._side(), torch.cuda.current_stream()
        with torch.cuda.stream(side):
            if done is not None:
                side.wait_event(done)
            out = torch.empty(shape, dtype=buf.dtype, device=device)
            out.view(-1).copy_(buf, non_blocking=True)
            back = torch.cuda.Event()
            back.record(side)
        cur.wait_event(back)
        out.record_stream(cur)
        self._release_later(buf, back)
        return out

    def _release_later(self, buf: torch.Tensor, ev: torch.cuda.Event) -> None:
        # the host buffer may be reused once the copy back has run
        pending = getattr(self, "_pending", None)
        if pending is None:
            pending = self._pending = deque()
        pending.append((buf, ev))
        while pending and pending[0][1].query():
            b, _ = pending.popleft()
            self.pool.setdefault((b.dtype, b.numel()), []).append(b)


class NoOpManager(contextlib.AbstractContextManager):
    def __exit__(self, *exc):
        return False


def get_act_offloading_ctx_manager(enable: bool, **kwargs):
    """Context manager to wrap the forward pass in (a fresh no-op when disabled)."""
    return OffloadActivations(**kwargs) if enable else NoOpManager()
