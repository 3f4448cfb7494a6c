"""Symmetric (peer-addressable) device buffers and the flag barrier built on them.

One process per GPU.  ``SymmetricBuffer`` allocates the same number of bytes on every rank with
cudaMalloc, exchanges CUDA IPC handles through the torch.distributed group and keeps a device pointer
to every peer's copy; kernels then read/write peers with plain loads and stores over NVLink.
``PeerBarrier`` is an all-to-all flag barrier executed by a tiny kernel with a bounded spin (a rank
that never arrives turns into a status code on the host instead of a hang).  NCCL stays the bootstrap
transport and the baseline collective implementation.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native as nv


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__`` (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _as_tensor(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``; ``peer_ptrs[r]`` addresses rank r's copy."""

    def __init__(self, nbytes: int, group=None, device=None):
        if not dist.is_initialized():
            raise RuntimeError("SymmetricBuffer needs an initialised process group")
        nv.load(required=True)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        out = ctypes.c_longlong(0)
        nv.call("ttcd_symm_alloc", nv.i64(self.nbytes), ctypes.byref(out))
        self.local_ptr = int(out.value)
        lib = nv.load(required=True)
        lib.ttcd_ipc_handle_size.restype = ctypes.c_int
        hsize = int(lib.ttcd_ipc_handle_size())
        handle = ctypes.create_string_buffer(hsize)
        nv.call("ttcd_ipc_get_handle", nv.i64(self.local_ptr), handle)
        handles: list[bytes | None] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.peer_ptrs: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            p = ctypes.c_longlong(0)
            nv.call("ttcd_ipc_open_handle", ctypes.create_string_buffer(h, hsize), ctypes.byref(p))
            self.peer_ptrs.append(int(p.value))
            self._opened.append(int(p.value))
        self._ptr_array = (ctypes.c_longlong * self.world)(*self.peer_ptrs)
        self.tensor = _as_tensor(self.local_ptr, self.nbytes, self.device)
        dist.barrier(group=group)

    def ptr_array(self, byte_offset: int = 0):
        """ctypes array of every rank's base pointer (+ offset) for the kernels' ``PeerPtrs`` argument."""
        if byte_offset == 0:
            return self._ptr_array
        return (ctypes.c_longlong * self.world)(*[p + byte_offset for p in self.peer_ptrs])

    def view(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        size = numel * torch.empty((), dtype=dtype).element_size()
        return self.tensor[byte_offset:byte_offset + size].view(dtype)

    def peer_view(self, rank: int, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """A tensor aliasing rank ``rank``'s copy.  Only hand this to this library's own kernels
        (plain loads/stores); never to a library kernel."""
        size = numel * torch.empty((), dtype=dtype).element_size()
        return _as_tensor(self.peer_ptrs[rank] + byte_offset, size, self.device).view(dtype)

    def close(self):
        for p in self._opened:
            try:
                nv.call("ttcd_ipc_close", nv.i64(p))
            except Exception:
                pass
        self._opened = []
        if self.local_ptr:
            self.tensor = None
            nv.call("ttcd_symm_free", nv.i64(self.local_ptr))
            self.local_ptr = 0


class PeerBarrier:
    """All-to-all flag barrier over a symmetric flag array (``slots`` independent barriers)."""

    def __init__(self, group=None, slots: int = 8, wait_ns: int = 0, fail: torch.Tensor | None = None):
        """``wait_ns``: budget of one wait (0: the library default, 10 s).  ``fail``: optional 1-element fp32 CUDA
        tensor that a wait which runs out sets to 1 (kernels later in the step take it as their skip flag)."""
        self.buf = SymmetricBuffer(slots * 64 * 4, group)
        self.rank, self.world, self.slots = self.buf.rank, self.buf.world, slots
        self.epochs = [0] * slots
        self.wait_ns = wait_ns
        self.fail = fail

    def sync(self, slot: int = 0, stream: torch.cuda.Stream | None = None) -> None:
        """Enqueue the barrier on ``stream`` (default: current).  Work enqueued after it on that stream
        sees every peer's writes enqueued before the peer's matching call."""
        self.epochs[slot] += 1
        s = ctypes.c_void_p((stream or torch.cuda.current_stream()).cuda_stream)
        nv.call("ttcd_comm_barrier", self.buf.ptr_array(), nv.i32(self.rank), nv.i32(self.world), nv.i32(slot),
                nv.i32(self.epochs[slot]), nv.i64(self.wait_ns), nv.ptr(self.fail), s)

    def check(self) -> None:
        """Raise if a bounded wait expired (a peer never arrived).  Synchronises the device."""
        torch.cuda.synchronize()
        code = nv.device_status()
        if code:
            raise RuntimeError(f"peer barrier wait expired (status {code}): rank {code - 500 if code >= 500 else '?'} never arrived")
