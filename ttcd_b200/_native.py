"""ctypes binding to the in-tree sm_100a library ``ttcd_b200/_lib/libttcd_b200.so``.

Every kernel is exported with C linkage and takes raw device pointers, sizes and
a ``cudaStream_t``; Python passes ``tensor.data_ptr()`` and the current torch
stream, so launches are ordered with the surrounding torch work and no torch C++
headers are needed at build time.  Entry points return 0 on success or a
non-zero ``cudaError_t`` / negative framework error code.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent / "_lib"
_LIB_PATH = _LIB_DIR / "libttcd_b200.so"
_lib: ctypes.CDLL | None = None
_load_error: str | None = None


class NativeError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load(required: bool = False) -> ctypes.CDLL | None:
    """Load the shared library once.  ``required`` raises if it is missing."""
    global _lib, _load_error
    if _lib is None and _load_error is None:
        if _LIB_PATH.exists():
            try:
                _lib = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
            except OSError as exc:  # pragma: no cover - depends on the machine
                _load_error = f"{exc}"
        else:
            _load_error = f"{_LIB_PATH} not built (run `python -m ttcd_b200._build`)"
    if _lib is None and required:
        raise NativeError(f"ttcd_b200 native library unavailable: {_load_error}")
    return _lib


def available() -> bool:
    return load() is not None


def torch_fallback_allowed() -> bool:
    """Bring-up switch: let CUDA tensors run the PyTorch statement of an op."""
    return os.environ.get("TTCD_TORCH_FALLBACK", "0") == "1"


def use_native(*tensors: torch.Tensor) -> bool:
    """True when the op must run on the hand-written kernels.

    CUDA bf16 tensors always take the native path; a missing library is an error
    (never a silent fallback) unless TTCD_TORCH_FALLBACK=1.  CPU tensors and fp32
    CUDA tensors take the PyTorch statement.
    """
    t = tensors[0]
    if not t.is_cuda or t.dtype != torch.bfloat16:
        return False
    if load() is None:
        if torch_fallback_allowed():
            return False
        raise NativeError(
            "CUDA bf16 tensors require the ttcd_b200 native library: " + str(_load_error)
        )
    return True


def has(symbol: str) -> bool:
    lib = load()
    return lib is not None and hasattr(lib, symbol)


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_ERRORS = {
    -1: "invalid argument (shape/stride/alignment)",
    -2: "device wait ran out (bounded spin expired)",
    -3: "size exceeds the built-in maximum",
    -4: "tensor-map encode failed",
}


launch_count = 0  # kernels launched through this binding (entry points that launch two count twice)
_MULTI_KERNEL = {"ttcd_attn_bwd": 2, "ttcd_attn_bwd_cp": 2, "ttcd_rmsnorm_bwd_no_alloc": 2, "ttcd_attn_small_q": 2,
                 # host-only entry points launch nothing
                 "ttcd_symm_alloc": 0, "ttcd_symm_free": 0, "ttcd_ipc_get_handle": 0, "ttcd_ipc_open_handle": 0,
                 "ttcd_ipc_close": 0}


def call(symbol: str, *args) -> None:
    """Invoke ``int symbol(args...)`` and raise on a non-zero status."""
    global launch_count
    launch_count += _MULTI_KERNEL.get(symbol, 1)
    lib = load(required=True)
    fn = getattr(lib, symbol, None)
    if fn is None:
        raise NativeError(f"native symbol {symbol} missing from {_LIB_PATH}")
    fn.restype = ctypes.c_int
    rc = fn(*args)
    if rc != 0:
        detail = _ERRORS.get(rc, f"cudaError {rc}")
        if rc == -4 and hasattr(lib, "ttcd_last_tmap_error"):
            buf = ctypes.create_string_buffer(320)
            lib.ttcd_last_tmap_error(buf, ctypes.c_int(320))
            detail += f" ({buf.value.decode(errors='replace')})"
        raise NativeError(f"{symbol} failed: {detail}")
    if _CHECK_EVERY_CALL and _MULTI_KERNEL.get(symbol, 1) > 0:
        _check_after(symbol)


# TTCD_CHECK_EVERY_CALL=1: debugging aid for locating a misbehaving launch.  After every kernel call the device is
# synchronised, so an asynchronous CUDA error surfaces at the call that caused it instead of at some later
# synchronisation, and the status words of the bounded waits are read, so an expired wait is attributed to its kernel.
# Serialises everything (no overlap, no graph capture): never a setting for timing runs.
_CHECK_EVERY_CALL = os.environ.get("TTCD_CHECK_EVERY_CALL", "0") == "1"


def _check_after(symbol: str) -> None:
    import torch
    if torch.cuda.is_current_stream_capturing():
        return
    try:
        torch.cuda.synchronize()
    except RuntimeError as exc:
        raise NativeError(f"{symbol}: the device reported an error after this launch: {exc}") from exc
    code = device_status(reset=True)
    if code:
        raise NativeError(f"{symbol}: a bounded device wait ran out in this launch (status {code})")


def i32(v) -> ctypes.c_int:
    return ctypes.c_int(int(v))


def i64(v) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(v))


def f32(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))


# translation units of the library that contain bounded waits; each exports ttcd_read_status_<unit>
STATUS_UNITS = ("gemm", "attn", "attn_bwd", "comm", "gemm_comm")


def device_status(reset: bool = True) -> int:
    """Read (and clear) the device-side error word written by bounded waits."""
    lib = load()
    if lib is None:
        return 0
    status = 0
    for unit in STATUS_UNITS:
        fn = getattr(lib, f"ttcd_read_status_{unit}", None)
        if fn is None:
            continue
        fn.restype = ctypes.c_int
        v = int(fn(ctypes.c_int(1 if reset else 0)))
        status = status or v
    return status
