"""ctypes binding of `libsumma_b200.so` (the in-tree sm_100a kernel library).

Every exported launcher takes raw device pointers plus the CUDA stream and returns
0 or a negative error code; `call()` turns a non-zero code into an exception. The
library is built by `summa_b200.ops.build`; on a machine with a GPU a missing
library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SUMMA_B200_LIB points at an alternative build of the kernel library (kernel tuning sweeps)
LIB_PATH = os.environ.get("SUMMA_B200_LIB") or os.path.join(_HERE, "libsumma_b200.so")
_lib: Optional[ctypes.CDLL] = None

P, I, L, F = c_void_p, c_int, c_long, c_float

_SIGNATURES = {
    "sb_read_error_flag": [P],
    "sb_num_sms": [],
    "sb_set_device": [I],
    "sb_gemm_bf16": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P],
    "sb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "sb_rmsnorm_bwd": [P, P, P, P, P, P, P, I, I, P],
    "sb_qk_rope": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
    "sb_swiglu_fwd": [P, P, L, I, L, P],
    "sb_swiglu_bwd": [P, P, P, L, I, L, P],
    "sb_mul_silu_fwd": [P, P, P, L, I, L, L, P],
    "sb_mul_silu_bwd": [P, P, P, P, P, L, I, L, L, L, L, P],
    "sb_adamw": [P, P, P, P, P, L, P, F, F, F, F, F, F, F, P],
    "sb_sumsq": [P, L, P, P],
    "sb_muon_momentum": [P, P, P, I, L, P, F, P],
    "sb_muon_apply": [P, P, P, I, L, F, P],
}


class NativeError(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeError(
                f"{LIB_PATH} is missing: build it with `python -m summa_b200.ops.build` "
                "(CUDA tensors never fall back to PyTorch ops)")
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


_RESTYPES = {}


def register(name: str, argtypes, restype=None) -> None:
    _SIGNATURES[name] = argtypes
    if restype is not None:
        _RESTYPES[name] = restype


_bound = {}


def fn(name: str):
    f = _bound.get(name)
    if f is None:
        f = getattr(lib(), name)
        f.argtypes = _SIGNATURES[name]
        f.restype = _RESTYPES.get(name, c_int)
        _bound[name] = f
    return f


_CODES = {-1: "bad argument", -2: "CUDA runtime error", -3: "tensor-map encode failed",
          -4: "size exceeds capacity"}


_tls = threading.local()


def _bind_device() -> None:
    """The library carries its own CUDA runtime instance, whose current device is
    per-thread state: mirror torch's current device into it (cheap after the first
    call on a thread)."""
    dev = torch.cuda.current_device()
    if getattr(_tls, "dev", None) != dev:
        rc = fn("sb_set_device")(dev)
        if rc != 0:
            raise NativeError(f"sb_set_device({dev}) failed")
        _tls.dev = dev


def call(name: str, *args) -> None:
    _bind_device()
    rc = fn(name)(*args)
    if rc != 0:
        raise NativeError(f"{name} failed: {_CODES.get(rc, rc)}")


def call_value(name: str, *args) -> int:
    """Call an entry point whose return value is a quantity, not a status code."""
    _bind_device()
    return int(fn(name)(*args))


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    """Raw handle of torch's current CUDA stream (the C accessor: `torch.cuda.current_stream()` builds a Python
    stream object on every call, ~16 us, which at ~550 launches per training step was 9 ms of host time)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def read_error_flag() -> int:
    """Device error word (0 = clean): bit 1 = an mbarrier wait timed out, bit 2 = a
    peer-flag wait timed out, bit 4 = a kernel saw a bad argument. Synchronises."""
    out = ctypes.c_uint(0)
    call("sb_read_error_flag", ctypes.byref(out))
    return int(out.value)
