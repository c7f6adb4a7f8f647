"""Shared plumbing of the kernel wrappers: library handle, error checks, dtype codes."""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

DTYPE_CODE = {
    torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3,
    torch.int8: 4, torch.uint8: 5, torch.bfloat16: 6, torch.float16: 7,
}

_launches = 0


class KernelError(RuntimeError):
    pass


def K():
    """The CUDA kernel library; raises if it is missing (no silent fallback)."""
    return _lib.kernels()


def check(rc: int, what: str) -> None:
    global _launches
    if rc != 0:
        msg = K().tipsk_last_error()
        raise KernelError(f"{what} failed ({rc}): {msg.decode() if msg else ''}")
    _launches += 1


def count_launches(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    """Number of successful launcher calls made through the wrappers so far."""
    return _launches


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def comm_stream() -> int:
    """Current stream for the collective launchers, where a null handle means "the library's own stream":
    the legacy default stream is passed as its explicit handle instead."""
    s = torch.cuda.current_stream().cuda_stream
    return s if s else 1  # cudaStreamLegacy


def code(t: torch.Tensor | torch.dtype) -> int:
    dt = t.dtype if isinstance(t, torch.Tensor) else t
    return DTYPE_CODE[dt]


def ptr(t):
    return None if t is None else t.data_ptr()


def ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if isinstance(t, torch.Tensor) else t
    return arr


def i64_array(values):
    return (ctypes.c_int64 * len(values))(*values)


def u64_array(values):
    return (ctypes.c_uint64 * len(values))(*values)
