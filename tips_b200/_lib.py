"""ctypes bindings to the native libraries.

Counterpart of the reference's loader (tips/tensorflow/basics.py:5-31, ops.py:11-30),
which opens ``libtipscore.so`` with ``ctypes.CDLL`` and calls ``tips_init`` at
import.  Here loading and initialisation are separate steps (``tips_b200.init()``),
and the CUDA kernels live in a second library that is only opened when a GPU is
present; if a GPU is present and that library is missing the import fails loudly
instead of falling back to another implementation.
"""
from __future__ import annotations

import ctypes
from ctypes import (CFUNCTYPE, POINTER, Structure, c_char_p, c_double, c_int, c_int32, c_int64, c_uint64,
                    c_void_p)
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"

ALLOC_FN = CFUNCTYPE(c_void_p, c_int64, c_int64, POINTER(c_int64), c_int32, c_void_p)


class TipsOp(Structure):
    _fields_ = [
        ("name", c_char_p), ("type", c_int32), ("dtype", c_int32), ("ndim", c_int32),
        ("shape", POINTER(c_int64)), ("in_", c_void_p), ("out", c_void_p), ("device", c_int32),
        ("root_rank", c_int32), ("reduce_op", c_int32), ("prescale", c_double), ("postscale", c_double),
        ("stream", c_void_p), ("ready_event", c_void_p), ("done_event", c_void_p),
        ("alloc", ALLOC_FN), ("alloc_user", c_void_p),
    ]


def _build_if_missing(name: str) -> Path:
    path = _LIB_DIR / name
    if not path.exists():
        from . import build
        if name == "libtips_core.so":
            build.build_core()
        else:
            build.build_kernels()
    return path


_core = None
_kernels = None


def core() -> ctypes.CDLL:
    """The host runtime library (built on first use if absent)."""
    global _core
    if _core is not None:
        return _core
    path = _build_if_missing("libtips_core.so")
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    lib.tips_last_error.restype = c_char_p
    lib.tips_counter_names.restype = c_char_p
    lib.tips_init_ex.argtypes = [c_int, c_int, c_char_p, c_int]
    lib.tips_enqueue.argtypes = [POINTER(TipsOp)]
    lib.tips_enqueue.restype = c_int64
    lib.tips_poll.argtypes = [c_int64]
    lib.tips_wait.argtypes = [c_int64, c_int]
    lib.tips_release.argtypes = [c_int64]
    lib.tips_handle_error.argtypes = [c_int64, c_char_p, c_int]
    lib.tips_handle_sizes.argtypes = [c_int64, POINTER(c_int64), c_int]
    lib.tips_handle_output.argtypes = [c_int64]
    lib.tips_handle_output.restype = c_void_p
    lib.tips_host_allgather.argtypes = [c_void_p, c_int64, c_void_p, c_int64, POINTER(c_int64)]
    lib.tips_host_broadcast.argtypes = [c_void_p, c_int64, c_int]
    lib.tips_group_new.argtypes = [POINTER(ctypes.c_int32), c_int]
    lib.tips_group_new.restype = c_int64
    for fn in (lib.tips_group_size, lib.tips_group_rank):
        fn.argtypes = [c_int64]
    lib.tips_group_to_world.argtypes = [c_int64, c_int]
    lib.tips_group_barrier.argtypes = [c_int64, c_int]
    lib.tips_group_allgather.argtypes = [c_int64, c_void_p, c_int64, c_void_p, c_int64, POINTER(c_int64), c_int]
    lib.tips_set_fusion_threshold.argtypes = [c_int64]
    lib.tips_set_device_executor.argtypes = [c_void_p]
    lib.tips_take_negotiated_order.argtypes = [c_char_p, c_int]
    lib.tips_freeze_schedule.argtypes = [c_char_p]
    lib.tips_timeline_dump.argtypes = [c_char_p]
    lib.tips_counters.argtypes = [POINTER(c_uint64), c_int]
    lib.tips_rank_ip.argtypes = [c_int, c_char_p, c_int]
    _core = lib
    return lib


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library. Raises if it cannot be loaded."""
    global _kernels
    if _kernels is not None:
        return _kernels
    path = _build_if_missing("libtips_kernels.so")
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m tips_b200.build` (needs nvcc)")
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    from .ops import _signatures
    _signatures.declare(lib)
    _kernels = lib
    return lib


def kernels_available() -> bool:
    return (_LIB_DIR / "libtips_kernels.so").exists()


def last_error() -> str:
    msg = core().tips_last_error()
    return msg.decode() if msg else ""
