"""Process lifecycle: init / shutdown / rank / size.

API parity with the reference's ``tips.tensorflow`` basics (tips/tensorflow/basics.py:8-31,
ops.py:26-30): ``init`` (the reference initialises at import time), ``shutdown``
(registered with ``atexit``), ``size``, ``rank``, ``initialized``; plus
``local_rank`` / ``local_size`` which a one-process-per-GPU job needs to pick
its device.
"""
from __future__ import annotations

import atexit
import os

from . import _lib
from .config import get_config

_atexit_registered = False
_device_state = None


class TipsError(RuntimeError):
    """A tips runtime or collective failure, with the native status code."""

    def __init__(self, message: str, code: int = 7):
        super().__init__(message)
        self.code = code


def _check(rc: int, what: str) -> int:
    if rc < 0:
        raise TipsError(f"{what}: {_lib.last_error()}", -rc)
    return rc


def init(rank: int | None = None, size: int | None = None, master_addr: str | None = None,
         master_port: int | None = None, device: bool | None = None) -> None:
    """Start the runtime on this process.

    Without arguments the rank, the world size and the rendezvous address are
    taken from the environment of a ``torchrun``-style launcher (RANK,
    WORLD_SIZE, MASTER_ADDR, MASTER_PORT).  With ``device`` true (default: when
    CUDA is available) the GPU data plane is set up as well: the process binds
    to ``cuda:local_rank`` and, for world sizes above one, maps the symmetric
    memory windows used by the fused kernels.
    """
    global _atexit_registered, _device_state
    lib = _lib.core()
    if lib.tips_is_initialized():
        return
    cfg = get_config()
    levels = {"INFO": 0, "WARNING": 1, "ERROR": 2, "FATAL": 3}
    if "TIPS_LOG_LEVEL" not in os.environ:
        lib.tips_set_log_level(levels.get(cfg.log_level.upper(), 1), int(os.environ.get("GLOG_v", "0") or 0))
    lib.tips_set_fusion_threshold(int(cfg.fusion_threshold_bytes))
    lib.tips_set_cycle_time_ms(int(cfg.cycle_time_ms))
    lib.tips_set_stall_check(int(cfg.stall_warn_s * 1000), int(cfg.stall_abort_s * 1000))
    if rank is None and size is None:
        _check(lib.tips_init(), "tips_init")
    else:
        env_rank = int(os.environ.get("RANK", "0"))
        env_size = int(os.environ.get("WORLD_SIZE", "1"))
        addr = master_addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
        _check(lib.tips_init_ex(env_rank if rank is None else rank, env_size if size is None else size,
                                addr.encode(), int(master_port or 0)), "tips_init")
    if not _atexit_registered:
        atexit.register(shutdown)
        _atexit_registered = True
    if cfg.timeline_path:
        lib.tips_timeline_enable(1)
    if device is None:
        import torch
        device = torch.cuda.is_available()
    if device:
        from .parallel import device as _device
        _device_state = _device.setup()
        if cfg.numa_bind:
            bind_to_gpu_numa_node()


def bind_to_gpu_numa_node(device_index: int | None = None, sysfs: str = "/sys", pci_bus_id: str | None = None):
    """Limit this process to the CPUs of the NUMA node its GPU hangs off, so that pinned host buffers allocated from
    here on sit next to the GPU that reads them (``numa_bind=True`` / ``TIPS_NUMA_BIND=1`` does this inside
    ``init()``; ``python -m tips_b200.launch --bind numa`` does it before the process starts).  Returns the CPU list,
    or None when the platform reports no node for the device or the node has no CPU this process may use."""
    from .launch import gpu_numa_cpus
    if not hasattr(os, "sched_setaffinity"):
        return None
    if pci_bus_id is None:
        import torch
        if not torch.cuda.is_available():
            return None
        props = torch.cuda.get_device_properties(torch.cuda.current_device() if device_index is None else device_index)
        if not hasattr(props, "pci_bus_id"):
            return None
        pci_bus_id = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    cpus = gpu_numa_cpus(0, sysfs, [pci_bus_id])
    if not cpus:
        return None
    cpus = sorted(set(cpus) & set(os.sched_getaffinity(0)))
    if not cpus:
        return None
    try:
        os.sched_setaffinity(0, cpus)
    except OSError:
        return None
    return cpus


def shutdown() -> None:
    """Stop the runtime; collectives still in flight fail with an "aborted" status."""
    global _device_state
    lib = _lib.core()
    if not lib.tips_is_initialized():
        return
    cfg = get_config()
    if cfg.timeline_path:
        path = cfg.timeline_path
        if lib.tips_size() > 1:
            path = f"{path}.rank{lib.tips_rank()}"
        lib.tips_timeline_dump(path.encode())
    if _device_state is not None:
        from .parallel import device as _device
        _device.teardown(_device_state)
        _device_state = None
    lib.tips_shutdown()


def is_initialized() -> bool:
    return bool(_lib.core().tips_is_initialized())


initialized = is_initialized


def _require_init():
    if not _lib.core().tips_is_initialized():
        raise TipsError("tips is not initialised; call tips_b200.init() first", 3)


def size() -> int:
    _require_init()
    return _lib.core().tips_size()


def rank() -> int:
    _require_init()
    return _lib.core().tips_rank()


def local_rank() -> int:
    _require_init()
    return _lib.core().tips_local_rank()


def local_size() -> int:
    _require_init()
    return _lib.core().tips_local_size()


def barrier() -> None:
    _require_init()
    _check(_lib.core().tips_barrier(), "barrier")


def reset_collectives() -> None:
    """Bring the collective machinery back to a clean state after a failed step, on every rank: collectives still
    in flight fail with status 4, partial negotiations and the frozen bucket order are forgotten, the flags, epochs
    and error state of the GPU data plane are cleared, and the ranks meet on a host barrier before any of them
    issues the next collective.  Raises if a rank does not arrive (the job cannot continue with the same ranks)."""
    _require_init()
    lib = _lib.core()
    _check(-abs(lib.tips_reset_collectives()), "reset_collectives")
    if _device_state is not None and _device_state.window is not None:
        k = _lib.kernels()
        if k.tipsk_comm_reset() != 0:
            raise TipsError("tipsk_comm_reset: " + k.tipsk_last_error().decode(), 7)
    if lib.tips_size() > 1:
        barrier()


def device_state():
    return _device_state


def metrics() -> dict:
    """Counters of the collective engine and the RPC layer."""
    import ctypes
    lib = _lib.core()
    names = lib.tips_counter_names().decode().split(",")
    buf = (ctypes.c_uint64 * len(names))()
    n = lib.tips_counters(buf, len(names))
    out = {names[i]: int(buf[i]) for i in range(n)}
    if _device_state is not None:
        out.update(_device_state.metrics())
    return out
