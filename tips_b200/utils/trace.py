"""NVTX ranges around the host-side phases of a step (bucket pack and hand-off to the engine, waits, parameter
-server pull and push), next to the engine's own Chrome-trace timeline and the ranges the device executor opens
around every collective launch.  Off unless ``TIPS_NVTX=1`` (a range costs two calls into the NVTX library; a
profiler is rarely attached).  The reference has no tracing beyond VLOG lines (tips/core/common/logging.h)."""
from __future__ import annotations

import contextlib
import os

_enabled = os.environ.get("TIPS_NVTX", "0") == "1"


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def _null():
    yield


def nvtx_range(name: str):
    """Context manager: an NVTX range on the calling thread when tracing is on and CUDA is available."""
    if not _enabled:
        return _null()
    import torch
    if not torch.cuda.is_available():
        return _null()
    return torch.cuda.nvtx.range(name)
