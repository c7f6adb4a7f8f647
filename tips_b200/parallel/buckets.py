"""Gradient fusion buckets.

A bucket is one flat gradient buffer that covers a run of parameters (in reverse
registration order, i.e. roughly the order in which backward produces their
gradients) up to ``fusion_threshold_bytes``.  On a multi-GPU job the buffer is
carved out of the symmetric memory window so the allreduce kernel can work on it
in place; gradients are gathered into it by ONE pack kernel per bucket (scale and
cast to the wire dtype fused), and the optimizer reads the reduced gradients
straight from it.

This is the "fusion buffer" that the reference's DistributedOptimizer lacks: it
issues one negotiated MPI_Allreduce per gradient tensor
(tips/tensorflow/__init__.py:203-222, tips/core/collective/coordinator.cc:256-274).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from ..config import get_config


class Bucket:
    def __init__(self, index: int, params: List[torch.nn.Parameter], wire_dtype: torch.dtype, device):
        self.index = index
        self.params = params
        self.wire_dtype = wire_dtype
        self.device = device
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            # every tensor starts on a 128-byte boundary (2-byte types): parameters are views of the flat buffer, and
            # a TMA box row of a weight matrix that straddles two 128-byte lines costs an extra sector per row
            off += (p.numel() + 63) // 64 * 64
        self.numel = max(off, 8)
        self.grad: Optional[torch.Tensor] = None      # flat [numel] wire dtype
        self.win_off: int = -1
        self.pending = 0
        self.ready_count = 0
        self.handle = None
        self.name = f"tips.bucket.{index}"
        # cached ctypes arrays for pack / unpack
        self._numels = (ctypes.c_int64 * len(params))(*[p.numel() for p in params])
        self._offsets = (ctypes.c_int64 * len(params))(*self.offsets)

    def allocate(self, device_state=None):
        nbytes = self.numel * torch.empty((), dtype=self.wire_dtype).element_size()
        if device_state is not None and device_state.window is not None and self.device.type == "cuda":
            self.grad, self.win_off = device_state.alloc_symmetric(nbytes, self.wire_dtype)
            self.grad.zero_()
        else:
            self.grad = torch.zeros(self.numel, dtype=self.wire_dtype, device=self.device)

    def view_of(self, i: int) -> torch.Tensor:
        p = self.params[i]
        return self.grad[self.offsets[i]:self.offsets[i] + p.numel()].view(p.shape)

    # -- pack / unpack ------------------------------------------------------------
    def slices(self, slice_bytes: int):
        """Cut the bucket into runs of consecutive parameters of about `slice_bytes`: [(first, last + 1, element
        offset, elements)].  Parameters sit in the buffer in the order backward produces their gradients, so a
        slice is complete, and can be reduced, while backward is still working on the later ones."""
        es = torch.empty((), dtype=self.wire_dtype).element_size()
        out, first, start = [], 0, 0
        for i in range(len(self.params)):
            end = self.offsets[i + 1] if i + 1 < len(self.params) else self.numel
            last = i + 1 == len(self.params)
            if (end - start) * es >= slice_bytes or last:
                out.append((first, i + 1, start, end - start))
                first, start = i + 1, end
        return out

    def pack(self, scale: float = 1.0, accumulate: bool = False, only=None):
        """Gather the parameters' .grad tensors into the flat buffer (one launch on CUDA); `only` = (first, last)
        restricts it to that run of parameters."""
        grads = [p.grad for p in self.params]
        if only is not None:
            grads = [g if only[0] <= i < only[1] else None for i, g in enumerate(grads)]
        if self.device.type == "cuda":
            from ..ops import base
            present = [(i, g) for i, g in enumerate(grads) if g is not None]
            if not present:
                return
            by_dtype = {}
            for i, g in present:
                by_dtype.setdefault(g.dtype, []).append((i, g if g.is_contiguous() else g.contiguous()))
            for dt, items in by_dtype.items():
                ptrs = (ctypes.c_void_p * len(items))(*[g.data_ptr() for _, g in items])
                offs = (ctypes.c_int64 * len(items))(*[self.offsets[i] for i, _ in items])
                nums = (ctypes.c_int64 * len(items))(*[g.numel() for _, g in items])
                base.check(base.K().tipsk_pack(ptrs, offs, nums, len(items), base.code(dt), self.grad.data_ptr(),
                                               base.code(self.wire_dtype), scale, int(accumulate), base.stream()),
                           "pack")
                self._keep = items  # keep the (possibly copied) sources alive until the next pack
        else:
            for i, g in enumerate(grads):
                if g is None:
                    continue
                v = self.view_of(i)
                if accumulate:
                    v.add_(g.to(self.wire_dtype), alpha=scale)
                else:
                    v.copy_(g if scale == 1.0 else g * scale)

    def unpack_to_grads(self, scale: float = 1.0):
        """Point every parameter's .grad at its slice of the bucket (copy only if dtypes differ)."""
        for i, p in enumerate(self.params):
            v = self.view_of(i)
            if v.dtype == p.dtype and scale == 1.0:
                p.grad = v
            else:
                g = v.to(p.dtype)
                if scale != 1.0:
                    g.mul_(scale)
                p.grad = g


def resolve_wire_dtype(params, wire: str) -> torch.dtype:
    if wire in ("bf16", "bfloat16"):
        return torch.bfloat16
    if wire in ("fp16", "float16", "half"):
        return torch.float16
    if wire in ("fp32", "float32"):
        return torch.float32
    # auto: the widest gradient dtype among the parameters
    dts = {p.dtype for p in params}
    if torch.float32 in dts or torch.float64 in dts:
        return torch.float32
    if torch.bfloat16 in dts:
        return torch.bfloat16
    return torch.float16 if torch.float16 in dts else torch.float32


def build_buckets(params, threshold_bytes: Optional[int] = None, wire_dtype="auto", device_state=None,
                  reverse: bool = True) -> List[Bucket]:
    params = [p for p in params if p.requires_grad]
    if not params:
        return []
    cfg = get_config()
    threshold = int(threshold_bytes if threshold_bytes is not None else cfg.fusion_threshold_bytes)
    ordered = list(reversed(params)) if reverse else list(params)
    buckets: List[Bucket] = []
    # one bucket never mixes devices; wire dtype is chosen per bucket group
    cur, cur_bytes, cur_dev = [], 0, None
    wd = resolve_wire_dtype(params, wire_dtype) if isinstance(wire_dtype, str) else wire_dtype
    es = torch.empty((), dtype=wd).element_size()

    def flush():
        nonlocal cur, cur_bytes
        if cur:
            b = Bucket(len(buckets), cur, wd, cur_dev)
            b.allocate(device_state)
            buckets.append(b)
        cur, cur_bytes = [], 0

    for p in ordered:
        nbytes = p.numel() * es
        if cur and (p.device != cur_dev or (threshold > 0 and cur_bytes + nbytes > threshold)):
            flush()
        if not cur:
            cur_dev = p.device
        cur.append(p)
        cur_bytes += nbytes
        if threshold <= 0:
            flush()
    flush()
    return buckets
