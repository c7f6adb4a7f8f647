"""Sub-groups of ranks with their own host collectives.

The reference builds sub-communicators with ``MpiGroup`` (a set of world ranks, the group-rank <-> world-rank map,
``Barrier``, ``AllReduce``: tips/core/mpi_group.h:15-96, mpi_group.cc:5-52) and uses one for the parameter
servers (tips/core/ps/route.h:58-76).  ``Group`` is the same object over this runtime's TCP control plane:
creating one is a collective over the world (every rank passes the same list, in the same order relative to
other groups), its barrier / allgather / allreduce involve the members only.

Tensor collectives (``allreduce_``, ``allgather``, ``broadcast_``) among the members: CUDA tensors go through the
device kernels of ``DeviceGroup`` (peer loads and stores inside the group's own slice of the symmetric window),
CPU tensors through the control plane.
"""
from __future__ import annotations

import ctypes
import pickle
from typing import Any, Iterable, List

from .. import _lib
from ..runtime import TipsError, _require_init


class Group:
    def __init__(self, world_ranks: Iterable[int]):
        _require_init()
        ranks = [int(r) for r in world_ranks]
        arr = (ctypes.c_int32 * len(ranks))(*ranks)
        gid = _lib.core().tips_group_new(arr, len(ranks))
        if gid < 0:
            raise TipsError("group: " + _lib.core().tips_last_error().decode(), int(-gid))
        self.id = int(gid)
        self._ranks = sorted(set(ranks))
        self._device = None
        # every rank of the job reserves the group's slice of the symmetric window here, members or not,
        # so that the slice sits at the same offset everywhere
        from . import device as D
        if D._state is not None and D._state.window is not None and not D._state.emulated:
            self._device = D.DeviceGroup(self._ranks, group_id=self.id)

    # -- membership ---------------------------------------------------------------
    @property
    def size(self) -> int:
        return _lib.core().tips_group_size(self.id)

    @property
    def rank(self) -> int:
        """Rank of this process inside the group, -1 if it is not a member."""
        return _lib.core().tips_group_rank(self.id)

    @property
    def is_member(self) -> bool:
        return self.rank >= 0

    def to_world_rank(self, group_rank: int) -> int:
        r = _lib.core().tips_group_to_world(self.id, group_rank)
        if r < 0:
            raise IndexError(f"group rank {group_rank} out of range")
        return r

    @property
    def world_ranks(self) -> List[int]:
        return [self.to_world_rank(i) for i in range(self.size)]

    # -- collectives among the members ----------------------------------------------
    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise TipsError(f"group {what}: " + _lib.core().tips_last_error().decode(), rc if rc > 0 else -rc)

    def barrier(self, timeout_s: float | None = None) -> None:
        self._check(_lib.core().tips_group_barrier(self.id, -1 if timeout_s is None else int(timeout_s * 1000)),
                    "barrier")

    def allgather_bytes(self, payload: bytes, max_bytes: int = 1 << 20, timeout_s: float | None = None) -> List[bytes]:
        n = self.size
        if len(payload) > max_bytes:
            raise ValueError("payload larger than max_bytes")
        out = ctypes.create_string_buffer(n * max_bytes)
        sizes = (ctypes.c_int64 * n)()
        self._check(_lib.core().tips_group_allgather(self.id, payload, len(payload), out, max_bytes, sizes,
                                                     -1 if timeout_s is None else int(timeout_s * 1000)), "allgather")
        return [out.raw[i * max_bytes:i * max_bytes + sizes[i]] for i in range(n)]

    def allgather_object(self, obj: Any) -> list:
        return [pickle.loads(b) for b in self.allgather_bytes(pickle.dumps(obj))]

    def allreduce(self, value: float) -> float:
        """Sum of a scalar over the members."""
        return float(sum(self.allgather_object(float(value))))

    # -- tensor collectives among the members -------------------------------------
    _OPS = {"Sum": 0, "Average": 0, "Max": 1, "Min": 2, "Product": 3}

    def _host_gather(self, t):
        import torch
        flat = t.detach().contiguous().cpu()
        blobs = self.allgather_bytes(pickle.dumps((tuple(flat.shape), flat.view(torch.uint8).numpy().tobytes()
                                                   if flat.numel() else b"")),
                                     max_bytes=max(1 << 16, 2 * flat.numel() * flat.element_size() + 4096))
        out = []
        for b in blobs:
            shape, raw = pickle.loads(b)
            out.append(torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(t.dtype).reshape(shape)
                       if raw else torch.empty(shape, dtype=t.dtype))
        return out

    def allreduce_(self, tensor, op: str = "Sum"):
        """Reduce `tensor` in place over the members (Sum, Average, Max, Min, Product)."""
        import torch
        if op not in self._OPS:
            raise ValueError(f"unknown reduction {op}")
        n = self.size
        if n == 1:
            return tensor
        if tensor.is_cuda and self._device is not None:
            if not tensor.is_contiguous():
                raise ValueError("group allreduce_ takes a contiguous tensor")
            self._device.allreduce_(tensor, self._OPS[op], 1.0, 1.0 / n if op == "Average" else 1.0)
            return tensor
        parts = torch.stack([p.to(torch.float64) if p.is_floating_point() else p for p in self._host_gather(tensor)])
        red = {"Sum": parts.sum(0), "Average": parts.sum(0) / n if tensor.is_floating_point() else parts.sum(0) // n,
               "Max": parts.amax(0), "Min": parts.amin(0), "Product": parts.prod(0)}[op]
        with torch.no_grad():
            tensor.copy_(red.to(tensor.dtype))
        return tensor

    def allgather(self, tensor):
        """Concatenate the members' tensors along dim 0 (first dimensions may differ), in group-rank order."""
        import torch
        if self.size == 1:
            return tensor.clone()
        if tensor.is_cuda and self._device is not None:
            dims = self.allgather_object(int(tensor.shape[0]))
            return self._device.allgatherv(tensor.contiguous(), dims)
        return torch.cat(self._host_gather(tensor), 0).to(tensor.device)

    def broadcast_(self, tensor, root: int = 0):
        """Overwrite `tensor` on every member with group rank `root`'s."""
        import torch
        if self.size == 1:
            return tensor
        if tensor.is_cuda and self._device is not None:
            if not tensor.is_contiguous():
                raise ValueError("group broadcast_ takes a contiguous tensor")
            self._device.broadcast_(tensor, root)
            return tensor
        parts = self._host_gather(tensor if self.rank == root else tensor.new_empty((0,)))
        with torch.no_grad():
            tensor.copy_(parts[root].reshape(tensor.shape))
        return tensor
