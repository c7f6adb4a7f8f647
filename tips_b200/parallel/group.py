"""Sub-groups of ranks with their own host collectives.

The reference builds sub-communicators with ``MpiGroup`` (a set of world ranks, the group-rank <-> world-rank map,
``Barrier``, ``AllReduce``: tips/core/mpi_group.h:15-96, mpi_group.cc:5-52) and uses one for the parameter
servers (tips/core/ps/route.h:58-76).  ``Group`` is the same object over this runtime's TCP control plane:
creating one is a collective over the world (every rank passes the same list, in the same order relative to
other groups), its barrier / allgather / allreduce involve the members only.
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
