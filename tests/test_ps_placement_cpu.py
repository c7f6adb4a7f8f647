"""Placement rule of the GPU parameter-server tables: the host-side mirror (ShardedEmbedding.place / global_ids)
against the rule the kernels compile (tipsk_ps_place), and the bijection id <-> (owner, local row)."""
import ctypes

import pytest
import torch

from tips_b200.ops import base
from tips_b200.ps.gpu import ShardedEmbedding


class _Geometry:
    """The fields of a ShardedEmbedding that the placement helpers read, without a device."""

    def __init__(self, n, rows):
        self.size, self.nservers, self.rows = n, n, rows
        self.rows_per_shard = (rows + n - 1) // n

    place = ShardedEmbedding.place
    global_ids = ShardedEmbedding.global_ids


@pytest.mark.parametrize("n", [1, 2, 3, 4, 8])
def test_python_rule_matches_the_compiled_rule(n):
    lib = base.K()
    g = _Geometry(n, 100_000)
    ids = torch.cat([torch.arange(0, 300), torch.randint(0, 1 << 40, (300,), generator=torch.Generator().manual_seed(n))])
    for f in (0, 1, 7, 25, 63):
        owner, lrow = g.place(ids, f)
        for k in range(ids.numel()):
            o, l = ctypes.c_int32(), ctypes.c_int64()
            assert lib.tipsk_ps_place(f, int(ids[k]), n, ctypes.byref(o), ctypes.byref(l)) == 0
            assert (o.value, l.value) == (int(owner[k]), int(lrow[k])), (f, int(ids[k]))


@pytest.mark.parametrize("n", [1, 2, 3, 8])
def test_placement_is_a_bijection(n):
    rows = 1000 * n
    g = _Geometry(n, rows)
    for f in (0, 5):
        seen = torch.zeros(rows, dtype=torch.int32)
        for r in range(n):
            ids = g.global_ids(f, r)
            owner, lrow = g.place(ids, f)
            assert torch.equal(owner, torch.full_like(owner, r))
            assert torch.equal(lrow, torch.arange(g.rows_per_shard))
            seen[ids] += 1
        assert torch.equal(seen, torch.ones_like(seen))
