"""Host arithmetic of the sharded optimizer state: take / assemble are inverse for every rank count."""
import pytest
import torch

from tips_b200.parallel.sharding import ShardLayout


@pytest.mark.parametrize("nranks", [1, 2, 3, 8])
@pytest.mark.parametrize("numel", [8, 4096, 100_000, 2048 * 8 * 8 + 40])
@pytest.mark.parametrize("elem_size", [2, 4])
def test_take_and_assemble_round_trip(nranks, numel, elem_size):
    lay = ShardLayout(numel, elem_size, nranks, subtile=2048)
    full = torch.arange(numel, dtype=torch.float32)
    shards = torch.stack([lay.take(full, r) for r in range(nranks)])
    assert shards.shape == (nranks, lay.shard_numel)
    assert torch.equal(lay.assemble(shards), full)
    # every element belongs to exactly one rank
    marks = torch.stack([lay.take(torch.ones(numel), r) for r in range(nranks)])
    assert int(marks.sum()) == numel


def test_ownership_matches_the_kernel_rule():
    # vector v of a bucket belongs to rank (v mod (subtile * n)) div subtile
    lay = ShardLayout(8 * 50, 2, 2, subtile=4)
    full = torch.arange(50).repeat_interleave(8).float()  # element value = its vector index
    for r in range(2):
        got = lay.take(full, r).view(-1, 8)[:, 0]
        want = [v for v in range(50) if (v % 8) // 4 == r]
        assert got[:len(want)].tolist() == [float(v) for v in want]


def test_rejects_partial_vectors():
    with pytest.raises(ValueError):
        ShardLayout(12, 2, 2, 2048)


def test_misc_helpers_without_a_gpu():
    from tips_b200.utils import misc
    assert misc.executing_eagerly()
    calls = []

    @misc.cache
    def f(a, b=1):
        calls.append((a, b))
        return a + b

    assert f(1, b=2) == 3 and f(1, b=2) == 3 and len(calls) == 1
    ps = [torch.nn.Parameter(torch.zeros(1)) for _ in range(3)]
    assert misc.refs_to_vars(misc.vars_to_refs(ps), ps) == ps

    def g(x):
        return x * 2

    assert misc.make_subgraph(g, torch.ones(3)) is g  # CPU tensors: the function itself


def test_bucket_offsets_start_on_128_byte_boundaries():
    """Parameters become views of the flat buffer: a weight matrix that starts off a 128-byte line makes every TMA
    box row straddle two lines (measured: 4 % of the ResNet-50 step)."""
    from tips_b200.parallel.buckets import Bucket
    ps = [torch.nn.Parameter(torch.zeros(n)) for n in (1000, 64 * 3 * 7 * 7, 1, 513)]
    b = Bucket(0, ps, torch.bfloat16, torch.device("cpu"))
    assert all(off % 64 == 0 for off in b.offsets)
    assert b.numel % 64 == 0 and b.numel >= sum(p.numel() for p in ps)
    b.allocate()
    for i, p in enumerate(ps):
        assert b.view_of(i).numel() == p.numel()
