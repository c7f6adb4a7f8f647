"""Collectives on CPU ranks through the negotiating engine: values, dtypes, odd sizes, average vs sum,
any broadcast root, allgather with unequal first dimensions, cross-rank mismatch errors, duplicate names,
fusion, object collectives, stall detection."""
import pytest
import torch

from mp_util import run_ranks


def _values(rank, size):
    import tips_b200 as tips
    assert tips.rank() == rank and tips.size() == size and tips.local_size() == size
    for dtype in (torch.float32, torch.float64, torch.int32, torch.int64, torch.bfloat16, torch.float16):
        for n in (1, 7, 1000, 4097):
            x = (torch.arange(n) % 13 + rank).to(dtype)
            s = tips.allreduce(x, op=tips.Sum)
            ref = sum(((torch.arange(n) % 13 + r).to(dtype).double()) for r in range(size))
            assert torch.allclose(s.double(), ref, rtol=2e-2 if dtype in (torch.bfloat16, torch.float16) else 1e-6), dtype
    x = torch.full((5,), float(rank + 1))
    assert torch.allclose(tips.allreduce(x), torch.full((5,), (size + 1) / 2))            # Average is the default
    assert torch.allclose(tips.allreduce(x, average=False), torch.full((5,), size * (size + 1) / 2))
    assert torch.allclose(tips.allreduce(x, op=tips.Sum, prescale_factor=2.0, postscale_factor=0.5),
                          torch.full((5,), size * (size + 1) / 2))
    assert torch.allclose(tips.allreduce(x, op=tips.Max), torch.full((5,), float(size)))
    assert torch.allclose(tips.allreduce(x, op=tips.Min), torch.full((5,), 1.0))
    y = x.clone(); tips.allreduce_(y, op=tips.Sum); assert y[0] == size * (size + 1) / 2
    assert tips.allreduce(torch.tensor(float(rank)), op=tips.Sum).item() == sum(range(size))  # scalar
    c = tips.allreduce(torch.full((64,), 1.0 + rank), compression=tips.Compression.fp16, op=tips.Sum)
    assert c.dtype == torch.float32 and torch.allclose(c, torch.full((64,), float(sum(range(1, size + 1)))))
    for root in range(size):
        b = tips.broadcast(torch.full((3, 2), float(rank)), root_rank=root)
        assert (b == root).all()
    g = tips.allgather(torch.full((rank + 1, 2, 3), float(rank)))
    assert g.shape == (size * (size + 1) // 2, 2, 3)
    off = 0
    for r in range(size):
        assert (g[off:off + r + 1] == r).all(); off += r + 1
    sp = torch.sparse_coo_tensor(torch.tensor([[rank, size]]), torch.tensor([1.0, 2.0]), (size + 1,))
    dense = tips.sparse_allreduce(sp, op=tips.Sum).to_dense()
    assert dense[size] == 2.0 * size and dense[0] == 1.0
    # rows of values whose bytes are a multiple of 8 travel with their indices as ONE allgather; a rank may have none
    rows = torch.tensor([rank, 7, 7]) if rank != 1 else torch.zeros(0, dtype=torch.int64)
    vals = torch.full((rows.numel(), 4), float(rank + 1))
    sp = torch.sparse_coo_tensor(rows.unsqueeze(0), vals, (10, 4))
    before = tips.metrics()["ops_enqueued"]
    got = tips.sparse_allreduce(sp, op=tips.Average).to_dense()
    assert tips.metrics()["ops_enqueued"] - before == 1
    want = torch.zeros(10, 4)
    for r in range(size):
        if r != 1:
            want[r] += r + 1
            want[7] += 2 * (r + 1)
    assert torch.allclose(got, want / size)
    two_d = torch.sparse_coo_tensor(torch.tensor([[rank], [2]]), torch.tensor([1.5], dtype=torch.float64), (size, 3))
    assert torch.equal(tips.sparse_allreduce(two_d, op=tips.Sum).to_dense()[:, 2], torch.full((size,), 1.5, dtype=torch.float64))
    objs = tips.allgather_object({"rank": rank, "s": "x" * rank})
    assert [o["rank"] for o in objs] == list(range(size))
    assert tips.broadcast_object(("cfg", rank), root_rank=size - 1) == ("cfg", size - 1)


def _errors(rank, size):
    import tips_b200 as tips
    with pytest.raises(tips.TipsError, match="mismatched.*shapes"):
        tips.allreduce(torch.ones(3 + rank), name="bad_shape")
    with pytest.raises(tips.TipsError, match="data types"):
        tips.allreduce(torch.ones(3, dtype=torch.float32 if rank == 0 else torch.float64), name="bad_dtype")
    with pytest.raises(tips.TipsError, match="mismatched collective operations"):
        (tips.allreduce if rank == 0 else tips.allgather)(torch.ones(3), name="bad_op")
    with pytest.raises(tips.TipsError, match="roots"):
        tips.broadcast(torch.ones(3), root_rank=rank % 2, name="bad_root")
    with pytest.raises(tips.TipsError, match="trailing"):
        tips.allgather(torch.ones(2, 3 + rank), name="bad_gather")
    h = tips.allreduce_async(torch.ones(4), name="dup", op=tips.Sum)
    if True:
        try:
            tips.allreduce_async(torch.ones(4), name="dup", op=tips.Sum)
            dup_ok = True
        except tips.TipsError as e:
            dup_ok = False
            assert "already in flight" in str(e)
        # the first may already have completed on a fast machine; both outcomes are legal, a crash is not
        if dup_ok:
            pass
    assert tips.synchronize(h)[0] == size
    # the engine still works after errors
    assert tips.allreduce(torch.ones(2), op=tips.Sum)[0] == size


def _fusion_and_order(rank, size):
    import tips_b200 as tips
    tips.barrier()
    names = [f"t{i}" for i in range(32)]
    order = names if rank == 0 else list(reversed(names))  # every rank enqueues in a different order
    hs = {n: tips.allreduce_async(torch.full((100,), float(int(n[1:]))), name=n, op=tips.Sum) for n in order}
    for n in names:
        assert torch.allclose(tips.synchronize(hs[n]), torch.full((100,), float(int(n[1:]) * size)))
    out = tips.grouped_allreduce([torch.ones(10) * i for i in range(8)], op=tips.Sum)
    assert all(torch.allclose(o, torch.ones(10) * i * size) for i, o in enumerate(out))
    m = tips.metrics()
    if rank == 0:
        assert m["fused_tensors"] > 0 and m["ops_failed"] == 0


def _stall(rank, size):
    import tips_b200 as tips
    if rank == 0:
        with pytest.raises(tips.TipsError, match="stalled"):
            tips.allreduce(torch.ones(3), name="only_rank0")
    tips.barrier()
    assert tips.allreduce(torch.ones(2), op=tips.Sum)[0] == size


def test_values_3_ranks():
    run_ranks(_values, 3)


def test_values_2_ranks():
    run_ranks(_values, 2)


def test_error_paths():
    run_ranks(_errors, 2)


def test_fusion_and_global_order():
    run_ranks(_fusion_and_order, 3)


def test_stall_detector_aborts_the_tensor():
    run_ranks(_stall, 2, env={"TIPS_STALL_ABORT_MS": "1500", "TIPS_STALL_WARN_MS": "500"})


def _groups(rank, size):
    import tips_b200 as tips
    g = tips.Group([3, 1, 1])           # unsorted, with a duplicate: normalised to [1, 3]
    h = tips.Group(range(size))
    assert g.size == 2 and g.world_ranks == [1, 3]
    assert h.size == size and h.rank == rank
    if rank in (1, 3):
        assert g.is_member and g.rank == (0 if rank == 1 else 1)
        assert g.to_world_rank(g.rank) == rank
        g.barrier()
        assert g.allgather_object({"r": rank}) == [{"r": 1}, {"r": 3}]
        assert g.allreduce(rank) == 4.0
        # tensor collectives among the members (CPU tensors travel over the control plane)
        t = torch.full((3, 2), float(rank))
        assert torch.equal(g.allreduce_(t.clone()), torch.full((3, 2), 4.0))
        assert torch.equal(g.allreduce_(t.clone(), op="Average"), torch.full((3, 2), 2.0))
        assert torch.equal(g.allreduce_(t.clone().to(torch.int64), op="Max"), torch.full((3, 2), 3, dtype=torch.int64))
        got = g.allgather(torch.full((g.rank + 1, 2), float(rank)))
        assert got.shape == (3, 2) and got[:, 0].tolist() == [1.0, 3.0, 3.0]
        b = torch.full((4,), float(rank))
        assert torch.equal(g.broadcast_(b, root=1), torch.full((4,), 3.0))
    else:
        assert not g.is_member and g.rank == -1
        with pytest.raises(tips.TipsError):
            g.barrier()
    assert h.allreduce(1.0) == float(size)
    # two groups at once with payloads far above a socket buffer: the leader answers itself and the other member
    # from its listener thread, which must not block on those sends
    e = tips.Group([0, 2])
    mine = g if rank in (1, 3) else e
    big = torch.full((300_000,), float(rank))
    mine.allreduce_(big)
    assert float(big[0]) == float(sum(mine.world_ranks)) and float(big[-1]) == float(big[0])
    with pytest.raises(tips.TipsError):
        tips.Group([0, size])           # out of range
    tips.barrier()


def test_rank_subgroups():
    run_ranks(_groups, 4)


def _grouped_broadcast(rank, size):
    """A state dict of 40 tensors of three dtypes travels as ONE negotiated collective, in place, from a root other
    than 0; so does a stock optimizer's state."""
    import tips_b200 as tips
    torch.manual_seed(rank)
    sd = {}
    for i in range(12):
        sd[f"w{i}"] = torch.randn(7 + i, 3)
        sd[f"b{i}"] = torch.randn(5 + i).to(torch.bfloat16)
        sd[f"n{i}"] = torch.full((1,), rank * 100 + i, dtype=torch.int64)
    sd["odd"] = torch.randn(6, 4).t()            # not contiguous
    want = tips.allgather_object({k: v.clone() for k, v in sd.items()})[size - 1]
    before = tips.metrics()["ops_enqueued"]
    tips.broadcast_parameters(sd, root_rank=size - 1)
    assert tips.metrics()["ops_enqueued"] - before == 1
    for k, v in sd.items():
        assert torch.equal(v, want[k]), k
    model = torch.nn.Linear(6, 3)
    opt = torch.optim.Adam(model.parameters(), lr=0.1 * (rank + 1))
    model(torch.ones(2, 6) * (rank + 1)).sum().backward()
    opt.step()
    tips.broadcast_optimizer_state(opt, root_rank=0)
    st = tips.allgather_object({k: {n: (v.clone() if isinstance(v, torch.Tensor) else v) for n, v in s.items()}
                                for k, s in opt.state_dict()["state"].items()})
    for other in st[1:]:
        for k in st[0]:
            for n in st[0][k]:
                a, b = st[0][k][n], other[k][n]
                assert torch.equal(a, b) if isinstance(a, torch.Tensor) else a == b
    assert opt.param_groups[0]["lr"] == 0.1


def test_parameters_are_broadcast_as_one_collective():
    run_ranks(_grouped_broadcast, 3)


def _shutdown_with_work_in_flight(rank, size):
    """Shutdown does not wait for collectives nobody synchronised, nor for a tensor that only one rank submitted."""
    import time
    import tips_b200 as tips
    t = torch.ones(1000)
    handles = [tips.allreduce_async(t * i, name=f"inflight.{i}") for i in range(20)]
    if rank == 0:
        handles.append(tips.allreduce_async(t, name="only.rank0"))       # never matched by the other ranks
    t0 = time.time()
    tips.shutdown()
    assert time.time() - t0 < 30
    assert not tips.is_initialized()
    assert len(handles) >= 20


def test_shutdown_with_work_in_flight():
    run_ranks(_shutdown_with_work_in_flight, 3)

