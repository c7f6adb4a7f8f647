"""Worker of the multi-GPU collective tests: one process per GPU, launched by torchrun.

Checks the fused NVLink kernels through the public API against values computed locally: allreduce
(staged and in-place bucket, sum/average/min/max, fp32/bf16/fp16/int), allgather with unequal sizes,
broadcast from every root, DistributedOptimizer on a small model against a single-process reference,
and the frozen schedule.  Prints "MULTI_GPU_OK" on rank 0 when everything passed.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import tips_b200 as tips  # noqa: E402


def main():
    tips.init()
    rank, size = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = tips.runtime.device_state()
    assert st is not None and st.window is not None
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64):
        for n in (1, 5, 1000, 65537, 3_000_001):
            torch.manual_seed(n)
            base = [torch.randint(-8, 8, (n,)).to(dtype) for _ in range(size)]
            x = base[rank].to(dev)
            out = tips.allreduce(x, op=tips.Sum, name=f"ar.{dtype}.{n}")
            ref = sum(b.double() for b in base)
            assert torch.equal(out.double().cpu(), ref), (dtype, n, (out.double().cpu() - ref).abs().max())
    x = torch.full((1000,), float(rank + 1), device=dev)
    assert torch.allclose(tips.allreduce(x), torch.full_like(x, (size + 1) / 2))
    assert torch.allclose(tips.allreduce(x, op=tips.Max), torch.full_like(x, float(size)))
    assert torch.allclose(tips.allreduce(x, op=tips.Min), torch.full_like(x, 1.0))
    y = x.clone()
    tips.allreduce_(y, op=tips.Sum)
    assert torch.allclose(y, torch.full_like(y, size * (size + 1) / 2))
    g = tips.allgather(torch.full((rank + 1, 3), float(rank), device=dev))
    assert g.shape[0] == size * (size + 1) // 2
    off = 0
    for r in range(size):
        assert (g[off:off + r + 1] == r).all()
        off += r + 1
    for root in range(size):
        b = tips.broadcast(torch.full((70001,), float(rank), device=dev, dtype=torch.bfloat16), root_rank=root)
        assert (b == root).all()
    st.check_status()
    # large messages: the gather above the pushing kernel's limit, the broadcast as scatter + allgather (forced for
    # two ranks too), an odd byte count, every root
    lib = tips._lib.kernels()
    assert lib.tipsk_comm_set_option(b"bcast_scatter_min_ranks", 2) == 0
    assert lib.tipsk_comm_set_option(b"bcast_scatter_bytes", 1 << 20) == 0
    assert lib.tipsk_comm_set_option(b"bcast_scatter_chunk_bytes", 4 << 20) == 0
    g = tips.allgather(torch.full(((rank + 1) * 3_000_001,), float(rank), device=dev))
    off = 0
    for r in range(size):
        part = g[off:off + (r + 1) * 3_000_001]
        assert float(part.min()) == r and float(part.max()) == r
        off += (r + 1) * 3_000_001
    for root in range(size):
        torch.manual_seed(root)
        want = torch.randn(9_000_001).to(torch.bfloat16)
        b = tips.broadcast(want.to(dev) if rank == root else torch.zeros(9_000_001, device=dev, dtype=torch.bfloat16),
                           root_rank=root)
        assert torch.equal(b.cpu(), want), root
    st.check_status()

    # DistributedOptimizer against a single-process reference on the concatenated batch
    from tips_b200.ops.optim import FusedSGD
    torch.manual_seed(7)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).to(dev)
    ref = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).to(dev)
    ref.load_state_dict(model.state_dict())
    tips.broadcast_parameters(model.state_dict(), 0)
    opt = tips.DistributedOptimizer(FusedSGD(model.parameters(), lr=0.1, momentum=0.9))
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    for step in range(6):
        torch.manual_seed(100 + step)
        xs = torch.randn(size * 16, 32, device=dev)
        ys = torch.randint(0, 10, (size * 16,), device=dev)
        loss = torch.nn.functional.cross_entropy(model(xs[rank * 16:(rank + 1) * 16]), ys[rank * 16:(rank + 1) * 16])
        loss.backward()
        opt.step()
        rl = torch.nn.functional.cross_entropy(ref(xs), ys)
        rl.backward()
        ropt.step()
        ropt.zero_grad()
    torch.cuda.synchronize()
    st.check_status()
    for (k, a), (_, b) in zip(model.state_dict().items(), ref.state_dict().items()):
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (k, (a - b).abs().max())
    # sub-groups: even and odd ranks run their own device collectives at the same time, then all ranks as a group
    even, odd = tips.Group(range(0, size, 2)), tips.Group(range(1, size, 2))
    everyone = tips.Group(range(size))
    mine = even if rank % 2 == 0 else odd
    peers = mine.world_ranks
    assert mine._device is not None and (odd if rank % 2 == 0 else even).rank == -1
    for n, dtype in [(3, torch.float32), (100003, torch.bfloat16), (12_000_001, torch.float32)]:
        t = torch.full((n,), float(rank + 1), device=dev, dtype=dtype)
        mine.allreduce_(t)
        assert (t == float(sum(p + 1 for p in peers))).all(), (n, dtype)
        t = torch.full((n,), float(rank + 1), device=dev, dtype=dtype)
        everyone.allreduce_(t, op="Max")
        assert (t == float(size)).all()
    t = torch.full((1000,), float(rank), device=dev)
    mine.allreduce_(t, op="Average")
    assert torch.allclose(t, torch.full_like(t, sum(peers) / len(peers)))
    g = mine.allgather(torch.full((mine.rank + 2, 5), float(rank), device=dev))
    assert g.shape[0] == sum(i + 2 for i in range(len(peers)))
    off = 0
    for i, p in enumerate(peers):
        assert (g[off:off + i + 2] == p).all()
        off += i + 2
    for root in range(len(peers)):
        b = torch.full((70001,), float(rank), device=dev, dtype=torch.bfloat16)
        mine.broadcast_(b, root=root)
        assert (b == peers[root]).all()
    torch.cuda.synchronize()
    st.check_status()
    m = tips.metrics()
    if rank == 0:
        assert m["frozen_executions"] > 0, m
        print("metrics", m)
    tips.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    tips.shutdown()


if __name__ == "__main__":
    main()
