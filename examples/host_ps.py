"""Host parameter server (the reference's PsServer / PsClient path): a sparse table with arbitrary 64-bit keys
and a dense table addressed by index range; ranks 0..servers-1 serve shards, every rank pulls and pushes.

    python -m torch.distributed.run --nproc-per-node 3 examples/host_ps.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.ps.host import HostDenseTable, HostSparseTable, Route  # noqa: E402


def main():
    tips.init(device=False)
    servers = list(range(max(1, tips.size() // 2)))
    table = HostSparseTable("demo", dim=8, route=Route(servers=servers), optimizer="adagrad", lr=0.1)
    rng = np.random.default_rng(tips.rank())
    for step in range(5):
        keys = rng.integers(0, 1000, size=64).astype(np.uint64)
        rows = table.pull(keys)
        grads = rows * 0.1 + 1.0
        table.push(keys, grads)
        tips.barrier()
    # asynchronous calls: the rows of the next batch travel while this batch's gradients are pushed
    batches = [rng.integers(0, 1000, size=64).astype(np.uint64) for _ in range(3)]
    nxt = table.pull_async(batches[0])
    for i, keys in enumerate(batches):
        rows = nxt.wait()
        if i + 1 < len(batches):
            nxt = table.pull_async(batches[i + 1])
        table.push_async(keys, rows * 0.1 + 1.0).wait()
    tips.barrier()
    print(f"rank {tips.rank()}: local rows {table.local_size()} counters {table.counters()}")
    table.close()
    # a dense vector of 10 000 weights: rank 0 sets it, every rank pushes a gradient for its own range
    dense = HostDenseTable("dense_demo", 10_000, route=Route(servers=servers), optimizer="sgd", lr=0.5)
    if tips.rank() == 0:
        dense.assign(np.ones(10_000, dtype=np.float32))
    tips.barrier()
    lo = 1000 * tips.rank()
    dense.push(np.full(500, 0.2, dtype=np.float32), begin=lo)
    tips.barrier()
    w = dense.pull(lo, lo + 502)
    print(f"rank {tips.rank()}: dense[{lo}:{lo + 3}] = {w[:3]}, dense[{lo + 500}] = {w[500]}  {dense.counters()}")
    dense.close()
    tips.shutdown()


if __name__ == "__main__":
    main()
