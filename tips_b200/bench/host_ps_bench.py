"""The CTR parameter-server step through the HOST parameter server on CPU ranks: the path the reference has.

    python -m tips_b200.bench.host_ps_bench [--ranks 2,4] [--batch 8192] [--steps 5]

Every rank is server and worker (the reference's default route, tips/core/ps/route.h:22-56).  A step pulls the
rows of one batch (batch x 26 keys drawn Zipf(1.05) from 10M ids per field, rows of 64 fp32, created on first
pull as in tips/core/ps/access_method.h:90-99), computes nothing, and pushes one gradient row per distinct key,
which the owning shard applies with Adagrad (tips/core/ps/ps_server.h:147-265 serves pull and push the same way:
hash-map shards behind RPC, one update per key).  The worker sends each distinct key once, as the reference's
client does (its request carries a key set).  Timed on the host with a barrier on both sides, max over ranks.

This is the timed stand-in for the reference's parameter-server mode on this machine; the GPU path's samples/s on
the same model shape are what `bench.py` reports.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import time

import numpy as np
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p if p < 60000 else p - 5000


def _zipf_ids(rng, n, rows, a=1.05):
    """Ids in [0, rows) with P(k) ~ 1 / (k + 1)^a, by inverting the continuous bound of the distribution."""
    u = rng.random(n)
    lo, hi = 1.0, float(rows + 1)
    x = ((hi ** (1 - a) - lo ** (1 - a)) * u + lo ** (1 - a)) ** (1 / (1 - a))
    return np.minimum(x.astype(np.int64) - 1, rows - 1)


def _rank_main(rank, size, port, a, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(size), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    tips.init(device=False)
    table = HostSparseTable("ctr", dim=a.dim, route=Route(), optimizer="adagrad", lr=0.05, local_shards=a.shards,
                            timeout_s=300.0)
    rng = np.random.default_rng(100 + rank)
    batches = []
    for _ in range(a.steps + 1):
        ids = _zipf_ids(rng, a.batch * a.fields, a.rows).reshape(a.batch, a.fields)
        keys = (np.arange(a.fields, dtype=np.uint64)[None, :] << np.uint64(40)) + ids.astype(np.uint64)
        batches.append(np.unique(keys.reshape(-1)))

    def step(keys):
        rows = table.pull(keys)
        table.push(keys, rows * 0.01 + 0.001)

    step(batches[0])                     # warm-up: creates rows, opens the connections
    tips.barrier()
    t0 = time.perf_counter()
    if a.overlap:
        # the pull of the next batch and the push of this one are in flight together (asynchronous calls)
        nxt = table.pull_async(batches[1])
        pending = None
        for s in range(a.steps):
            keys = batches[1 + s]
            rows = nxt.wait()
            if s + 1 < a.steps:
                nxt = table.pull_async(batches[2 + s])
            if pending is not None:
                pending.wait()
            pending = table.push_async(keys, rows * 0.01 + 0.001)
        pending.wait()
    else:
        for s in range(a.steps):
            step(batches[1 + s])
    tips.barrier()
    dt = (time.perf_counter() - t0) / a.steps
    worst = max(tips.allgather_object(dt))
    if rank == 0:
        distinct = float(np.mean([b.size for b in batches[1:]]))
        out.put({"ranks": size, "overlap": bool(a.overlap), "batch_per_rank": a.batch, "fields": a.fields, "dim": a.dim,
                 "distinct_keys_per_step_per_rank": round(distinct), "ms_per_step": round(worst * 1e3, 1),
                 "samples_per_s": round(a.batch * size / worst, 1),
                 "rows_per_s_per_rank": round(2 * distinct / worst, 1)})
    table.close()
    tips.shutdown()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", default="2,4")
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--fields", type=int, default=26)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=10_000_000)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--shards", type=int, default=4, help="shard threads per server")
    ap.add_argument("--overlap", action="store_true", help="asynchronous calls: next pull and this push in flight together")
    a = ap.parse_args(argv)
    res = []
    ctx = mp.get_context("spawn")
    for n in [int(v) for v in a.ranks.split(",") if v]:
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, n, port, a, q)) for r in range(n)]
        for p in procs:
            p.start()
        res.append(q.get(timeout=900))
        for p in procs:
            p.join()
    print(json.dumps({"workload": "CTR step through the host parameter server (CPU ranks)", "rounds": res}))


if __name__ == "__main__":
    sys.exit(main())
