"""Host parameter server on CPU ranks: routing, lazy rows, server-side update rules, dumps.

Mirrors the reference's PS integration tests (tips/core/ps/ps_server_test.cc:55-131: pull of unknown keys gives
zeros, push of rows; ps_client_test.cc:11-85: one server, several clients, keys {0, 3, 200}) and closes their gaps:
numeric checks of the update rules, several servers, duplicate keys, dump and reload under another sharding.
"""
import os

import numpy as np
import pytest

from mp_util import run_ranks


def _one_server_many_clients(rank, size):
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    table = HostSparseTable("t1", dim=4, route=Route(servers=[0]), optimizer="sgd", lr=0.5)
    keys = np.array([0, 3, 200], dtype=np.uint64)
    rows = table.pull(keys)
    assert rows.shape == (3, 4)
    tips.barrier()
    # every rank pushes a gradient of ones for key 3
    table.push(np.array([3], dtype=np.uint64), np.ones((1, 4), dtype=np.float32))
    tips.barrier()
    got = table.pull(np.array([3, 0], dtype=np.uint64))
    assert np.allclose(got[0], -0.5 * size), got  # w -= lr * g, once per pushing rank
    assert np.allclose(got[1], 0.0)
    assert all(table.server_of(int(k)) == 0 for k in keys)
    if rank == 0:
        assert table.local_size() >= 3
    else:
        assert table.local_size() == 0
    table.close()


def test_one_server_many_clients():
    run_ranks(_one_server_many_clients, 4)


def _multi_server_rules(rank, size, rule):
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    servers = [0, 1, 2]
    lr, eps = 0.1, 1e-8
    table = HostSparseTable("t2", dim=8, route=Route(servers=servers), optimizer=rule, lr=lr, eps=eps, local_shards=2)
    rng = np.random.default_rng(7)  # same stream on every rank
    keys = rng.integers(0, 2**40, size=64).astype(np.uint64)
    keys[10] = keys[3]  # duplicates inside one request
    keys[11] = keys[3]
    owners = {table.server_of(int(k)) for k in keys}
    assert owners <= set(servers) and len(owners) > 1
    w = {int(k): np.zeros(8, dtype=np.float64) for k in keys}
    acc = {int(k): np.zeros(8, dtype=np.float64) for k in keys}
    assert np.all(table.pull(keys) == 0)
    tips.barrier()
    for step in range(3):
        grads = rng.standard_normal((keys.size, 8)).astype(np.float32)
        if rank == step % size:  # one pusher per step keeps the expected order of updates well defined
            missing = table.push(keys, grads)
            assert missing == 0
        for k, g in zip(keys, grads.astype(np.float64)):
            k = int(k)
            if rule == "sgd":
                w[k] -= lr * g
            else:
                acc[k] += g * g
                w[k] -= lr * g / (np.sqrt(acc[k]) + eps)
        tips.barrier()
        got = table.pull(keys)
        want = np.stack([w[int(k)] for k in keys])
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5), (rule, step, np.abs(got - want).max())
        tips.barrier()
    c = table.counters()
    assert c["rows_pulled"] >= 0 and c["rows_pushed"] >= 0
    table.close()


@pytest.mark.parametrize("rule", ["sgd", "adagrad"])
def test_multi_server_update_rules(rule):
    run_ranks(_multi_server_rules, 3, rule)


def _dump(rank, size, folder, servers, binary, phase):
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    table = HostSparseTable("t3", dim=3, route=Route(servers=servers), optimizer="sgd", lr=1.0)
    keys = np.arange(1, 41, dtype=np.uint64) * 7919
    if phase == "write":
        table.pull(keys)
        tips.barrier()
        if rank == 0:
            table.push(keys, np.tile(-keys.astype(np.float32)[:, None], (1, 3)))  # row of key k becomes k
        tips.barrier()
        table.save(os.path.join(folder, f"dump.{rank}"), binary=binary)
        if not binary and table.local_size():
            line = open(os.path.join(folder, f"dump.{rank}")).readline()
            key, tag, rest = line.rstrip("\n").split("\t")
            assert tag == "Vec:" and len(rest.split()) == 3  # "<key>\tVec:\t<e> <e> <e> "
    else:
        for src in range(size):  # every rank reads every file and keeps the rows it owns now
            path = os.path.join(folder, f"dump.{src}")
            if os.path.exists(path) and os.path.getsize(path):
                table.load(path, binary=binary)
        tips.barrier()
        got = table.pull(keys)
        assert np.allclose(got, np.tile(keys.astype(np.float32)[:, None], (1, 3)))
        total = tips.allreduce_value(float(table.local_size()), name="t3.rows", average=False)
        assert int(total.item()) == keys.size
    table.close()


@pytest.mark.parametrize("binary", [False, True])
def test_dump_and_reload_under_another_sharding(tmp_path, binary):
    run_ranks(_dump, 3, str(tmp_path), [0, 1, 2], binary, "write")
    run_ranks(_dump, 3, str(tmp_path), [1, 2], binary, "read")


def _dense_table(rank, size, servers, rule, tmp):
    """Dense table over `servers`: assign, pull by range, pushes from every rank, rule numerics, dump and reload
    under another sharding."""
    import tips_b200 as tips
    from tips_b200.ps.host import HostDenseTable, Route
    n, lr, eps = 1003, 0.1, 1e-8
    table = HostDenseTable("d_" + rule, n, route=Route(servers=servers), optimizer=rule, lr=lr, eps=eps, local_shards=2)
    init = np.linspace(-1.0, 1.0, n).astype(np.float32)
    if rank == 0:
        table.assign(init)
    tips.barrier()
    assert np.array_equal(table.pull(), init)
    assert np.array_equal(table.pull(100, 777), init[100:777])   # a range that crosses several shards
    cnt, total = table.local_count_and_sum()
    counts = tips.allgather_object(cnt)
    assert sum(counts) == n
    assert all((c > 0) == (r in servers) for r, c in enumerate(counts))
    assert abs(sum(tips.allgather_object(total)) - float(init.astype(np.float64).sum())) < 1e-3
    tips.barrier()
    # every rank pushes its own gradient for a different range, one after the other (order of updates is defined)
    w = init.astype(np.float64).copy()
    acc = np.zeros(n)
    rng = np.random.default_rng(3)
    for step in range(2):
        for r in range(size):
            lo, hi = 50 * r, n - 31 * r
            g = rng.standard_normal(hi - lo).astype(np.float32)
            if rank == r:
                table.push(g, begin=lo)
            tips.barrier()
            g64 = g.astype(np.float64)
            if rule == "sgd":
                w[lo:hi] -= lr * g64
            elif rule == "adagrad":
                acc[lo:hi] += g64 * g64
                w[lo:hi] -= lr * g64 / (np.sqrt(acc[lo:hi]) + eps)
            else:
                w[lo:hi] = lr * g64
    got = table.pull()
    assert np.allclose(got, w, atol=2e-5), np.abs(got - w).max()
    with pytest.raises(ValueError):
        table.pull(5, n + 1)
    # dump: every server writes its shards; reload into a table sharded over ONE server
    path = os.path.join(tmp, f"dense_{rule}.rank{rank}.bin")
    if rank in servers:
        table.save(path)
    tips.barrier()
    single = HostDenseTable("d2_" + rule, n, route=Route(servers=[size - 1]), optimizer=rule, lr=lr)
    for r in servers:
        single.load(os.path.join(tmp, f"dense_{rule}.rank{r}.bin"))
    tips.barrier()
    assert np.allclose(single.pull(), got)
    c = table.counters()
    assert (c["elements_pulled"] > 0) == (rank in servers)
    single.close()
    table.close()


@pytest.mark.parametrize("servers,rule", [([0], "sgd"), ([0, 1], "adagrad"), ([0, 1, 2], "sgd"),
                                          ([1, 2], "literal_reference")])
def test_dense_table(tmp_path, servers, rule):
    run_ranks(_dense_table, 3, servers, rule, str(tmp_path))


def _large_crossing_traffic(rank, size):
    """Both ranks serve and both pull and push tens of MB at the same time: requests and responses far above a socket
    buffer cross in both directions (and each server also answers itself), which must neither stall nor mix rows up.
    Also the packed wire form: a row that exists with another length is refused, an unknown row is counted."""
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    dim, n = 64, 60_000
    table = HostSparseTable("big", dim=dim, route=Route(), optimizer="sgd", lr=1.0, local_shards=2, timeout_s=120.0)
    keys = (np.arange(n, dtype=np.uint64) * np.uint64(2654435761) + np.uint64(rank)) % np.uint64(1 << 40)
    keys = np.unique(keys)
    assert np.all(table.pull(keys) == 0)                      # creates the rows, about half of them on the other rank
    grads = -(keys % np.uint64(1000)).astype(np.float32)[:, None] * np.ones((1, dim), dtype=np.float32)
    for _ in range(2):
        assert table.push(keys, grads) == 0                   # w -= 1.0 * g, twice
    got = table.pull(keys)
    want = 2.0 * (keys % np.uint64(1000)).astype(np.float32)
    assert np.array_equal(got[:, 0], want) and np.array_equal(got[:, dim - 1], want)
    tips.barrier()
    never_pulled = np.array([(1 << 41) + rank, (1 << 41) + 7 + rank], dtype=np.uint64)
    assert table.push(never_pulled, np.ones((2, dim), dtype=np.float32)) == 2
    other = HostSparseTable("big2", dim=8, route=Route(), optimizer="sgd", lr=1.0)
    k = np.array([5 + rank], dtype=np.uint64)
    other.pull(k)
    other.dim = 16                                            # ask for the same row with another length
    with pytest.raises(tips.TipsError, match="different length or dtype"):
        other.pull(k)
    other.dim = 8
    other.close()
    table.close()


def test_large_crossing_traffic():
    run_ranks(_large_crossing_traffic, 2)


def _async_calls(rank, size):
    """Pulls and pushes that return at once: the next batch's rows travel while this batch is used; results equal
    the blocking calls'; a cancelled pull never writes into its buffer later."""
    import tips_b200 as tips
    from tips_b200.ps.host import HostSparseTable, Route
    table = HostSparseTable("async", dim=16, route=Route(), optimizer="sgd", lr=0.5, local_shards=2)
    batches = [np.arange(2000, dtype=np.uint64) * np.uint64(7919) + np.uint64(1000 * b + rank) for b in range(4)]
    for b in batches:
        table.pull(b)                                          # create every row
    tips.barrier()
    nxt = table.pull_async(batches[0])
    pushes = []
    for i, keys in enumerate(batches):
        rows = nxt.wait()
        assert rows.shape == (2000, 16) and np.all(rows == 0)
        if i + 1 < len(batches):
            nxt = table.pull_async(batches[i + 1])             # overlaps with the "compute" below
        pushes.append(table.push_async(keys, np.full((2000, 16), float(i + 1), dtype=np.float32)))
    assert all(p.wait() == 0 for p in pushes)
    assert pushes[0].done() and pushes[0].wait() == 0          # waiting twice is harmless
    for i, keys in enumerate(batches):
        assert np.all(table.pull(keys) == -0.5 * (i + 1))
    missing = table.push_async(np.array([1 << 50], dtype=np.uint64), np.ones((1, 16), dtype=np.float32))
    assert missing.wait() == 1
    call = table.pull_async(batches[1])
    call.cancel()                                              # the answer may still arrive; nobody reads it
    call.cancel()
    assert call.done()
    tips.barrier()
    table.close()


def test_asynchronous_pull_and_push():
    run_ranks(_async_calls, 2)


def _host_embedding_layer(rank, size, sync=False):
    """The host table as a layer: two data-parallel steps of a tiny model against a dense single-process model that
    sees the concatenated batch (SGD on the table, averaged over the ranks; duplicate ids inside a batch)."""
    import torch
    import tips_b200 as tips
    from tips_b200.ps.host import HostEmbedding
    fields, dim, rows, batch, lr = 3, 4, 50, 6, 0.5
    layer = HostEmbedding("emb", fields, dim, optimizer="sgd", lr=lr, sync=sync)
    torch.manual_seed(0)
    head = torch.nn.Linear(fields * dim, 1)
    dense = torch.nn.Embedding(fields * rows, dim)             # the oracle: one dense matrix, row = field * rows + id
    torch.nn.init.zeros_(dense.weight)                         # rows of the server table start at zero too
    ref_head = torch.nn.Linear(fields * dim, 1)
    ref_head.load_state_dict(head.state_dict())
    opt = tips.DistributedOptimizer(torch.optim.SGD(head.parameters(), lr=0.1))
    ref_opt = torch.optim.SGD([{"params": ref_head.parameters(), "lr": 0.1}, {"params": [dense.weight], "lr": lr}])
    for step in range(2):
        g = torch.Generator().manual_seed(10 + step)
        ids_all = torch.randint(0, rows, (size * batch, fields), generator=g)
        ids_all[1] = ids_all[0]                                # duplicates inside one rank's batch
        y_all = torch.rand(size * batch, 1, generator=g)
        ids, y = ids_all[rank * batch:(rank + 1) * batch], y_all[rank * batch:(rank + 1) * batch]
        if step == 1:
            layer.prefetch(ids)
        x = layer(ids)
        if not sync:
            tips.barrier()      # synchronous step for the comparison: every rank has pulled before any rank pushes
        out = head(x + 1.0)
        loss = torch.nn.functional.mse_loss(out, y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        assert layer.wait() == 0
        if not sync:
            tips.barrier()                                     # every rank's push has been applied
        flat = (ids_all + torch.arange(fields) * rows).reshape(-1)
        ref_out = ref_head(dense(flat).reshape(size * batch, fields * dim) + 1.0)
        ref_loss = torch.nn.functional.mse_loss(ref_out, y_all)
        ref_opt.zero_grad()
        ref_loss.backward()
        ref_opt.step()
        probe = ids_all[:4]
        got = layer(probe).detach()
        want = dense((probe + torch.arange(fields) * rows).reshape(-1)).reshape(4, fields * dim).detach()
        assert torch.allclose(got, want, atol=1e-5), (step, (got - want).abs().max())
        assert torch.allclose(head.weight, ref_head.weight, atol=1e-5)
        tips.barrier()
    layer.close()


@pytest.mark.parametrize("sync", [False, True])
def test_host_embedding_layer_matches_dense_model(sync):
    run_ranks(_host_embedding_layer, 2, sync)


def _host_embedding_checkpoint(rank, size, folder, phase):
    import torch
    import tips_b200 as tips
    from tips_b200.ps.host import HostEmbedding
    layer = HostEmbedding("ckpt", 2, 4, optimizer="sgd", lr=1.0, average_over_ranks=False)
    ids = torch.tensor([[1, 2], [3, 2], [1, 7]])
    path = os.path.join(folder, "emb")
    if phase == "write":
        x = layer(ids)
        (x * (rank + 1.0)).sum().backward()                   # d/dx = rank + 1 for every element
        layer.save(path)
    else:
        layer.load(path, nfiles=3)                             # written by 3 ranks, read by 2
    got = layer(ids).detach().reshape(3, 2, 4)
    total = -sum(r + 1.0 for r in range(3))                    # every writer pushed -(r + 1) per occurrence
    assert torch.allclose(got[0, 0], torch.full((4,), 2 * total))      # key (0, 1) occurs twice in the batch
    assert torch.allclose(got[1, 0], torch.full((4,), total))          # key (0, 3) once
    assert torch.allclose(got[0, 1], torch.full((4,), 2 * total))      # key (1, 2) twice
    tips.barrier()
    layer.close()


def test_host_embedding_checkpoint_under_another_rank_count(tmp_path):
    run_ranks(_host_embedding_checkpoint, 3, str(tmp_path), "write")
    run_ranks(_host_embedding_checkpoint, 2, str(tmp_path), "read")
