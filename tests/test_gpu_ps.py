"""Parameter-server kernels (pull / push with server-side SGD and Adagrad) against a dense PyTorch model of
the same tables; single rank and 4 emulated ranks on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dense_tables(table, fields, rows, dim):
    """Reassemble the global [rows, dim] tables (and Adagrad state) from the shards."""
    out = [table.dense_table(f) for f in range(fields)]
    state = [table.dense_table(f, state=True) if table.has_state else torch.zeros_like(out[f]) for f in range(fields)]
    return out, state


def _reference_update(ws, ss, ids_all, grads_all, rule, lr, eps, dim):
    for f in range(len(ws)):
        g = torch.zeros_like(ws[f])
        for ids, grads in zip(ids_all, grads_all):
            g.index_add_(0, ids[:, f], grads[:, f * dim:(f + 1) * dim].float())
        touched = g.abs().sum(1) != 0
        if rule == "adagrad":
            ss[f] += g * g
            ws[f] -= torch.where(touched[:, None], lr * g / (ss[f].sqrt() + eps), torch.zeros_like(g))
        else:
            ws[f] -= lr * g


@pytest.mark.parametrize("rule", ["sgd", "adagrad"])
@pytest.mark.parametrize("dim", [16, 64])
def test_pull_push_single_rank(rule, dim):
    from tips_b200.ps.gpu import ShardedEmbedding
    dev = torch.device("cuda", 0)
    fields, rows, batch = 3, 5000, 2048
    t = ShardedEmbedding(fields, rows, dim, optimizer=rule, lr=0.1, init_scale=0.1, seed=3, expected_batch=batch,
                         device=dev)
    ws, ss = _dense_tables(t, fields, rows, dim)
    torch.manual_seed(0)
    ids = (torch.rand(batch, fields, device=dev) ** 4 * rows).long().clamp_(0, rows - 1)  # skewed: many duplicates
    out = t.pull(ids, dtype=torch.float32)
    ref = torch.cat([ws[f][ids[:, f]] for f in range(fields)], dim=1)
    assert torch.equal(out, ref)
    out16 = t.pull(ids, dtype=torch.bfloat16)
    assert torch.equal(out16, ref.to(torch.bfloat16))
    assert torch.equal(t.pull(ids, dtype=torch.float32, index=True), ref)      # distinct rows fetched once
    assert torch.equal(t.pull(ids, dtype=torch.bfloat16, index=True), ref.to(torch.bfloat16))
    for step in range(2):
        grads = torch.randn(batch, fields * dim, device=dev)
        if step == 1:
            t.pull(ids, dtype=torch.float32, index=True)
        t.push(ids, grads, grad_scale=0.5, reuse_index=step == 1)
        _reference_update(ws, ss, [ids], [grads * 0.5], rule, 0.1, t.eps, dim)
    assert t.check() > 0
    got, got_s = _dense_tables(t, fields, rows, dim)
    for f in range(fields):
        assert torch.allclose(got[f], ws[f], atol=2e-4, rtol=1e-4)
        if rule == "adagrad":
            assert torch.allclose(got_s[f], ss[f], atol=1e-3, rtol=1e-4)


def test_pull_push_emulated_ranks():
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import ShardedEmbedding
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8)
    st = device.setup(emulate_ranks=4)
    try:
        dev = st.device
        fields, rows, dim, batch = 2, 3001, 32, 1024
        t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.1, seed=9,
                             expected_batch=batch * 4, device=dev)
        assert t.size == 4 and t.emulated
        ws, ss = _dense_tables(t, fields, rows, dim)
        # the initial contents do not depend on the sharding
        t1_vals = ws[0][:5].clone()
        torch.manual_seed(1)
        ids = [(torch.rand(batch, fields, device=dev) ** 3 * rows).long().clamp_(0, rows - 1) for _ in range(4)]
        outs = t.pull(ids, dtype=torch.float32)
        for r in range(4):
            ref = torch.cat([ws[f][ids[r][:, f]] for f in range(fields)], dim=1)
            assert torch.equal(outs[r], ref)
        grads = [torch.randn(batch, fields * dim, device=dev) for _ in range(4)]
        t.push(ids, grads, grad_scale=0.25)
        _reference_update(ws, ss, ids, [g * 0.25 for g in grads], "adagrad", 0.05, t.eps, dim)
        t.check()
        st.check_status()
        got, got_s = _dense_tables(t, fields, rows, dim)
        for f in range(fields):
            assert torch.allclose(got[f], ws[f], atol=2e-4, rtol=1e-4)
            assert torch.allclose(got_s[f], ss[f], atol=1e-3, rtol=1e-4)
        assert t1_vals.abs().sum() > 0
    finally:
        device.teardown(st)


@pytest.mark.parametrize("wire", ["fp32", "grad"])
@pytest.mark.parametrize("indexed", [False, True])
@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_push_with_mostly_duplicate_ids_emulated(ranks, indexed, wire):
    """Three synchronous steps on 2, 4 and 8 emulated ranks with ids drawn from 40 hot rows for 70 % of the batch
    (so most of every batch is duplicates, within a rank and across ranks): the tables equal the dense model, the
    number of rows sent to owners is the number of distinct ids per rank, not the batch size."""
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import ShardedEmbedding
    # wire "grad": the bf16 gradients of this test make every rank's per-row sum cross as bf16 (one rounding)
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8, ps_wire_dtype=wire)

    def close(a, b, atol=3e-4, rtol=1e-4):
        if wire == "fp32":
            return torch.allclose(a, b, atol=atol, rtol=rtol)
        # bf16 on the wire: a row's gradient is exact to 2^-9 of each rank's partial sum, and where the partial sums
        # of the ranks nearly cancel Adagrad turns that into a visible step (lr * g / |g| on a first update), so
        # the comparison is statistical: nearly all elements agree closely and the mean error is small
        d = (a - b).abs()
        return float((d > 4e-3).float().mean()) < 0.02 and float(d.mean()) < 5e-4

    st = device.setup(emulate_ranks=ranks)
    try:
        dev = st.device
        fields, rows, dim, batch = 3, 2503, 64, 768
        t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.1, seed=21,
                             expected_batch=batch, device=dev)
        ws, ss = _dense_tables(t, fields, rows, dim)
        torch.manual_seed(7)
        total_distinct = 0
        for step in range(3):
            ids, distinct = [], 0
            for r in range(ranks):
                hot = torch.randint(0, 40, (batch, fields), device=dev)
                cold = torch.randint(0, rows, (batch, fields), device=dev)
                ids.append(torch.where(torch.rand(batch, fields, device=dev) < 0.7, hot, cold))
                distinct += sum(int(ids[-1][:, f].unique().numel()) for f in range(fields))
            total_distinct += distinct
            outs = t.pull(ids, dtype=torch.float32, index=indexed)
            for r in range(ranks):
                ref = torch.cat([ws[f][ids[r][:, f]] for f in range(fields)], dim=1)
                assert close(outs[r], ref)
            pulls = 1
            if indexed and step == 1:
                t.pull(ids, dtype=torch.bfloat16, index=True)   # an index that nothing consumes is dropped
                outs = t.pull(ids, dtype=torch.float32, index=True)
                pulls = 3
            grads = [torch.randn(batch, fields * dim, device=dev).to(torch.bfloat16) for _ in range(ranks)]
            t.push(ids, grads, grad_scale=1.0 / ranks, reuse_index=indexed)
            _reference_update(ws, ss, ids, [g.float() / ranks for g in grads], "adagrad", 0.05, t.eps, dim)
            sent, remote, fetched = t.traffic()
            assert sent == distinct, (sent, distinct)
            assert 0 < remote < sent
            assert fetched == (pulls * remote if indexed else 0)
        t.check()
        st.check_status()
        assert total_distinct < 0.6 * 3 * ranks * batch * fields
        got, got_s = _dense_tables(t, fields, rows, dim)
        # bf16 pulls read the owners' bf16 copy of the rows, which the apply pass keeps current
        assert t.shadow_base > 0
        outs16 = t.pull(ids, dtype=torch.bfloat16, index=True)
        for r in range(ranks):
            want16 = torch.cat([got[f][ids[r][:, f]] for f in range(fields)], dim=1).to(torch.bfloat16)
            assert torch.equal(outs16[r], want16)
        t.pull(ids, dtype=torch.float32)   # a plain pull drops the unused index
        for f in range(fields):
            assert close(got[f], ws[f])
            assert close(got_s[f], ss[f], atol=1e-3) if wire == "fp32" else torch.allclose(got_s[f], ss[f], atol=0.5, rtol=5e-2)
    finally:
        set_config(ps_wire_dtype="grad")
        device.teardown(st)


def test_hot_rows_are_spread_over_the_ranks():
    """The smallest ids of every field (the most frequent under a Zipf distribution) must not share an owner."""
    from tips_b200.ops import base
    import ctypes
    lib = base.K()
    for n in (2, 4, 8):
        counts = [0] * n
        for f in range(26):
            for i in range(4):
                o, l = ctypes.c_int32(), ctypes.c_int64()
                assert lib.tipsk_ps_place(f, i, n, ctypes.byref(o), ctypes.byref(l)) == 0
                counts[o.value] += 1
        assert max(counts) - min(counts) <= 2, counts


def test_ctr_trainer_loss_decreases():
    from tips_b200.models.ctr import CtrTrainer, synthetic_ctr_batch
    dev = torch.device("cuda", 0)
    t = CtrTrainer(num_fields=4, rows_per_table=2000, dim=16, dense_features=5, hidden=(64, 32), device=dev,
                   expected_batch=512, table_lr=0.1, mlp_lr=5e-3)
    ids, dense, labels = [x.to(dev) for x in synthetic_ctr_batch(512, 4, 2000, 5, seed=5)]
    losses = [t.train_step(ids, dense, labels).item() for _ in range(30)]
    t.check()
    assert losses[-1] < losses[0] * 0.8, losses


def test_table_dump_reloads_under_another_sharding(tmp_path):
    """Dump 4 emulated ranks' shards, reload them into a single-rank table: same dense contents and optimizer
    state; the text dump has the reference's "<key>\\tVec:\\t<e> <e> ... " lines."""
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import ShardedEmbedding
    fields, rows, dim, batch = 2, 1501, 16, 256
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8)
    st = device.setup(emulate_ranks=4)
    try:
        dev = st.device
        t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.1, seed=3,
                             expected_batch=batch * 4, device=dev)
        torch.manual_seed(2)
        ids = [(torch.rand(batch, fields, device=dev) * rows).long().clamp_(0, rows - 1) for _ in range(4)]
        t.push(ids, [torch.randn(batch, fields * dim, device=dev) for _ in range(4)])
        t.check()
        want_w, want_s = _dense_tables(t, fields, rows, dim)
        paths = t.save(str(tmp_path / "ctr"))
        assert len(paths) == 4
        t.save_text(str(tmp_path / "field0.txt"), 0)
    finally:
        device.teardown(st)
    lines = open(tmp_path / "field0.txt").read().splitlines()
    assert len(lines) == rows
    key, tag, rest = lines[5].split("\t")
    assert tag == "Vec:" and len(rest.split()) == dim
    row = torch.tensor([float(v) for v in rest.split()])
    assert torch.allclose(row, want_w[0][int(key)].cpu(), rtol=1e-4, atol=1e-6)
    single = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.0, seed=0,
                              expected_batch=batch, device=torch.device("cuda", 0))
    assert single.size == 1
    single.load(str(tmp_path / "ctr"))
    got_w, got_s = _dense_tables(single, fields, rows, dim)
    for f in range(fields):
        assert torch.equal(got_w[f], want_w[f])
        assert torch.equal(got_s[f], want_s[f])


@pytest.mark.parametrize("rule", ["sgd", "adagrad"])
def test_async_push_emulated_ranks(rule):
    """Fence-free pushes: with SGD the result equals the synchronous one (sums commute); with Adagrad and distinct
    ids per step it equals the reference update as well."""
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import ShardedEmbedding
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8)
    st = device.setup(emulate_ranks=4)
    try:
        dev = st.device
        fields, rows, dim, batch = 2, 4001, 32, 512
        t = ShardedEmbedding(fields, rows, dim, optimizer=rule, lr=0.05, init_scale=0.1, seed=5,
                             expected_batch=batch * 4, device=dev, sync=False)
        ws, ss = _dense_tables(t, fields, rows, dim)
        torch.manual_seed(3)
        if rule == "sgd":
            ids = [(torch.rand(batch, fields, device=dev) ** 3 * rows).long().clamp_(0, rows - 1) for _ in range(4)]
        else:  # distinct rows over all ranks and samples, so the order of application does not matter
            perm = [torch.randperm(rows, device=dev)[:4 * batch].view(4, batch) for _ in range(fields)]
            ids = [torch.stack([perm[f][r] for f in range(fields)], dim=1) for r in range(4)]
        grads = [torch.randn(batch, fields * dim, device=dev) for _ in range(4)]
        t.push(ids, grads, grad_scale=0.5)
        torch.cuda.synchronize()
        _reference_update(ws, ss, ids, [g * 0.5 for g in grads], rule, 0.05, t.eps, dim)
        t.check()
        got, got_s = _dense_tables(t, fields, rows, dim)
        for f in range(fields):
            assert torch.allclose(got[f], ws[f], atol=3e-4, rtol=1e-4)
            if rule == "adagrad":
                assert torch.allclose(got_s[f], ss[f], atol=1e-3, rtol=1e-4)
        outs = t.pull(ids, dtype=torch.float32)
        for r in range(4):
            assert torch.allclose(outs[r], torch.cat([got[f][ids[r][:, f]] for f in range(fields)], dim=1))
    finally:
        device.teardown(st)


@pytest.mark.parametrize("rule,dtype", [("sgd", torch.float32), ("sgd", torch.bfloat16), ("adam", torch.bfloat16)])
def test_dense_table_single_rank(rule, dtype):
    """ShardedDense on one rank against torch's optimizer on an fp32 copy: assign, three pushes, pull, state
    round trip."""
    from tips_b200.ps.gpu import ShardedDense
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    n = 10_000
    kw = dict(lr=0.05, momentum=0.9) if rule == "sgd" else dict(lr=0.01, weight_decay=0.0)
    t = ShardedDense(n, dtype=dtype, optimizer=rule, device=dev, **kw)
    init = torch.randn(n, device=dev)
    t.assign(init)
    ref = init.clone().to(dtype).float().requires_grad_()
    ropt = torch.optim.SGD([ref], **kw) if rule == "sgd" else torch.optim.Adam([ref], **kw)
    for step in range(3):
        g = torch.randn(n, device=dev).to(dtype)
        t.push(g)
        ref.grad = g.float()
        ropt.step()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(t.pull().float(), ref.detach(), atol=tol, rtol=tol)
    assert t.pull(10, 20).shape == (10,)
    saved = t.state()
    t2 = ShardedDense(n, dtype=dtype, optimizer=rule, device=dev, **kw)
    t2.load_state(saved)
    g = torch.randn(n, device=dev).to(dtype)
    t.push(g)
    t2.push(g)
    assert torch.equal(t.pull(), t2.pull())


@pytest.mark.parametrize("ranks,rule", [(1, "sgd"), (4, "sgd"), (4, "adagrad")])
def test_hashed_table_creates_rows_on_first_pull(ranks, rule):
    """Arbitrary 64-bit keys (negative, huge, duplicates): unknown keys pull zeros and exist afterwards, a push to
    a key that was never pulled is counted as missing, updates match a dictionary model; 1 rank and 4 emulated."""
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import HashedEmbedding
    st = None
    if ranks > 1:
        set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8)
        st = device.setup(emulate_ranks=ranks)
    try:
        dev = st.device if st else torch.device("cuda", 0)
        dim, lr = 16, 0.1
        t = HashedEmbedding(dim, capacity_per_rank=4096, optimizer=rule, lr=lr, device=dev)
        g = torch.Generator().manual_seed(3)
        pool = torch.randint(-2**62, 2**62, (600,), generator=g)
        pool[:3] = torch.tensor([0, -5, 2**62 + 12345])
        wrap = (lambda x: [x.to(dev)] * 1 if False else x.to(dev))
        per_rank = [pool[torch.randint(0, 600, (512,), generator=g)] for _ in range(max(ranks, 1))]
        arg = [k.to(dev) for k in per_rank] if ranks > 1 else per_rank[0].to(dev)
        first = t.pull(arg)
        for o in (first if ranks > 1 else [first]):
            assert float(o.abs().sum()) == 0.0                      # created as zeros
        seen = set(int(v) for k in per_rank for v in k)
        total = sum(t.local_size(r) for r in range(ranks)) if ranks > 1 else t.local_size()
        assert total == len(seen)
        model, acc = {}, {}
        for step in range(2):
            grads = [torch.randn(512, dim, generator=g) for _ in per_rank]
            garg = [x.to(dev) for x in grads] if ranks > 1 else grads[0].to(dev)
            t.push(arg, garg)
            torch.cuda.synchronize()
            if rule == "sgd":
                for k, gr in zip(per_rank, grads):
                    for i in range(512):
                        model[int(k[i])] = model.get(int(k[i]), torch.zeros(dim)) - lr * gr[i]
        assert t.check() == 0
        if rule == "sgd":
            got = t.pull(arg)
            for k, o in zip(per_rank, got if ranks > 1 else [got]):
                want = torch.stack([model[int(v)] for v in k])
                assert torch.allclose(o.cpu(), want, atol=1e-4, rtol=1e-4)
        else:
            got = t.pull(arg)
            assert all(float(o.abs().sum()) > 0 for o in (got if ranks > 1 else [got]))
        never = torch.tensor([7_000_000_001], dtype=torch.int64)
        nk = [never.to(dev)] * ranks if ranks > 1 else never.to(dev)
        ng = [torch.ones(1, dim, device=dev)] * ranks if ranks > 1 else torch.ones(1, dim, device=dev)
        t.push(nk, ng)
        torch.cuda.synchronize()
        assert t.check() == max(ranks, 1)
    finally:
        if st is not None:
            device.teardown(st)


def test_server_subgroup_emulated(tmp_path):
    """Four ranks, of which ranks 1 and 3 hold the tables (servers) and all four pull and push (workers): rows live
    on the two servers only, the update equals the dense model, and the dump reloads into a one-rank table."""
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    from tips_b200.ps.gpu import ShardedEmbedding
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=8, ps_wire_dtype="fp32")
    st = device.setup(emulate_ranks=4)
    try:
        dev = st.device
        fields, rows, dim, batch = 2, 1777, 32, 512
        t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.1, seed=2,
                             expected_batch=batch, device=dev, servers=[3, 1])
        assert t.servers == [1, 3] and t.rows_per_shard == (rows + 1) // 2
        ws, ss = _dense_tables(t, fields, rows, dim)
        torch.manual_seed(11)
        for step in range(2):
            ids = [(torch.rand(batch, fields, device=dev) ** 2 * rows).long().clamp_(0, rows - 1) for _ in range(4)]
            outs = t.pull(ids, dtype=torch.float32, index=step == 1)
            for r in range(4):
                ref = torch.cat([ws[f][ids[r][:, f]] for f in range(fields)], dim=1)
                assert torch.allclose(outs[r], ref, atol=3e-4, rtol=1e-4)
            grads = [torch.randn(batch, fields * dim, device=dev) for _ in range(4)]
            t.push(ids, grads, grad_scale=0.25, reuse_index=step == 1)
            _reference_update(ws, ss, ids, [g * 0.25 for g in grads], "adagrad", 0.05, t.eps, dim)
        t.check()
        st.check_status()
        sent, remote, _ = t.traffic()
        assert 0 < remote < sent              # the servers' own rows never left them, the workers' all did
        got, got_s = _dense_tables(t, fields, rows, dim)
        for f in range(fields):
            assert torch.allclose(got[f], ws[f], atol=3e-4, rtol=1e-4)
            assert torch.allclose(got_s[f], ss[f], atol=1e-3, rtol=1e-4)
        assert len(t.save(str(tmp_path / "sub"))) == 2
    finally:
        set_config(ps_wire_dtype="grad")
        device.teardown(st)
    single = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, device=torch.device("cuda", 0),
                              expected_batch=batch)
    single.load(str(tmp_path / "sub"))
    again, _ = _dense_tables(single, fields, rows, dim)
    for f in range(fields):
        assert torch.equal(again[f], got[f])
