"""The multi-rank NVLink collectives, exercised on ONE GPU: every rank's window lives on the
same device and one cooperative launch runs all ranks (gridDim.y = ranks), so the barrier,
reduce-scatter / push and staging logic is the code that runs across GPUs."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3, torch.bfloat16: 6, torch.float16: 7}


@pytest.fixture(scope="module")
def comm4():
    from tips_b200 import _lib
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    set_config(symm_window_bytes=8 << 20, device_wait_budget_ms=2000, comm_blocks=16)
    st = device.setup(emulate_ranks=4)
    yield st, _lib.kernels()
    device.teardown(st)


def _arr(ptrs):
    a = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        a[i] = p
    return a


def _check(lib, rc):
    assert rc == 0, lib.tipsk_last_error().decode()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.float64])
@pytest.mark.parametrize("n", [1, 3, 1000, 4097, 300001])
def test_allreduce_staged_sum(comm4, dtype, n):
    st, lib = comm4
    torch.manual_seed(n)
    dev = st.device
    if dtype.is_floating_point:
        xs = [torch.randn(n, device=dev).to(dtype) for _ in range(4)]
    else:
        xs = [torch.randint(-100, 100, (n,), device=dev, dtype=dtype) for _ in range(4)]
    outs = [torch.empty_like(x) for x in xs]
    es = xs[0].element_size()
    _check(lib, lib.tipsk_allreduce(_arr([x.data_ptr() for x in xs]), _arr([o.data_ptr() for o in outs]), -1, n * es,
                                    DT[dtype], 0, 1.0, 0.25, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st.check_status()
    if dtype.is_floating_point:
        ref = sum(x.double() for x in xs) * 0.25
        tol = 1e-5 if dtype in (torch.float32, torch.float64) else 3e-2
        for o in outs:
            assert torch.allclose(o.double(), ref, atol=tol, rtol=tol)
    else:
        ref = (sum(x.to(torch.int64) for x in xs).double() * 0.25).to(dtype)
        for o in outs:
            assert torch.equal(o, ref)


@pytest.mark.parametrize("op,fn", [(1, torch.maximum), (2, torch.minimum)])
def test_allreduce_minmax(comm4, op, fn):
    st, lib = comm4
    xs = [torch.randn(5000, device=st.device) for _ in range(4)]
    outs = [torch.empty_like(x) for x in xs]
    _check(lib, lib.tipsk_allreduce(_arr([x.data_ptr() for x in xs]), _arr([o.data_ptr() for o in outs]), -1,
                                    5000 * 4, 0, op, 1.0, 1.0, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    ref = xs[0]
    for x in xs[1:]:
        ref = fn(ref, x)
    for o in outs:
        assert torch.equal(o, ref)


def test_allreduce_in_place_window(comm4):
    st, lib = comm4
    n = 1 << 20
    off = st.heap_off
    views = [w[off:off + n * 4].view(torch.float32) for w in st.windows]
    for r, v in enumerate(views):
        v.copy_(torch.full((n,), float(r + 1), device=st.device) + torch.arange(n, device=st.device) % 7)
    ref = sum(v.clone() for v in views) / 4
    _check(lib, lib.tipsk_allreduce(None, None, off, n * 4, 0, 0, 1.0, 0.25, 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st.check_status()
    for v in views:
        assert torch.allclose(v, ref)


def test_allgatherv_and_broadcast(comm4):
    st, lib = comm4
    dev = st.device
    sizes = [5, 0, 1000, 77777]
    xs = [torch.randn(s, device=dev) for s in sizes]
    total = sum(sizes)
    outs = [torch.zeros(total, device=dev) for _ in range(4)]
    nbytes = (ctypes.c_uint64 * 4)(*[s * 4 for s in sizes])
    _check(lib, lib.tipsk_allgatherv(_arr([x.data_ptr() if x.numel() else 0 for x in xs]),
                                     _arr([o.data_ptr() for o in outs]), nbytes, 0,
                                     torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st.check_status()
    ref = torch.cat(xs)
    for o in outs:
        assert torch.equal(o, ref)
    src = torch.randn(123457, device=dev).to(torch.bfloat16)
    outs = [torch.zeros_like(src) for _ in range(4)]
    srcs = [torch.zeros_like(src) for _ in range(4)]
    srcs[2] = src
    _check(lib, lib.tipsk_broadcast(_arr([s.data_ptr() for s in srcs]), _arr([o.data_ptr() for o in outs]),
                                    src.numel() * 2, 2, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st.check_status()
    for o in outs:
        assert torch.equal(o, src)


@pytest.mark.parametrize("push", [True, False])
def test_allgatherv_pushed_and_pulled(comm4, push):
    """The same ragged gather through the pushing kernel (small slabs) and through the pulling one; the byte counts
    are odd on purpose and one output is misaligned."""
    st, lib = comm4
    dev = st.device
    _check(lib, lib.tipsk_comm_set_option(b"allgather_push_bytes", (32 << 20) if push else 0))
    try:
        for sizes in ([3, 0, 70001, 1], [65536 * 3 + 5, 17, 16, 250001], [0, 0, 9, 0]):
            xs = [torch.randint(0, 255, (s,), dtype=torch.uint8, device=dev) for s in sizes]
            total = sum(sizes)
            raw = [torch.full((total + 64,), 0xEE, dtype=torch.uint8, device=dev) for _ in range(4)]
            outs = [r[3 * (i % 2):3 * (i % 2) + total] for i, r in enumerate(raw)]   # ranks 1, 3: odd address
            nbytes = (ctypes.c_uint64 * 4)(*sizes)
            _check(lib, lib.tipsk_allgatherv(_arr([x.data_ptr() if x.numel() else 0 for x in xs]),
                                             _arr([o.data_ptr() for o in outs]), nbytes, 0,
                                             torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            st.check_status()
            ref = torch.cat(xs)
            for i, (o, r) in enumerate(zip(outs, raw)):
                assert torch.equal(o, ref), (sizes, i)
                assert bool((r[3 * (i % 2) + total:] == 0xEE).all()) and bool((r[:3 * (i % 2)] == 0xEE).all())
    finally:
        _check(lib, lib.tipsk_comm_set_option(b"allgather_push_bytes", 2 << 20))


@pytest.mark.parametrize("chunk", [65536, 1 << 20, 8 << 20])
def test_broadcast_scatter_then_allgather(comm4, chunk):
    """Large broadcasts: the root scatters tiles to their owners, the owners forward them, in a pipeline over
    chunks.  Every root, byte counts that end inside a vector, a misaligned input and output, and a message larger
    than the staging area (several launches)."""
    st, lib = comm4
    dev = st.device
    _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_bytes", 1 << 20))
    _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_min_ranks", 2))
    _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_chunk_bytes", chunk))
    try:
        for nbytes, root, shift in [(1 << 20, 0, 0), ((3 << 20) + 7, 1, 0), ((2 << 20) + 4097, 3, 5),
                                    ((19 << 20) + 13, 2, 0)]:
            src = torch.randint(0, 255, (nbytes + 16,), dtype=torch.uint8, device=dev)[shift:shift + nbytes]
            raw = [torch.full((nbytes + 64,), 0xEE, dtype=torch.uint8, device=dev) for _ in range(4)]
            outs = [r[shift:shift + nbytes] for r in raw]
            srcs = [torch.zeros(16, dtype=torch.uint8, device=dev) for _ in range(4)]
            srcs[root] = src
            _check(lib, lib.tipsk_broadcast(_arr([s.data_ptr() for s in srcs]), _arr([o.data_ptr() for o in outs]),
                                            nbytes, root, 0, torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            st.check_status()
            for i, (o, r) in enumerate(zip(outs, raw)):
                assert torch.equal(o, src), (nbytes, root, i)
                assert bool((r[shift + nbytes:] == 0xEE).all()) and bool((r[:shift] == 0xEE).all())
        # in place on the root (input and output are the same buffer)
        buf = [torch.randint(0, 255, (3 << 20,), dtype=torch.uint8, device=dev) for _ in range(4)]
        want = buf[1].clone()
        ptrs = _arr([b.data_ptr() for b in buf])
        _check(lib, lib.tipsk_broadcast(ptrs, ptrs, 3 << 20, 1, 0, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        st.check_status()
        for b in buf:
            assert torch.equal(b, want)
    finally:
        _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_bytes", 128 << 20))
        _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_min_ranks", 8))
        _check(lib, lib.tipsk_comm_set_option(b"bcast_scatter_chunk_bytes", 32 << 20))


def _reference_step(kind, w, state, g, step, hp):
    """fp32 reference of one optimizer step (the rules of torch.optim.SGD / AdamW)."""
    if kind == "sgd":
        lr, mom, damp, wd, nesterov = hp
        g = g + wd * w
        if step == 1:
            state["m"] = g.clone()
        else:
            state["m"] = mom * state["m"] + (1 - damp) * g
        g = g + mom * state["m"] if nesterov else state["m"]
        return w - lr * g
    lr, b1, b2, eps, wd, _ = hp
    state["m"] = b1 * state.get("m", torch.zeros_like(w)) + (1 - b1) * g
    state["v"] = b2 * state.get("v", torch.zeros_like(w)) + (1 - b2) * g * g
    mhat = state["m"] / (1 - b1 ** step)
    denom = (state["v"] / (1 - b2 ** step)).sqrt() + eps
    return w * (1 - lr * wd) - lr * mhat / denom


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["sgd", "adam"])
@pytest.mark.parametrize("numel", [8 * 1000, 2048 * 4 * 8 * 2 + 4096 + 64])
def test_allreduce_fused_with_optimizer_step(comm4, dtype, kind, numel):
    """One launch reduces the gradient bucket, steps the share of the master weights each rank owns and stores the
    new parameters into every rank's window; three steps against an fp32 reference."""
    from tips_b200.parallel.sharding import ShardLayout
    st, lib = comm4
    dev = st.device
    n = 4
    es = torch.empty((), dtype=dtype).element_size()
    nbytes = numel * es
    # canary words before, between and after the two buffers: the kernel must not write outside them
    guards = []
    _, g0 = st.alloc_symmetric(256)
    _, goff = st.alloc_symmetric(nbytes)
    _, g1 = st.alloc_symmetric(256)
    _, poff = st.alloc_symmetric(nbytes)
    _, g2 = st.alloc_symmetric(256)
    for w in st.windows:
        for off in (g0, g1, g2):
            w[off:off + 256].fill_(0xA5)
            guards.append(w[off:off + 256])
    grads = [w[goff:goff + nbytes].view(dtype) for w in st.windows]
    params = [w[poff:poff + nbytes].view(dtype) for w in st.windows]
    torch.manual_seed(numel + es)
    w0 = (torch.randn(numel, device=dev) * 0.5).to(dtype)
    for p in params:
        p.copy_(w0)
    lay = ShardLayout(numel, es, n, int(lib.tipsk_comm_update_subtile()))
    assert lay.shard_numel * es == int(lib.tipsk_comm_update_shard_vecs(nbytes)) * 16
    masters = [lay.take(w0.float(), r) for r in range(n)]
    s0 = [torch.zeros_like(m) for m in masters]
    s1 = [torch.zeros_like(m) for m in masters]
    code = 0 if kind == "sgd" else 1
    _check(lib, lib.tipsk_comm_attach_update(goff, nbytes, DT[dtype], poff, code, _arr([m.data_ptr() for m in masters]),
                                             _arr([m.data_ptr() for m in s0]), _arr([m.data_ptr() for m in s1])))
    assert lib.tipsk_comm_update_attached(goff, nbytes) == 1
    hp = [0.1, 0.9, 0.0, 1e-3, 1.0] if kind == "sgd" else [1e-2, 0.9, 0.999, 1e-8, 0.01, 1.0]
    ref_w = w0.float().clone()
    ref_state = {}
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for step in range(1, 4):
        gs = [(torch.randn(numel, device=dev) * 0.3).to(dtype) for _ in range(n)]
        for g, src in zip(grads, gs):
            g.copy_(src)
        _check(lib, lib.tipsk_comm_set_update_hyper(goff, (ctypes.c_float * len(hp))(*hp), len(hp), step))
        _check(lib, lib.tipsk_allreduce_update(goff, 0.25, 1, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        st.check_status()
        gsum = sum(g.float() for g in gs) * 0.25
        ref_w = _reference_step(kind, ref_w, ref_state, gsum, step, hp)
        got_master = lay.assemble(torch.stack(masters))
        assert torch.allclose(got_master, ref_w, atol=2e-5, rtol=1e-4), (step, (got_master - ref_w).abs().max())
        for p in params:
            assert torch.allclose(p.float(), ref_w, atol=tol, rtol=tol)
            assert torch.equal(p, params[0])
    if kind == "sgd":
        assert torch.allclose(lay.assemble(torch.stack(s0)), ref_state["m"], atol=2e-5, rtol=1e-4)
    else:
        assert torch.allclose(lay.assemble(torch.stack(s1)), ref_state["v"], atol=1e-6, rtol=1e-4)
    assert lib.tipsk_comm_update_launches(goff) == 3
    assert all(bool((g == 0xA5).all()) for g in guards)
    lib.tipsk_comm_detach_update(goff)
    assert lib.tipsk_comm_update_attached(goff, nbytes) == 0


def test_bounded_wait_reports_timeout(comm4):
    """A wait on a flag that nothing sets must give up inside the budget and leave a status."""
    st, lib = comm4
    lib.tipsk_comm_set_budget_ms(200)
    _check(lib, lib.tipsk_comm_wait_never(3, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    from tips_b200.runtime import TipsError
    with pytest.raises(TipsError, match="timed out"):
        st.check_status()
    st.check_status()  # cleared
    lib.tipsk_comm_set_budget_ms(2000)
    x = [torch.ones(100, device=st.device) for _ in range(4)]
    o = [torch.empty_like(t) for t in x]
    _check(lib, lib.tipsk_allreduce(_arr([t.data_ptr() for t in x]), _arr([t.data_ptr() for t in o]), -1, 400, 0, 0,
                                    1.0, 1.0, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st.check_status()
    assert torch.equal(o[0], torch.full((100,), 4.0, device=st.device))


def test_optimizer_step_raises_after_a_device_wait_ran_out(comm4):
    """A kernel that gave up on a peer must stop the training loop: DistributedOptimizer.step() raises TipsError
    (code 5) instead of applying gradients that were never combined, and keeps raising until the collectives are
    reset.  The wait runs out on a flag that nothing sets; no fault is injected on the device."""
    import os
    import tips_b200 as tips
    from tips_b200.ops.optim import FusedSGD
    from tips_b200.runtime import TipsError
    st, lib = comm4
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    tips.init(device=False)
    try:
        model = torch.nn.Linear(64, 64).to(st.device)
        opt = tips.DistributedOptimizer(FusedSGD(model.parameters(), lr=0.1))
        model(torch.ones(4, 64, device=st.device)).sum().backward()
        opt.step()                                        # healthy step
        w0 = model.weight.detach().clone()
        lib.tipsk_comm_set_budget_ms(200)
        _check(lib, lib.tipsk_comm_wait_never(3, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        model(torch.ones(4, 64, device=st.device)).sum().backward()
        with pytest.raises(TipsError) as e:
            opt.step()
        assert e.value.code == 5 and "timed out" in str(e.value)
        assert torch.equal(model.weight.detach(), w0)     # the update was not applied
        with pytest.raises(TipsError):
            tips.parallel.collectives._check_device_status()
        _check(lib, lib.tipsk_comm_reset())
        opt.reset()
        lib.tipsk_comm_set_budget_ms(2000)
        model(torch.ones(4, 64, device=st.device)).sum().backward()
        opt.step()
        assert not torch.equal(model.weight.detach(), w0)
    finally:
        tips.shutdown()


def test_subgroup_collectives(comm4):
    """Two disjoint groups of two ranks and the four ranks together, interleaved: every group has flags, epochs
    and a staging area of its own, so neither disturbs the others; sizes above the group's staging area are
    chunked."""
    from tips_b200.parallel.device import DeviceGroup
    st, lib = comm4
    dev = st.device
    ga = DeviceGroup([1, 3], stage_bytes=1 << 20)
    gb = DeviceGroup([2, 0], stage_bytes=1 << 20)
    assert ga.members == [1, 3] and gb.members == [0, 2] and ga.area_off != gb.area_off
    torch.manual_seed(5)
    for n, dtype in [(7, torch.float32), (70001, torch.float32), (700001, torch.bfloat16), (4096, torch.int64)]:
        def rand():
            if dtype.is_floating_point:
                return torch.randn(n, device=dev).to(dtype)
            return torch.randint(-50, 50, (n,), device=dev, dtype=dtype)
        xa, xb, xw = [rand() for _ in range(2)], [rand() for _ in range(2)], [rand() for _ in range(4)]
        ra, rb = xa[0].double() + xa[1].double(), xb[0].double() + xb[1].double()
        rw = sum(x.double() for x in xw)
        ow = [torch.empty_like(x) for x in xw]
        ga.allreduce_(xa)
        _check(lib, lib.tipsk_allreduce(_arr([x.data_ptr() for x in xw]), _arr([o.data_ptr() for o in ow]), -1,
                                        n * xw[0].element_size(), DT[dtype], 0, 1.0, 1.0, 0,
                                        torch.cuda.current_stream().cuda_stream))
        gb.allreduce_(xb, postscale=0.5)
        torch.cuda.synchronize()
        st.check_status()
        tol = 1e-5 if dtype != torch.bfloat16 else 3e-2
        for got, want in [(xa, ra), (xb, rb * 0.5), (ow, rw)]:
            for t in got:
                assert torch.allclose(t.double(), want.to(dtype).double() if not dtype.is_floating_point else want,
                                      atol=tol, rtol=tol)
    # max over a group
    xs = [torch.randn(3000, device=dev) for _ in range(2)]
    want = torch.maximum(xs[0], xs[1])
    ga.allreduce_(xs, op_code=1)
    torch.cuda.synchronize()
    assert torch.equal(xs[0], want) and torch.equal(xs[1], want)
    # allgatherv with different first dimensions, one of them above the staging area
    parts = [torch.randn(5, 33, device=dev), torch.randn(9000, 33, device=dev)]
    outs = gb.allgatherv(parts, [5, 9000])
    torch.cuda.synchronize()
    st.check_status()
    for o in outs:
        assert torch.equal(o, torch.cat(parts, 0))
    # broadcast from group rank 1 (the job's rank 3)
    bs = [torch.full((300001,), float(i), device=dev) for i in range(2)]
    ga.broadcast_(bs, root=1)
    torch.cuda.synchronize()
    st.check_status()
    assert float(bs[0].min()) == 1.0 and float(bs[0].max()) == 1.0 and float(bs[1].min()) == 1.0
    with pytest.raises(ValueError):
        DeviceGroup([0, 4])
    ga.close()
    gb.close()
