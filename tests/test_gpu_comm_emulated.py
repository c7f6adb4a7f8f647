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
