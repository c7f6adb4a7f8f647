"""Exhaustive small-size sweep of the NVLink collectives on ONE GPU: 2, 4 and 8 ranks emulated in one cooperative
launch, every element count from 1 to 4097 for allreduce, allgatherv (ragged parts) and broadcast (every root),
with canary words on both sides of every input and output buffer and around the staging area of every rank's
window, so that a write one element out of place fails the test wherever it lands."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

CANARY = 0x5A


def _arr(ptrs):
    a = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        a[i] = p
    return a


class _Guarded:
    """A device buffer with 256 canary bytes in front of and behind the payload."""

    def __init__(self, nbytes, device):
        self.raw = torch.full((nbytes + 512,), CANARY, dtype=torch.uint8, device=device)
        self.nbytes = nbytes

    def view(self, dtype):
        return self.raw[256:256 + self.nbytes].view(dtype)

    def intact(self):
        return bool((self.raw[:256] == CANARY).all()) and bool((self.raw[256 + self.nbytes:] == CANARY).all())


@pytest.fixture(scope="module", params=[2, 4, 8])
def comm(request):
    from tips_b200 import _lib
    from tips_b200.config import set_config
    from tips_b200.parallel import device
    set_config(symm_window_bytes=1 << 20, device_wait_budget_ms=2000, comm_blocks=4)
    st = device.setup(emulate_ranks=request.param)
    lib = _lib.kernels()
    # canaries in the window heap right behind the staging area (the collectives must stay inside staging)
    for w in st.windows:
        w[st.heap_off:st.heap_off + 4096] = CANARY
    yield st, lib, request.param
    for w in st.windows:
        assert bool((w[st.heap_off:st.heap_off + 4096] == CANARY).all()), "a collective wrote past the staging area"
    device.teardown(st)


def _stream():
    """The stream the test's torch ops run on, as the collective launchers want it (a null handle would mean the
    library's own communication stream, which is not ordered with the fills and comparisons below)."""
    from tips_b200.ops import base
    return base.comm_stream()


def _ok(lib, rc):
    assert rc == 0, lib.tipsk_last_error().decode()


def test_allreduce_every_size_up_to_4097(comm):
    st, lib, n = comm
    dev, stream = st.device, _stream()
    torch.manual_seed(n)
    full = [torch.randint(-8, 9, (4097,), device=dev).float() for _ in range(n)]   # exact in fp32
    want = sum(full)
    ins = [_Guarded(4097 * 4, dev) for _ in range(n)]
    outs = [_Guarded(4097 * 4, dev) for _ in range(n)]
    for g, x in zip(ins, full):
        g.view(torch.float32).copy_(x)
    bad = []
    for count in range(1, 4098):
        for o in outs:
            o.view(torch.float32).fill_(-777.0)
        _ok(lib, lib.tipsk_allreduce(_arr([g.view(torch.float32).data_ptr() for g in ins]),
                                     _arr([o.view(torch.float32).data_ptr() for o in outs]), -1, count * 4, 0, 0, 1.0,
                                     1.0, 0, stream))
        got = torch.stack([o.view(torch.float32) for o in outs])
        ok = bool((got[:, :count] == want[:count]).all()) and bool((got[:, count:] == -777.0).all())
        if not ok:
            bad.append(count)
    torch.cuda.synchronize()
    st.check_status()
    assert not bad, f"wrong sums or writes past the end for counts {bad[:20]}"
    assert all(g.intact() for g in ins + outs)


def test_allgatherv_every_size_up_to_4097(comm):
    st, lib, n = comm
    dev, stream = st.device, _stream()
    src = [torch.arange(4097, device=dev, dtype=torch.int32) + 10000 * (r + 1) for r in range(n)]
    ins = [_Guarded(4097 * 4, dev) for _ in range(n)]
    for g, x in zip(ins, src):
        g.view(torch.int32).copy_(x)
    outs = [_Guarded(4097 * 4 * n, dev) for _ in range(n)]
    bad = []
    for count in range(1, 4098):
        sizes = [max(0, count - 3 * r) for r in range(n)]          # ragged: every rank contributes another length
        total = sum(sizes)
        for o in outs:
            o.view(torch.int32).fill_(-1)
        nbytes = (ctypes.c_uint64 * n)(*[s * 4 for s in sizes])
        _ok(lib, lib.tipsk_allgatherv(_arr([g.view(torch.int32).data_ptr() for g in ins]),
                                      _arr([o.view(torch.int32).data_ptr() for o in outs]), nbytes, 0, stream))
        ref = torch.cat([src[r][:sizes[r]] for r in range(n)])
        got = torch.stack([o.view(torch.int32) for o in outs])
        if not (bool((got[:, :total] == ref).all()) and bool((got[:, total:] == -1).all())):
            bad.append(count)
    torch.cuda.synchronize()
    st.check_status()
    assert not bad, f"allgatherv wrong for counts {bad[:20]}"
    assert all(g.intact() for g in ins + outs)


def test_broadcast_every_size_up_to_4097(comm):
    st, lib, n = comm
    dev, stream = st.device, _stream()
    bufs = [_Guarded(4097 * 2, dev) for _ in range(n)]
    outs = [_Guarded(4097 * 2, dev) for _ in range(n)]
    bad = []
    for count in range(1, 4098):
        root = count % n
        for r, b in enumerate(bufs):
            b.view(torch.int16).copy_((torch.arange(4097, device=dev) % 1000 + 1000 * r).to(torch.int16))
        for o in outs:
            o.view(torch.int16).fill_(-3)
        _ok(lib, lib.tipsk_broadcast(_arr([b.view(torch.int16).data_ptr() for b in bufs]),
                                     _arr([o.view(torch.int16).data_ptr() for o in outs]), count * 2, root, 0, stream))
        ref = bufs[root].view(torch.int16)[:count]
        got = torch.stack([o.view(torch.int16) for o in outs])
        if not (bool((got[:, :count] == ref).all()) and bool((got[:, count:] == -3).all())):
            bad.append(count)
    torch.cuda.synchronize()
    st.check_status()
    assert not bad, f"broadcast wrong for counts {bad[:20]}"
    assert all(g.intact() for g in bufs + outs)
