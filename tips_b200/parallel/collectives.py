"""Tensor collectives: allreduce / allgather / broadcast, sync and async.

API parity with the reference's op wrappers and ``allreduce`` front end
(tips/tensorflow/ops.py:33-88, tips/tensorflow/__init__.py:20-103), following the
documented semantics rather than the reference's shortcuts: ``op`` defaults to
``Average`` and is honoured together with ``prescale_factor`` /
``postscale_factor`` (the reference accepts and ignores them, __init__.py:78-91),
``broadcast`` takes any ``root_rank`` (the reference CHECKs root == 0,
tips/tensorflow/ops.cc:219), and every collective skips the engine when the
world has one rank (``_allreduce_cond``, __init__.py:94-103).

Each call enqueues an op record with the native collective engine, which
negotiates one global order through rank 0 and executes on its background
thread; the handle completes when the op has run (host tensors) or has been
launched on the communication stream (device tensors, ordered by CUDA events).
"""
from __future__ import annotations

import ctypes
import itertools
import threading
from typing import Optional

import torch

from .. import _lib
from ..runtime import TipsError, _require_init, size as _size, rank as _rank
from .compression import Compression

Average = "Average"
Sum = "Sum"
Min = "Min"
Max = "Max"
Product = "Product"
_REDUCE_CODE = {Sum: 0, Average: 0, Max: 1, Min: 2, Product: 3}

_DTYPE_CODE = {
    torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3,
    torch.int8: 4, torch.uint8: 5, torch.bfloat16: 6, torch.float16: 7, torch.bool: 5,
}

_name_counter = itertools.count()
_handles = {}
_handles_lock = threading.Lock()


class _Handle:
    __slots__ = ("id", "keep", "output", "post", "done_event", "ready_event", "alloc_cb", "gathered", "kind", "name",
                 "first_dims")

    def __init__(self):
        self.id = 0
        self.keep = []
        self.output = None
        self.post = None
        self.done_event = None
        self.ready_event = None
        self.alloc_cb = None
        self.gathered = None
        self.kind = ""
        self.name = ""
        self.first_dims = None   # allgather: dimension 0 of every rank, known once the collective was negotiated


def _auto_name(kind: str, name: Optional[str]) -> str:
    # The reference derives "Tips<Op>_<tensor name>" in graph mode (ops.py:61-65);
    # eager tensors have no name, so unnamed calls are numbered, which matches
    # across ranks as long as they make the same calls in the same order.
    return name if name else f"{kind}.noname.{next(_name_counter)}"


def _resolve_op(average, op):
    if op is not None and average is not None:
        raise ValueError("pass either `op` or the deprecated `average`, not both")
    if op is None:
        op = Average if (average is None or average) else Sum
    if op not in _REDUCE_CODE:
        raise ValueError(f"unknown reduce op {op!r}")
    return op


def _enqueue(h: _Handle, kind: int, name: str, tensor_in, tensor_out, shape, dtype, root=0, reduce_op=0,
             prescale=1.0, postscale=1.0, alloc=None):
    lib = _lib.core()
    op = _lib.TipsOp()
    op.name = name.encode()
    op.type = kind
    if dtype not in _DTYPE_CODE:
        raise TipsError(f"dtype {dtype} is not supported by tips collectives", 2)
    op.dtype = _DTYPE_CODE[dtype]
    op.ndim = len(shape)
    arr = (ctypes.c_int64 * max(len(shape), 1))(*shape)
    op.shape = arr
    op.in_ = tensor_in.data_ptr() if tensor_in is not None else None
    op.out = tensor_out.data_ptr() if tensor_out is not None else None
    is_cuda = tensor_in.is_cuda
    op.device = 1 if is_cuda else 0
    op.root_rank = root
    op.reduce_op = reduce_op
    op.prescale = prescale
    op.postscale = postscale
    if is_cuda:
        from . import device as _device
        st = _device.state()
        ready, done = st.events_for_op()
        _device.record_event(ready, torch.cuda.current_stream().cuda_stream)
        op.stream = torch.cuda.current_stream().cuda_stream
        op.ready_event = ready
        op.done_event = done
        h.done_event = done
        h.ready_event = ready
    if alloc is not None:
        op.alloc = alloc
    hid = lib.tips_enqueue(ctypes.byref(op))
    if hid < 0:
        _recycle_events(h)
        raise TipsError(f"{name}: {_lib.last_error()}", int(-hid))
    h.id = hid
    h.name = name
    with _handles_lock:
        _handles[hid] = h
    return h


def poll(handle: _Handle) -> bool:
    """True once the collective behind `handle` has completed (or failed)."""
    return _lib.core().tips_poll(handle.id) != 1


def _recycle_events(handle: _Handle) -> None:
    """Return the CUDA events of a finished (or failed) device collective to the pool.  Safe once the engine has
    answered the handle: its executor has issued the stream wait on `ready` and recorded `done` by then."""
    if handle.done_event is None and handle.ready_event is None:
        return
    from . import device as _device
    st = _device._state
    for ev in (handle.ready_event, handle.done_event):
        if ev is not None and st is not None:
            st.recycle_event(ev)
    handle.ready_event = handle.done_event = None


def _check_device_status(wait: bool = False) -> None:
    """Raise TipsError(code 5) if a kernel of the GPU data plane gave up on a bounded wait (a lost or late peer).

    The status block lives in mapped host memory, so reading it costs nothing and does not wait for the device;
    `wait` (or ``device_status_check="sync"``) first waits for the current stream, which makes the failing step
    itself raise instead of a later one.  The status stays set until ``tips_b200.reset_collectives()``."""
    from ..config import get_config
    mode = get_config().device_status_check
    if mode == "off":
        return
    from . import device as _device
    st = _device._state
    if st is None or st.window is None:
        return
    if wait or mode == "sync":
        torch.cuda.current_stream().synchronize()
    st.check_status(clear=False)


def synchronize(handle: _Handle, timeout_s: float | None = None):
    """Wait for an asynchronous collective and return its output tensor."""
    lib = _lib.core()
    if handle.id:
        rc = lib.tips_wait(handle.id, -1 if timeout_s is None else int(timeout_s * 1000))
        if rc == 5 and lib.tips_poll(handle.id) == 1:
            raise TipsError(f"{handle.name}: timed out after {timeout_s} s (still in flight)", 5)
        if rc != 0:
            buf = ctypes.create_string_buffer(1024)
            lib.tips_handle_error(handle.id, buf, 1024)
            lib.tips_release(handle.id)
            with _handles_lock:
                _handles.pop(handle.id, None)
            handle.id = 0
            _recycle_events(handle)
            raise TipsError(f"{handle.name}: {buf.value.decode()}", rc)
        if handle.kind == "allgather" and handle.gathered is not None:
            handle.output = handle.gathered[0]
        lib.tips_release(handle.id)
        with _handles_lock:
            _handles.pop(handle.id, None)
        if handle.done_event is not None:
            from . import device as _device
            _device.stream_wait_event(torch.cuda.current_stream().cuda_stream, handle.done_event)
            _recycle_events(handle)
            _check_device_status()
        handle.id = 0
    out = handle.output
    if handle.post is not None:
        out = handle.post(out)
        handle.post = None
        handle.output = out
    handle.keep = []
    return out


def abandon(handle: _Handle) -> None:
    """Forget a collective that will never be waited for (after a failed step): releases the engine handle if the
    engine has answered it, and returns its events."""
    lib = _lib.core()
    if handle.id:
        if lib.tips_poll(handle.id) != 1:
            lib.tips_release(handle.id)
            _recycle_events(handle)
        with _handles_lock:
            _handles.pop(handle.id, None)
        handle.id = 0
    handle.keep = []


# ------------------------------------------------------------------ allreduce


def allreduce_async(tensor: torch.Tensor, average=None, name=None, compression=Compression.none, op=None,
                    prescale_factor=1.0, postscale_factor=1.0, _inplace=False) -> _Handle:
    _require_init()
    op = _resolve_op(average, op)
    h = _Handle()
    h.kind = "allreduce"
    n = _size()
    post = postscale_factor / n if op == Average else postscale_factor
    if tensor.is_sparse:
        raise TypeError("use sparse_allreduce for sparse tensors")
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    wire, ctx = compression.compress(src)
    if n == 1:
        out = wire if (_inplace and wire is tensor) else wire.clone()
        scale = prescale_factor * post
        if scale != 1.0:
            out = out.mul_(scale) if out.is_floating_point() else (out * scale).to(out.dtype)
        result = compression.decompress(out, ctx)
        if _inplace and result is not tensor:
            tensor.copy_(result)
            result = tensor
        h.output = result
        return h
    if wire.is_cuda:
        from . import device as _device
        if _device.state().backend == "nccl":
            return _device.nccl_allreduce(h, tensor, wire, ctx, compression, _REDUCE_CODE[op], prescale_factor, post,
                                          _inplace)
    out = wire if (_inplace and wire is tensor) or (wire is not src) else torch.empty_like(wire)
    h.keep = [src, wire, out]
    h.output = out

    def finish(o, ctx=ctx, tensor=tensor):
        r = compression.decompress(o, ctx)
        if _inplace and r is not tensor:
            tensor.copy_(r)
            return tensor
        return r

    h.post = finish
    return _enqueue(h, 0, _auto_name("allreduce", name), wire, out, tuple(wire.shape), wire.dtype,
                    reduce_op=_REDUCE_CODE[op], prescale=prescale_factor, postscale=post)


def allreduce(tensor, average=None, name=None, compression=Compression.none, op=None, prescale_factor=1.0,
              postscale_factor=1.0):
    """Reduce `tensor` over all ranks; returns a new tensor (Average by default)."""
    return synchronize(allreduce_async(tensor, average, name, compression, op, prescale_factor, postscale_factor))


def allreduce_async_(tensor, average=None, name=None, op=None, prescale_factor=1.0, postscale_factor=1.0,
                     compression=Compression.none):
    return allreduce_async(tensor, average, name, compression, op, prescale_factor, postscale_factor, _inplace=True)


def allreduce_(tensor, average=None, name=None, op=None, prescale_factor=1.0, postscale_factor=1.0,
               compression=Compression.none):
    """In-place allreduce."""
    return synchronize(allreduce_async_(tensor, average, name, op, prescale_factor, postscale_factor, compression))


def grouped_allreduce(tensors, average=None, name=None, compression=Compression.none, op=None,
                      prescale_factor=1.0, postscale_factor=1.0):
    """Allreduce a list of tensors; they are enqueued together so the engine can fuse them."""
    base = _auto_name("grouped_allreduce", name)
    hs = [allreduce_async(t, average, f"{base}.{i}", compression, op, prescale_factor, postscale_factor)
          for i, t in enumerate(tensors)]
    return [synchronize(h) for h in hs]


def sparse_allreduce(tensor: torch.Tensor, name=None, op=Average):
    """Allreduce of a sparse COO tensor as two allgathers (values, indices).

    Mirrors the reference's tf.IndexedSlices branch (tips/tensorflow/__init__.py:61-76):
    gathered values are divided by the world size when `op` is Average.
    """
    _require_init()
    t = tensor.coalesce()
    base = _auto_name("sparse_allreduce", name)
    values = t.values()
    sparse_dim, nnz = t.indices().shape
    indices = t.indices().t().reshape(-1).reshape(nnz, sparse_dim)   # [nnz, sparse_dim] int64, unit inner stride
    inner = values.shape[1:]
    vbytes = values.element_size()
    for d in inner:
        vbytes *= d
    if vbytes % 8 == 0 or nnz == 0:
        # One collective instead of two: a row of the gathered matrix is [the entry's indices | its values] as bytes
        # (one negotiation through the coordinator per step instead of two; the reference gathers values and indices
        # separately, tips/tensorflow/__init__.py:61-76).
        packed = torch.cat([indices.view(torch.uint8).reshape(nnz, sparse_dim * 8),
                            values.reshape(-1).view(torch.uint8).reshape(nnz, vbytes)], dim=1)
        gathered = allgather(packed, name=base + ".entries")
        total = gathered.shape[0]
        indices = gathered[:, :sparse_dim * 8].reshape(-1).view(torch.int64).reshape(total, sparse_dim).t()
        values = gathered[:, sparse_dim * 8:].reshape(-1).view(values.dtype).reshape((total,) + tuple(inner))
    else:  # value rows that are not a multiple of 8 bytes would leave the int64 indices misaligned
        values = allgather(values, name=base + ".values")
        indices = allgather(indices, name=base + ".indices").t()
    if op == Average:
        values = values / _size()
    return torch.sparse_coo_tensor(indices, values, t.shape).coalesce()


# ------------------------------------------------------------------ allgather


def allgather_async(tensor: torch.Tensor, name=None) -> _Handle:
    _require_init()
    h = _Handle()
    h.kind = "allgather"
    src = tensor.contiguous()
    if src.dim() == 0:
        src = src.reshape(1)
    if _size() == 1:
        h.output = src.clone()
        return h
    if src.is_cuda:
        from . import device as _device
        if _device.state().backend == "nccl":
            return _device.nccl_allgather(h, src)
    gathered = []
    trailing = tuple(src.shape[1:])

    def _alloc(handle, nbytes, first_dims, n, user):
        h.first_dims = [int(first_dims[i]) for i in range(n)]   # every rank's dimension 0, in rank order
        total = sum(h.first_dims)
        out = torch.empty((total,) + trailing, dtype=src.dtype, device=src.device)
        gathered.append(out)
        return out.data_ptr() if out.numel() else 0

    cb = _lib.ALLOC_FN(_alloc)
    h.alloc_cb = cb
    h.gathered = gathered
    h.keep = [src]
    return _enqueue(h, 1, _auto_name("allgather", name), src, None, tuple(src.shape), src.dtype, alloc=cb)


def allgather(tensor, name=None):
    """Concatenate `tensor` from all ranks along dimension 0 (first dimensions may differ)."""
    return synchronize(allgather_async(tensor, name))


# ------------------------------------------------------------------ broadcast


def broadcast_async(tensor: torch.Tensor, root_rank: int = 0, name=None, _inplace=False) -> _Handle:
    _require_init()
    h = _Handle()
    h.kind = "broadcast"
    n = _size()
    if not 0 <= root_rank < n:
        raise ValueError(f"root_rank {root_rank} out of range for world size {n}")
    if n == 1:
        h.output = tensor if _inplace else tensor.clone()
        return h
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    if src.is_cuda:
        from . import device as _device
        if _device.state().backend == "nccl":
            return _device.nccl_broadcast(h, tensor, src, root_rank, _inplace)
    out = src if (_inplace and src is tensor) else src.clone()
    h.keep = [src, out]
    h.output = out
    if _inplace and out is not tensor:
        h.post = lambda o, tensor=tensor: tensor.copy_(o)
    return _enqueue(h, 2, _auto_name("broadcast", name), out, out, tuple(out.shape), out.dtype, root=root_rank)


def broadcast(tensor, root_rank=0, name=None):
    """Return root_rank's `tensor` on every rank."""
    return synchronize(broadcast_async(tensor, root_rank, name))


def broadcast_async_(tensor, root_rank=0, name=None):
    return broadcast_async(tensor, root_rank, name, _inplace=True)


def broadcast_(tensor, root_rank=0, name=None):
    """In-place broadcast."""
    return synchronize(broadcast_async_(tensor, root_rank, name))
