"""Parameter / optimizer-state broadcast and collectives on Python objects.

API parity with the reference's tips/tensorflow/functions.py: ``broadcast_variables``
(functions.py:14-46; here ``broadcast_parameters``), ``broadcast_object`` /
``broadcast_object_fn`` (cloudpickle -> uint8 tensor, size first then payload,
functions.py:49-124) and ``allgather_object`` (sizes allgather + payload
allgatherv, sliced by prefix sums, functions.py:127-168); plus
``broadcast_optimizer_state`` which the reference covers by broadcasting
``optimizer.variables()`` in its Keras callback (_keras/callbacks.py:30-45).
"""
from __future__ import annotations

import io
import pickle
from typing import Any

import torch

from . import collectives as C

try:  # cloudpickle serialises lambdas and local classes too
    import cloudpickle as _pickle
except Exception:  # pragma: no cover
    _pickle = pickle


def broadcast_tensors_(tensors, root_rank: int = 0, name: str = "tips.bcast.group") -> None:
    """Broadcast a list of tensors in place as ONE collective per device kind: the tensors are packed byte-wise
    into a flat buffer (every tensor on a 16-byte boundary), the buffer is broadcast once and cut up again, so a
    model's state dict costs one negotiation instead of one per tensor.

    The reference groups its variable broadcasts the same way (one ``tf.group`` of assign ops,
    tips/tensorflow/functions.py:36-46); its ops still negotiate tensor by tensor."""
    tensors = [t for t in tensors if isinstance(t, torch.Tensor) and t.numel() > 0]
    if not tensors or C._size() == 1:
        return
    by_device = {}
    for t in tensors:
        by_device.setdefault(t.device, []).append(t)
    for k, (device, group) in enumerate(sorted(by_device.items(), key=lambda kv: str(kv[0]))):
        if len(group) == 1 and group[0].is_contiguous():
            C.broadcast_(group[0], root_rank, name=f"{name}.{k}")
            continue
        offsets, total = [], 0
        for t in group:
            offsets.append(total)
            total += (t.numel() * t.element_size() + 15) // 16 * 16
        flat = torch.empty(total, dtype=torch.uint8, device=device)
        views = [flat[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offsets, group)]
        if C._rank() == root_rank:
            torch._foreach_copy_(views, [t.detach() for t in group])
        C.broadcast_(flat, root_rank, name=f"{name}.{k}")
        if C._rank() != root_rank:
            with torch.no_grad():
                torch._foreach_copy_([t.detach() for t in group], views)


def broadcast_parameters(params, root_rank: int = 0, prefix: str = "tips.bcast", optimizer=None) -> None:
    """Broadcast parameters (a state_dict, a list of (name, tensor) or an iterable of tensors) in place, all of
    them in one collective per device kind (`broadcast_tensors_`).
    A fused optimizer that already owns these parameters is found through its flat buffers and its fp32 master
    weights follow the new values (`optimizer` may still be passed; it is refreshed as a whole)."""
    if isinstance(params, dict):
        items = sorted(params.items())
    else:
        items = list(params)
        if items and not isinstance(items[0], tuple):
            items = [(str(i), t) for i, t in enumerate(items)]
    broadcast_tensors_([t.data if isinstance(t, torch.nn.Parameter) else t for _, t in items
                        if isinstance(t, torch.Tensor)], root_rank, name=prefix)
    if optimizer is not None and hasattr(optimizer, "refresh_master_from_params"):
        optimizer.refresh_master_from_params()
    else:
        from ..ops.optim import refresh_masters_of
        refresh_masters_of(t for _, t in items)


broadcast_variables = broadcast_parameters


def broadcast_object(obj: Any = None, root_rank: int = 0, name: str | None = None) -> Any:
    """Return root_rank's `obj` on every rank."""
    name = name or "tips.bcast_object"
    if C._size() == 1:
        return obj
    # One collective: an allgather to which only the root contributes bytes.  The negotiation carries every
    # rank's length, so the other ranks need not learn the size first (the reference broadcasts the size and then
    # the payload, tips/tensorflow/functions.py:49-124).
    if C._rank() == root_rank:
        buf = io.BytesIO()
        _pickle.dump(obj, buf)
        payload = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
    else:
        payload = torch.empty(0, dtype=torch.uint8)
    payload = C.allgather(payload, name=name + ".data")
    return pickle.loads(payload.numpy().tobytes())


def broadcast_object_fn(root_rank: int = 0, name: str | None = None):
    def fn(obj=None):
        return broadcast_object(obj, root_rank, name)
    return fn


def allgather_object(obj: Any, name: str | None = None) -> list:
    """Return the list of every rank's `obj`, in rank order."""
    name = name or "tips.allgather_object"
    buf = io.BytesIO()
    _pickle.dump(obj, buf)
    payload = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
    if C._size() == 1:
        return [pickle.loads(payload.numpy().tobytes())]
    # one collective: the allgather negotiates every rank's length anyway and the handle keeps them
    # (the reference gathers the sizes first and the payloads second, tips/tensorflow/functions.py:127-168)
    h = C.allgather_async(payload, name=name + ".data")
    gathered = C.synchronize(h)
    sizes = getattr(h, "first_dims", None)
    if sizes is None:
        sizes = C.allgather(torch.tensor([payload.numel()], dtype=torch.int64), name=name + ".size").tolist()
    out, off = [], 0
    for s in sizes:
        out.append(pickle.loads(gathered[off:off + s].numpy().tobytes()))
        off += s
    return out


def broadcast_optimizer_state(optimizer: torch.optim.Optimizer, root_rank: int = 0) -> None:
    """Make every rank's optimizer state equal to root_rank's (tensors in place, scalars via objects)."""
    from ..ops.optim import _FusedOptimizer
    if isinstance(optimizer, _FusedOptimizer):
        flat = optimizer.build()
        meta = broadcast_object([(fs.steps, sorted(fs.state.keys())) for fs in flat] if C._rank() == root_rank else None,
                                root_rank, name="tips.bcast_opt.meta")
        for i, (fs, (steps, keys)) in enumerate(zip(flat, meta)):
            fs.steps = steps
            if fs.sharded:
                # Every rank holds its own share, so there is nothing to copy unless the root has just loaded
                # full-size tensors (a checkpoint) that the other ranks have not seen: those travel whole and
                # every rank cuts its share out.
                pending = broadcast_object(sorted(fs._pending_full.keys()) if C._rank() == root_rank else None,
                                           root_rank, name=f"tips.bcast_opt.{i}.pending")
                for k in pending:
                    full = fs._pending_full.get(k) if C._rank() == root_rank else None
                    if full is None:
                        full = torch.empty(fs.layout.numel, dtype=torch.float32, device=fs.master.device)
                    C.broadcast_(full, root_rank, name=f"tips.bcast_opt.{i}.{k}")
                    if k == "master":
                        fs.load_master(full)
                    else:
                        fs.load_state(k, full)
                fs._pending_full = {}
                continue
            for k in keys:
                if k not in fs.state:
                    fs.state[k] = torch.zeros_like(fs.master)
                C.broadcast_(fs.state[k], root_rank, name=f"tips.bcast_opt.{i}.{k}")
            C.broadcast_(fs.master, root_rank, name=f"tips.bcast_opt.{i}.master")
            if fs.low:
                fs.flat_param.copy_(fs.master)
        groups = broadcast_object([{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
                                  if C._rank() == root_rank else None, root_rank, name="tips.bcast_opt.groups")
        for g, src in zip(optimizer.param_groups, groups):
            g.update(src)
        return
    state = optimizer.state_dict()
    if C._rank() == root_rank:
        skeleton = {"param_groups": state["param_groups"],
                    "state": {k: {n: (("tensor", tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("value", v))
                                  for n, v in s.items()} for k, s in state["state"].items()}}
    else:
        skeleton = None
    skeleton = broadcast_object(skeleton, root_rank, name="tips.bcast_opt.skeleton")
    params = [p for g in optimizer.param_groups for p in g["params"]]
    new_state = {}
    together = []
    for k in sorted(skeleton["state"].keys()):
        entry = {}
        device = params[k].device if isinstance(k, int) and k < len(params) else torch.device("cpu")
        for n, spec in sorted(skeleton["state"][k].items()):
            if spec[0] == "tensor":
                cur = state["state"].get(k, {}).get(n)
                if not (isinstance(cur, torch.Tensor) and tuple(cur.shape) == spec[1] and cur.dtype == spec[2]):
                    cur = torch.zeros(spec[1], dtype=spec[2], device=device)
                elif C._rank() != root_rank:
                    cur = cur.clone()
                entry[n] = cur
                together.append(cur)
            else:
                entry[n] = spec[1]
        new_state[k] = entry
    broadcast_tensors_(together, root_rank, name="tips.bcast_opt.tensors")
    optimizer.load_state_dict({"param_groups": skeleton["param_groups"], "state": new_state})


def metric_average(value, name: str):
    """Average a Python number or a tensor over all ranks."""
    t = value if isinstance(value, torch.Tensor) else torch.tensor(float(value), dtype=torch.float64)
    out = C.allreduce(t.detach().cpu().reshape(1) if t.dim() == 0 else t.detach().cpu(), name=name, op=C.Average)
    return out.item() if out.numel() == 1 else out


# ---- value-level collectives and small op wrappers --------------------------------------------------
# Counterparts of the reference's Keras value helpers (tips/_keras/__init__.py:193-212: allreduce /
# allgather / broadcast of constants) and of its raw size_op / rank_op (tips/tensorflow/ops.py:33-45).

def size_op() -> torch.Tensor:
    """World size as an int32 tensor."""
    return torch.tensor(C._size(), dtype=torch.int32)


def rank_op() -> torch.Tensor:
    """Rank as an int32 tensor."""
    return torch.tensor(C._rank(), dtype=torch.int32)


def local_size_op() -> torch.Tensor:
    """Number of ranks on this node as an int32 tensor."""
    from .. import runtime
    return torch.tensor(runtime.local_size(), dtype=torch.int32)


def local_rank_op() -> torch.Tensor:
    """Rank within this node as an int32 tensor."""
    from .. import runtime
    return torch.tensor(runtime.local_rank(), dtype=torch.int32)


def _as_tensor(value):
    if isinstance(value, torch.Tensor):
        return value
    return torch.as_tensor(value)


def allreduce_value(value, name=None, average=True):
    """Allreduce a Python number / sequence / array; returns a tensor."""
    t = _as_tensor(value)
    if not t.is_floating_point() and average:
        t = t.to(torch.float64)
    return C.allreduce(t, name=name, op=C.Average if average else C.Sum)


def allgather_value(value, name=None):
    t = _as_tensor(value)
    return C.allgather(t.reshape(1) if t.dim() == 0 else t, name=name)


def broadcast_value(value, root_rank=0, name=None):
    return C.broadcast(_as_tensor(value), root_rank, name=name)


def broadcast_global_variables(model: torch.nn.Module, root_rank: int = 0, optimizer=None) -> None:
    """Broadcast every parameter and buffer of `model` (and the optimizer state) from root_rank;
    the reference's broadcast_global_variables / BroadcastGlobalVariablesHook (tips/tensorflow/__init__.py:106-186)."""
    broadcast_parameters(model.state_dict(), root_rank)
    if optimizer is not None:
        broadcast_optimizer_state(optimizer, root_rank)


def allreduce_gradients(parameters, op=C.Average, compression=None, name="tips.grads") -> None:
    """Allreduce the .grad of every parameter in place, for hand-written training loops: what the
    reference's DistributedGradientTape does to the gradients a tape returns
    (tips/tensorflow/__init__.py:459-568)."""
    from .compression import Compression
    comp = compression or Compression.none
    params = [p for p in parameters if p.grad is not None]
    handles = [C.allreduce_async(p.grad, name=f"{name}.{i}", op=op, compression=comp) for i, p in enumerate(params)]
    for p, h in zip(params, handles):
        out = C.synchronize(h)
        if out is not p.grad:
            p.grad.copy_(out)
