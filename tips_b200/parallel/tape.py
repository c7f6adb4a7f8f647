"""Hand-written training loops: a gradient "tape" whose gradients come back reduced over the ranks, and the
start-of-training broadcast as a hook object.

The reference wraps a ``tf.GradientTape`` so that ``tape.gradient(loss, variables)`` returns allreduced gradients
(tips/tensorflow/__init__.py:461-568: compression, sparse gradients as allgathers or densified, ``op``,
``gradient_predivide_factor``, explicit ``groups``) and ships a session hook that broadcasts all variables from a
root rank once (tips/tensorflow/__init__.py:152-186).  PyTorch records the graph by itself, so the tape here is a
thin context manager around ``torch.autograd.grad``; the reduction of the gradients is the same code path the
other collectives use (negotiated once, then the frozen schedule on CUDA).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch

from . import collectives as C
from . import functions as F
from .compression import Compression


def _split(items: Sequence, parts: int) -> List[list]:
    """`items` cut into `parts` contiguous runs whose lengths differ by at most one."""
    parts = max(1, min(parts, len(items))) if items else 1
    base, extra = divmod(len(items), parts)
    out, at = [], 0
    for i in range(parts):
        n = base + (1 if i < extra else 0)
        out.append(list(items[at:at + n]))
        at += n
    return out


class DistributedGradientTape:
    """``with DistributedGradientTape() as tape: loss = ...`` then ``tape.gradient(loss, params)`` returns the
    gradients of `loss` reduced over all ranks (averaged by default), in the order of `params`; parameters the loss
    does not depend on give ``None``.

    compression              wire format of dense gradients (``Compression.fp16`` / ``bf16``)
    sparse_as_dense          densify sparse gradients and allreduce them; otherwise they travel as two allgathers
    op                       ``Average`` (default), ``Sum``, ...
    gradient_predivide_factor  with Average: scale by 1/f before the sum and by f/size after it
    groups                   None: one collective per gradient (the engine fuses what is ready together);
                             an integer n: the dense gradients are packed into n flat buffers, one collective each;
                             a list of parameter lists: one buffer per inner list, the rest on their own
    persistent               keep the graph so that ``gradient`` can be called more than once
    """

    def __init__(self, compression=Compression.none, sparse_as_dense: bool = False, op=C.Average,
                 gradient_predivide_factor: float = 1.0, groups=None, persistent: bool = False,
                 name: str = "DistributedGradientTape"):
        if gradient_predivide_factor != 1.0 and op != C.Average:
            raise ValueError("gradient_predivide_factor not supported with op != Average")
        if groups is not None and not isinstance(groups, (list, tuple)) and not (isinstance(groups, int) and groups > 0):
            raise ValueError("groups should be a positive integer or a list of lists of parameters")
        self.compression = compression
        self.sparse_as_dense = sparse_as_dense
        self.op = op
        self.predivide = float(gradient_predivide_factor)
        self.groups = groups
        self.persistent = persistent
        self.name = name
        self._calls = 0

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    # -- reduction ------------------------------------------------------------------
    def _scales(self):
        if self.op == C.Average and self.predivide != 1.0:
            # Average divides by the size after the sum: together with the postscale this gives f / size
            return 1.0 / self.predivide, self.predivide
        return 1.0, 1.0

    def _reduce_dense(self, grads: List[torch.Tensor], sources: List[torch.Tensor], tag: str) -> List[torch.Tensor]:
        pre, post = self._scales()
        if self.groups is None:
            handles = [C.allreduce_async(g, name=f"{tag}.{i}", compression=self.compression, op=self.op,
                                         prescale_factor=pre, postscale_factor=post) for i, g in enumerate(grads)]
            return [C.synchronize(h) for h in handles]
        if isinstance(self.groups, int):
            buckets = _split(list(range(len(grads))), self.groups)
        else:
            index = {id(s): i for i, s in enumerate(sources)}
            taken, buckets = set(), []
            for plist in self.groups:
                members = [index[id(p)] for p in plist if id(p) in index and index[id(p)] not in taken]
                taken.update(members)
                if members:
                    buckets.append(members)
            buckets += [[i] for i in range(len(grads)) if i not in taken]
        out: List[Optional[torch.Tensor]] = [None] * len(grads)
        pending = []
        for b, members in enumerate(buckets):
            # one flat buffer per (bucket, dtype, device): tensors of different kinds cannot share storage
            kinds = {}
            for i in members:
                kinds.setdefault((grads[i].dtype, grads[i].device), []).append(i)
            for k, (kind, idx) in enumerate(sorted(kinds.items(), key=lambda kv: str(kv[0]))):
                flat = torch.cat([grads[i].reshape(-1) for i in idx])
                h = C.allreduce_async(flat, name=f"{tag}.group{b}.{k}", compression=self.compression, op=self.op,
                                      prescale_factor=pre, postscale_factor=post)
                pending.append((h, idx))
        for h, idx in pending:
            flat = C.synchronize(h)
            at = 0
            for i in idx:
                n = grads[i].numel()
                out[i] = flat[at:at + n].view_as(grads[i])
                at += n
        return out

    def reduce(self, grads: Sequence[Optional[torch.Tensor]], sources: Sequence[torch.Tensor]) -> list:
        """The reduction alone, for gradients computed elsewhere (e.g. by ``loss.backward()``)."""
        self._calls += 1
        tag = f"{self.name}.{self._calls}" if self.persistent else self.name
        if C._size() == 1:
            return list(grads)
        out = list(grads)
        dense_i, dense_g = [], []
        for i, g in enumerate(grads):
            if g is None:
                continue
            if g.is_sparse:
                if self.sparse_as_dense:
                    g = g.to_dense()
                else:
                    out[i] = C.sparse_allreduce(g, name=f"{tag}.sparse.{i}", op=self.op)
                    continue
            dense_i.append(i)
            dense_g.append(g.contiguous())
        reduced = self._reduce_dense(dense_g, [sources[i] for i in dense_i], tag)
        for i, g in zip(dense_i, reduced):
            out[i] = g
        return out

    def gradient(self, target: torch.Tensor, sources: Iterable[torch.Tensor], output_gradients=None) -> list:
        sources = list(sources)
        grads = torch.autograd.grad(target, sources, grad_outputs=output_gradients, retain_graph=self.persistent,
                                    allow_unused=True)
        return self.reduce(list(grads), sources)


class BroadcastGlobalVariablesHook:
    """Broadcasts a model's parameters and buffers (and an optimizer's state) from `root_rank` once, at the start of
    training or after restoring a checkpoint on the root, so that all workers start identical.  Use it from a
    hand-written loop: ``hook = BroadcastGlobalVariablesHook(0, model, optimizer); hook.begin()`` (``hook()`` and
    ``after_create_session()`` do the same; later calls are no-ops until ``reset()``)."""

    def __init__(self, root_rank: int = 0, model: Optional[torch.nn.Module] = None, optimizer=None):
        self.root_rank = root_rank
        self.model = model
        self.optimizer = optimizer
        self.done = False

    def begin(self, model: Optional[torch.nn.Module] = None, optimizer=None) -> None:
        model = model if model is not None else self.model
        optimizer = optimizer if optimizer is not None else self.optimizer
        if self.done:
            return
        if model is None:
            raise ValueError("BroadcastGlobalVariablesHook needs a model")
        F.broadcast_global_variables(model, self.root_rank, optimizer)
        self.done = True

    def after_create_session(self, session=None, coord=None) -> None:
        self.begin()

    __call__ = begin

    def reset(self) -> None:
        self.done = False
