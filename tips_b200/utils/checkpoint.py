"""Checkpoint / resume helpers.

The reference checkpoints with Keras ``ModelCheckpoint`` on rank 0 only
(examples/tensorflow2_keras_mnist.py:83-86), resumes with ``load_model`` that re-wraps the
optimizer (tips/_keras/__init__.py:215-231) and re-synchronises the ranks by broadcasting
variables (tips/_keras/callbacks.py:22-45).  Same scheme here: rank 0 writes one file with model,
optimizer and extra state; every rank may read it; ``resume`` loads on rank 0 and broadcasts.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

from .. import runtime
from ..parallel import functions as F


def _optimizer_state(optimizer):
    from ..ops.optim import _FusedOptimizer
    if isinstance(optimizer, _FusedOptimizer):
        return {"fused": True,
                "flat": [{k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in s.items()}
                         for s in optimizer.flat_state()],
                "masters": [fs.full_master().cpu() for fs in optimizer.build()],
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]}
    return {"fused": False, "state_dict": optimizer.state_dict()}


def _load_optimizer_state(optimizer, state):
    from ..ops.optim import _FusedOptimizer
    if state.get("fused"):
        if not isinstance(optimizer, _FusedOptimizer):
            raise TypeError("the checkpoint holds fused-optimizer state but the optimizer is not a fused one")
        optimizer.load_flat_state(state["flat"])
        for fs, m in zip(optimizer.build(), state["masters"]):
            fs.load_master(m)
        for g, src in zip(optimizer.param_groups, state["param_groups"]):
            g.update(src)
    else:
        optimizer.load_state_dict(state["state_dict"])


def save_checkpoint(path: str, model: torch.nn.Module, optimizer=None, extra: Optional[dict] = None,
                    rank0_only: bool = True) -> bool:
    """Write a checkpoint. With rank0_only (default) only rank 0 writes; returns True if this rank wrote."""
    opt_state = None
    if optimizer is not None and any(getattr(fs, "sharded", False) for fs in getattr(optimizer, "_flat", [])):
        opt_state = _optimizer_state(optimizer)  # assembling a sharded state is a collective: every rank takes part
    if rank0_only and runtime.is_initialized() and runtime.rank() != 0:
        return False
    payload = {"model": {k: v.detach().cpu() for k, v in model.state_dict().items()}, "extra": dict(extra or {}),
               "optimizer_class": type(optimizer).__name__ if optimizer is not None else None}
    if optimizer is not None:
        payload["optimizer"] = opt_state if opt_state is not None else _optimizer_state(optimizer)
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)
    return True


def load_checkpoint(path: str, model: torch.nn.Module, optimizer=None, map_location="cpu") -> dict:
    payload = torch.load(path, map_location=map_location, weights_only=False)
    model.load_state_dict(payload["model"])
    # a fused optimizer that owns these parameters keeps fp32 master copies: they follow the loaded values
    from ..ops.optim import refresh_masters_of
    refresh_masters_of(model.state_dict().values())
    if optimizer is not None and "optimizer" in payload:
        _load_optimizer_state(optimizer, payload["optimizer"])
    return payload.get("extra", {})


def resume(path: str, model: torch.nn.Module, optimizer=None, root_rank: int = 0) -> dict:
    """Load on root_rank, then broadcast parameters, optimizer state and the extra dict to every rank."""
    extra: Any = None
    if not runtime.is_initialized() or runtime.rank() == root_rank:
        extra = load_checkpoint(path, model, optimizer)
    if runtime.is_initialized() and runtime.size() > 1:
        F.broadcast_parameters(model.state_dict(), root_rank, prefix="tips.resume")
        if optimizer is not None:
            F.broadcast_optimizer_state(optimizer, root_rank)
        extra = F.broadcast_object(extra, root_rank, name="tips.resume.extra")
    return extra or {}


def load_model(path: str, model: torch.nn.Module, optimizer=None, root_rank: int = 0, **distributed_kwargs):
    """Resume a training job from a checkpoint and hand back an optimizer that is ready for distributed training.

    The reference's ``load_model`` loads a saved Keras model and re-wraps whatever stock optimizer class the file
    names in its DistributedOptimizer, so the caller never wraps by hand after a restart
    (tips/_keras/__init__.py:215-231).  Here the optimizer object is built by the caller (a torch checkpoint holds
    state, not objects); it may be a plain or fused torch optimizer or one that is wrapped already.  If it is not
    wrapped yet and the runtime is initialised it is wrapped with ``DistributedOptimizer(**distributed_kwargs)``
    first; then the checkpoint is loaded on `root_rank` and broadcast (``resume``).  The optimizer class recorded in
    the file must match.  Returns ``(optimizer, extra)``."""
    from ..parallel.optimizer import DistributedOptimizer, _DistributedMixin
    if optimizer is not None:
        # every rank learns the class the file names, so that a mismatch raises everywhere and not only on the root
        saved = None
        if not runtime.is_initialized() or runtime.rank() == root_rank:
            saved = torch.load(path, map_location="cpu", weights_only=False).get("optimizer_class")
        if runtime.is_initialized() and runtime.size() > 1:
            saved = F.broadcast_object(saved, root_rank, name="tips.load_model.class")
        if saved is not None and saved != type(optimizer).__name__:
            raise TypeError(f"the checkpoint was written with a {saved} optimizer, got {type(optimizer).__name__}")
        if runtime.is_initialized() and not isinstance(optimizer, _DistributedMixin):
            optimizer = DistributedOptimizer(optimizer, **distributed_kwargs)
    extra = resume(path, model, optimizer, root_rank)
    return optimizer, extra
