"""A small training loop that drives the callbacks, the role Keras ``model.fit`` plays in the
reference's example (examples/tensorflow2_keras_mnist.py:93-98)."""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .callbacks import Callback


def fit(model: torch.nn.Module, optimizer, loss_fn: Callable, batches: Callable[[int, int], tuple], epochs: int,
        steps_per_epoch: int, callbacks: Optional[List[Callback]] = None, initial_epoch: int = 0,
        metrics: Optional[Callable] = None, verbose: int = 0) -> list:
    """Train for `epochs` x `steps_per_epoch` steps.

    `batches(epoch, step)` returns (inputs, targets); `loss_fn(outputs, targets)` the loss; `metrics(outputs,
    targets)` an optional dict of extra logged values.  Returns the per-epoch logs.
    """
    callbacks = list(callbacks or [])
    params = {"epochs": epochs, "steps": steps_per_epoch}
    for cb in callbacks:
        cb.set_context(model, optimizer, params)
        cb.params = params  # shared, so one callback can shorten an epoch for the loop
    history = []
    for cb in callbacks:
        cb.on_train_begin({})
    for epoch in range(initial_epoch, epochs):
        logs = {}
        for cb in callbacks:
            cb.on_epoch_begin(epoch, logs)
        total, count = 0.0, 0
        extra = {}
        for step in range(params["steps"]):
            for cb in callbacks:
                cb.on_batch_begin(step, logs)
            x, y = batches(epoch, step)
            out = model(x)
            loss = loss_fn(out, y)
            loss.backward()
            optimizer.step()
            optimizer.zero_grad()
            total += float(loss.detach())
            count += 1
            if metrics is not None:
                for k, v in metrics(out.detach(), y).items():
                    extra[k] = extra.get(k, 0.0) + float(v)
            for cb in callbacks:
                cb.on_batch_end(step, logs)
        logs["loss"] = total / max(count, 1)
        for k, v in extra.items():
            logs[k] = v / max(count, 1)
        for cb in callbacks:
            cb.on_epoch_end(epoch, logs)
        if verbose:
            print(f"epoch {epoch + 1}/{epochs} " + " ".join(f"{k}={v:.4g}" for k, v in sorted(logs.items())))
        history.append(dict(logs))
    for cb in callbacks:
        cb.on_train_end({})
    return history
