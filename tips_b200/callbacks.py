"""Training-loop callbacks.

API parity with the reference's Keras callbacks (tips/_keras/callbacks.py:22-225,
tips/tensorflow/keras/callbacks.py:168-182), for a PyTorch loop (``tips_b200.trainer.fit``
or any loop that calls the ``on_*`` hooks):

* ``BroadcastGlobalVariablesCallback``: broadcast model and optimizer state from
  ``root_rank`` once, after the first batch (so lazily created optimizer state exists).
* ``MetricAverageCallback``: average every logged metric over the ranks at epoch end,
  in sorted-name order (the reference sums, because its allreduce ignores ``op``).
* ``LearningRateScheduleCallback``: multiply the initial learning rate by a constant or a
  function of the epoch between ``start_epoch`` and ``end_epoch``; ``staircase`` adjusts once
  per epoch, otherwise every batch with a fractional epoch; with ``momentum_correction`` the
  momentum is scaled by new_lr/old_lr for the batch in which the rate changes and restored
  afterwards.
* ``LearningRateWarmupCallback``: ramp from lr/size to lr over ``warmup_epochs``:
  multiplier(epoch) = 1/size * (epoch * (size - 1) / warmup_epochs + 1).
* ``BestModelCheckpoint``: rank-0 checkpoint whenever the monitored metric improves.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Union

import torch

from . import runtime
from .parallel import functions as F


class Callback:
    """Base class; a training loop sets `model`, `optimizer` and `params` before training."""

    model = None
    optimizer = None
    params: dict = {}

    def set_context(self, model, optimizer, params=None):
        self.model, self.optimizer, self.params = model, optimizer, dict(params or {})

    def on_train_begin(self, logs=None): ...
    def on_train_end(self, logs=None): ...
    def on_epoch_begin(self, epoch, logs=None): ...
    def on_epoch_end(self, epoch, logs=None): ...
    def on_batch_begin(self, batch, logs=None): ...
    def on_batch_end(self, batch, logs=None): ...


class BroadcastGlobalVariablesCallback(Callback):
    def __init__(self, root_rank: int = 0):
        self.root_rank = root_rank
        self.broadcast_done = False

    def on_batch_end(self, batch, logs=None):
        if self.broadcast_done:
            return
        F.broadcast_parameters(self.model.state_dict(), self.root_rank)
        if self.optimizer is not None:
            F.broadcast_optimizer_state(self.optimizer, self.root_rank)
        self.broadcast_done = True


class MetricAverageCallback(Callback):
    def on_epoch_end(self, epoch, logs=None):
        if logs is None:
            return
        for name in sorted(logs.keys()):
            value = logs[name]
            if isinstance(value, (int, float)) or (isinstance(value, torch.Tensor) and value.numel() == 1):
                logs[name] = F.metric_average(value, name=f"tips.metric.{name}")


class LearningRateScheduleCallback(Callback):
    def __init__(self, initial_lr: float, multiplier: Union[float, Callable[[float], float]], start_epoch: int = 0,
                 end_epoch: Optional[int] = None, staircase: bool = True, momentum_correction: bool = True,
                 steps_per_epoch: Optional[int] = None):
        self.initial_lr = initial_lr
        self.start_epoch = start_epoch
        self.end_epoch = end_epoch
        self.staircase = staircase
        self.momentum_correction = momentum_correction
        self.steps_per_epoch = steps_per_epoch
        self.current_epoch = 0
        self.restore_momentum = None
        if callable(multiplier):
            self.multiplier = multiplier
        else:
            self.staircase = True
            self.multiplier = lambda epoch: multiplier
        if self.initial_lr is None:
            raise ValueError("initial_lr is required")

    def _autodetect_steps(self):
        if self.steps_per_epoch is None:
            self.steps_per_epoch = self.params.get("steps")
        if self.steps_per_epoch is None:
            raise ValueError("steps_per_epoch is needed for a non-staircase schedule")

    def _adjust(self, epoch: float):
        new_lr = self.initial_lr * self.multiplier(epoch)
        for index, group in enumerate(self.optimizer.param_groups):
            old_lr = group["lr"]
            group["lr"] = new_lr
            if self.momentum_correction and "momentum" in group and old_lr > 0 and new_lr != old_lr:
                if self.restore_momentum is None:
                    self.restore_momentum = []
                # remembered by index: another callback may replace the group dicts (load_state_dict)
                self.restore_momentum.append((index, group["momentum"]))
                group["momentum"] = group["momentum"] * new_lr / old_lr

    def _restore(self):
        if self.restore_momentum:
            for index, m in self.restore_momentum:
                self.optimizer.param_groups[index]["momentum"] = m
        self.restore_momentum = None

    def _in_range(self, epoch):
        return epoch >= self.start_epoch and (self.end_epoch is None or epoch < self.end_epoch)

    def on_train_begin(self, logs=None):
        if not self.staircase:
            self._autodetect_steps()

    def on_epoch_begin(self, epoch, logs=None):
        self.current_epoch = epoch

    def on_batch_begin(self, batch, logs=None):
        if not self._in_range(self.current_epoch):
            return
        if self.staircase and batch == 0:
            self._adjust(self.current_epoch)
        elif not self.staircase:
            self._adjust(self.current_epoch + float(batch) / self.steps_per_epoch)

    def on_batch_end(self, batch, logs=None):
        self._restore()

    def on_epoch_end(self, epoch, logs=None):
        if logs is not None:
            logs["lr"] = self.optimizer.param_groups[0]["lr"]


class LearningRateWarmupCallback(LearningRateScheduleCallback):
    def __init__(self, initial_lr: float, warmup_epochs: int = 5, momentum_correction: bool = True,
                 steps_per_epoch: Optional[int] = None, verbose: int = 0):
        size = runtime.size()

        def multiplier(epoch):
            epoch += 1.0 / self.steps_per_epoch  # end the warm-up exactly at warmup_epochs
            return 1.0 / size * (epoch * (size - 1) / warmup_epochs + 1)

        super().__init__(initial_lr, multiplier, start_epoch=0, end_epoch=warmup_epochs, staircase=False,
                         momentum_correction=momentum_correction, steps_per_epoch=steps_per_epoch)
        self.verbose = verbose
        self.warmup_epochs = warmup_epochs

    def on_epoch_end(self, epoch, logs=None):
        super().on_epoch_end(epoch, logs)
        if epoch == self.end_epoch - 1 and self.verbose > 0 and runtime.rank() == 0:
            print(f"\nEpoch {epoch + 1}: finished gradual learning rate warmup to "
                  f"{self.optimizer.param_groups[0]['lr']:g}.")


class BestModelCheckpoint(Callback):
    """Save model (and optimizer) on rank 0 whenever `monitor` improves."""

    def __init__(self, filepath: str, monitor: str = "val_loss", mode: str = "auto", save_optimizer: bool = True):
        self.filepath = filepath
        self.monitor = monitor
        if mode == "auto":
            mode = "max" if ("acc" in monitor or monitor.startswith("fmeasure")) else "min"
        self.better = (lambda a, b: a > b) if mode == "max" else (lambda a, b: a < b)
        self.best = -math.inf if mode == "max" else math.inf
        self.save_optimizer = save_optimizer

    def on_epoch_end(self, epoch, logs=None):
        if not logs or self.monitor not in logs:
            return
        current = float(logs[self.monitor])
        if self.better(current, self.best):
            self.best = current
            if runtime.rank() == 0:
                from .utils.checkpoint import save_checkpoint
                save_checkpoint(self.filepath.format(epoch=epoch + 1, **logs), self.model,
                                self.optimizer if self.save_optimizer else None, extra={"epoch": epoch, "best": current})
