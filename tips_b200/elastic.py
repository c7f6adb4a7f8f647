"""Elastic training state and its loop hooks.

The reference ships three Keras callback implementations for an elastic ``state`` object
(tips/_keras/elastic.py:17-86: CommitStateCallbackImpl, UpdateBatchStateCallbackImpl,
UpdateEpochStateCallbackImpl) but no State class and no driver.  Here ``State`` holds model,
optimizer and progress counters with ``commit`` (snapshot in host memory), ``restore`` (roll back to
the last commit) and ``sync`` (adopt rank 0's state, e.g. after the set of ranks changed), and
``run`` retries a training function after a recoverable collective failure.
"""
from __future__ import annotations

import copy
from typing import Callable

import torch

from . import runtime
from .callbacks import Callback
from .parallel import functions as F


class State:
    def __init__(self, model: torch.nn.Module = None, optimizer=None, **counters):
        self.model = model
        self.optimizer = optimizer
        self.epoch = 0
        self.batch = 0
        self.commits = 0
        for k, v in counters.items():
            setattr(self, k, v)
        self._user_keys = list(counters.keys())
        self._saved = None
        self._reset_callbacks = []
        self.commit()

    def register_reset_callbacks(self, callbacks):
        self._reset_callbacks.extend(callbacks)

    def on_reset(self):
        for cb in self._reset_callbacks:
            cb()

    def _counters(self):
        return {k: getattr(self, k) for k in ["epoch", "batch", *self._user_keys]}

    def commit(self):
        """Snapshot model, optimizer and counters in host memory."""
        from .utils.checkpoint import _optimizer_state
        self._saved = {
            "model": {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()} if self.model else None,
            "optimizer": copy.deepcopy(_optimizer_state(self.optimizer)) if self.optimizer is not None else None,
            "counters": copy.deepcopy(self._counters()),
        }
        self.commits += 1

    def restore(self):
        """Roll back to the last commit."""
        from .utils.checkpoint import _load_optimizer_state
        if self._saved is None:
            return
        if self.model is not None:
            self.model.load_state_dict(self._saved["model"])
        if self.optimizer is not None and self._saved["optimizer"] is not None:
            _load_optimizer_state(self.optimizer, self._saved["optimizer"])
        for k, v in self._saved["counters"].items():
            setattr(self, k, copy.deepcopy(v))

    def sync(self, root_rank: int = 0):
        """Make every rank's state equal to root_rank's."""
        if not runtime.is_initialized() or runtime.size() == 1:
            return
        if self.model is not None:
            F.broadcast_parameters(self.model.state_dict(), root_rank, prefix="tips.elastic")
        if self.optimizer is not None:
            F.broadcast_optimizer_state(self.optimizer, root_rank)
        counters = F.broadcast_object(self._counters(), root_rank, name="tips.elastic.counters")
        for k, v in counters.items():
            setattr(self, k, v)
        self.commit()


def run(train_fn: Callable[[State], object], max_retries: int = 3):
    """Decorator-style driver: call ``train_fn(state)``; if a collective fails with a recoverable
    error (a rank left, a timeout) restore the last commit, re-sync and try again."""

    def wrapper(state: State, *args, **kwargs):
        attempts = 0
        while True:
            try:
                return train_fn(state, *args, **kwargs)
            except runtime.TipsError as e:
                attempts += 1
                if attempts > max_retries or e.code not in (5, 6):  # timeout, unavailable
                    raise
                # the failed step left handles, counters, a frozen schedule and device flags behind: clear them on
                # every rank (the ranks meet on a barrier inside), then roll back and adopt rank 0's state
                runtime.reset_collectives()
                if state.optimizer is not None and hasattr(state.optimizer, "reset"):
                    state.optimizer.reset()
                state.restore()
                state.on_reset()
                state.sync()

    return wrapper


class CommitStateCallback(Callback):
    """Commit every `batches_per_commit` batches and at the end of every epoch."""

    def __init__(self, state: State, batches_per_commit: int = 1):
        self.state = state
        self.batches_per_commit = batches_per_commit
        self.batches_remaining = batches_per_commit

    def on_batch_end(self, batch, logs=None):
        self.batches_remaining -= 1
        if self.batches_remaining == 0:
            self.state.commit()
            self.batches_remaining = self.batches_per_commit

    def on_epoch_end(self, epoch, logs=None):
        self.state.commit()


class UpdateBatchStateCallback(Callback):
    """Track the batch index in the state; after a reset, shorten the first epoch by the batches already done."""

    def __init__(self, state: State):
        self.state = state
        self.steps_per_epoch = None

    def on_train_begin(self, logs=None):
        self.steps_per_epoch = self.params.get("steps")

    def on_epoch_begin(self, epoch, logs=None):
        if self.steps_per_epoch is not None and self.state.batch > 0:
            self.params["steps"] = self.steps_per_epoch - self.state.batch  # resume mid-epoch
        elif self.steps_per_epoch is not None:
            self.params["steps"] = self.steps_per_epoch

    def on_batch_end(self, batch, logs=None):
        self.state.batch = batch + 1

    def on_epoch_end(self, epoch, logs=None):
        self.state.batch = 0


class UpdateEpochStateCallback(Callback):
    """Keep a global epoch number in the state that survives resets."""

    def __init__(self, state: State):
        self.state = state
        self.initial_epoch = state.epoch

    def on_train_begin(self, logs=None):
        self.initial_epoch = self.state.epoch

    def on_epoch_end(self, epoch, logs=None):
        # `epoch` counts from 0 in every (re)started loop, as in the reference (tips/_keras/elastic.py:80-86)
        self.state.epoch = self.initial_epoch + epoch + 1
