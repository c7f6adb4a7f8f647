"""DistributedOptimizer: data-parallel training by allreducing gradients.

API parity with the reference's ``DistributedOptimizer`` / ``DistributedGradientTape``
(tips/tensorflow/__init__.py:252-456,459-568, tips/_keras/__init__.py:27-177): wrap
an optimizer so that gradients are combined across ranks before they are applied;
``compression``, ``op`` (Average / Sum), ``gradient_predivide_factor``,
``backward_passes_per_step`` with ``average_aggregated_gradients``,
``sparse_as_dense``; the wrapper is a dynamic subclass carrying the wrapped
optimizer's class name, so a checkpoint loads without this package
(_keras/__init__.py:161-166); using gradients that were never aggregated is an
error (_keras/__init__.py:130-159).

What differs: the reference issues one negotiated allreduce per gradient tensor.
Here gradients are fused into buckets (``fusion_threshold_bytes``, 64 MB by
default); a bucket is packed by one kernel as soon as backward has produced its
last gradient, handed to the collective engine, and reduced in place in
symmetric memory by one fused kernel on the communication stream while backward
continues.  After the first step the bucket order is frozen, and later steps
need no control messages at all.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..config import get_config
from ..runtime import TipsError, _require_init
from . import collectives as C
from .buckets import build_buckets
from .compression import Compression
from ..utils.trace import nvtx_range


_optimizer_counter = 0


class _DistributedMixin:
    """Behaviour mixed into a dynamic subclass of the user's optimizer class."""

    def _tips_setup(self, named_parameters, compression, backward_passes_per_step, op, gradient_predivide_factor,
                    sparse_as_dense, average_aggregated_gradients, groups, fused_update=None):
        _require_init()
        if op not in (C.Average, C.Sum):
            raise ValueError("op must be Average or Sum")
        if gradient_predivide_factor != 1.0 and op != C.Average:
            raise ValueError("gradient_predivide_factor is only supported with op=Average")
        if backward_passes_per_step < 1:
            raise ValueError("backward_passes_per_step must be >= 1")
        self._tips_compression = compression
        self._tips_op = op
        self._tips_predivide = float(gradient_predivide_factor)
        self._tips_passes = int(backward_passes_per_step)
        self._tips_avg_aggregated = bool(average_aggregated_gradients)
        self._tips_sparse_as_dense = bool(sparse_as_dense)
        self._tips_groups = groups
        self._tips_size = C._size()
        params = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        if named_parameters is not None:
            named = list(named_parameters)
            ids = {id(p) for _, p in named}
            missing = [p for p in params if id(p) not in ids]
            if missing:
                raise ValueError("named_parameters does not cover every parameter of the optimizer")
            names = [n for n, _ in named]
            if len(set(names)) != len(names):
                raise ValueError("parameter names must be unique")
        self._tips_params = params
        self._tips_pass_count = {id(p): 0 for p in params}
        self._tips_sparse = []
        self._tips_synchronized = False
        self._tips_should_sync = True
        self._tips_step_count = 0
        self._tips_frozen = False
        self._tips_hooks = []

        from ..ops.optim import _FusedOptimizer
        self._tips_fused = isinstance(self, _FusedOptimizer)
        dev_state = None
        if any(p.is_cuda for p in params):
            from .. import runtime
            dev_state = runtime.device_state()
        wire = get_config().wire_dtype
        if compression is Compression.fp16:
            wire = "fp16"
        elif compression is Compression.bf16:
            wire = "bf16"
        self._tips_update_in_allreduce = False
        # `groups` (tips/tensorflow/__init__.py:394-404): explicit grouping of the gradient allreduces.  An integer is
        # the number of groups the parameters are cut into; a list of parameter lists puts every inner list into one
        # group and leaves every other parameter in a group of its own.  A group is a fusion bucket here.
        if groups is not None and not isinstance(groups, int):
            groups = [list(g) for g in groups]
            known = {id(p) for p in params}
            flat_ids = [id(p) for g in groups for p in g]
            if len(set(flat_ids)) != len(flat_ids) or not set(flat_ids) <= known:
                raise ValueError("groups must hold parameters of this optimizer, each at most once")
        if isinstance(groups, int) and groups < 0:
            raise ValueError("groups must be a non-negative integer or a list of parameter lists")
        total_bytes = sum(p.numel() * p.element_size() for p in params)
        group_threshold = None
        if isinstance(groups, int) and groups > 0:
            group_threshold = max(1, -(-total_bytes // groups))
        if self._tips_fused:
            if groups is not None and not isinstance(groups, int):
                raise ValueError("explicit parameter lists in `groups` need a stock torch optimizer; a fused "
                                 "optimizer takes an integer number of groups")
            if group_threshold is not None and not self._built:
                self._bucket_bytes = group_threshold
            self._wire_dtype = wire
            self._tips_buckets = [fs.bucket for fs in self.build(dev_state)]
            if fused_update is None:
                fused_update = get_config().fused_update
            if fused_update and self._tips_size > 1 and dev_state is not None and get_config().backend == "fused":
                if op != C.Average and op != C.Sum:
                    raise ValueError("the update inside the allreduce needs op Average or Sum")
                self._tips_update_in_allreduce = self.shard_for_fused_update(dev_state)
                self._tips_fs_of = {id(fs.bucket): fs for fs in self._flat}
        else:
            self._tips_buckets = []

            def add(plist, threshold):
                by_kind = {}
                for p in plist:
                    by_kind.setdefault((p.dtype, p.device), []).append(p)
                for same in by_kind.values():
                    for b in build_buckets(same, threshold, wire, dev_state):
                        b.index = len(self._tips_buckets)
                        b.name = f"tips.bucket.{b.index}"
                        self._tips_buckets.append(b)

            if groups is not None and not isinstance(groups, int):
                grouped = {id(p) for g in groups for p in g}
                for g in groups:
                    add([p for p in g if p.requires_grad], 1 << 62)   # one bucket per list (per dtype and device)
                for p in params:
                    if id(p) not in grouped:
                        add([p], 1 << 62)
            else:
                add(params, group_threshold)
        # Bucket names are the negotiation keys: unique per optimizer instance, identical across ranks as
        # long as every rank creates its optimizers in the same order.
        global _optimizer_counter
        prefix = f"tips.opt{_optimizer_counter}"
        _optimizer_counter += 1
        for i, b in enumerate(self._tips_buckets):
            b.index = i
            b.name = f"{prefix}.bucket.{i}"
        # A bucket is reduced in slices: runs of consecutive parameters of about fusion_slice_bytes that are handed
        # to the engine as soon as backward has produced their gradients, so that only the last slice of the last
        # bucket is left when backward ends.  One slice = the whole bucket when slicing does not apply.
        self._tips_slice_of = {}
        slice_bytes = int(get_config().fusion_slice_bytes)
        for b in self._tips_buckets:
            b.pending = len(b.params)
            es = b.grad.element_size()
            sliced = (slice_bytes > 0 and self._tips_size > 1 and not self._tips_update_in_allreduce
                      and b.numel * es >= 2 * slice_bytes)
            b.slice_list = b.slices(slice_bytes) if sliced else [(0, len(b.params), 0, b.numel)]
            b.slice_ready = [0] * len(b.slice_list)
            b.slice_launched = [False] * len(b.slice_list)
            b.handles = [None] * len(b.slice_list)
            b.slice_names = [b.name if len(b.slice_list) == 1 else f"{b.name}.s{k}" for k in range(len(b.slice_list))]
            for k, (i0, i1, _, _) in enumerate(b.slice_list):
                for p in b.params[i0:i1]:
                    self._tips_slice_of[id(p)] = (b, k)
        for p in params:
            self._tips_hooks.append(p.register_post_accumulate_grad_hook(self._tips_make_hook()))
        import ctypes
        _lib.core().tips_take_negotiated_order(ctypes.create_string_buffer(1 << 16), 1 << 16)  # clear the log

    # ------------------------------------------------------------------ hooks
    def _tips_make_hook(self):
        def hook(p):
            pid = id(p)
            self._tips_pass_count[pid] += 1
            if self._tips_pass_count[pid] < self._tips_passes:
                return
            if self._tips_pass_count[pid] > self._tips_passes:
                raise TipsError("a gradient was computed more than backward_passes_per_step times since the last "
                                "step(); call step() or synchronize() first, or raise backward_passes_per_step", 3)
            if p.grad is not None and p.grad.is_sparse:
                if self._tips_sparse_as_dense:
                    p.grad = p.grad.to_dense()
                else:
                    self._tips_sparse.append(p)
            b, k = self._tips_slice_of[pid]
            b.ready_count += 1
            b.slice_ready[k] += 1
            i0, i1, _, _ = b.slice_list[k]
            if b.slice_ready[k] == i1 - i0:
                self._tips_launch(b, k)
        return hook

    def _tips_launch(self, b, k):
        """Pack slice `k` of the bucket and hand it to the collective engine."""
        n = self._tips_size
        pre = 1.0
        post = 1.0
        if self._tips_op == C.Average:
            pre = 1.0 / self._tips_predivide
            post = self._tips_predivide / n
        if self._tips_avg_aggregated and self._tips_passes > 1:
            pre /= self._tips_passes
        i0, i1, off, count = b.slice_list[k]
        params = b.params[i0:i1]
        part = b.grad[off:off + count]
        dense = [p for p in params if not (p.grad is not None and p.grad.is_sparse)]
        if any(p.grad is None for p in dense) or len(dense) != len(params):
            part.zero_()
        saved = None
        if len(dense) != len(params):  # sparse gradients travel separately
            saved = {id(p): p.grad for p in params if p.grad is not None and p.grad.is_sparse}
            for p in params:
                if id(p) in saved:
                    p.grad = None
        with nvtx_range(f"tips.pack {b.slice_names[k]}"):
            b.pack(scale=pre, only=(i0, i1))
        if saved:
            for p in params:
                if id(p) in saved:
                    p.grad = saved[id(p)]
        b.slice_launched[k] = True
        b.launched = True
        if n == 1:
            if post != 1.0:
                part.mul_(post)
            b.handles[k] = None
            return
        if self._tips_update_in_allreduce:
            if saved:
                raise TipsError("sparse gradients cannot be combined with the update inside the allreduce; use "
                                "sparse_as_dense=True", 3)
            # the kernel that reduces this bucket also applies the step: it needs this step's hyper-parameters
            self.push_update_hyper(self._tips_fs_of[id(b)])
        h = C._Handle()
        h.kind = "allreduce"
        h.output = part
        h.keep = [part]
        with nvtx_range(f"tips.enqueue {b.slice_names[k]}"):
            b.handles[k] = C._enqueue(h, 0, b.slice_names[k], part, part, (count,), part.dtype, reduce_op=0,
                                      prescale=1.0, postscale=post)

    # ------------------------------------------------------------- public API
    def synchronize(self):
        """Wait for every gradient allreduce of this step and make the reduced gradients visible."""
        for b in self._tips_buckets:
            for k in range(len(b.slice_list)):
                if not b.slice_launched[k]:
                    # no (or not every) gradient of the slice on this rank: still take part, with zeros for the
                    # missing ones, so that the ranks stay in step
                    self._tips_launch(b, k)
        timeout = get_config().collective_timeout_s
        for b in self._tips_buckets:
            for k, h in enumerate(b.handles):
                if h is not None:
                    with nvtx_range(f"tips.wait {b.slice_names[k]}"):
                        C.synchronize(h, timeout if timeout > 0 else None)
                    b.handles[k] = None
        # a kernel that gave up on a peer skipped its reduction (and, with the update inside the allreduce, its
        # update): stop here, before the optimizer applies gradients that were never combined
        if any(b.grad.is_cuda for b in self._tips_buckets):
            C._check_device_status()
        for p in self._tips_sparse:
            p.grad = C.sparse_allreduce(p.grad, name=f"tips.sparse.{id(p)}", op=self._tips_op)
        self._tips_sparse = []
        if self._tips_fused:
            for fs in self._flat:
                fs.grads_packed = True
        else:
            for b in self._tips_buckets:
                sparse_ids = {id(p) for p in b.params if p.grad is not None and p.grad.is_sparse}
                for i, p in enumerate(b.params):
                    if id(p) in sparse_ids:
                        continue
                    v = b.view_of(i)
                    p.grad = v if v.dtype == p.dtype else v.to(p.dtype)
        self._tips_synchronized = True
        self._tips_maybe_freeze()

    def _tips_maybe_freeze(self):
        cfg = get_config()
        if self._tips_frozen or not cfg.static_schedule or self._tips_size == 1:
            return
        if not all(b.grad.is_cuda for b in self._tips_buckets):
            return
        lib = _lib.core()
        import ctypes
        buf = ctypes.create_string_buffer(1 << 16)
        n = lib.tips_take_negotiated_order(buf, 1 << 16)
        if n <= 0:
            return
        names = buf.value.decode().split("\n")
        mine = {name for b in self._tips_buckets for name in b.slice_names}
        order = [x for x in names if x in mine]
        if len(order) != len(mine):
            return
        if lib.tips_freeze_schedule("\n".join(order).encode()) == 0:
            self._tips_frozen = True

    class _SkipSync:
        def __init__(self, opt):
            self.opt = opt

        def __enter__(self):
            self.opt._tips_should_sync = False

        def __exit__(self, *a):
            self.opt._tips_should_sync = True

    def skip_synchronize(self):
        """Context manager: ``step()`` inside it does not synchronize (the caller already did)."""
        return _DistributedMixin._SkipSync(self)

    def step(self, closure=None, **kwargs):
        if self._tips_should_sync:
            if self._tips_synchronized:
                import warnings
                warnings.warn("step() called after synchronize() without skip_synchronize(); "
                              "gradients are synchronized only once")
            else:
                self.synchronize()
        elif not self._tips_synchronized:
            raise TipsError("step() inside skip_synchronize() but synchronize() was not called: the gradients "
                            "have not been aggregated across ranks", 3)
        self._tips_synchronized = False
        out = super().step(closure, **kwargs) if closure is not None or kwargs else super().step()
        self._tips_after_step()
        return out

    def _tips_after_step(self):
        self._tips_step_count += 1
        for b in self._tips_buckets:
            b.ready_count = 0
            b.launched = False
            b.slice_ready = [0] * len(b.slice_list)
            b.slice_launched = [False] * len(b.slice_list)
        for k in self._tips_pass_count:
            self._tips_pass_count[k] = 0
        if not self._tips_fused:
            # reduced gradients were consumed; drop the views so that the next backward
            # writes fresh gradients instead of accumulating into the bucket
            for p in self._tips_params:
                p.grad = None

    def reset(self):
        """Forget the step in progress after a failure: drop the handles of the buckets in flight, clear the
        per-step counters and the frozen bucket order, so that the next backward pass starts a clean step that is
        negotiated again.  Call it on every rank after ``tips_b200.reset_collectives()`` (``elastic.run`` does)."""
        for b in self._tips_buckets:
            for k, h in enumerate(b.handles):
                if h is not None:
                    C.abandon(h)
                    b.handles[k] = None
            b.ready_count = 0
            b.launched = False
            b.slice_ready = [0] * len(b.slice_list)
            b.slice_launched = [False] * len(b.slice_list)
        for k in self._tips_pass_count:
            self._tips_pass_count[k] = 0
        self._tips_sparse = []
        self._tips_synchronized = False
        self._tips_should_sync = True
        self._tips_frozen = False
        if self._tips_fused:
            for fs in self._flat:
                fs.grads_packed = False
        else:
            for p in self._tips_params:
                p.grad = None

    def zero_grad(self, set_to_none: bool = True):
        if any(h is not None for b in self._tips_buckets for h in b.handles):
            raise TipsError("zero_grad() called while gradient allreduces are in flight; call step() or "
                            "synchronize() first", 3)
        return super().zero_grad(set_to_none)


def DistributedOptimizer(optimizer, named_parameters=None, compression=Compression.none,
                         backward_passes_per_step=1, op=C.Average, gradient_predivide_factor=1.0,
                         sparse_as_dense=False, average_aggregated_gradients=True, groups=None, fused_update=None):
    """Wrap `optimizer` so that `step()` applies gradients combined over all ranks.

    ``fused_update`` (default: the ``fused_update`` configuration field) makes a FusedSGD / FusedAdam step run
    inside the kernel that reduces each gradient bucket: every rank reduces its share of the bucket, updates the
    fp32 master weights and state of that share (the only copy of them in the job) and stores the new parameters
    into every rank's parameter buffer in symmetric memory.  The reduced gradients are then never materialised, so
    code that reads or clips ``p.grad`` between ``synchronize()`` and ``step()`` cannot use it."""
    cls = type(optimizer.__class__.__name__, (_DistributedMixin, optimizer.__class__), {})
    optimizer.__class__ = cls
    optimizer._tips_setup(named_parameters, compression, backward_passes_per_step, op, gradient_predivide_factor,
                          sparse_as_dense, average_aggregated_gradients, groups, fused_update)
    return optimizer
