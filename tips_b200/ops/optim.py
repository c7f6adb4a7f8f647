"""Fused optimizers on flat parameter slabs: SGD with momentum and Adam / AdamW.

Parameters of one (param group, dtype) partition are flattened into buckets;
each bucket owns a flat fp32 master copy (the parameters themselves when they
are fp32), flat optimizer state and a flat gradient buffer.  ``step()`` is one
kernel launch per bucket (csrc/kernels/elementwise.cu): it reads the gradient
once and writes master weights, state and — for bf16 / fp16 models — the
low-precision parameters in the same pass.

The reference has no optimizer kernels (TensorFlow applies the gradients); its
server-side SGD rule lives in the parameter server
(tips/core/ps/sparse_access_method.h:41-61).  These optimizers are what
``DistributedOptimizer`` drives on the bucketed fast path.
"""
from __future__ import annotations

import weakref
from typing import List

import torch

from ..parallel.buckets import Bucket, build_buckets
from . import base


# Every flat parameter buffer alive in this process: code that overwrites parameters from outside an optimizer
# (a broadcast, a loaded state dict) finds the fused optimizer state that owns them here and refreshes its fp32
# master copy, which would otherwise be written back over the new values by the next step.
_flat_registry = weakref.WeakSet()


def refresh_masters_of(tensors) -> int:
    """Re-read the fp32 master weights of every fused optimizer that owns one of `tensors` (parameters that were
    just overwritten in place).  Returns the number of flat buffers refreshed."""
    states = list(_flat_registry)
    if not states:
        return 0
    spans = [(fs, fs.flat_param.data_ptr(), fs.flat_param.data_ptr() + fs.flat_param.numel() * fs.flat_param.element_size())
             for fs in states]
    hit = []
    for t in tensors:
        if not isinstance(t, torch.Tensor) or t.numel() == 0:
            continue
        ptr = t.data_ptr()
        for fs, lo, hi in spans:
            if lo <= ptr < hi and fs not in hit:
                hit.append(fs)
    for fs in hit:
        fs.refresh_master_from_params()
    return len(hit)


class _FlatBucketState:
    def __init__(self, bucket: Bucket, group: dict):
        self.bucket = bucket
        self.group = group
        dev = bucket.device
        pdtype = bucket.params[0].dtype
        self.low = pdtype in (torch.bfloat16, torch.float16)
        flat = torch.zeros(bucket.numel, dtype=pdtype, device=dev)
        for i, p in enumerate(bucket.params):
            v = flat[bucket.offsets[i]:bucket.offsets[i] + p.numel()].view(p.shape)
            v.copy_(p.data)
            p.data = v
        self.flat_param = flat
        self.master = flat.float() if self.low else flat
        self.state = {}
        self.steps = 0
        self.grads_packed = False  # set by DistributedOptimizer when the bucket already holds reduced grads
        self.layout = None         # ShardLayout when the update runs inside the allreduce kernel
        self.rank = 0
        self.param_off = -1
        self._pending_full = {}    # full-size tensors loaded on this rank and not yet shared with the others
        _flat_registry.add(self)

    # -- update inside the allreduce: this rank keeps master weights and state of the vectors it owns -------------
    @property
    def sharded(self) -> bool:
        return self.layout is not None

    def shard(self, device_state, state_keys):
        """Move the parameters into the symmetric window and cut master weights / state down to this rank's share.
        `state_keys` names the state tensors the optimizer's rule needs; they start at zero."""
        from ..parallel.sharding import ShardLayout
        b = self.bucket
        if b.win_off < 0 or b.grad.dtype != self.flat_param.dtype:
            raise ValueError("the fused update needs the gradient bucket in the window and in the parameters' dtype")
        lib = base.K()
        es = self.flat_param.element_size()
        nbytes = b.numel * es
        pbuf, poff = device_state.alloc_symmetric(nbytes, self.flat_param.dtype)
        pbuf.copy_(self.flat_param)
        for i, p in enumerate(b.params):
            p.data = pbuf[b.offsets[i]:b.offsets[i] + p.numel()].view(p.shape)
        full_master = self.master.float() if self.master is self.flat_param else self.master
        self.flat_param = pbuf
        self.param_off = poff
        self.rank = device_state.rank
        self.layout = ShardLayout(b.numel, es, device_state.size, int(lib.tipsk_comm_update_subtile()))
        assert self.layout.shard_numel * es == int(lib.tipsk_comm_update_shard_vecs(nbytes)) * 16
        self.master = self.layout.take(full_master, self.rank)
        self.state = {k: torch.zeros_like(self.master) for k in state_keys}
        return self

    def attach(self, kind: int, s0=None, s1=None):
        import ctypes
        b = self.bucket

        def arr(t):
            return (ctypes.c_void_p * 1)(t.data_ptr()) if t is not None else None

        base.check(base.K().tipsk_comm_attach_update(
            b.win_off, b.numel * self.flat_param.element_size(), base.code(self.flat_param), self.param_off, kind,
            arr(self.master), arr(s0), arr(s1)), "attach_update")

    def full(self, shard: torch.Tensor) -> torch.Tensor:
        """Full-size tensor assembled from every rank's share (a collective: every rank calls it)."""
        if not self.sharded:
            return shard
        from ..parallel import collectives as C
        gathered = C.allgather(shard.reshape(1, -1), name=None)
        return self.layout.assemble(gathered)

    def full_master(self) -> torch.Tensor:
        return self.full(self.master)

    def load_master(self, full: torch.Tensor) -> None:
        full = full.to(self.master.device, torch.float32).reshape(-1)
        if self.sharded:
            self.master.copy_(self.layout.take(full, self.rank))
            self._pending_full["master"] = full
        else:
            self.master.copy_(full)
        if self.low or self.sharded:
            self.flat_param.copy_(full)

    def load_state(self, key: str, full: torch.Tensor) -> None:
        if key == "step_dev":  # rebuilt from `steps` by the optimizer
            return
        full = full.to(self.master.device, torch.float32).reshape(-1)
        if self.sharded:
            if key not in self.state:
                raise KeyError(f"the attached update has no state tensor {key!r}")
            self.state[key].copy_(self.layout.take(full, self.rank))  # in place: the kernel holds this pointer
            self._pending_full[key] = full
        else:
            self.state[key] = full.clone()

    def refresh_master_from_params(self) -> None:
        """After the parameters were overwritten from outside (a broadcast, a loaded state dict)."""
        if self.sharded:
            self.master.copy_(self.layout.take(self.flat_param.float(), self.rank))
        elif self.low:
            self.master.copy_(self.flat_param)


class _FusedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, defaults, bucket_bytes=None, wire_dtype="auto"):
        super().__init__(params, defaults)
        self._bucket_bytes = bucket_bytes
        self._wire_dtype = wire_dtype
        self._flat: List[_FlatBucketState] = []
        self._built = False

    # -- bucket construction ---------------------------------------------------
    def build(self, device_state=None):
        """Flatten the parameters (idempotent). Called lazily by step(), or by
        DistributedOptimizer with the device state so gradient buffers are symmetric."""
        if self._built:
            return self._flat
        index = 0
        for group in self.param_groups:
            by_dtype = {}
            for p in group["params"]:
                if p.requires_grad:
                    by_dtype.setdefault((p.dtype, p.device), []).append(p)
            for (_, _), plist in by_dtype.items():
                buckets = build_buckets(plist, self._bucket_bytes, self._wire_dtype, device_state)
                for b in buckets:
                    b.index = index
                    b.name = f"tips.bucket.{index}"
                    index += 1
                    self._flat.append(_FlatBucketState(b, group))
        self._built = True
        return self._flat

    @property
    def buckets(self) -> List[Bucket]:
        return [f.bucket for f in self.build()]

    def zero_grad(self, set_to_none: bool = True):
        for group in self.param_groups:
            for p in group["params"]:
                p.grad = None

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for fs in self.build():
            b = fs.bucket
            if fs.sharded:
                # the allreduce kernel of this bucket already applied the update to the share each rank owns
                if not fs.grads_packed:
                    raise RuntimeError("this optimizer's update runs inside the gradient allreduce: call step() "
                                       "through DistributedOptimizer, after backward")
                if grad_scale != 1.0:
                    raise ValueError("grad_scale is not supported when the update runs inside the allreduce")
                fs.grads_packed = False
                fs.steps += 1
                for p in b.params:
                    p.grad = None
                continue
            if not fs.grads_packed:
                if all(p.grad is None for p in b.params):
                    continue
                b.pack()
            fs.grads_packed = False
            fs.steps += 1
            self._update(fs, grad_scale)
            for p in b.params:
                p.grad = None
        return loss

    def _update(self, fs, grad_scale):
        raise NotImplementedError

    # -- update inside the allreduce --------------------------------------------
    _update_kind = -1  # 0 SGD, 1 Adam: which rule the allreduce kernel applies

    def shard_for_fused_update(self, device_state) -> bool:
        """Run this optimizer's update inside the gradient allreduce (csrc/kernels/comm.cu): parameters move into
        the symmetric window, every rank keeps 1/N of the master weights and state.  Returns False, and changes
        nothing, when a bucket does not qualify (no window, gradients in another dtype than the parameters)."""
        flat = self.build(device_state)
        if self._update_kind < 0 or device_state is None or device_state.window is None or device_state.emulated:
            return False
        if any(fs.sharded for fs in flat):
            return True
        if any(fs.bucket.win_off < 0 or fs.bucket.grad.dtype != fs.flat_param.dtype or fs.steps for fs in flat):
            return False
        for fs in flat:
            fs.shard(device_state, self._shard_state_keys(fs))
            self._attach(fs)
        return True

    def _shard_state_keys(self, fs):
        return []

    def _attach(self, fs):
        raise NotImplementedError

    def _hyper(self, fs):
        raise NotImplementedError

    def push_update_hyper(self, fs) -> None:
        """Hand the hyper-parameters of the coming step to the allreduce kernel of that bucket."""
        import ctypes
        h = [float(x) for x in self._hyper(fs)]
        base.check(base.K().tipsk_comm_set_update_hyper(fs.bucket.win_off, (ctypes.c_float * len(h))(*h), len(h),
                                                        fs.steps + 1), "set_update_hyper")

    def refresh_master_from_params(self) -> None:
        """Call after overwriting parameters from outside the optimizer (broadcast_parameters, load_state_dict):
        the fp32 master weights are re-read from the parameters."""
        for fs in self.build():
            fs.refresh_master_from_params()

    # state_dict: flat state is exposed per bucket, always as full-size tensors (with a sharded update this is a
    # collective: every rank has to call it)
    def flat_state(self):
        return [{"steps": fs.steps, **{k: fs.full(v) for k, v in fs.state.items() if k != "step_dev"}}
                for fs in self.build()]

    def load_flat_state(self, states):
        for fs, s in zip(self.build(), states):
            fs.steps = int(s.get("steps", 0))
            for k, v in s.items():
                if k == "steps":
                    continue
                fs.load_state(k, v)


class FusedSGD(_FusedOptimizer):
    """SGD with momentum, dampening, Nesterov and (coupled) weight decay; torch.optim.SGD semantics."""

    def __init__(self, params, lr=0.01, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                 bucket_bytes=None, wire_dtype="auto"):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        defaults = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)
        super().__init__(params, defaults, bucket_bytes, wire_dtype)

    _update_kind = 0

    def _shard_state_keys(self, fs):
        return ["momentum_buffer"] if float(fs.group["momentum"]) != 0.0 else []

    def _attach(self, fs):
        fs.attach(0, fs.state.get("momentum_buffer"))

    def _hyper(self, fs):
        g = fs.group
        return [g["lr"], g["momentum"], g["dampening"], g["weight_decay"], 1.0 if g["nesterov"] else 0.0]

    def _update(self, fs, grad_scale):
        g, b = fs.group, fs.bucket
        mom = float(g["momentum"])
        first = 0
        if mom != 0.0 and "momentum_buffer" not in fs.state:
            fs.state["momentum_buffer"] = torch.zeros_like(fs.master)
            first = 1
        buf = fs.state.get("momentum_buffer")
        if fs.master.is_cuda:
            base.check(base.K().tipsk_sgd_momentum_flat(
                fs.master.data_ptr(), fs.flat_param.data_ptr() if fs.low else None,
                base.code(fs.flat_param) if fs.low else 6, b.grad.data_ptr(), base.code(b.grad), base.ptr(buf),
                b.numel, float(g["lr"]), mom, float(g["dampening"]), float(g["weight_decay"]), int(g["nesterov"]),
                float(grad_scale), first, base.stream()), "sgd_momentum_flat")
        else:
            grad = b.grad.float() * grad_scale + float(g["weight_decay"]) * fs.master
            if mom != 0.0:
                if first:
                    buf.copy_(grad)
                else:
                    buf.mul_(mom).add_(grad, alpha=1.0 - float(g["dampening"]))
                grad = grad + mom * buf if g["nesterov"] else buf
            fs.master.add_(grad, alpha=-float(g["lr"]))
            if fs.low:
                fs.flat_param.copy_(fs.master)


class FusedAdam(_FusedOptimizer):
    """Adam; with ``decoupled_weight_decay`` (default) it is AdamW."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 decoupled_weight_decay=True, bucket_bytes=None, wire_dtype="auto", capturable=False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                        decoupled_weight_decay=decoupled_weight_decay)
        super().__init__(params, defaults, bucket_bytes, wire_dtype)
        self.capturable = capturable

    _update_kind = 1

    def _shard_state_keys(self, fs):
        return ["exp_avg", "exp_avg_sq"]

    def _attach(self, fs):
        fs.attach(1, fs.state["exp_avg"], fs.state["exp_avg_sq"])

    def _hyper(self, fs):
        g = fs.group
        return [g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                1.0 if g["decoupled_weight_decay"] else 0.0]

    def _update(self, fs, grad_scale):
        g, b = fs.group, fs.bucket
        if "exp_avg" not in fs.state:
            fs.state["exp_avg"] = torch.zeros_like(fs.master)
            fs.state["exp_avg_sq"] = torch.zeros_like(fs.master)
        m, v = fs.state["exp_avg"], fs.state["exp_avg_sq"]
        b1, b2 = g["betas"]
        if fs.master.is_cuda:
            step_ptr = None
            if self.capturable:
                # the step count lives on the device so that a captured graph can be replayed
                if "step_dev" not in fs.state:
                    fs.state["step_dev"] = torch.full((1,), fs.steps - 1, dtype=torch.int64, device=fs.master.device)
                fs.state["step_dev"].add_(1)
                step_ptr = fs.state["step_dev"].data_ptr()
            base.check(base.K().tipsk_adam_flat_devstep(
                fs.master.data_ptr(), fs.flat_param.data_ptr() if fs.low else None,
                base.code(fs.flat_param) if fs.low else 6, b.grad.data_ptr(), base.code(b.grad), m.data_ptr(),
                v.data_ptr(), b.numel, float(g["lr"]), float(b1), float(b2), float(g["eps"]),
                float(g["weight_decay"]), max(fs.steps, 1), step_ptr, float(grad_scale),
                int(g["decoupled_weight_decay"]), base.stream()), "adam_flat")
        else:
            grad = b.grad.float() * grad_scale
            if not g["decoupled_weight_decay"]:
                grad = grad + float(g["weight_decay"]) * fs.master
            m.mul_(b1).add_(grad, alpha=1 - b1)
            v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
            bias1 = 1 - b1 ** fs.steps
            bias2 = 1 - b2 ** fs.steps
            if g["decoupled_weight_decay"]:
                fs.master.mul_(1 - float(g["lr"]) * float(g["weight_decay"]))
            fs.master.addcdiv_(m / bias1, (v / bias2).sqrt_().add_(float(g["eps"])), value=-float(g["lr"]))
            if fs.low:
                fs.flat_param.copy_(fs.master)


class FusedAdamW(FusedAdam):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, bucket_bytes=None,
                 wire_dtype="auto"):
        super().__init__(params, lr, betas, eps, weight_decay, True, bucket_bytes, wire_dtype)
