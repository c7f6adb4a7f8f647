"""Benchmark workloads driven through the public API: ResNet-50 data-parallel training and the
CTR parameter-server model.  Each returns the device-timed rate with resident inputs (`value`)
and the end-to-end rate with per-step host-to-device input copies and a loss read-back (`e2e`)."""
from __future__ import annotations

import os

import torch

import tips_b200 as tips
from tips_b200.ops import base as kbase


def _max_over_ranks(ms: float) -> float:
    if tips.size() == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64)
    return float(tips.allreduce(t, op=tips.Max, name=None)[0])


def _launch_count() -> int:
    n = kbase.launches()
    st = tips.runtime.device_state()
    if st is not None and st.window is not None:
        from tips_b200 import _lib
        n += int(_lib.kernels().tipsk_comm_launches())
    return n


def timed(step_fn, steps: int, warmup: int, inner: int = 1):
    """Run `warmup` untimed and `steps * inner` timed calls of step_fn between CUDA events; max over ranks.
    Returns (milliseconds for the whole timed region, launcher calls made inside it)."""
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    tips.barrier()
    torch.cuda.synchronize()
    l0 = _launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps * inner):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    l1 = _launch_count()
    tips.barrier()
    ms = _max_over_ranks(e0.elapsed_time(e1))
    return ms, l1 - l0


def inner_repeats(step_fn, steps: int, target_ms: float = 1200.0, probe: int = 20) -> int:
    """How many times a short step must be repeated per counted step so that the timed region lasts about
    `target_ms`; measured on `probe` calls, the same value on every rank."""
    torch.cuda.synchronize()
    tips.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(probe):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    per_step = max(_max_over_ranks(e0.elapsed_time(e1)) / probe, 1e-3)
    return max(1, int(round(target_ms / (per_step * max(steps, 1)) + 0.5)))


class _LossReader:
    """Device -> host read of every step's loss without stalling the step loop: each loss is copied into a pinned
    slot on the compute stream (4 bytes per step, inside the timed region) and read on the host a few steps later,
    when its copy has certainly finished; `drain()` reads the rest."""

    def __init__(self, depth: int = 4):
        self.slots = torch.zeros(depth, dtype=torch.float32).pin_memory()
        self.events = [None] * depth
        self.i = 0
        self.last = None
        self.read = 0

    def push(self, loss: torch.Tensor) -> None:
        k = self.i % len(self.events)
        if self.events[k] is not None:
            self.events[k].synchronize()
            self.last = float(self.slots[k])
            self.read += 1
        self.slots[k:k + 1].copy_(loss.detach().reshape(1).float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[k] = ev
        self.i += 1

    def drain(self):
        n = len(self.events)
        for j in range(self.i, self.i + n):
            k = j % n
            if self.events[k] is not None:
                self.events[k].synchronize()
                self.last = float(self.slots[k])
                self.read += 1
                self.events[k] = None
        return self.last


class _Prefetcher:
    """Double-buffered pinned-host -> device input pipeline on a side stream."""

    def __init__(self, host_batches):
        self.host = host_batches
        self.stream = torch.cuda.Stream()
        self.i = 0
        self.next = None
        self.bytes_per_step = sum(t.numel() * t.element_size() for t in host_batches[0])
        self._issue()

    def _issue(self):
        batch = self.host[self.i % len(self.host)]
        self.i += 1
        with torch.cuda.stream(self.stream):
            self.next = [t.cuda(non_blocking=True) for t in batch]
            self.ev = torch.cuda.Event()
            self.ev.record(self.stream)

    def get(self):
        torch.cuda.current_stream().wait_event(self.ev)
        cur = self.next
        for t in cur:
            t.record_stream(torch.cuda.current_stream())
        self._issue()
        return cur


def _image_batches(batch: int, count: int):
    """`count` pinned host batches of the named input: fp32 N(0,1) images in NCHW layout, labels uniform over 1000."""
    g = torch.Generator().manual_seed(100 + tips.rank())
    host = []
    for _ in range(count):
        x = torch.randn(batch, 3, 224, 224, generator=g)
        y = torch.randint(0, 1000, (batch,), generator=g)
        host.append((x.pin_memory(), y.pin_memory()))
    return host


def run_resnet50(batch: int, steps: int, warmup: int, fused_update=None):
    from tips_b200.models.resnet50 import resnet50
    from tips_b200.ops.optim import FusedSGD
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234)
    # TIPS_RESNET_LIBRARY_CONV=1 swaps the tcgen05 convolutions for library ones (for A/B measurements)
    model = resnet50(device=dev, library_conv=os.environ.get("TIPS_RESNET_LIBRARY_CONV", "0") == "1")
    model.train()
    opt = FusedSGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    opt = tips.DistributedOptimizer(opt, named_parameters=model.named_parameters(), fused_update=fused_update)
    tips.broadcast_parameters(model.state_dict(), root_rank=0, optimizer=opt)
    host = _image_batches(batch, 3)
    # inputs stay fp32 NCHW on the device as well: the stem's padding copy changes the layout and casts to bf16
    x_dev = host[0][0].to(dev, non_blocking=True)
    y_dev = host[0][1].to(dev, non_blocking=True)

    def step_resident():
        loss = model.loss(x_dev, y_dev)
        loss.backward()
        opt.step()
        return loss

    ms, launches = timed(step_resident, steps, warmup)
    st = tips.runtime.device_state()
    if st is not None and st.window is not None:
        st.check_status()
    value = batch * tips.size() * steps / (ms / 1e3)

    pre = _Prefetcher(host)
    last = {}
    reader = _LossReader()

    def step_e2e():
        x, y = pre.get()
        loss = model.loss(x, y)
        loss.backward()
        opt.step()
        reader.push(loss)

    ms2, _ = timed(step_e2e, steps, max(5, warmup))
    last["loss"] = reader.drain()
    e2e = {"value": batch * tips.size() * steps / (ms2 / 1e3), "unit": "images/s", "ms_per_step": ms2 / steps,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    update_in_allreduce = bool(getattr(opt, "_tips_update_in_allreduce", False))
    del pre, model, opt, x_dev, y_dev
    release_cached_memory()
    return {"value": value, "ms_per_step": ms / steps, "gpu_launches": launches, "e2e": e2e,
            "update_in_allreduce": update_in_allreduce}


def run_resnet50_floor(batch: int, steps: int, warmup: int):
    """Library floor: cuDNN batch norm, torch SGD (foreach), torch cross-entropy, NCCL DistributedDataParallel."""
    import torch.distributed as dist
    from tips_b200.models.resnet50 import resnet50
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234)
    model = resnet50(device=dev, library_norm=True).train()
    if tips.size() > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index], bucket_cap_mb=64,
                                                          gradient_as_bucket_view=True)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    host = _image_batches(batch, 3)
    x_dev, y_dev = host[0][0].to(dev), host[0][1].to(dev)

    def prep(x):  # the same fp32 NCHW input as the product arm; layout change and cast by library kernels
        return x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)

    def step_resident():
        loss = torch.nn.functional.cross_entropy(model(prep(x_dev)).float(), y_dev)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    ms, _ = timed(step_resident, steps, warmup)
    pre = _Prefetcher(host)
    last = {}
    reader = _LossReader()

    def step_e2e():
        xb, yb = pre.get()
        loss = torch.nn.functional.cross_entropy(model(prep(xb)).float(), yb)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        reader.push(loss)

    ms2, _ = timed(step_e2e, steps, max(5, warmup))
    last["loss"] = reader.drain()
    e2e = {"value": batch * tips.size() * steps / (ms2 / 1e3), "unit": "images/s", "ms_per_step": ms2 / steps,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    out = {"value": batch * tips.size() * steps / (ms / 1e3), "ms_per_step": ms / steps, "gpu_launches": 0, "e2e": e2e}
    del pre, model, opt, x_dev, y_dev
    release_cached_memory()
    return out


def release_cached_memory():
    import gc
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def run_ctr(batch: int, rows: int, steps: int, warmup: int, graph: bool = True, sync_ps: bool = True):
    from tips_b200.models.ctr import CtrTrainer, synthetic_ctr_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    release_cached_memory()
    # tables + Adagrad state for this rank's shards; refuse to start a step that cannot fit
    need = 26 * ((rows + tips.size() - 1) // tips.size()) * 64 * 4 * 2 + (6 << 30)
    free, _ = torch.cuda.mem_get_info()
    if need > free:
        raise MemoryError(f"CTR tables need {need >> 30} GiB on this GPU, {free >> 30} GiB are free")
    trainer = CtrTrainer(num_fields=26, rows_per_table=rows, dim=64, dense_features=13, hidden=(512, 256),
                         device=dev, expected_batch=batch, graph=graph, sync_ps=sync_ps)
    nhost = 8
    host = [tuple(t.pin_memory() for t in synthetic_ctr_batch(batch, 26, rows, 13, seed=7 * tips.rank() + 1000 * i))
            for i in range(nhost)]
    # eight different batches in rotation: the ids, hence the rows of the 133 GB of tables that a step touches, change
    # from step to step
    resident = [[t.to(dev) for t in b] for b in host]
    cursor = {"i": 0}

    def step_resident():
        b = resident[cursor["i"] % nhost]
        cursor["i"] += 1
        return trainer.train_step(*b)

    # kernels per step: launcher calls of one eager step (the captured graph replays exactly those)
    l0 = _launch_count()
    step_resident()
    per_step_launches = _launch_count() - l0
    for _ in range(max(warmup, 4)):
        step_resident()
    inner = inner_repeats(step_resident, steps)
    ms, launches = timed(step_resident, steps, 2, inner)
    if graph:
        launches = per_step_launches * steps * inner
    trainer.check()
    value = batch * tips.size() * steps * inner / (ms / 1e3)
    pre = _Prefetcher(host)
    last = {}
    reader = _LossReader()

    def step_e2e():
        ids, dense, labels = pre.get()
        reader.push(trainer.train_step(ids, dense, labels))

    for _ in range(max(5, warmup)):
        step_e2e()
    inner2 = inner_repeats(step_e2e, steps)
    ms2, _ = timed(step_e2e, steps, 2, inner2)
    last["loss"] = reader.drain()
    trainer.check()
    e2e = {"value": batch * tips.size() * steps * inner2 / (ms2 / 1e3), "unit": "samples/s",
           "ms_per_step": ms2 / (steps * inner2), "timed_region_ms": ms2, "repeats_per_step": inner2,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    out = {"value": value, "ms_per_step": ms / (steps * inner), "timed_region_ms": ms, "repeats_per_step": inner,
           "gpu_launches": launches, "e2e": e2e}
    trainer.close()
    del pre, trainer, resident
    release_cached_memory()
    return out


class _FloorCtr:
    """Library floor of the parameter-server workload: the same tables, sharded over the ranks by `id % N`, looked
    up with torch's embedding kernel, exchanged with NCCL all-to-all, updated by torch's sparse Adagrad; the MLP is
    torch Linear layers (cuBLAS) under DistributedDataParallel with torch Adam."""

    def __init__(self, fields, rows, dim, dense, hidden, dev):
        import torch.distributed as dist
        self.world, self.rank = tips.size(), tips.rank()
        self.fields, self.dim, self.dense, self.dev = fields, dim, dense, dev
        self.rps = (rows + self.world - 1) // self.world
        self.table = torch.empty(fields * self.rps, dim, device=dev).uniform_(-0.05, 0.05).requires_grad_()
        self.topt = torch.optim.Adagrad([self.table], lr=0.05)
        dims = [fields * dim + dense] + list(hidden)
        layers = []
        for i in range(len(hidden)):
            layers += [torch.nn.Linear(dims[i], dims[i + 1]), torch.nn.ReLU()]
        layers.append(torch.nn.Linear(dims[-1], 1))
        torch.manual_seed(17)
        self.mlp = torch.nn.Sequential(*layers).to(dev).to(torch.bfloat16)
        if self.world > 1:
            self.mlp = torch.nn.parallel.DistributedDataParallel(self.mlp, device_ids=[dev.index])
        self.mopt = torch.optim.Adam(self.mlp.parameters(), lr=1e-3)
        self.dist = dist
        self.field_base = (torch.arange(fields, device=dev) * self.rps).view(1, fields)

    def lookup(self, ids):
        n = self.world
        key = (ids // n + self.field_base).view(-1)
        if n == 1:
            return torch.nn.functional.embedding(key, self.table, sparse=True)
        import torch.distributed.nn.functional as dfn
        owner = (ids % n).view(-1)
        order = torch.argsort(owner, stable=True)
        send = torch.bincount(owner, minlength=n)
        recv = torch.empty_like(send)
        self.dist.all_to_all_single(recv, send)
        send_l, recv_l = send.tolist(), recv.tolist()
        keys_in = torch.empty(sum(recv_l), dtype=key.dtype, device=self.dev)
        self.dist.all_to_all_single(keys_in, key[order], recv_l, send_l)
        rows_out = torch.nn.functional.embedding(keys_in, self.table, sparse=True)
        back = torch.empty(key.numel(), self.dim, device=self.dev)
        back = dfn.all_to_all_single(back, rows_out, send_l, recv_l)
        emb = torch.empty_like(back)
        return emb.index_copy(0, order, back)  # the gradient flows back through the all-to-all

    def step(self, ids, dense, labels):
        emb = self.lookup(ids).view(ids.shape[0], self.fields * self.dim)
        if self.world > 1:
            emb.register_hook(lambda g: g / self.world)
        x = torch.cat([emb.to(torch.bfloat16), dense], dim=1)
        logit = self.mlp(x).view(-1).float()
        loss = torch.nn.functional.binary_cross_entropy_with_logits(logit, labels)
        loss.backward()
        self.topt.step()
        self.mopt.step()
        self.topt.zero_grad(set_to_none=True)
        self.mopt.zero_grad(set_to_none=True)
        return loss.detach()


def run_ctr_floor(batch: int, rows: int, steps: int, warmup: int):
    from tips_b200.models.ctr import synthetic_ctr_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    release_cached_memory()
    need = 26 * ((rows + tips.size() - 1) // tips.size()) * 64 * 4 * 2 + (8 << 30)
    free, _ = torch.cuda.mem_get_info()
    if need > free:
        raise MemoryError(f"CTR floor tables need {need >> 30} GiB on this GPU, {free >> 30} GiB are free")
    model = _FloorCtr(26, rows, 64, 13, (512, 256), dev)
    nhost = 8
    host = [tuple(t.pin_memory() for t in synthetic_ctr_batch(batch, 26, rows, 13, seed=7 * tips.rank() + 1000 * i))
            for i in range(nhost)]
    resident = [[t.to(dev) for t in b] for b in host]
    cursor = {"i": 0}

    def step_resident():
        b = resident[cursor["i"] % nhost]
        cursor["i"] += 1
        return model.step(*b)

    for _ in range(max(warmup, 4)):
        step_resident()
    inner = inner_repeats(step_resident, steps, probe=10)
    ms, _ = timed(step_resident, steps, 2, inner)
    pre = _Prefetcher(host)
    reader = _LossReader()

    def step_e2e():
        ids, dense, labels = pre.get()
        reader.push(model.step(ids, dense, labels))

    for _ in range(5):
        step_e2e()
    inner2 = inner_repeats(step_e2e, steps, probe=10)
    ms2, _ = timed(step_e2e, steps, 2, inner2)
    loss = reader.drain()
    e2e = {"value": batch * tips.size() * steps * inner2 / (ms2 / 1e3), "unit": "samples/s",
           "ms_per_step": ms2 / (steps * inner2), "timed_region_ms": ms2, "repeats_per_step": inner2,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": loss}
    out = {"value": batch * tips.size() * steps * inner / (ms / 1e3), "ms_per_step": ms / (steps * inner),
           "timed_region_ms": ms, "repeats_per_step": inner, "gpu_launches": 0, "e2e": e2e}
    del pre, model, resident
    release_cached_memory()
    return out


def run_bert(batch: int, seq: int, steps: int, warmup: int, layers: int = 24, fused_update=None):
    """BERT-large-shaped MLM training, data-parallel, AdamW (tokens/s)."""
    from tips_b200.models.bert import bert_large, synthetic_mlm_batch
    from tips_b200.ops.optim import FusedAdamW
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(4321)
    model = bert_large(device=dev, layers=layers, max_seq=seq).train()
    opt = tips.DistributedOptimizer(FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01),
                                    fused_update=fused_update)
    tips.broadcast_parameters(model.state_dict(), root_rank=0, optimizer=opt)
    host = [tuple(t.pin_memory() for t in synthetic_mlm_batch(batch, seq, 30522, seed=31 * tips.rank() + i))
            for i in range(3)]
    resident = [t.to(dev) for t in host[0]]

    def step_resident():
        loss = model.loss(*resident)
        loss.backward()
        opt.step()
        return loss

    ms, launches = timed(step_resident, steps, warmup)
    from tips_b200.ops.linear import gemm_status
    assert gemm_status() == 0
    value = batch * seq * tips.size() * steps / (ms / 1e3)
    pre = _Prefetcher(host)
    last = {}
    reader = _LossReader()

    def step_e2e():
        ids, pos, lab = pre.get()
        loss = model.loss(ids, pos, lab)
        loss.backward()
        opt.step()
        reader.push(loss)

    ms2, _ = timed(step_e2e, steps, max(5, warmup))
    last["loss"] = reader.drain()
    e2e = {"value": batch * seq * tips.size() * steps / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / steps,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    return {"value": value, "ms_per_step": ms / steps, "gpu_launches": launches, "e2e": e2e,
            "update_in_allreduce": bool(getattr(opt, "_tips_update_in_allreduce", False))}
