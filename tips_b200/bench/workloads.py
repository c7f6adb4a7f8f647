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


def timed(step_fn, steps: int, warmup: int):
    """Run `warmup` untimed and `steps` timed calls of step_fn between CUDA events; max over ranks."""
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    tips.barrier()
    torch.cuda.synchronize()
    l0 = _launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    l1 = _launch_count()
    tips.barrier()
    ms = _max_over_ranks(e0.elapsed_time(e1))
    return ms, l1 - l0


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
    g = torch.Generator().manual_seed(100 + tips.rank())
    nhost = 3
    host = []
    for _ in range(nhost):
        x = torch.randn(batch, 3, 224, 224, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, 1000, (batch,), generator=g)
        host.append((x.pin_memory(), y.pin_memory()))
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
    g = torch.Generator().manual_seed(100 + tips.rank())
    x = torch.randn(batch, 3, 224, 224, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (batch,), generator=g)
    host = [(x.pin_memory(), y.pin_memory())] * 3
    x_dev, y_dev = x.to(dev), y.to(dev)

    def step_resident():
        loss = torch.nn.functional.cross_entropy(model(x_dev).float(), y_dev)
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
        loss = torch.nn.functional.cross_entropy(model(xb).float(), yb)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        reader.push(loss)

    ms2, _ = timed(step_e2e, steps, max(5, warmup))
    last["loss"] = reader.drain()
    e2e = {"value": batch * tips.size() * steps / (ms2 / 1e3), "unit": "images/s", "ms_per_step": ms2 / steps,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    return {"value": batch * tips.size() * steps / (ms / 1e3), "ms_per_step": ms / steps, "gpu_launches": 0, "e2e": e2e}


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
    nhost = 3
    host = [tuple(t.pin_memory() for t in synthetic_ctr_batch(batch, 26, rows, 13, seed=7 * tips.rank() + i))
            for i in range(nhost)]
    resident = [t.to(dev) for t in host[0]]

    def step_resident():
        return trainer.train_step(*resident)

    ms, launches = timed(step_resident, steps, warmup)
    trainer.check()
    value = batch * tips.size() * steps / (ms / 1e3)
    pre = _Prefetcher(host)
    last = {}
    reader = _LossReader()

    def step_e2e():
        ids, dense, labels = pre.get()
        reader.push(trainer.train_step(ids, dense, labels))

    ms2, _ = timed(step_e2e, steps, max(5, warmup))
    last["loss"] = reader.drain()
    trainer.check()
    e2e = {"value": batch * tips.size() * steps / (ms2 / 1e3), "unit": "samples/s", "ms_per_step": ms2 / steps,
           "h2d_bytes_per_step": pre.bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}
    return {"value": value, "ms_per_step": ms / steps, "gpu_launches": launches, "e2e": e2e}


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
