"""Per-phase device timing of the parameter-server step on the named CTR geometry (26 fields x dim 64, batch
8192 per GPU, ids ~ Zipf(1.05)): pull, and the scatter / send / fence / reduce / apply phases of the synchronous
push, with the rows and bytes that cross NVLink against the rows of the batch.

    python -m tips_b200.bench.ps_phases [--rows 10000000] [--iters 20]                      (one GPU)
    python -m torch.distributed.run --nproc-per-node N -m tips_b200.bench.ps_phases ...    (N GPUs)

Each phase is timed with CUDA events recorded on the launching stream between the kernels of an eager pull and
push (tipsk_ps_phase_timing); the figures are the max over ranks of the per-rank mean over `iters` steps after 5
warm-up steps.  Every step uses a fresh batch of ids, so the rows touched differ from step to step.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import torch

import tips_b200 as tips
from tips_b200.models.ctr import synthetic_ctr_batch
from tips_b200.ops import base
from tips_b200.ps.gpu import ShardedEmbedding

PHASES = ("scatter", "send", "fence", "reduce", "apply")
PULL_PHASES = ("index", "pull fence", "fetch", "expand")


def _max_over_ranks(values):
    t = torch.tensor(values, dtype=torch.float64)
    if tips.is_initialized() and tips.size() > 1:
        t = tips.allreduce(t, op=tips.Max, name=None)
    return [float(v) for v in t]


def _sum_over_ranks(values):
    t = torch.tensor(values, dtype=torch.float64)
    if tips.is_initialized() and tips.size() > 1:
        t = tips.allreduce(t, op=tips.Sum, name=None)
    return [float(v) for v in t]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=10_000_000)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--fields", type=int, default=26)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--plain", action="store_true", help="plain pull and push (no index shared between them)")
    ap.add_argument("--emulate", type=int, default=0,
                    help="run that many ranks on ONE GPU (one launch covers all of them): the kernels without NVLink")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    em = a.emulate if a.emulate > 1 else 0
    if em:
        from tips_b200.config import set_config
        from tips_b200.parallel import device as _device
        set_config(symm_window_bytes=1 << 20, comm_blocks=8)
        _device.setup(emulate_ranks=em)
        rank, n = 0, em
    else:
        tips.init()
        rank, n = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    table = ShardedEmbedding(a.fields, a.rows, a.dim, optimizer="adagrad", lr=0.05, init_scale=0.05, seed=0,
                             expected_batch=a.batch, device=dev)
    lib = base.K()
    warm = 5

    def ids_of(i):
        mk = lambda r: synthetic_ctr_batch(a.batch, a.fields, a.rows, 13, seed=1000 * r + i)[0].to(dev)
        return [mk(r) for r in range(em)] if em else mk(rank)

    batches = [ids_of(i) for i in range(a.iters + warm)]
    mk_g = lambda: torch.randn(a.batch, a.fields * a.dim, device=dev).to(torch.bfloat16)
    mk_o = lambda: torch.empty(a.batch, a.fields * a.dim, dtype=torch.bfloat16, device=dev)
    grads = [mk_g() for _ in range(em)] if em else mk_g()
    out = [mk_o() for _ in range(em)] if em else mk_o()
    distinct = sum(int(t[:, f].unique().numel()) for b in batches[warm:] for t in (b if em else [b])
                   for f in range(a.fields))
    base.check(lib.tipsk_ps_phase_timing(1), "phase_timing")
    acc = [0.0] * 5
    pacc = [0.0] * 4
    pull_ms = 0.0
    step_ms = 0.0
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ms5 = (ctypes.c_float * 5)()
    ms4 = (ctypes.c_float * 4)()
    for i, ids in enumerate(batches):
        if i == warm:
            table.check()
            table.traffic()
        e[0].record()
        table.pull(ids, out=out, index=not a.plain)
        e[1].record()
        table.push(ids, grads, grad_scale=1.0 / n, reuse_index=not a.plain)
        e[2].record()
        torch.cuda.synchronize()
        if i >= warm:
            base.check(lib.tipsk_ps_phase_ms(ms5), "phase_ms")
            for k in range(5):
                acc[k] += ms5[k]
            base.check(lib.tipsk_ps_pull_phase_ms(ms4), "pull_phase_ms")
            for k in range(4):
                pacc[k] += ms4[k]
            pull_ms += e[0].elapsed_time(e[1])
            step_ms += e[0].elapsed_time(e[2])
    base.check(lib.tipsk_ps_phase_timing(0), "phase_timing")
    applied = table.check()
    sent, remote, fetched = table.traffic()
    it = a.iters
    per = _max_over_ranks([1e3 * v / it for v in acc] + [1e3 * pull_ms / it, 1e3 * step_ms / it] +
                          [1e3 * v / it for v in pacc])
    tot = _sum_over_ranks([sent, remote, applied, distinct, fetched])
    if rank == 0:
        # bytes per row on the wire: pushed rows travel in the gradients' dtype (bf16 here) unless the wire is set
        # to fp32, plus the 8-byte key; pulled rows are read from the owner's bf16 copy when there is one
        from tips_b200.config import get_config
        row_bytes = a.dim * (4 if get_config().ps_wire_dtype == "fp32" else 2) + 8
        pull_row_bytes = a.dim * (2 if (table.shadow_base and not a.plain) else 4)
        items = a.batch * a.fields
        res = {"n_gpus": 1 if em else n, "emulated_ranks": em, "rows_per_table": a.rows, "batch_per_gpu": a.batch, "fields": a.fields, "dim": a.dim,
               "iters": it, "indexed": not a.plain,
               "us": {**{p: round(per[7 + k], 1) for k, p in enumerate(PULL_PHASES) if not a.plain},
                      "pull (with its fence)": round(per[5], 1),
                      **{p: round(per[k], 1) for k, p in enumerate(PHASES)}, "pull + push": round(per[6], 1)},
               "per_step_per_gpu": {
                   "items (sample, field)": items,
                   "distinct ids in the batch": round(tot[3] / it / n),
                   "rows pulled over NVLink": round(tot[4] / it / n) if not a.plain else round(items * (n - 1) / n),
                   "rows pushed over NVLink": round(tot[1] / it / n),
                   "rows applied by the owner": round(tot[2] / it / n),
                   "NVLink bytes (pull)": round((tot[4] / it / n if not a.plain else items * (n - 1) / n) * pull_row_bytes),
                   "NVLink bytes (push)": round(tot[1] / it / n * row_bytes),
                   "bytes if every item were sent as fp32": round(items * (a.dim * 4 + 8) * (n - 1) / n)}}
        line = json.dumps(res)
        print(line)
        if a.out:
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if not em:
        tips.shutdown()


if __name__ == "__main__":
    main()
