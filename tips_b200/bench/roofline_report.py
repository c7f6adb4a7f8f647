"""Achieved fraction of the roofline, as one generated report.

    python -m tips_b200.bench.roofline_report --kernels kernel_bench.json [--sweep sweep_8gpu.json ...] \
        [--bench bench.json ...] [--out report.md]

Inputs are the JSON files the benchmarks of this package write (``kernel_bench --json``, ``collective_sweep
--out``, the line ``bench.py`` prints); nothing is measured here and no GPU is needed.  Every fraction is taken
against the peaks recorded inside the input (measured copy bandwidth and cuBLAS bf16 throughput of the pool's B200s,
or the stated fallback) and says which; NVLink bounds use the measured 770 GB/s peer copy per direction.

The reference has no profiling output to match (its only timing is a log line in
tips/core/message/flatbuffers_test.cc:30-44); this is the report its build plan lacks.
"""
from __future__ import annotations

import argparse
import json
import sys

LINK_GBS = 770.0


def _fmt(v, digits=3):
    if v is None:
        return "—"
    if isinstance(v, float):
        if abs(v) >= 100:
            return f"{v:,.0f}".replace(",", " ")
        return f"{v:.{digits}g}"
    return str(v)


def _shape(r):
    for k in ("shape", "elements", "batch"):
        if k in r:
            v = r[k]
            return "x".join(str(x) for x in v) if isinstance(v, (list, tuple)) else f"{k} {v}"
    if "hw" in r:
        return f"{r['hw']}x{r['hw']} {r['cin']}->{r['cout']} k{r['k']} s{r['stride']}"
    return ""


def kernel_rows(doc):
    """Rows (kernel, shape, ms, achieved, unit, fraction, library ms, speed-up) of one kernel_bench document."""
    peaks = doc.get("peaks", {})
    src = peaks.get("source", "measured")
    rows = []
    for r in doc.get("results", []):
        if "kernel" not in r:
            continue
        if r["kernel"] == "conv":
            for part in ("fwd", "dgrad", "wgrad"):
                ms = r.get(part + "_ms")
                if ms is None:
                    continue
                tf = r.get(part + "_tflops") or (r["gflop"] / ms / 1e3 if "gflop" in r else None)
                frac = tf / peaks["bf16_tflops"] if tf and peaks.get("bf16_tflops") else None
                lib = r.get(part + "_lib_ms")
                rows.append(("conv " + part, _shape(r), ms, tf, "TFLOP/s", frac, lib, lib / ms if lib else None))
            continue
        ms = r.get("ms")
        lib = next((v for k, v in r.items() if k.startswith("library_ms")), None)
        if "tflops" in r:
            ach, unit = r["tflops"], "TFLOP/s"
            frac = ach / peaks["bf16_tflops"] if peaks.get("bf16_tflops") else None
        elif "gbs" in r:
            ach, unit = r["gbs"], "GB/s"
            frac = ach / peaks["hbm_gbs"] if peaks.get("hbm_gbs") else None
        else:
            ach, unit, frac = None, "", None
        rows.append((r["kernel"], _shape(r), ms, ach, unit, frac, lib, lib / ms if lib and ms else None))
    return rows, src, peaks


def sweep_rows(doc):
    """Rows (dtype, bytes, allreduce bus GB/s, fraction of its NVLS bound, NCCL, allgather, NCCL, broadcast, NCCL)."""
    n = doc.get("ranks", 0)
    rows = []
    for r in doc.get("rows", []):
        b = r["bytes"]
        ar_ms = r.get("allreduce_inplace_ms")
        bound = (b * (n + 1) / n / (LINK_GBS * 1e6)) / ar_ms if ar_ms and n else None
        rows.append((r.get("dtype"), b, r.get("allreduce_inplace_busbw"), bound, r.get("nccl_allreduce_busbw"),
                     r.get("allgather_busbw"), r.get("nccl_allgather_busbw"),
                     r.get("broadcast_gbs"), r.get("nccl_broadcast_gbs")))
    return n, rows


def bench_rows(doc):
    """Rows (workload, GPUs, value, unit, ms/step, end to end, floor, ratio) of one bench.py line."""
    rows = []
    floors = doc.get("floor", {})
    ratios = doc.get("vs_floor", {})

    def one(name, d, key):
        f = floors.get(key, {})
        rows.append((name, doc.get("n_gpus"), d.get("value"), d.get("unit"), d.get("ms_per_step"),
                     (d.get("e2e") or {}).get("value"), f.get("value"), ratios.get(key)))
    one(doc.get("metric", "step"), doc, "resnet50")
    if "ps" in doc:
        one(doc["ps"].get("metric", "ps"), doc["ps"], "ps")
    return rows


def render(kernel_docs, sweep_docs, bench_docs) -> str:
    out = ["# Achieved fraction of the roofline", ""]
    for doc in kernel_docs:
        rows, src, peaks = kernel_rows(doc)
        out += [f"## Kernels (one GPU; peaks {src}: copy {_fmt(float(peaks.get('hbm_gbs', 0)))} GB/s, "
                f"bf16 GEMM {_fmt(float(peaks.get('bf16_tflops', 0)))} TFLOP/s)", "",
                f"| kernel | shape | ms | achieved | of {src} peak | library ms | vs library |", "|---|---|---|---|---|---|---|"]
        for k, shape, ms, ach, unit, frac, lib, sp in rows:
            out.append(f"| {k} | {shape} | {_fmt(ms)} | {_fmt(ach)} {unit} | {_fmt(frac, 2)} | {_fmt(lib)} | "
                       f"{_fmt(sp, 3) + 'x' if sp else '—'} |")
        out.append("")
    for doc in sweep_docs:
        n, rows = sweep_rows(doc)
        out += [f"## Collectives on {n} GPUs (bus GB/s; bound = time against bytes x (N+1)/N over {LINK_GBS:.0f} GB/s)", "",
                "| dtype | bytes | allreduce | of bound | NCCL | allgather | NCCL | broadcast | NCCL |",
                "|---|---|---|---|---|---|---|---|---|"]
        for dt, b, ar, bound, arn, ag, agn, bc, bcn in rows:
            out.append(f"| {dt} | {b} | {_fmt(ar)} | {_fmt(bound, 2)} | {_fmt(arn)} | {_fmt(ag)} | {_fmt(agn)} | "
                       f"{_fmt(bc)} | {_fmt(bcn)} |")
        out.append("")
    if bench_docs:
        out += ["## Training steps (device-timed, max over ranks)", "",
                "| workload | GPUs | value | ms/step | end to end | library floor | vs floor |", "|---|---|---|---|---|---|---|"]
        for doc in bench_docs:
            for name, n, v, unit, ms, e2e, floor, ratio in bench_rows(doc):
                out.append(f"| {name} | {n} | {_fmt(v)} {unit or ''} | {_fmt(ms)} | {_fmt(e2e)} | {_fmt(floor)} | "
                           f"{_fmt(ratio, 3) + 'x' if ratio else '—'} |")
        out.append("")
    return "\n".join(out)


def _load(path):
    text = open(path).read().strip()
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        return json.loads(text.splitlines()[-1])  # bench.py prints log lines before its JSON line on some runs


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels", nargs="*", default=[])
    ap.add_argument("--sweep", nargs="*", default=[])
    ap.add_argument("--bench", nargs="*", default=[])
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    text = render([_load(p) for p in a.kernels], [_load(p) for p in a.sweep], [_load(p) for p in a.bench])
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
    else:
        print(text)


if __name__ == "__main__":
    main(sys.argv[1:])
