"""Single-GPU kernel microbenchmarks with roofline fractions against MEASURED_PEAKS.json.

    python -m tips_b200.bench.kernel_bench [--only gemm,bn,ln,optim,ps,conv] [--json out.json]

Timing: CUDA events on the launching stream, >= 3 warm-up launches, inputs larger than L2 (or an L2 flush
between launches for the small ones); every figure is "of measured" copy bandwidth / cuBLAS bf16 throughput.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters=20, warmup=3, flush=False):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not flush:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    for _ in range(iters):
        flush_l2()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bench_gemm(out):
    from tips_b200.ops.linear import gemm_status, gemm_tn
    pk = peaks()
    shapes = [(8192, 512, 1680), (8192, 256, 512), (16384, 1024, 1024), (16384, 4096, 1024), (16384, 1024, 4096),
              (16384, 3072, 1024), (8192, 8192, 8192), (4096, 4096, 4096)]
    for m, n, k in shapes:
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
        bias = torch.randn(n, device="cuda").to(torch.bfloat16)
        ms = time_ms(lambda: gemm_tn(a, b, bias, "relu"), flush=(m * k + n * k) * 2 < (200 << 20))
        ms_lib = time_ms(lambda: torch.relu(torch.nn.functional.linear(a, b, bias)),
                         flush=(m * k + n * k) * 2 < (200 << 20))
        assert gemm_status() == 0
        tf = 2.0 * m * n * k / ms / 1e9
        out.append({"kernel": "gemm_tcgen05+bias+relu", "shape": [m, n, k], "ms": ms, "tflops": tf,
                    "frac_of_" + pk["source"] + "_cublas": tf / pk["bf16_tflops"],
                    "library_ms(linear+relu)": ms_lib, "speedup_vs_library": ms_lib / ms})
        print(out[-1], flush=True)


def bench_bn(out):
    from tips_b200.ops.norm import BatchNorm2d
    pk = peaks()
    for (n, c, h, w) in [(256, 64, 112, 112), (256, 256, 56, 56), (256, 512, 28, 28), (256, 2048, 7, 7)]:
        x = torch.randn(n, c, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        r = torch.randn_like(x)
        bn = BatchNorm2d(c, relu=True).cuda()
        ref = torch.nn.BatchNorm2d(c).cuda().to(torch.bfloat16)
        nbytes = x.numel() * 2
        flush = nbytes * 4 < (256 << 20)
        ms = time_ms(lambda: bn(x, residual=r), flush=flush)
        ms_lib = time_ms(lambda: torch.relu(ref(x) + r), flush=flush)
        gbs = nbytes * (4 + 1 / 16) / ms / 1e6  # read x twice (stats + apply), read residual, write y and the sign bits
        out.append({"kernel": "bn_fwd_train+residual+relu", "shape": [n, c, h, w], "ms": ms, "gbs": gbs,
                    "frac_of_" + pk["source"] + "_copy": gbs / pk["hbm_gbs"], "library_ms": ms_lib,
                    "speedup_vs_library": ms_lib / ms})
        print(out[-1], flush=True)
        xg = x.clone().requires_grad_()
        y = bn(xg, residual=r.clone().requires_grad_())
        dy = torch.randn_like(y)
        ms = time_ms(lambda: torch.autograd.grad(y, xg, dy, retain_graph=True), flush=flush)
        gbs = nbytes * (6 + 2 / 16) / ms / 1e6  # (dy, x, sign bits) twice (reduce + apply), write dx and dres
        out.append({"kernel": "bn_bwd+relu_mask+dresidual", "shape": [n, c, h, w], "ms": ms, "gbs": gbs,
                    "frac_of_" + pk["source"] + "_copy": gbs / pk["hbm_gbs"]})
        print(out[-1], flush=True)


def bench_ln(out):
    from tips_b200.ops.norm import LayerNorm
    pk = peaks()
    rows, cols = 32 * 512, 1024
    x = torch.randn(rows * 8, cols, device="cuda").to(torch.bfloat16)
    ln = LayerNorm(cols).cuda()
    ms = time_ms(lambda: ln(x))
    ref = torch.nn.LayerNorm(cols).cuda().to(torch.bfloat16)
    ms_lib = time_ms(lambda: ref(x))
    gbs = x.numel() * 2 * 2 / ms / 1e6
    out.append({"kernel": "layernorm_fwd", "shape": [rows * 8, cols], "ms": ms, "gbs": gbs,
                "frac_of_" + pk["source"] + "_copy": gbs / pk["hbm_gbs"], "library_ms": ms_lib})
    print(out[-1], flush=True)


def bench_optim(out):
    from tips_b200.ops.optim import FusedAdamW, FusedSGD
    pk = peaks()
    n = 128 << 20
    for name, make, bpe in [("fused_sgd_momentum(bf16 param, fp32 master)", lambda p: FusedSGD([p], lr=0.1, momentum=0.9, weight_decay=1e-4), 2 + 4 + 4 + 4 + 4 + 2),
                            ("fused_adamw(bf16 param, fp32 master)", lambda p: FusedAdamW([p], lr=1e-3), 2 + 4 * 6 + 2)]:
        p = torch.nn.Parameter(torch.randn(n, device="cuda").to(torch.bfloat16))
        opt = make(p)
        fs = opt.build()[0]
        p.grad = torch.randn_like(p)
        opt.step()

        def step():
            fs.grads_packed = True
            fs.steps += 1
            opt._update(fs, 1.0)

        ms = time_ms(step)
        gbs = n * bpe / ms / 1e6
        out.append({"kernel": name, "elements": n, "ms": ms, "gbs": gbs,
                    "frac_of_" + pk["source"] + "_copy": gbs / pk["hbm_gbs"]})
        print(out[-1], flush=True)
        del opt, p, fs


def bench_ps(out):
    from tips_b200.models.ctr import synthetic_ctr_batch
    from tips_b200.ps.gpu import ShardedEmbedding
    pk = peaks()
    rows, fields, dim, batch = 2_000_000, 26, 64, 8192
    t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.05, expected_batch=batch)
    ids, _, _ = synthetic_ctr_batch(batch, fields, rows, 13, seed=3)
    ids = ids.cuda()
    outbuf = torch.empty(batch, fields * dim, dtype=torch.bfloat16, device="cuda")
    ms = time_ms(lambda: t.pull(ids, out=outbuf), flush=True)
    gbs = batch * fields * dim * (4 + 2) / ms / 1e6
    out.append({"kernel": "ps_pull_lookup(fp32 rows -> bf16)", "batch": batch, "ms": ms, "gbs": gbs,
                "frac_of_" + pk["source"] + "_copy": gbs / pk["hbm_gbs"]})
    print(out[-1], flush=True)
    grads = torch.randn(batch, fields * dim, device="cuda").to(torch.bfloat16)
    ms = time_ms(lambda: t.push(ids, grads), flush=True)
    out.append({"kernel": "ps_push(scatter-reduce + adagrad)", "batch": batch, "ms": ms,
                "unique_rows_per_push": t.check() // 24})
    print(out[-1], flush=True)


# The distinct convolutions of ResNet-50 v1.5 at 224x224 (stem excluded): h = w of the input, cin, cout, k, stride.
RESNET50_CONVS = [
    (56, 64, 64, 1, 1), (56, 64, 64, 3, 1), (56, 64, 256, 1, 1), (56, 256, 64, 1, 1),
    (56, 256, 128, 1, 1), (56, 128, 128, 3, 2), (28, 128, 512, 1, 1), (56, 256, 512, 1, 2),
    (28, 512, 128, 1, 1), (28, 128, 128, 3, 1),
    (28, 512, 256, 1, 1), (28, 256, 256, 3, 2), (14, 256, 1024, 1, 1), (28, 512, 1024, 1, 2),
    (14, 1024, 256, 1, 1), (14, 256, 256, 3, 1),
    (14, 1024, 512, 1, 1), (14, 512, 512, 3, 2), (7, 512, 2048, 1, 1), (14, 1024, 2048, 1, 2),
    (7, 2048, 512, 1, 1), (7, 512, 512, 3, 1),
]


def bench_conv(out, batch=256):
    """Forward / data-gradient / weight-gradient time of every ResNet-50 convolution shape: the tcgen05 kernels
    against the library convolution on the same channels-last bf16 tensors."""
    import torch.nn.functional as F
    from tips_b200.ops import conv as C
    pk = peaks()
    for (hw, cin, cout, k, stride) in RESNET50_CONVS:
        pad = k // 2
        x = torch.randn(batch, cin, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        w = (torch.randn(cout, k, k, cin, device="cuda") * 0.05).to(torch.bfloat16)
        w_lib = w.permute(0, 3, 1, 2)  # OIHW view with channels-last strides
        _, y = C.conv2d_forward(x, w, stride, pad)
        dy = torch.randn_like(y)
        ho = y.shape[2]
        flops = 2.0 * batch * ho * ho * cout * cin * k * k
        row = {"kernel": "conv", "hw": hw, "cin": cin, "cout": cout, "k": k, "stride": stride, "gflop": flops / 1e9}
        ours = {
            "fwd": lambda: C.conv2d_forward(x, w, stride, pad),
            "dgrad": lambda: C.conv2d_dgrad(dy, w, tuple(x.shape), stride, pad),
            "wgrad": lambda: C.conv2d_wgrad(x, dy, tuple(w.shape), stride, pad),
        }
        lib = {
            "fwd": lambda: F.conv2d(x, w_lib, stride=stride, padding=pad),
            "dgrad": lambda: torch.ops.aten.convolution_backward(
                dy, x, w_lib, None, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1, [True, False, False]),
            "wgrad": lambda: torch.ops.aten.convolution_backward(
                dy, x, w_lib, None, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1, [False, True, False]),
        }
        for name in ("fwd", "dgrad", "wgrad"):
            ms = time_ms(ours[name], iters=10, flush=True)
            ms_lib = time_ms(lib[name], iters=10, flush=True)
            row[name + "_ms"] = round(ms, 4)
            row[name + "_lib_ms"] = round(ms_lib, 4)
            row[name + "_tflops"] = round(flops / ms / 1e9, 1)
            row[name + "_speedup_vs_lib"] = round(ms_lib / ms, 3)
        row["fwd_frac_of_" + pk["source"] + "_gemm"] = round(row["fwd_tflops"] / pk["bf16_tflops"], 3)
        out.append(row)
        print(row, flush=True)
    tot = {n: sum(r[n + "_ms"] for r in out if r.get("kernel") == "conv") for n in ("fwd", "dgrad", "wgrad")}
    tot_lib = {n: sum(r[n + "_lib_ms"] for r in out if r.get("kernel") == "conv") for n in ("fwd", "dgrad", "wgrad")}
    print({"conv_total_ms": tot, "conv_total_lib_ms": tot_lib}, flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="gemm,bn,ln,optim,ps")
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    sys.path.insert(0, REPO)
    out = []
    table = {"gemm": bench_gemm, "bn": bench_bn, "ln": bench_ln, "optim": bench_optim, "ps": bench_ps, "conv": bench_conv}
    for k in a.only.split(","):
        table[k](out)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"peaks": peaks(), "results": out}, f, indent=1)


if __name__ == "__main__":
    main(sys.argv[1:])
