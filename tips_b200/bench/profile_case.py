"""Small single-kernel cases for profiler captures: each runs ONE kernel a handful of times on inputs a
little larger than L2, holds well under a GB on the device and exits by itself in seconds.

    python -m tips_b200.bench.profile_case {bn_fwd,bn_bwd,gemm,gemm_persistent,ln,sgd,ps_pull,ps_push,conv1x1,conv3x3,conv_dgrad,conv_wgrad,adam,ln_bwd,bias_act_bwd,softmax_xent}
"""
from __future__ import annotations

import sys

import torch


def main(argv=None):
    case = (argv or sys.argv[1:])[0]
    dev = torch.device("cuda", 0)
    reps = 3
    if case in ("bn_fwd", "bn_bwd"):
        from tips_b200.ops.norm import BatchNorm2d
        x = torch.randn(128, 256, 56, 56, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        r = torch.randn_like(x)
        bn = BatchNorm2d(256, relu=True).to(dev)
        if case == "bn_fwd":
            for _ in range(reps):
                bn(x, residual=r)
        else:
            xg = x.requires_grad_()
            y = bn(xg, residual=r)
            dy = torch.randn_like(y)
            for _ in range(reps):
                torch.autograd.grad(y, xg, dy, retain_graph=True)
    elif case in ("gemm", "gemm_persistent"):
        from tips_b200.ops.linear import gemm_tn
        k = 4096 if case == "gemm" else 1024  # the short-K shape takes the persistent double-buffered variant
        a = torch.randn(16384, k, device=dev).to(torch.bfloat16)
        b = torch.randn(4096, k, device=dev).to(torch.bfloat16)
        bias = torch.randn(4096, device=dev).to(torch.bfloat16)
        for _ in range(reps):
            gemm_tn(a, b, bias, "relu")
    elif case in ("conv1x1", "conv3x3", "conv_dgrad", "conv_wgrad"):
        from tips_b200.ops import conv as C
        k, cin, cout = (1, 64, 256) if case == "conv1x1" else (3, 64, 64)
        x = torch.randn(128, cin, 56, 56, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        w = (torch.randn(cout, k, k, cin, device=dev) * 0.05).to(torch.bfloat16)
        stats = torch.zeros(2, cout, dtype=torch.float32, device=dev)
        _, y = C.conv2d_forward(x, w, 1, k // 2, stats)
        dy = torch.randn_like(y)
        for _ in range(reps):
            if case == "conv_dgrad":
                C.conv2d_dgrad(dy, w, tuple(x.shape), 1, k // 2)
            elif case == "conv_wgrad":
                C.conv2d_wgrad(x, dy, tuple(w.shape), 1, k // 2)
            else:
                C.conv2d_forward(x, w, 1, k // 2, stats)
    elif case == "ln":
        from tips_b200.ops.norm import LayerNorm
        x = torch.randn(131072, 1024, device=dev).to(torch.bfloat16)
        ln = LayerNorm(1024).to(dev)
        for _ in range(reps):
            ln(x)
    elif case == "sgd":
        from tips_b200.ops.optim import FusedSGD
        p = torch.nn.Parameter(torch.randn(64 << 20, device=dev).to(torch.bfloat16))
        opt = FusedSGD([p], lr=0.1, momentum=0.9, weight_decay=1e-4)
        for _ in range(reps + 1):
            p.grad = torch.randn_like(p)
            opt.step()
    elif case == "adam":
        from tips_b200.ops.optim import FusedAdamW
        p = torch.nn.Parameter(torch.randn(64 << 20, device=dev).to(torch.bfloat16))
        opt = FusedAdamW([p], lr=1e-3)
        for _ in range(reps + 1):
            p.grad = torch.randn_like(p)
            opt.step()
    elif case == "ln_bwd":
        from tips_b200.ops.norm import LayerNorm
        x = torch.randn(131072, 1024, device=dev).to(torch.bfloat16).requires_grad_()
        ln = LayerNorm(1024).to(dev)
        y = ln(x)
        dy = torch.randn_like(y)
        for _ in range(reps):
            torch.autograd.grad(y, x, dy, retain_graph=True)
    elif case == "bias_act_bwd":
        from tips_b200.ops.linear import Linear
        lin = Linear(1024, 4096, act="gelu").to(dev).to(torch.bfloat16)
        x = torch.randn(16384, 1024, device=dev).to(torch.bfloat16).requires_grad_()
        y = lin(x)
        dy = torch.randn_like(y)
        for _ in range(reps):
            torch.autograd.grad(y, x, dy, retain_graph=True)
    elif case == "softmax_xent":
        from tips_b200.ops.pointwise import softmax_cross_entropy
        logits = torch.randn(16384, 30528, device=dev).to(torch.bfloat16).requires_grad_()
        labels = torch.randint(0, 30522, (16384,), device=dev)
        for _ in range(reps):
            softmax_cross_entropy(logits, labels).backward()
    elif case in ("ps_pull", "ps_push"):
        from tips_b200.models.ctr import synthetic_ctr_batch
        from tips_b200.ps.gpu import ShardedEmbedding
        t = ShardedEmbedding(26, 200_000, 64, optimizer="adagrad", lr=0.05, init_scale=0.05, expected_batch=8192)
        ids = synthetic_ctr_batch(8192, 26, 200_000, 13, seed=1)[0].to(dev)
        out = torch.empty(8192, 26 * 64, dtype=torch.bfloat16, device=dev)
        g = torch.randn_like(out)
        for _ in range(reps):
            if case == "ps_pull":
                t.pull(ids, out=out)
            else:
                t.push(ids, g)
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    print("done", case)


if __name__ == "__main__":
    main()
