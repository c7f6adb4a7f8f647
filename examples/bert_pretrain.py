"""Data-parallel masked-language-model pre-training of a BERT-large-shaped encoder on synthetic tokens: tcgen05 GEMMs
with fused bias / GELU epilogues, layer norms with the residual add inside, fused AdamW on flat buffers, gradient
buckets reduced over NVLink while the backward pass is still running.  With --fused-update the optimizer step runs
inside the allreduce kernel and every rank keeps 1/N of the AdamW state.  Needs CUDA.

    python -m torch.distributed.run --nproc-per-node 8 examples/bert_pretrain.py --steps 50 --fused-update
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.models.bert import bert_large, synthetic_mlm_batch  # noqa: E402
from tips_b200.ops.optim import FusedAdamW  # noqa: E402
from tips_b200.utils.checkpoint import save_checkpoint  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=32, help="sequences per GPU")
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--warmup-steps", type=int, default=10)
    ap.add_argument("--fused-update", action="store_true")
    ap.add_argument("--checkpoint", default="", help="file that rank 0 writes at the end")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("this example needs a CUDA device")
    tips.init()
    rank, size = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234)
    model = bert_large(device=dev, layers=a.layers, max_seq=a.seq).train()
    opt = tips.DistributedOptimizer(FusedAdamW(model.parameters(), lr=a.lr, weight_decay=0.01),
                                    fused_update=a.fused_update if size > 1 else None)
    tips.broadcast_parameters(model.state_dict(), root_rank=0, optimizer=opt)
    # three host batches in pinned memory, copied while the previous step computes
    host = [tuple(t.pin_memory() for t in synthetic_mlm_batch(a.batch, a.seq, 30522, seed=31 * rank + i)) for i in range(3)]
    copy_stream = torch.cuda.Stream()
    nxt = [t.to(dev, non_blocking=True) for t in host[0]]
    t0 = None
    for step in range(a.steps):
        if step == 5:
            torch.cuda.synchronize()
            t0 = time.time()
        ids, pos, labels = nxt
        with torch.cuda.stream(copy_stream):
            nxt = [t.to(dev, non_blocking=True) for t in host[(step + 1) % 3]]
        for g in opt.param_groups:                      # linear warm-up; the fused kernels read lr every step
            g["lr"] = a.lr * min(1.0, (step + 1) / max(1, a.warmup_steps))
        loss = model.loss(ids, pos, labels)
        loss.backward()
        opt.step()
        torch.cuda.current_stream().wait_stream(copy_stream)
        if step % 10 == 0 or step == a.steps - 1:
            avg = tips.metric_average(loss.detach().float(), "loss")
            if rank == 0:
                print(f"step {step}: loss {avg:.4f} lr {opt.param_groups[0]['lr']:.2e}", flush=True)
    torch.cuda.synchronize()
    if t0 is not None and a.steps > 5 and rank == 0:
        dt = (time.time() - t0) / (a.steps - 5)
        print(f"{a.batch * a.seq * size / dt:,.0f} tokens/s on {size} GPU(s), {dt * 1e3:.1f} ms/step", flush=True)
    if a.checkpoint:
        save_checkpoint(a.checkpoint, model, opt, extra={"steps": a.steps})
    tips.shutdown()


if __name__ == "__main__":
    main()
