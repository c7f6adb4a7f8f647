"""Data-parallel ResNet-50 training on synthetic ImageNet-shaped data: the reference's headline workload
(a TensorFlow ResNet-50 under its DistributedOptimizer, README.md:12) on this framework's own kernels.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        examples/resnet50_data_parallel.py --steps 100 --fused-update

Each rank owns one GPU.  Inputs come from pinned host memory through a side stream; gradients are packed into
64 MB buckets and reduced in place over NVLink while backward runs; with ``--fused-update`` the SGD step runs
inside the reduction kernel and every rank keeps 1/N of the optimizer state.  ``--tiny --cpu`` runs a small
network on the CPU (one process) to try the script without a GPU.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.models import resnet50 as R  # noqa: E402
from tips_b200.ops.optim import FusedSGD  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=256, help="images per GPU")
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--fused-update", action="store_true", help="optimizer step inside the gradient allreduce")
    ap.add_argument("--tiny", action="store_true", help="one block per stage, 64x64 images")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--checkpoint", default="", help="write a checkpoint here at the end (rank 0)")
    a = ap.parse_args()
    use_cuda = torch.cuda.is_available() and not a.cpu
    tips.init(device=use_cuda)
    rank, size = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    torch.manual_seed(1234)
    side = 64 if a.tiny else 224
    classes = 10 if a.tiny else 1000
    dtype = torch.bfloat16 if use_cuda else torch.float32
    if a.tiny:
        model = R.tiny_resnet(classes, dtype=dtype, device=dev, width=64 if use_cuda else 16)
    else:
        model = R.resnet50(classes, dtype=dtype, device=dev)
    model.train()
    opt = tips.DistributedOptimizer(FusedSGD(model.parameters(), lr=a.lr, momentum=0.9, weight_decay=1e-4),
                                    named_parameters=model.named_parameters(), fused_update=a.fused_update)
    tips.broadcast_parameters(model.state_dict(), root_rank=0, optimizer=opt)

    g = torch.Generator().manual_seed(100 + rank)
    host = []
    for _ in range(3):  # a few pinned batches, cycled
        x = torch.randn(a.batch, 3, side, side, generator=g).to(dtype).contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, classes, (a.batch,), generator=g)
        host.append((x.pin_memory(), y.pin_memory()) if use_cuda else (x, y))
    copy_stream = torch.cuda.Stream() if use_cuda else None

    def fetch(i):
        x, y = host[i % len(host)]
        if not use_cuda:
            return x, y, None
        with torch.cuda.stream(copy_stream):
            xd, yd = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return xd, yd, ev

    nxt = fetch(0)
    t0 = time.time()
    for step in range(a.steps):
        x, y, ev = nxt
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            x.record_stream(torch.cuda.current_stream())
            y.record_stream(torch.cuda.current_stream())
        nxt = fetch(step + 1)
        loss = model.loss(x, y)
        loss.backward()
        opt.step()
        if step % 10 == 0 or step == a.steps - 1:
            avg = tips.metric_average(loss.detach().float(), name="loss")
            if rank == 0:
                print(f"step {step:4d}  loss {float(avg):.4f}  "
                      f"{(step + 1) * a.batch * size / (time.time() - t0):9.0f} images/s", flush=True)
    if a.checkpoint:
        tips.save_checkpoint(a.checkpoint, model, opt, extra={"step": a.steps})
    tips.barrier()
    tips.shutdown()


if __name__ == "__main__":
    main()
