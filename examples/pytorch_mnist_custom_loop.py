"""A hand-written training loop, the counterpart of the reference's examples/tensorflow_mnist.py (a custom
`train_step` around a DistributedGradientTape): the gradients of an ordinary backward pass are averaged over the
ranks by a `DistributedGradientTape`, a stock optimizer applies them, metrics are averaged with `metric_average`.
Synthetic data (28x28x1 uniform, labels 0..9).

    python -m torch.distributed.run --nproc-per-node 2 examples/pytorch_mnist_custom_loop.py --steps 200
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.models.mnist_cnn import MnistCNN, synthetic_batch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--compression", default="none", choices=["none", "fp16", "bf16"])
    a = ap.parse_args()
    use_cuda = torch.cuda.is_available() and not a.cpu
    tips.init(device=use_cuda)
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    torch.manual_seed(1 + tips.rank())
    model = MnistCNN().to(device)
    optimizer = torch.optim.Adam(model.parameters(), lr=1e-3)
    # every rank starts from rank 0's weights and optimizer state
    tips.broadcast_global_variables(model, 0, optimizer)
    compression = getattr(tips.Compression, a.compression)

    def train_step(images, labels):
        with tips.DistributedGradientTape(compression=compression) as tape:
            logits = model(images)
            loss = torch.nn.functional.cross_entropy(logits, labels)
        params = list(model.parameters())
        for p, g in zip(params, tape.gradient(loss, params)):      # gradients averaged over the ranks
            p.grad = g
        optimizer.step()
        return loss.detach(), (logits.argmax(1) == labels).float().mean()

    for step in range(a.steps):
        x, y = synthetic_batch(a.batch, seed=step * tips.size() + tips.rank(), device=device)
        loss, acc = train_step(x, y)
        if step % 50 == 0 or step == a.steps - 1:
            loss = tips.metric_average(loss, "loss")
            acc = tips.metric_average(acc, "accuracy")
            if tips.rank() == 0:
                print(f"step {step}: loss {loss:.4f} accuracy {acc:.3f}", flush=True)
    # the replicas never diverge: same averaged gradients, same optimizer
    w = tips.allgather_object(next(model.parameters()).detach().cpu())
    assert all(torch.allclose(w[0], other, atol=1e-6) for other in w), "the replicas diverged"
    if tips.rank() == 0:
        print("replicas identical on", tips.size(), "ranks")
    tips.shutdown()


if __name__ == "__main__":
    main()
