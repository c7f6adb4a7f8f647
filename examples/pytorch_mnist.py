"""Data-parallel training of the MNIST-shaped CNN, the counterpart of the reference's
examples/tensorflow2_keras_mnist.py: DistributedOptimizer, broadcast of the initial state, metric
averaging, learning-rate warm-up, rank-0 checkpoints.  Synthetic data (28x28x1 uniform, labels 0..9).

    python -m torch.distributed.run --nproc-per-node 2 examples/pytorch_mnist.py --epochs 3
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200 import callbacks as cb  # noqa: E402
from tips_b200.models.mnist_cnn import MnistCNN, synthetic_batch  # noqa: E402
from tips_b200.trainer import fit  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--steps", type=int, default=0, help="steps per epoch (default 500 // size)")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--checkpoint-dir", default="")
    a = ap.parse_args()
    use_cuda = torch.cuda.is_available() and not a.cpu
    tips.init(device=use_cuda)
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    torch.manual_seed(1 + tips.rank())
    model = MnistCNN(dropout=True).to(device)
    scaled_lr = 0.001 * tips.size()  # the reference scales Adam's rate by the number of workers
    opt = tips.DistributedOptimizer(torch.optim.Adam(model.parameters(), lr=scaled_lr),
                                    named_parameters=model.named_parameters())
    steps = a.steps or max(1, 500 // tips.size())
    callbacks = [cb.BroadcastGlobalVariablesCallback(0), cb.MetricAverageCallback(),
                 cb.LearningRateWarmupCallback(initial_lr=scaled_lr, warmup_epochs=min(3, a.epochs), verbose=1)]
    if a.checkpoint_dir:
        callbacks.append(cb.BestModelCheckpoint(os.path.join(a.checkpoint_dir, "checkpoint-{epoch}.pt"), monitor="loss"))

    def batches(epoch, step):
        return synthetic_batch(a.batch, seed=(epoch * steps + step) * tips.size() + tips.rank(), device=device)

    def accuracy(out, y):
        return {"accuracy": (out.argmax(1) == y).float().mean()}

    history = fit(model, opt, torch.nn.functional.cross_entropy, batches, a.epochs, steps, callbacks,
                  metrics=accuracy, verbose=1 if tips.rank() == 0 else 0)
    if tips.rank() == 0:
        print("final", history[-1])
    tips.shutdown()


if __name__ == "__main__":
    main()
