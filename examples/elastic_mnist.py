"""Training that survives a failed step: `elastic.State` keeps the last committed model, optimizer and progress
in host memory, `elastic.run` catches a recoverable collective failure, resets the collectives on every rank, rolls
back to the commit and calls the training function again.  The failure here is made on the host: one rank's request
to the coordinator is dropped once, so the step times out everywhere.  The reference ships the callbacks of this
flow (tips/_keras/elastic.py:17-86) without a state object or a driver.

    python -m torch.distributed.run --nproc-per-node 2 examples/elastic_mnist.py --cpu
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200 import _lib, elastic  # noqa: E402
from tips_b200.models.mnist_cnn import MnistCNN, synthetic_batch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--fail-at", type=int, default=5, help="step whose allreduce is made to time out once (-1: never)")
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    use_cuda = torch.cuda.is_available() and not a.cpu
    tips.init(device=use_cuda)
    tips.set_config(collective_timeout_s=4.0)             # a stalled collective becomes an error after 4 s
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    torch.manual_seed(3)
    model = MnistCNN().to(device)
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9))
    state = elastic.State(model, opt)
    state.sync()
    pending = {"failure": a.fail_at >= 0 and tips.size() > 1, "retries": 0}

    @elastic.run
    def train(state):
        for step in range(state.batch, a.steps):
            if step == a.fail_at and pending["failure"] and tips.rank() == tips.size() - 1:
                _lib.core().tips_inject_drop_requests(0, 1)          # this rank's next request never arrives
            if step == a.fail_at:
                pending["failure"] = False
            x, y = synthetic_batch(a.batch, seed=step * tips.size() + tips.rank(), device=device)
            loss = torch.nn.functional.cross_entropy(state.model(x), y)
            loss.backward()
            try:
                state.optimizer.step()
            except tips.TipsError:
                pending["retries"] += 1
                raise                                                # elastic.run resets, restores and calls train again
            state.optimizer.zero_grad()
            state.batch = step + 1
            state.commit()
        return float(loss.detach())

    last = train(state)
    w = tips.allgather_object(next(model.parameters()).detach().cpu())
    assert all(torch.allclose(w[0], other, atol=1e-6) for other in w), "the replicas diverged"
    if tips.rank() == 0:
        print(f"finished {a.steps} steps, loss {last:.4f}, failed steps retried: {pending['retries']}, "
              f"commits {state.commits}", flush=True)
    tips.shutdown()


if __name__ == "__main__":
    main()
