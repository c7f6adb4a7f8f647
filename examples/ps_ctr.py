"""Parameter-server mode: a CTR model whose sparse embedding tables are sharded over the GPUs
(pull = fused lookup over NVLink, push = scatter-reduce + server-side Adagrad) while the MLP is data-parallel.

    python -m torch.distributed.run --nproc-per-node 2 examples/ps_ctr.py --steps 50
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.models.ctr import CtrTrainer, synthetic_ctr_batch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--rows", type=int, default=1_000_000)
    a = ap.parse_args()
    tips.init()
    dev = torch.device("cuda", torch.cuda.current_device())
    trainer = CtrTrainer(rows_per_table=a.rows, device=dev, expected_batch=a.batch)
    for step in range(a.steps):
        ids, dense, labels = [t.to(dev) for t in synthetic_ctr_batch(a.batch, 26, a.rows, 13, seed=step * tips.size() + tips.rank())]
        loss = trainer.train_step(ids, dense, labels)
        if step % 10 == 0:
            avg = tips.metric_average(loss.item(), name="loss")
            if tips.rank() == 0:
                print(f"step {step} loss {avg:.4f}")
    trainer.check()
    tips.shutdown()


if __name__ == "__main__":
    main()
