"""Parameter-server mode on CPU ranks: a small CTR model whose embedding rows live in the host parameter server
(every rank serves a share of the rows and trains on its own batches; pull in the forward pass, push with
server-side Adagrad in the backward pass) while the dense layers are data-parallel through DistributedOptimizer.
The GPU version of the same model is examples/ps_ctr.py.

    python -m tips_b200.launch -np 2 examples/host_ps_ctr.py --steps 30
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402
from tips_b200.models.ctr import synthetic_ctr_batch  # noqa: E402
from tips_b200.ps.host import HostEmbedding  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--rows", type=int, default=100_000)
    ap.add_argument("--fields", type=int, default=8)
    ap.add_argument("--dim", type=int, default=16)
    a = ap.parse_args()
    tips.init(device=False)
    rank, size = tips.rank(), tips.size()
    emb = HostEmbedding("ctr", a.fields, a.dim, optimizer="adagrad", lr=0.05)
    torch.manual_seed(0)
    mlp = torch.nn.Sequential(torch.nn.Linear(a.fields * a.dim + 13, 64), torch.nn.ReLU(), torch.nn.Linear(64, 1))
    opt = tips.DistributedOptimizer(torch.optim.Adam(mlp.parameters(), lr=1e-3))
    tips.broadcast_parameters(mlp.state_dict(), root_rank=0)
    batches = [synthetic_ctr_batch(a.batch, a.fields, a.rows, 13, seed=s * size + rank) for s in range(a.steps)]
    emb.prefetch(batches[0][0])
    for step, (ids, dense, labels) in enumerate(batches):
        x = torch.cat([emb(ids), dense], dim=1)               # rows prefetched during the previous step
        if step + 1 < a.steps:
            emb.prefetch(batches[step + 1][0])
        loss = torch.nn.functional.binary_cross_entropy_with_logits(mlp(x).squeeze(1), labels.float())
        loss.backward()                                        # pushes the embedding gradients to their servers
        opt.step()
        opt.zero_grad()
        if step % 10 == 0 or step == a.steps - 1:
            avg = tips.metric_average(loss.item(), name="loss")
            if rank == 0:
                print(f"step {step} loss {avg:.4f}", flush=True)
    emb.wait()
    tips.barrier()
    print(f"rank {rank}: serves {emb.table.local_size()} rows, {emb.table.counters()}", flush=True)
    emb.close()
    tips.shutdown()


if __name__ == "__main__":
    main()
