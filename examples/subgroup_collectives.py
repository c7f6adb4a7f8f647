"""Sub-groups of ranks: the ranks split into an even and an odd group, each reduces, gathers and broadcasts among
its own members only, at the same time as the other (the reference's MpiGroup, tips/core/mpi/mpi_group.h:15-96,
which its parameter-server mode uses for the server ranks).  CUDA tensors go through the device kernels of the
group (peer loads and stores over NVLink), CPU tensors through the control plane.

    python -m torch.distributed.run --nproc-per-node 4 examples/subgroup_collectives.py
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tips_b200 as tips  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    use_cuda = torch.cuda.is_available() and not a.cpu
    tips.init(device=use_cuda)
    rank, size = tips.rank(), tips.size()
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    # creating a group is a collective over ALL ranks, members or not, in the same order everywhere
    even = tips.Group(range(0, size, 2))
    odd = tips.Group(range(1, size, 2)) if size > 1 else None
    mine = even if rank % 2 == 0 else odd
    members = mine.world_ranks

    t = torch.full((1 << 16,), float(rank), device=device)
    mine.allreduce_(t)                                    # sum over my group only
    assert float(t[0]) == float(sum(members))
    mean = mine.allreduce_(torch.full((4,), float(rank), device=device), op="Average")
    parts = mine.allgather(torch.full((mine.rank + 1, 3), float(rank), device=device))   # ragged first dimension
    assert parts.shape[0] == sum(i + 1 for i in range(len(members)))
    b = torch.full((1000,), float(rank), device=device)
    mine.broadcast_(b, root=len(members) - 1)             # from the last member of the group
    assert float(b[0]) == float(members[-1])
    mine.barrier()
    print(f"rank {rank}: group {members}, sum {float(t[0]):.0f}, mean {float(mean[0]):.2f}, "
          f"gathered rows {parts.shape[0]}, broadcast from {members[-1]}", flush=True)
    tips.barrier()
    tips.shutdown()


if __name__ == "__main__":
    main()
