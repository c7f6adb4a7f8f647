"""Worker of the multi-GPU dense parameter-server test: a ShardedDense table over all GPUs, every rank pushes its
own gradient; after three pushes every rank's copy equals a single-process optimizer run on the mean gradient, and
a state saved under N ranks reloads.  Prints "MULTI_GPU_DENSE_OK" on rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import tips_b200 as tips  # noqa: E402
from tips_b200.ps.gpu import ShardedDense  # noqa: E402


def main():
    tips.init()
    rank, n = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    size = 300_007
    for rule, kw in (("sgd", dict(lr=0.05, momentum=0.9)), ("adam", dict(lr=0.01))):
        t = ShardedDense(size, dtype=torch.bfloat16, optimizer=rule, device=dev, **kw)
        assert t.sharded
        g0 = torch.Generator().manual_seed(5)
        init = torch.randn(size, generator=g0).to(dev)
        t.assign(init)
        ref = init.to(torch.bfloat16).float().requires_grad_()
        ropt = torch.optim.SGD([ref], **kw) if rule == "sgd" else torch.optim.Adam([ref], **kw)
        for step in range(3):
            gens = [torch.Generator().manual_seed(100 * step + r) for r in range(n)]
            grads = [torch.randn(size, generator=g).to(torch.bfloat16) for g in gens]
            t.push(grads[rank].to(dev))
            ref.grad = (torch.stack([g.float() for g in grads]).sum(0) / n).to(dev)
            ropt.step()
        torch.cuda.synchronize()
        tips.runtime.device_state().check_status()
        got = t.pull().float()
        assert torch.allclose(got, ref.detach(), atol=3e-2, rtol=3e-2), (rule, (got - ref.detach()).abs().max())
        every = tips.allgather(t.pull().reshape(1, -1))
        assert all(torch.equal(every[r], every[0]) for r in range(n))     # one copy, identical on every rank
        saved = t.state()
        t2 = ShardedDense(size, dtype=torch.bfloat16, optimizer=rule, device=dev, **kw)
        t2.load_state(saved)
        g = torch.randn(size, generator=torch.Generator().manual_seed(77)).to(torch.bfloat16).to(dev)
        t.push(g)
        t2.push(g)
        torch.cuda.synchronize()
        assert torch.equal(t.pull(), t2.pull())
    tips.barrier()
    if rank == 0:
        print("MULTI_GPU_DENSE_OK")
    tips.shutdown()


if __name__ == "__main__":
    main()
