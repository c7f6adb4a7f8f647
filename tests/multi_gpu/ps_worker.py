"""Worker of the multi-GPU parameter-server test: tables sharded over the GPUs, every rank pulls and pushes
its own batch; the result must equal a dense single-process model of the same tables updated with the
gradients of ALL ranks (synchronous Adagrad).  Prints "MULTI_GPU_PS_OK" on rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import tips_b200 as tips  # noqa: E402
from tips_b200.ps.gpu import ShardedEmbedding  # noqa: E402


def main():
    tips.init()
    rank, n = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    fields, rows, dim, batch = 3, 10007, 64, 4096
    t = ShardedEmbedding(fields, rows, dim, optimizer="adagrad", lr=0.05, init_scale=0.1, seed=11,
                         expected_batch=batch * n, device=dev)
    # dense reference of the whole table, rebuilt from every rank's shard
    def gather_tables(state=False):
        out = []
        for f in range(fields):
            shard = t.local_shard(f, state=state).contiguous()
            allsh = tips.allgather(shard.reshape(1, -1)).reshape(n, t.rows_per_shard, dim)
            w = torch.zeros(t.rows_per_shard * n, dim, device=dev)
            for r in range(n):
                w[t.global_ids(f, r, device=dev)] = allsh[r]
            out.append(w[:rows].clone())
        return out
    ws = gather_tables()
    ss = [torch.zeros_like(w) for w in ws]
    for step in range(3):
        gens = [torch.Generator().manual_seed(1000 * step + r) for r in range(n)]
        ids_all = [(torch.rand(batch, fields, generator=g) ** 3 * rows).long().clamp_(0, rows - 1) for g in gens]
        grads_all = [torch.randn(batch, fields * dim, generator=g) for g in gens]
        ids, grads = ids_all[rank].to(dev), grads_all[rank].to(dev)
        out = t.pull(ids, dtype=torch.float32)
        ref = torch.cat([ws[f][ids[:, f]] for f in range(fields)], dim=1)
        # the reference sums the ranks' gradients in a fixed order, the device in arrival order
        assert torch.allclose(out, ref, atol=3e-4, rtol=1e-4), (step, (out - ref).abs().max())
        t.push(ids, grads, grad_scale=1.0 / n)
        for f in range(fields):
            g = torch.zeros_like(ws[f])
            for r in range(n):
                g.index_add_(0, ids_all[r][:, f].to(dev), grads_all[r][:, f * dim:(f + 1) * dim].to(dev) / n)
            touched = g.abs().sum(1) != 0
            ss[f] += g * g
            ws[f] -= torch.where(touched[:, None], 0.05 * g / (ss[f].sqrt() + t.eps), torch.zeros_like(g))
    t.check()
    tips.runtime.device_state().check_status()
    # a fence so that every owner has applied its updates before the shards are read back
    t.pull(ids, dtype=torch.float32)
    torch.cuda.synchronize()
    got = gather_tables()
    # the hottest rows sum hundreds of fp32 gradient rows per step in arrival order (more with more ranks), and
    # Adagrad divides by the root of the accumulated squares: the last bits of those sums show after three steps
    for f in range(fields):
        assert torch.allclose(got[f], ws[f], atol=1e-3, rtol=1e-4), (f, (got[f] - ws[f]).abs().max())
    tips.barrier()
    if rank == 0:
        print("MULTI_GPU_PS_OK")
    tips.shutdown()


if __name__ == "__main__":
    main()
