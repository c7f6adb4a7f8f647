"""Worker of the multi-GPU test of the optimizer step inside the gradient allreduce: one process per GPU.

For SGD with momentum (fp32 and bf16 models) and AdamW (bf16) it trains the same small model twice on the same
data, once with the separate allreduce + optimizer kernels and once with ``fused_update=True``, and compares the
parameters; it checks that the fused kernel really ran, that every rank holds 1/N of the state, that all ranks end
with identical parameters, and that a checkpoint written from the sharded state resumes into the same
trajectory.  Prints "FUSED_UPDATE_OK" on rank 0.
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import tips_b200 as tips  # noqa: E402
from tips_b200 import _lib  # noqa: E402
from tips_b200.ops.optim import FusedAdamW, FusedSGD  # noqa: E402
from tips_b200.utils.checkpoint import resume, save_checkpoint  # noqa: E402


def make_model(dev, dtype):
    torch.manual_seed(11)
    m = torch.nn.Sequential(torch.nn.Linear(64, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512), torch.nn.ReLU(),
                            torch.nn.Linear(512, 16))
    return m.to(dev).to(dtype)


def make_opt(kind, model, fused):
    if kind == "sgd":
        base = FusedSGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4, bucket_bytes=300_000)
    else:
        base = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.01, bucket_bytes=300_000)
    return tips.DistributedOptimizer(base, fused_update=fused)


def train(model, opt, steps, first, rank, size, dev, dtype):
    for step in range(first, first + steps):
        torch.manual_seed(1000 + step)
        xs = torch.randn(size * 32, 64, device=dev).to(dtype)
        ys = torch.randint(0, 16, (size * 32,), device=dev)
        sl = slice(rank * 32, (rank + 1) * 32)
        loss = torch.nn.functional.cross_entropy(model(xs[sl]).float(), ys[sl])
        loss.backward()
        opt.step()
    torch.cuda.synchronize()


def flat(model):
    return torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])


def main():
    tips.init()
    rank, size = tips.rank(), tips.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = tips.runtime.device_state()
    lib = _lib.kernels()
    for kind, dtype in (("sgd", torch.float32), ("sgd", torch.bfloat16), ("adam", torch.bfloat16)):
        plain_model, fused_model = make_model(dev, dtype), make_model(dev, dtype)
        plain = make_opt(kind, plain_model, False)
        fused = make_opt(kind, fused_model, True)
        assert fused._tips_update_in_allreduce and not plain._tips_update_in_allreduce
        assert len(fused._flat) >= 2  # several buckets
        for fs in fused._flat:
            assert fs.sharded and st.in_window(fs.flat_param)
            assert fs.master.numel() < fs.bucket.numel or size == 1 or fs.bucket.numel <= 2048 * 8
            assert all(st.in_window(p.data) for p in fs.bucket.params)
        train(plain_model, plain, 6, 0, rank, size, dev, dtype)
        train(fused_model, fused, 6, 0, rank, size, dev, dtype)
        st.check_status()
        a, b = flat(plain_model), flat(fused_model)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(a, b, atol=tol, rtol=tol), (kind, dtype, (a - b).abs().max())
        for fs in fused._flat:
            assert lib.tipsk_comm_update_launches(fs.bucket.win_off) == 6, "the fused kernel did not run"
        # every rank holds the same parameters, bit for bit
        sums = tips.allgather(b.double().sum().reshape(1))
        assert bool((sums == sums[0]).all()), sums
        # full-size state assembled from the shares equals the unsharded optimizer's state
        fstate, pstate = fused.flat_state(), plain.flat_state()
        for fs_f, fs_p, sf, sp in zip(fused._flat, plain._flat, fstate, pstate):
            assert sf["steps"] == sp["steps"] == 6
            for k in sp:
                if k == "steps":
                    continue
                assert sf[k].shape == sp[k].shape
                assert torch.allclose(sf[k], sp[k], atol=tol, rtol=tol), (kind, k)
            assert torch.allclose(fs_f.full_master(), fs_p.master.float(), atol=tol, rtol=tol)

        # checkpoint from the sharded state, resume into a fresh model / optimizer, continue both
        path = os.path.join(tempfile.gettempdir(), f"tips_fused_update_{kind}_{dtype}.pt".replace("torch.", ""))
        save_checkpoint(path, fused_model, fused, extra={"step": 6})
        tips.barrier()
        again_model = make_model(dev, dtype)
        with torch.no_grad():
            for p in again_model.parameters():
                p.add_(1.0)  # make sure the values come from the file
        again = make_opt(kind, again_model, True)
        extra = resume(path, again_model, again)
        assert extra["step"] == 6
        assert torch.equal(flat(again_model), flat(fused_model))
        train(fused_model, fused, 2, 6, rank, size, dev, dtype)
        train(again_model, again, 2, 6, rank, size, dev, dtype)
        st.check_status()
        a, b = flat(fused_model), flat(again_model)
        assert torch.allclose(a, b, atol=tol * 0.1, rtol=tol * 0.1), (kind, dtype, "resume", (a - b).abs().max())
        tips.barrier()
        if rank == 0 and os.path.exists(path):
            os.remove(path)
    tips.barrier()
    if rank == 0:
        print("FUSED_UPDATE_OK")
    tips.shutdown()


if __name__ == "__main__":
    main()
