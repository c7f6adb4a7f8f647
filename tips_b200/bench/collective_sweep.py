"""Collective sweep: allreduce(sum) / allgather / broadcast, 1 KB .. 1 GB, fp32 and bf16, fused NVLink kernels
vs NCCL on the same GPUs.  Device-timed with CUDA events on the launching stream, max over ranks.

    python -m torch.distributed.run --nproc-per-node N -m tips_b200.bench.collective_sweep [--max-mb 1024]

Bus bandwidth uses the usual conventions: allreduce algbw * 2(N-1)/N, allgather and broadcast algbw * (N-1)/N
with algbw = total bytes / time.  The roofline reference is the measured 770 GB/s peer copy per direction.
``--ops update`` times the allreduce followed by the Adam kernel on full-size state against the single kernel that
reduces, updates the share of the state this rank owns and stores the parameters to every rank.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys

import torch

import tips_b200 as tips
from tips_b200 import _lib

LINK_GBS = 770.0


def _checked(lib, call):
    def run():
        rc = call()
        if rc != 0:
            raise RuntimeError("kernel launcher failed: " + lib.tipsk_last_error().decode())
    return run


def _opt(lib, name, value):
    """Kernel selection of the library; every rank sets the same value between two timed runs."""
    if lib.tipsk_comm_set_option(name.encode(), int(value)):
        raise RuntimeError(lib.tipsk_last_error().decode())


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tips.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    t = torch.tensor([ms], dtype=torch.float64)
    return float(tips.allreduce(t, op=tips.Max)[0])


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--min-kb", type=int, default=1)
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--ops", default="allreduce,allgather,broadcast")
    ap.add_argument("--scatter-chunks-mb", default="32", help="also time the scatter broadcast with these pipeline "
                    "chunk sizes, e.g. 2,4,16")
    ap.add_argument("--verify", type=int, default=1, help="compare the alternative kernels' results with NCCL's")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    tips.init()
    import torch.distributed as dist
    rank, n = tips.rank(), tips.size()
    assert n > 1, "the sweep needs at least 2 GPUs"
    st = tips.runtime.device_state()
    lib = _lib.kernels()
    dev = st.device
    work_stream = torch.cuda.Stream()  # a real stream: a null handle would select the library's own
    torch.cuda.set_stream(work_stream)
    stream = work_stream.cuda_stream
    dts = {"fp32": (torch.float32, 0), "bf16": (torch.bfloat16, 6)}
    rows = []
    max_bytes = a.max_mb << 20
    sym, sym_off = st.alloc_symmetric(max_bytes)
    upd_max = min(max_bytes, 256 << 20)
    if "update" in a.ops:
        _, par_off = st.alloc_symmetric(upd_max)
    size = a.min_kb << 10
    sizes = []
    while size <= max_bytes:
        sizes.append(size)
        size *= 2
    for name in a.dtypes.split(","):
        dtype, code = dts[name]
        es = torch.empty((), dtype=dtype).element_size()
        for nbytes in sizes:
            numel = nbytes // es
            iters = 50 if nbytes <= (1 << 20) else 20 if nbytes <= (64 << 20) else 5
            x = torch.randn(numel, device=dev).to(dtype)
            y = torch.empty_like(x)
            res = {"dtype": name, "bytes": nbytes, "ranks": n}
            if "allreduce" in a.ops:
                srcs = (ctypes.c_void_p * 1)(x.data_ptr())
                dsts = (ctypes.c_void_p * 1)(y.data_ptr())
                ms = _time(_checked(lib, lambda: lib.tipsk_allreduce(srcs, dsts, -1, nbytes, code, 0, 1.0, 1.0, 3, stream)), iters)
                res["allreduce_staged_ms"] = ms
                ms = _time(_checked(lib, lambda: lib.tipsk_allreduce(None, None, sym_off, nbytes, code, 0, 1.0, 1.0 / n, 3, stream)), iters)
                res["allreduce_inplace_ms"] = ms
                res["allreduce_inplace_busbw"] = nbytes / ms / 1e6 * 2 * (n - 1) / n
                ms = _time(lambda: dist.all_reduce(x), iters)
                res["nccl_allreduce_ms"] = ms
                res["nccl_allreduce_busbw"] = nbytes / ms / 1e6 * 2 * (n - 1) / n
                res["allreduce_roofline_frac"] = (nbytes * (n - 1) / n / (LINK_GBS * 1e6)) / res["allreduce_inplace_ms"]
            if "allgather" in a.ops and nbytes * n <= (2 << 30):
                out = torch.empty(numel * n, dtype=dtype, device=dev)
                per = (ctypes.c_uint64 * n)(*([nbytes] * n))
                srcs = (ctypes.c_void_p * 1)(x.data_ptr())
                dsts = (ctypes.c_void_p * 1)(out.data_ptr())
                ms = _time(_checked(lib, lambda: lib.tipsk_allgatherv(srcs, dsts, per, 3, stream)), iters)
                res["allgather_ms"] = ms
                res["allgather_busbw"] = nbytes * n / ms / 1e6 * (n - 1) / n
                if nbytes * n <= (64 << 20):
                    # the same gather through each of the two kernels (slabs of up to 2 MiB are pushed by default)
                    _opt(lib, "allgather_push_bytes", 0)
                    ms = _time(_checked(lib, lambda: lib.tipsk_allgatherv(srcs, dsts, per, 3, stream)), iters)
                    res["allgather_pull_busbw"] = nbytes * n / ms / 1e6 * (n - 1) / n
                    _opt(lib, "allgather_push_bytes", 256 << 20)
                    ms = _time(_checked(lib, lambda: lib.tipsk_allgatherv(srcs, dsts, per, 3, stream)), iters)
                    res["allgather_push_busbw"] = nbytes * n / ms / 1e6 * (n - 1) / n
                    if a.verify:
                        want = torch.empty_like(out)
                        dist.all_gather_into_tensor(want, x)
                        if not torch.equal(out, want):
                            raise RuntimeError(f"pushed allgather of {nbytes} bytes per rank is wrong")
                    _opt(lib, "allgather_push_bytes", 2 << 20)
                ms = _time(lambda: dist.all_gather_into_tensor(out, x), iters)
                res["nccl_allgather_busbw"] = nbytes * n / ms / 1e6 * (n - 1) / n
                del out
            if "broadcast" in a.ops:
                srcs = (ctypes.c_void_p * 1)(x.data_ptr())
                dsts = (ctypes.c_void_p * 1)(y.data_ptr())
                ms = _time(_checked(lib, lambda: lib.tipsk_broadcast(srcs, dsts, nbytes, 0, 3, stream)), iters)
                res["broadcast_ms"] = ms
                res["broadcast_gbs"] = nbytes / ms / 1e6
                ms = _time(lambda: dist.broadcast(x, 0), iters)
                res["nccl_broadcast_gbs"] = nbytes / ms / 1e6
                if nbytes >= (2 << 20) and n >= 3:
                    # the same message stored to everybody by the root alone, and as scatter + allgather with
                    # several pipeline chunk sizes (by default: with 8 ranks, from 128 MiB on, 32 MiB chunks)
                    _opt(lib, "bcast_scatter_bytes", 0)
                    ms = _time(_checked(lib, lambda: lib.tipsk_broadcast(srcs, dsts, nbytes, 0, 3, stream)), iters)
                    res["broadcast_direct_gbs"] = nbytes / ms / 1e6
                    _opt(lib, "bcast_scatter_bytes", 2 << 20)
                    _opt(lib, "bcast_scatter_min_ranks", 3)
                    for mb in [int(c) for c in a.scatter_chunks_mb.split(",") if c]:
                        _opt(lib, "bcast_scatter_chunk_bytes", mb << 20)
                        ms = _time(_checked(lib, lambda: lib.tipsk_broadcast(srcs, dsts, nbytes, 0, 3, stream)), iters)
                        res[f"broadcast_scatter_gbs_chunk{mb}mb"] = nbytes / ms / 1e6
                        if a.verify:
                            want = x.clone()
                            dist.broadcast(want, 0)
                            if not torch.equal(y, want):
                                raise RuntimeError(f"scatter broadcast of {nbytes} bytes (chunk {mb} MiB) is wrong")
                    _opt(lib, "bcast_scatter_chunk_bytes", 32 << 20)
                    _opt(lib, "bcast_scatter_bytes", 128 << 20)
                    _opt(lib, "bcast_scatter_min_ranks", 8)
            if "update" in a.ops and 16 <= nbytes <= upd_max:
                # allreduce + Adam as two kernels on full-size state, against the one kernel that reduces this
                # rank's share, updates 1/n of the state and stores the parameters to every rank
                shard = int(lib.tipsk_comm_update_shard_vecs(nbytes)) * (16 // es)
                full = [torch.zeros(numel, device=dev) for _ in range(3)]
                part = [torch.zeros(shard, device=dev) for _ in range(3)]
                low = torch.zeros(numel, dtype=dtype, device=dev)
                hp = (ctypes.c_float * 6)(1e-4, 0.9, 0.999, 1e-8, 0.01, 1.0)

                def two_kernels():
                    rc = lib.tipsk_allreduce(None, None, sym_off, nbytes, code, 0, 1.0, 1.0 / n, 3, stream)
                    return rc or lib.tipsk_adam_flat_devstep(
                        full[0].data_ptr(), low.data_ptr() if es == 2 else None, code if es == 2 else 6,
                        sym.data_ptr(), code, full[1].data_ptr(), full[2].data_ptr(), numel, 1e-4, 0.9, 0.999, 1e-8,
                        0.01, 2, None, 1.0, 1, stream)

                res["allreduce_then_adam_ms"] = _time(_checked(lib, two_kernels), iters)
                arr = [(ctypes.c_void_p * 1)(t.data_ptr()) for t in part]
                rc = lib.tipsk_comm_attach_update(sym_off, nbytes, code, par_off, 1, arr[0], arr[1], arr[2])
                rc = rc or lib.tipsk_comm_set_update_hyper(sym_off, hp, 6, 2)
                if rc:
                    raise RuntimeError(lib.tipsk_last_error().decode())
                res["allreduce_adam_fused_ms"] = _time(
                    _checked(lib, lambda: lib.tipsk_allreduce_update(sym_off, 1.0 / n, 3, stream)), iters)
                lib.tipsk_comm_detach_update(sym_off)
                del full, part, low
            st.check_status()
            rows.append(res)
            if rank == 0:
                print(json.dumps(res), flush=True)
            del x, y
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"ranks": n, "uses_multimem": bool(lib.tipsk_comm_uses_multimem()), "rows": rows}, f, indent=1)
    tips.shutdown()


if __name__ == "__main__":
    main(sys.argv[1:])
