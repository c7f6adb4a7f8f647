"""Cost of the control plane on CPU ranks: message encode / decode, and the latency of one negotiated collective
(request to rank 0, validation, response, execution of a 1-element allreduce over the TCP mesh) at 2..N ranks.

    python -m tips_b200.bench.control_plane [--ranks 2,4] [--iters 2000]

The reference times only its serializer (tips/core/message/flatbuffers_test.cc:12-66, FlatBuffers against its
NaiveBuffer, 1000 x build / read, numbers logged and never recorded); the negotiated round trip has no
counterpart there.  This is also the timed row of the MNIST-sized configuration: a step of that model issues one
bucket per step, so its communication cost is one of these round trips plus the bytes; the same step is timed a
second time the way the reference runs it (one negotiated allreduce per gradient tensor, every step).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import socket
import sys
import time

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p if p < 60000 else p - 5000


def _rank_main(rank, size, port, iters, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(size), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import tips_b200 as tips
    tips.init(device=False)
    x = torch.ones(1)
    for i in range(50):
        tips.allreduce(x, op=tips.Sum, name=f"warm.{i}")
    tips.barrier()
    t0 = time.perf_counter()
    for i in range(iters):
        tips.allreduce(x, op=tips.Sum, name=f"lat.{i}")
    one = (time.perf_counter() - t0) / iters
    big = torch.ones(1 << 20)   # 4 MB fp32: the bandwidth of the host data mesh
    tips.barrier()
    t0 = time.perf_counter()
    for i in range(20):
        tips.allreduce(big, op=tips.Sum, name=f"bw.{i}")
    bw = (time.perf_counter() - t0) / 20
    # MNIST-sized data-parallel step (the first named configuration): CNN, batch 64 per rank, SGD 0.01
    from tips_b200.models.mnist_cnn import MnistCNN, synthetic_batch
    torch.manual_seed(0)
    model = MnistCNN()
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01))
    tips.broadcast_parameters(model.state_dict(), root_rank=0)
    xb, yb = synthetic_batch(64, rank)
    for _ in range(3):
        torch.nn.functional.cross_entropy(model(xb), yb).backward()
        opt.step()
        opt.zero_grad()
    tips.barrier()
    t0 = time.perf_counter()
    steps = 10
    for _ in range(steps):
        torch.nn.functional.cross_entropy(model(xb), yb).backward()
        opt.step()
        opt.zero_grad()
    step = (time.perf_counter() - t0) / steps
    # The same step the way the reference runs it (tips/tensorflow/__init__.py:230-300 and
    # tips/core/collective/coordinator.cc:243-353): one allreduce per gradient tensor, each negotiated through
    # rank 0 in every step, nothing fused and no order frozen.
    from tips_b200 import _lib
    _lib.core().tips_set_fusion_threshold(0)
    tips.barrier()
    torch.manual_seed(0)
    model_ref = MnistCNN()   # a model of its own: the first one carries the distributed optimizer's gradient hooks
    plain = torch.optim.SGD(model_ref.parameters(), lr=0.01)

    def reference_step():
        plain.zero_grad()
        torch.nn.functional.cross_entropy(model_ref(xb), yb).backward()
        tips.allreduce_gradients(model_ref.parameters(), name="ref.grads")
        plain.step()

    for _ in range(3):
        reference_step()
    tips.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        reference_step()
    ref_step = (time.perf_counter() - t0) / steps
    if rank == 0:
        out.put({"ranks": size, "negotiated_allreduce_us": round(one * 1e6, 1),
                 "allreduce_4MB_ms": round(bw * 1e3, 2), "allreduce_4MB_GBs_per_rank": round(4.194304e-3 / bw, 2),
                 "mnist_cnn_step_ms": round(step * 1e3, 1),
                 "mnist_cnn_images_per_s": round(64 * size / step, 1),
                 "mnist_cnn_step_ms_per_tensor_negotiated": round(ref_step * 1e3, 1),
                 "mnist_cnn_images_per_s_per_tensor_negotiated": round(64 * size / ref_step, 1)})
    tips.shutdown()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", default="2,4")
    ap.add_argument("--iters", type=int, default=2000)
    a = ap.parse_args(argv)
    from tips_b200 import _lib
    lib = _lib.core()
    lib.tips_bench_messages.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    out4 = (ctypes.c_double * 4)()
    lib.tips_bench_messages(200000, out4)
    res = {"message_ns": {"request_encode": round(out4[0], 1), "request_decode": round(out4[1], 1),
                          "response_encode": round(out4[2], 1), "response_decode": round(out4[3], 1)}, "rounds": []}
    ctx = mp.get_context("spawn")
    for n in [int(v) for v in a.ranks.split(",") if v]:
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, n, port, a.iters, q)) for r in range(n)]
        for p in procs:
            p.start()
        res["rounds"].append(q.get(timeout=600))
        for p in procs:
            p.join()
    print(json.dumps(res))


if __name__ == "__main__":
    sys.exit(main())
