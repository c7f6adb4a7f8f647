"""Run a function on N CPU ranks (spawned processes) with the tips runtime initialised."""
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p if p < 60000 else p - 5000


def _entry(rank, size, port, fn, args, env):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(size), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      TIPS_HOST_TIMEOUT_MS="60000")
    os.environ.update(env or {})
    import tips_b200 as tips
    try:
        tips.init(device=False)
        fn(rank, size, *args)
        tips.shutdown()
    except Exception:
        traceback.print_exc()
        raise


def run_ranks(fn, size, *args, env=None):
    mp.spawn(_entry, args=(size, free_port(), fn, args, env), nprocs=size, join=True)
