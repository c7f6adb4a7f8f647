"""Start one process per rank on this node: ``python -m tips_b200.launch -np 4 train.py --epochs 3``.

The reference is started with ``mpirun -np N python train.py`` and reads rank and size from MPI
(tips/core/mpi/mpi_context.cc); this runtime reads them from the environment, so any launcher that sets ``RANK``,
``WORLD_SIZE``, ``LOCAL_RANK``, ``MASTER_ADDR`` and ``MASTER_PORT`` works (``torch.distributed.run`` does).  This one
has no dependency beyond the standard library and adds what a training job on one 8-GPU box wants:

* a free rendezvous port on 127.0.0.1 unless one is given;
* the CPUs of each rank limited to the NUMA node of its GPU when the system exposes that (``--bind numa``; pinned
  host buffers are then allocated next to the GPU that reads them), or an equal share of the allowed CPUs
  (``--bind split``), or nothing (``--bind none``, the default);
* when one rank exits with an error the others get SIGTERM (then SIGKILL after ``--grace`` seconds), so a failed
  job ends instead of waiting in a collective, and the launcher's exit code is the first failure's;
* SIGINT / SIGTERM to the launcher are forwarded to every rank.
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port if port < 60000 else port - 5000  # the runtime derives a second port 1000 above this one


def parse_cpulist(text: str) -> List[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11]"""
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def gpu_numa_cpus(local_rank: int, sysfs: str = "/sys", pci_bus_ids: Optional[Sequence[str]] = None) -> Optional[List[int]]:
    """CPUs of the NUMA node that GPU `local_rank` hangs off, or None when the system does not say.
    `pci_bus_ids` lists the GPUs' PCI addresses in device order; by default they are read from the NVIDIA driver's
    procfs entries, sorted by address (the order CUDA uses with CUDA_DEVICE_ORDER=PCI_BUS_ID)."""
    try:
        if pci_bus_ids is None:
            root = "/proc/driver/nvidia/gpus"
            pci_bus_ids = sorted(os.listdir(root)) if os.path.isdir(root) else []
        if local_rank >= len(pci_bus_ids):
            return None
        dev = os.path.join(sysfs, "bus", "pci", "devices", pci_bus_ids[local_rank].lower())
        with open(os.path.join(dev, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return None


def cpu_share(local_rank: int, nproc: int, allowed: Sequence[int]) -> List[int]:
    """An equal contiguous share of the allowed CPUs (everything when there are fewer CPUs than ranks)."""
    allowed = sorted(allowed)
    if len(allowed) < nproc:
        return list(allowed)
    per = len(allowed) // nproc
    return list(allowed[local_rank * per:(local_rank + 1) * per])


def rank_env(rank: int, nproc: int, addr: str, port: int, base: Optional[Dict[str, str]] = None) -> Dict[str, str]:
    env = dict(os.environ if base is None else base)
    env.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(nproc), LOCAL_WORLD_SIZE=str(nproc),
               MASTER_ADDR=addr, MASTER_PORT=str(port))
    env.setdefault("OMP_NUM_THREADS", "1")
    return env


def _bind(local_rank: int, nproc: int, mode: str):
    """Returns a function for `preexec_fn` that limits the child's CPUs, or None."""
    if mode == "none" or not hasattr(os, "sched_setaffinity"):
        return None
    allowed = sorted(os.sched_getaffinity(0))
    cpus = None
    if mode == "numa":
        node = gpu_numa_cpus(local_rank)
        if node:
            cpus = [c for c in node if c in allowed]
    if not cpus and mode in ("numa", "split"):
        cpus = cpu_share(local_rank, nproc, allowed) if mode == "split" else None
    if not cpus:
        return None
    return lambda: os.sched_setaffinity(0, cpus)


def launch(nproc: int, command: Sequence[str], addr: str = "127.0.0.1", port: int = 0, bind: str = "none",
           grace: float = 10.0, module: bool = False) -> int:
    """Runs `command` (a script path and its arguments, or with `module` a module name) once per rank and waits.
    Returns 0 if every rank did, else the exit code of the first rank that failed."""
    port = port or free_port()
    argv = [sys.executable] + (["-m"] if module else []) + list(command)
    procs: List[subprocess.Popen] = []
    for r in range(nproc):
        procs.append(subprocess.Popen(argv, env=rank_env(r, nproc, addr, port), preexec_fn=_bind(r, nproc, bind)))

    def forward(signum, _frame):
        for p in procs:
            if p.poll() is None:
                p.send_signal(signum)

    old = {s: signal.signal(s, forward) for s in (signal.SIGINT, signal.SIGTERM)}
    first_failure = 0
    try:
        alive = set(range(nproc))
        while alive:
            for r in sorted(alive):
                code = procs[r].poll()
                if code is None:
                    continue
                alive.discard(r)
                if code != 0 and first_failure == 0:
                    first_failure = code if code > 0 else 128 - code
                    print(f"[tips launch] rank {r} exited with {code}; stopping the other ranks", file=sys.stderr, flush=True)
                    for q in alive:
                        procs[q].terminate()
                    deadline = time.time() + grace
                    while time.time() < deadline and any(procs[q].poll() is None for q in alive):
                        time.sleep(0.05)
                    for q in alive:
                        if procs[q].poll() is None:
                            procs[q].kill()
            time.sleep(0.05)
    finally:
        for s, h in old.items():
            signal.signal(s, h)
    return first_failure


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tips_b200.launch", description=__doc__.split("\n\n")[0])
    ap.add_argument("-np", "--nproc", type=int, required=True, help="ranks to start on this node")
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=0, help="0: pick a free one")
    ap.add_argument("--bind", default="none", choices=["none", "numa", "split"])
    ap.add_argument("--grace", type=float, default=10.0, help="seconds between SIGTERM and SIGKILL after a failure")
    ap.add_argument("-m", dest="module", action="store_true", help="the command is a module name, as with python -m")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="script (or module) and its arguments")
    a = ap.parse_args(argv)
    if not a.command:
        ap.error("no script given")
    return launch(a.nproc, a.command, a.master_addr, a.master_port, a.bind, a.grace, a.module)


if __name__ == "__main__":
    sys.exit(main())
