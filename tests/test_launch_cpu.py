"""The stand-alone launcher: environment of the ranks, CPU binding helpers (against a fake sysfs), a job that runs
to the end, and a job in which one rank fails while the other would wait for ever."""
import os
import subprocess
import sys
import time

from tips_b200 import launch as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpu_lists_and_shares():
    assert L.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert L.parse_cpulist("") == []
    assert L.cpu_share(1, 4, range(16)) == [4, 5, 6, 7]
    assert L.cpu_share(3, 4, [0, 1, 2, 3, 4, 5, 6, 7, 8]) == [6, 7]      # the remainder stays unused
    assert L.cpu_share(2, 8, [0, 1, 2]) == [0, 1, 2]                     # fewer CPUs than ranks: no split
    env = L.rank_env(2, 4, "127.0.0.1", 23456, base={"OMP_NUM_THREADS": "6"})
    assert env["RANK"] == "2" and env["WORLD_SIZE"] == "4" and env["LOCAL_RANK"] == "2"
    assert env["MASTER_PORT"] == "23456" and env["OMP_NUM_THREADS"] == "6"
    assert L.rank_env(0, 1, "127.0.0.1", 1, base={})["OMP_NUM_THREADS"] == "1"


def test_numa_node_of_a_gpu_from_sysfs(tmp_path):
    sysfs = tmp_path / "sys"
    for bus, node in (("0000:1b:00.0", "1"), ("0000:43:00.0", "-1")):
        d = sysfs / "bus" / "pci" / "devices" / bus
        d.mkdir(parents=True)
        (d / "numa_node").write_text(node + "\n")
    n1 = sysfs / "devices" / "system" / "node" / "node1"
    n1.mkdir(parents=True)
    (n1 / "cpulist").write_text("8-11,24-27\n")
    ids = ["0000:1B:00.0", "0000:43:00.0"]
    assert L.gpu_numa_cpus(0, str(sysfs), ids) == [8, 9, 10, 11, 24, 25, 26, 27]
    assert L.gpu_numa_cpus(1, str(sysfs), ids) is None          # the platform reports no node for this device
    assert L.gpu_numa_cpus(5, str(sysfs), ids) is None          # more ranks than GPUs
    assert L.gpu_numa_cpus(0, str(tmp_path / "nowhere"), ids) is None


def _script(tmp_path, body):
    p = tmp_path / "job.py"
    p.write_text("import os, sys, time\nsys.path.insert(0, %r)\n" % ROOT + body)
    return str(p)


def test_job_runs_to_the_end(tmp_path):
    script = _script(tmp_path, """
import torch
import tips_b200 as tips
tips.init(device=False)
out = tips.allreduce(torch.full((4,), float(tips.rank())), op=tips.Sum)
assert float(out[0]) == sum(range(tips.size())) and tips.size() == int(sys.argv[1])
assert len(os.sched_getaffinity(0)) >= 1
open(os.path.join(os.path.dirname(__file__), f"done.{tips.rank()}"), "w").write("ok")
tips.shutdown()
""")
    r = subprocess.run([sys.executable, "-m", "tips_b200.launch", "-np", "3", "--bind", "split", script, "3"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    assert sorted(f for f in os.listdir(tmp_path) if f.startswith("done.")) == ["done.0", "done.1", "done.2"]


def test_a_failed_rank_ends_the_job(tmp_path):
    script = _script(tmp_path, """
if os.environ["RANK"] == "1":
    sys.exit(3)
time.sleep(120)          # stands for a rank waiting in a collective for the one that died
""")
    t0 = time.time()
    code = L.launch(2, [script], grace=2.0)
    assert code == 3 and time.time() - t0 < 30


def test_bind_process_to_the_numa_node_of_its_gpu(tmp_path):
    """The in-process form of the binding, against a fake sysfs; run in a child so that this process keeps its CPUs."""
    allowed = sorted(os.sched_getaffinity(0))
    sysfs = tmp_path / "sys"
    d = sysfs / "bus" / "pci" / "devices" / "0000:1b:00.0"
    d.mkdir(parents=True)
    (d / "numa_node").write_text("0\n")
    node = sysfs / "devices" / "system" / "node" / "node0"
    node.mkdir(parents=True)
    (node / "cpulist").write_text(f"{allowed[0]},9999\n")     # one CPU we may use, one that does not exist here
    code = (f"import os, sys; sys.path.insert(0, {ROOT!r}); from tips_b200 import runtime\n"
            f"got = runtime.bind_to_gpu_numa_node(sysfs={str(sysfs)!r}, pci_bus_id='0000:1b:00.0')\n"
            f"assert got == [{allowed[0]}] and sorted(os.sched_getaffinity(0)) == [{allowed[0]}], got\n"
            f"assert runtime.bind_to_gpu_numa_node(sysfs={str(sysfs)!r}, pci_bus_id='0000:ff:00.0') is None\n"
            "print('BOUND')")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "BOUND" in r.stdout, r.stderr[-2000:]
