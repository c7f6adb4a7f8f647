"""The examples run as a user would start them: two CPU ranks under torchrun, a few steps each."""
import os
import subprocess
import sys

from mp_util import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args, nproc=2, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "examples", script), *args]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


def test_keras_style_mnist_example(tmp_path):
    out = _run("pytorch_mnist.py", "--cpu", "--epochs", "2", "--steps", "3", "--batch", "8",
               "--checkpoint-dir", str(tmp_path))
    assert "final" in out
    assert any(f.startswith("checkpoint-") for f in os.listdir(tmp_path))


def test_custom_loop_example():
    out = _run("pytorch_mnist_custom_loop.py", "--cpu", "--steps", "4", "--batch", "8", "--compression", "fp16")
    assert "replicas identical on 2 ranks" in out


def test_subgroup_example():
    out = _run("subgroup_collectives.py", "--cpu", nproc=4)
    assert "rank 3: group [1, 3], sum 4" in out and "rank 0: group [0, 2], sum 2" in out


def test_elastic_example_retries_the_failed_step():
    out = _run("elastic_mnist.py", "--cpu", "--steps", "6", "--fail-at", "2")
    assert "failed steps retried: 1" in out


def test_host_parameter_server_example():
    out = _run("host_ps.py")
    assert out.strip()


def test_parameter_server_mode_on_cpu_ranks():
    out = _run("host_ps_ctr.py", "--steps", "6", "--batch", "64", "--rows", "5000")
    assert "step 5 loss" in out and "rank 1: serves" in out

