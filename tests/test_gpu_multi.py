"""Multi-GPU tests: spawn one process per GPU with torchrun (skipped on boxes with one GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(worker, nproc, env=None, timeout=600):
    e = dict(os.environ)
    e.update(env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "multi_gpu", worker)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_collectives_two_gpus(multimem):
    r = _run("collectives_worker.py", 2, env={"TIPS_DISABLE_MULTIMEM": "0" if multimem == "1" else "1"})
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_optimizer_step_inside_the_allreduce(multimem):
    n = min(torch.cuda.device_count(), 4)
    r = _run("fused_update_worker.py", n, env={"TIPS_DISABLE_MULTIMEM": "0" if multimem == "1" else "1"})
    assert r.returncode == 0 and "FUSED_UPDATE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_parameter_server_two_gpus():
    r = _run("ps_worker.py", 2)
    assert r.returncode == 0 and "MULTI_GPU_PS_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_dense_parameter_server_table():
    r = _run("dense_worker.py", min(torch.cuda.device_count(), 4))
    assert r.returncode == 0 and "MULTI_GPU_DENSE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs at least 4 GPUs")
def test_collectives_and_ps_all_gpus():
    n = torch.cuda.device_count()
    r = _run("collectives_worker.py", n)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
    r = _run("ps_worker.py", n)
    assert r.returncode == 0 and "MULTI_GPU_PS_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
