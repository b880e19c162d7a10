"""Fused operators over real peer-mapped memory: one process per GPU under torchrun.  Needs two or
more GPUs in the box; on a one-GPU box the test is skipped (the same kernels are then covered by
the emulated-rank tests of test_gemm_gpu.py)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(nproc, port):
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(here, "multigpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    return res


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_two_ranks():
    res = _run(2, 29611)
    assert res.returncode == 0 and "MULTIGPU_OK" in res.stdout, (res.stdout + res.stderr)[-4000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs >= 4 GPUs")
def test_all_ranks_of_the_box():
    n = 8 if torch.cuda.device_count() >= 8 else 4
    res = _run(n, 29612)
    assert res.returncode == 0 and "MULTIGPU_OK" in res.stdout, (res.stdout + res.stderr)[-4000:]
