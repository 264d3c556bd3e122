"""Fused row-parallel linear across real GPUs: child processes, one per GPU, launched with
torchrun (skipped on a machine with fewer than two GPUs).  NVLS is switched off for the NCCL
traffic that carries the comparison data; the kernel under test uses plain peer stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_rowlinear_allreduce_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29540 + world),
           os.path.join(ROOT, "tests", "multi_gpu", "rowlinear_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and f"ROWLINEAR_OK world={world}" in r.stdout, \
        (r.stdout[-2000:], r.stderr[-2000:])
