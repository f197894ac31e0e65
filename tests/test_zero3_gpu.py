"""Parameter-sharded learner on GPUs: equals the resident learner on one GPU (the gather is a copy) and on two
(NCCL and peer-kernel transports)."""

import os
import subprocess
import sys

import pytest

from helpers import free_port
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "_zero3_gpu_worker.py")


@pytest.mark.gpu
def test_sharded_learner_single_gpu():
    res = subprocess.run([sys.executable, WORKER], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "WORLD_SIZE": "1", "RANK": "0", "LOCAL_RANK": "0"})
    assert res.returncode == 0 and "ZERO3_GPU_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
def test_sharded_learner_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), WORKER]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and res.stdout.count("ZERO3_GPU_OK") == 2, res.stdout[-3000:] + res.stderr[-3000:]
