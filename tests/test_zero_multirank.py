"""Sharded-optimizer state machine across ranks: gloo on CPU here, NCCL and the fused
symmetric-memory kernels on 2 GPUs."""

import os
import subprocess
import sys

import pytest

from helpers import free_port
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(nproc, extra, port, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "_zero_worker.py"), *extra]
    e = dict(os.environ)
    e.update(env or {})
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=e)
    assert res.returncode == 0 and "ZERO_WORKER_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_ranks_match_single_process(world):
    _launch(world, ["--device", "cpu", "--comms", "nccl"], free_port())


@pytest.mark.gpu
def test_fused_comm_matches_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _launch(2, ["--device", "cuda", "--comms", "nccl,fused,fused+overlap"], free_port(), env={"NCCL_NVLS_ENABLE": "0"})
