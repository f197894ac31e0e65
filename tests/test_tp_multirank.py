"""Tensor-parallel rollout on two GPUs (fused all-reduce + residual + norm kernel, sharded engine)."""

import os
import subprocess
import sys

import pytest

from helpers import free_port
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_tp2_engine_and_fused_allreduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "_tp_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and "TP_WORKER_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
def test_ulysses_sequence_parallel_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "_sp_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and "SP_WORKER_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
def test_training_tensor_parallel_fused_path():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "_tp_train_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and res.stdout.count("TP_TRAIN_GPU_OK") == 2, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
def test_sequence_parallel_groups_inside_data_parallel_world():
    """Ulysses groups of 2 inside a world of 4, with resident and with sharded parameters."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "_sp_dp_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and "SP_DP_WORKER_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
