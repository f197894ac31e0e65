"""Failure detection without touching a GPU: failures are made on the host (a rank that leaves, a worker that raises,
a checkpoint that was cut short, an actor that died) and must surface as errors, not hangs."""

import os
import subprocess
import sys
import time

import pytest

from helpers import free_port
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rank_leaving_between_steps_is_detected():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "_failure_worker.py"), "leave"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
    out = res.stdout + res.stderr
    assert "RANK1_LEFT" in out and "RANK0_SAW_FAILURE" in out and "UNEXPECTED_SUCCESS" not in out, out[-2000:]


def test_incomplete_checkpoint_is_skipped(tmp_path):
    from open_instruct_b200.ckpt.train_state import load_train_state, save_train_state
    from open_instruct_b200.parallel.zero import ZeroOptimizer, padded_numel
    from open_instruct_b200.utils.common import get_last_checkpoint, is_checkpoint_folder

    n = padded_numel(100, 1)
    opt = ZeroOptimizer(torch.randn(n), 100, 80, comm="none")
    opt.step(torch.randn(n))
    save_train_state(str(tmp_path / "step_1"), opt, {"completed_steps": 1, "epoch": 0, "loader": {}})
    save_train_state(str(tmp_path / "step_2"), opt, {"completed_steps": 2, "epoch": 0, "loader": {}})
    # a crash in the middle of the second save: completion marker gone, one file cut short
    marker = [f for f in os.listdir(tmp_path / "step_2") if "COMPLETE" in f.upper()]
    assert marker, os.listdir(tmp_path / "step_2")
    for m in marker:
        os.remove(tmp_path / "step_2" / m)
    victim = next(f for f in os.listdir(tmp_path / "step_2") if f.endswith((".pt", ".safetensors", ".bin")))
    with open(tmp_path / "step_2" / victim, "r+b") as f:
        f.truncate(10)
    last = get_last_checkpoint(str(tmp_path))
    assert last is not None and last.endswith("step_1") and is_checkpoint_folder(last)
    assert get_last_checkpoint(str(tmp_path), incomplete=True).endswith("step_2")  # only on explicit request
    assert load_train_state(last, opt)["completed_steps"] == 1


class _Boom:
    def ping(self):
        return "pong"

    def die(self):
        os._exit(3)


def test_dead_actor_raises_instead_of_hanging():
    from open_instruct_b200.actors import ray_compat as ray

    try:
        h = ray.remote(_Boom).remote()
        assert ray.get(h.ping.remote()) == "pong"
        with pytest.raises(ray.ActorError):
            ray.get(h.die.remote(), timeout=20)
        t0 = time.time()
        with pytest.raises(ray.ActorError):
            ray.get(h.ping.remote(), timeout=20)
        assert time.time() - t0 < 10
    finally:
        ray.shutdown()


def test_engine_loop_error_reaches_the_driver():
    """An exception inside the engine's background loop is kept and re-raised by the per-step health check."""
    from open_instruct_b200.actors import ray_compat as ray
    from open_instruct_b200.data_types import PromptRequest, SamplingConfig
    from open_instruct_b200.grpo_fast import EngineWorker
    from open_instruct_b200.models.spec import get_spec

    class BadReward:
        def build(self):
            def fn(*a, **k):
                raise RuntimeError("verifier exploded")
            return fn

    pq, rq = ray.Queue(local=True), ray.Queue(local=True)
    w = EngineWorker(get_spec("tiny"), pq, rq, None, BadReward(), tokenizer=None, device="cpu", ops="ref", num_blocks=64, max_model_len=64)
    try:
        w.check_background_threads()
        pq.put(PromptRequest(prompt=[1, 2, 3], generation_config=SamplingConfig(max_tokens=2, n=1), index=0, prompt_id="p"))
        deadline = time.time() + 20
        while w.error is None and time.time() < deadline:
            time.sleep(0.05)
        with pytest.raises(RuntimeError, match="engine loop died"):
            w.check_background_threads()
    finally:
        w.shutdown()
