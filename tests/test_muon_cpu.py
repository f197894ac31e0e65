"""Muon (orthogonalised momentum for the decoder matrices, AdamW elsewhere) on the sharded flat buffer."""
import os
import subprocess
import sys

import pytest

from helpers import free_port

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [1, 2, 3])
def test_muon_sharded_equals_single_process_and_plain_statement(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "_muon_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("MUON_OK") == world


def test_muon_through_the_dpo_trainer_config():
    """`optimizer_type muon` reaches the learner (it used to be parsed and ignored); combinations that are not built refuse."""
    import torch

    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.parallel.muon import MuonOptimizer

    spec = get_spec("tiny128").replace(num_layers=1)
    lr = Learner(spec, LearnerConfig(ops="ref", optimizer_type="muon", optimizer_kwargs={"mu": 0.9}, learning_rate=1e-2), device="cpu")
    assert isinstance(lr.opt, MuonOptimizer) and lr.opt.mu == 0.9
    before = lr.model.flat.detach().clone()
    ids = torch.randint(0, spec.vocab_size, (64,))
    lp, _ = lr.model.token_logprobs(ids, torch.arange(64), torch.tensor([0, 64], dtype=torch.int32), torch.cat([ids[1:], torch.tensor([-100])]))
    lr.backward(-lp.sum() / 63)
    lr.optimizer_step()
    assert not torch.equal(before, lr.model.flat.detach())
    with pytest.raises(ValueError):
        Learner(spec, LearnerConfig(ops="ref", optimizer_type="lion"), device="cpu")
    with pytest.raises(NotImplementedError):
        Learner(spec, LearnerConfig(ops="ref", optimizer_type="muon", offload_optimizer=True), device="cpu")
