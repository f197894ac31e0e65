"""Worker for sequence parallelism INSIDE a data-parallel world (four ranks under torchrun, one GPU each): Ulysses groups of
two consecutive ranks, two such groups side by side.  The ranks of a group train on the same packed micro-batches (each on
its half of the tokens), the groups on different ones; gradients are exchanged over all four ranks.  Compared with one
unsharded learner that sees all micro-batches - with the parameters resident and with the parameters sharded (the
combination the reference requires for sequence parallelism)."""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.data.collate import to_device  # noqa: E402
from open_instruct_b200.data.synthetic import sft_step_batches  # noqa: E402
from open_instruct_b200.learner import Learner, LearnerConfig  # noqa: E402
from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.ops import lib  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402


def main():
    rank, world, device = pdist.init_distributed()
    assert world == 4
    sp = 2
    dp_rank, dp_world = rank // sp, world // sp
    spec = get_spec("tiny128-tp").replace(num_layers=3, qk_norm=True, model_type="qwen3")
    seq = 512
    kw = dict(ops="fused", learning_rate=1e-3, lr_scheduler_type="constant", max_grad_norm=1.0, weight_decay=0.01, seed=7)
    oracle = Learner(spec, LearnerConfig(comm="none", **kw), device=device, group=pdist.SOLO)
    total = ParamLayout(spec).total
    init = oracle.model.flat.detach()[:total].clone()
    for shard in (None, True):
        oracle.load_full_weights(init)
        oracle.opt.m.zero_(); oracle.opt.v.zero_(); oracle.opt.step_count = 0; oracle.global_step = 0
        lr_ = Learner(spec, LearnerConfig(sequence_parallel_size=sp, sp_max_tokens=seq, shard_parameters=shard, **kw), device=device,
                      flat_init=init.clone())
        assert lr_.sp == sp and (lr_.z3 is not None) == bool(shard)
        for step in range(3):
            mine = [to_device(b, device) for b in sft_step_batches(2, seq, spec.vocab_size, seed=100 * step + dp_rank)]
            every = [to_device(b, device) for g in range(dp_world) for b in sft_step_batches(2, seq, spec.vocab_size, seed=100 * step + g)]
            got, want = lr_.sft_step(mine), oracle.sft_step(every)
            assert abs(float(got["grad_norm"]) - float(want["grad_norm"])) < 3e-2 * max(1.0, float(want["grad_norm"])), (shard, step, got["grad_norm"], want["grad_norm"])
        torch.cuda.synchronize()
        lib.check_status()
        a, b = lr_.full_flat().float()[:total], oracle.model.flat.detach()[:total].float()
        rel = ((a - b).norm() / b.norm()).item()
        assert rel < 1e-2, (shard, rel)
        del lr_
    pdist.barrier()
    if rank == 0:
        print("SP_DP_WORKER_OK")
    pdist.destroy()


if __name__ == "__main__":
    main()
