"""Worker for sequence parallelism inside a data-parallel world on CPU: four gloo ranks, Ulysses groups of two consecutive
ranks, the learner's hand-driven path over PyTorch restatements of the kernels.  The ranks of a group train on the same packed
micro-batches (each on its half of the tokens), the groups on different ones; gradients are exchanged over all four ranks.
Compared with one unsharded learner that sees all micro-batches - with resident and with sharded parameters, for Qwen3-style
per-head q/k norm and for OLMo-2 blocks (q/k norm over all heads)."""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.data.synthetic import sft_step_batches  # noqa: E402
from open_instruct_b200.learner import Learner, LearnerConfig  # noqa: E402
from open_instruct_b200.models import ModelSpec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402


def main():
    rank, world, device = pdist.init_distributed()
    assert world == 4
    sp = 2
    dp_rank, dp_world = rank // sp, world // sp
    base = ModelSpec(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16)
    seq = 128
    for spec in (base.replace(qk_norm=True, model_type="qwen3"), base.replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo2")):
        kw = dict(learning_rate=1e-2, lr_scheduler_type="constant", max_grad_norm=1.0, weight_decay=0.01, seed=7, dtype=torch.float32)
        oracle = Learner(spec, LearnerConfig(ops="ref", comm="none", **kw), device=device, group=pdist.SOLO)
        total = ParamLayout(spec).total
        init = oracle.model.flat.detach()[:total].clone()
        for shard in (False, True):
            oracle.load_full_weights(init)
            oracle.opt.m.zero_(); oracle.opt.v.zero_(); oracle.opt.step_count = 0; oracle.global_step = 0
            lr_ = Learner(spec, LearnerConfig(ops="emulated", sequence_parallel_size=sp, sp_max_tokens=seq, shard_parameters=shard, **kw),
                          device=device, flat_init=init.clone())
            assert lr_.sp == sp and (lr_.z3 is not None) == shard
            for step in range(3):
                mine = sft_step_batches(2, seq, spec.vocab_size, seed=100 * step + dp_rank)
                every = [b for g in range(dp_world) for b in sft_step_batches(2, seq, spec.vocab_size, seed=100 * step + g)]
                got, want = lr_.sft_step(mine), oracle.sft_step(every)
                assert abs(float(got["grad_norm"]) - float(want["grad_norm"])) < 1e-3 * max(1.0, float(want["grad_norm"])), (spec.model_type, shard, step, got["grad_norm"], want["grad_norm"])
            a, b = lr_.full_flat().float()[:total], oracle.model.flat.detach()[:total].float()
            lay = ParamLayout(spec)
            worst = max(((lay.view(a, n) - lay.view(b, n)).abs().max().item(), n) for n in lay.entries)
            moved = (b - init.float()).abs().max().item()
            # Adam divides by the gradient's own scale: entries whose gradient is rounding noise may differ by a step or so
            assert worst[0] < 0.05 * moved, (spec.model_type, shard, worst, moved)
            assert ((a - b).norm() / (b - init.float()).norm()).item() < 0.02, (spec.model_type, shard, worst)
            del lr_
    pdist.barrier()
    print(f"SP_DP_EMUL_OK rank={rank}")
    pdist.destroy()


if __name__ == "__main__":
    main()
