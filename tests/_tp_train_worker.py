"""Worker for the training-time tensor-parallel test (gloo ranks on CPU, PyTorch path): a learner whose layers are split
over TP groups of two ranks (data parallel across the groups) must follow the same trajectory as one unsharded process
that sees all the micro-batches."""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.learner import Learner, LearnerConfig  # noqa: E402
from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402


def batch(spec, seed):
    g = torch.Generator().manual_seed(seed)
    lens = [9, 14, 5]
    ids = torch.randint(1, spec.vocab_size, (sum(lens),), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])
    cu = torch.tensor([0, 9, 23, 28], dtype=torch.int32)
    labels = torch.roll(ids, -1)
    labels[cu[1:].long() - 1] = -100
    return {"input_ids": ids, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels}


def main():
    rank, world, device = pdist.init_distributed()
    tp = 2
    dp_world, dp_rank = world // tp, rank // tp
    family = os.environ.get("FAMILY", "llama")
    spec = get_spec("tiny").replace(num_layers=3)
    if family == "qwen3":
        spec = spec.replace(qk_norm=True, attention_bias=True, model_type="qwen3")
    kw = dict(ops="ref", learning_rate=1e-2, weight_decay=0.1, max_grad_norm=1.0, total_steps=10, lr_scheduler_type="constant", seed=4,
              dtype=torch.float32)
    oracle = Learner(spec, LearnerConfig(**kw, comm="none"), device=device, group=pdist.SOLO)
    if family == "qwen3":  # move biases / q-k norm weights off their initial values so that their gradients matter
        with torch.no_grad():
            for name, v in oracle.model.layout.views(oracle.model.flat.detach()).items():
                if name.endswith(("bqkv", "q_norm", "k_norm")):
                    v.add_(0.2 * torch.randn(v.shape, generator=torch.Generator().manual_seed(1)))
            oracle.opt.master.copy_(oracle.model.flat.detach()[oracle.opt.lo:oracle.opt.hi])
    total = ParamLayout(spec).total
    # OPS=emulated: the fused path's hand-driven forward / backward (its all-reduces after the row-parallel projections and
    # before the column-parallel ones' input gradients, the vocabulary-parallel head) over PyTorch restatements of the kernels
    kw_sharded = {**kw, "ops": os.environ.get("OPS", "ref")}
    sharded = Learner(spec, LearnerConfig(**kw_sharded, tensor_parallel_degree=tp), device=device, flat_init=oracle.model.flat.detach()[:total].clone())
    assert sharded.tp is not None and sharded.world == dp_world and sharded.rank == dp_rank
    assert sharded.spec.num_heads == spec.num_heads // tp and sharded.full_spec.num_heads == spec.num_heads
    assert torch.equal(sharded.full_flat(), oracle.model.flat.detach()[:total])   # shard -> unshard round trip
    # the log-prob head runs vocabulary-parallel over the TP group: log-probs and entropy still equal the unsharded model's
    assert sharded.model.vocab_parallel_head()
    b0 = batch(spec, 7)
    with torch.no_grad():
        lp_o, ent_o = oracle.token_logprobs(b0, temperature=0.7, want_entropy=True)
        lp_s, ent_s = sharded.token_logprobs(b0, temperature=0.7, want_entropy=True)
    assert torch.allclose(lp_o, lp_s, atol=1e-5) and torch.allclose(ent_o, ent_s, atol=1e-5)
    for step in range(3):
        want = oracle.sft_step([batch(spec, 100 * step + d) for d in range(dp_world)])
        got = sharded.sft_step([batch(spec, 100 * step + dp_rank)])
        loss = got["loss"].clone()
        if dp_world > 1:
            torch.distributed.all_reduce(loss, group=sharded.group)
            loss /= dp_world
        assert abs(loss.item() - want["loss"].item()) < 1e-4, (step, loss.item(), want["loss"].item())
        assert abs(got["grad_norm"].item() - want["grad_norm"].item()) < 1e-3 * max(1.0, want["grad_norm"].item()), (step, got["grad_norm"], want["grad_norm"])
    full = sharded.full_flat()
    err = (full - oracle.model.flat.detach()[:total]).abs().max().item()
    assert err < 2e-4, err
    pdist.barrier()
    print(f"TP_TRAIN_OK rank={rank}")


if __name__ == "__main__":
    main()
