"""Worker for the training-time tensor-parallel GPU test (two ranks, one GPU each, fused kernels): the TP = 2 learner
against an unsharded learner with the same weights and micro-batches, on every rank."""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.learner import Learner, LearnerConfig  # noqa: E402
from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.ops import lib  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402


def batch(spec, device, seed):
    g = torch.Generator().manual_seed(seed)
    lens = [150, 300, 62]
    ids = torch.randint(1, spec.vocab_size, (sum(lens),), generator=g).to(device)
    pos = torch.cat([torch.arange(n) for n in lens]).to(device)
    cu = torch.tensor([0, 150, 450, 512], dtype=torch.int32, device=device)
    labels = torch.roll(ids, -1)
    labels[cu[1:].long() - 1] = -100
    return {"input_ids": ids, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels}


def main():
    rank, world, device = pdist.init_distributed()
    assert world == 2
    from open_instruct_b200.models import llama

    for ckpt in (False, True):
        # second pass: also push the head through its token-chunked form (512 tokens in chunks of 256, logits recomputed in backward)
        llama.LOGIT_CHUNK_TOKENS = 256 if ckpt else 8192
        spec = get_spec("tiny128-tp").replace(num_layers=3)
        kw = dict(ops="fused", learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0, total_steps=10, lr_scheduler_type="constant", seed=4,
                  gradient_checkpointing=ckpt)
        oracle = Learner(spec, LearnerConfig(**kw, comm="none"), device=device, group=pdist.SOLO)
        total = ParamLayout(spec).total
        tp = Learner(spec, LearnerConfig(**kw, tensor_parallel_degree=2), device=device, flat_init=oracle.model.flat.detach()[:total].clone())
        assert tp.tp is not None and tp.world == 1 and tp.spec.num_heads == spec.num_heads // 2
        assert tp.model.vocab_parallel_head()  # the log-prob head is split over the vocabulary: [T]-sized partials are exchanged
        with torch.no_grad():
            b0 = batch(spec, device, 99)
            lp_o, ent_o = oracle.token_logprobs(b0, temperature=0.8, want_entropy=True)
            lp_t, ent_t = tp.token_logprobs(b0, temperature=0.8, want_entropy=True)
        assert (lp_o - lp_t).abs().max().item() < 5e-2 and (ent_o - ent_t).abs().max().item() < 5e-2
        for step in range(3):
            mbs = [batch(spec, device, 10 * step + i) for i in range(2)]
            want, got = oracle.sft_step(mbs), tp.sft_step(mbs)
            assert abs(want["loss"].item() - got["loss"].item()) < 2e-2 * max(1.0, abs(want["loss"].item())), (step, want["loss"], got["loss"])
            assert abs(want["grad_norm"].item() - got["grad_norm"].item()) < 3e-2 * max(1.0, want["grad_norm"].item()), (step, want["grad_norm"], got["grad_norm"])
        torch.cuda.synchronize()
        lib.check_status()
        a, b = tp.full_flat().float(), oracle.model.flat.detach()[:total].float()
        rel = ((a - b).norm() / b.norm()).item()
        # bf16 partial sums are added in another order than the unsharded GEMM rounds: Adam turns sign flips of tiny gradients
        # into full-size steps, so the weights agree to a fraction of a percent, not bitwise
        assert rel < 1e-2, rel
    pdist.barrier()
    print(f"TP_TRAIN_GPU_OK rank={rank}")


if __name__ == "__main__":
    main()
