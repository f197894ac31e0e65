"""Worker for the parameter-sharding GPU test (one rank per GPU; also run as a single process).

Three learners start from the same weights and see the same micro-batches (different per rank): the resident design
(NCCL exchange), parameter sharding over NCCL and parameter sharding over this package's peer kernels.  Their losses,
gradient norms and final weights must agree to bf16 rounding; checkpoint round trip included."""

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
    for tied, ckpt in ((False, False), (True, True)):
        spec = get_spec("tiny128").replace(num_heads=4, num_kv_heads=2, hidden_size=512, intermediate_size=1024, num_layers=5,
                                           tie_word_embeddings=tied)
        layout = ParamLayout(spec)
        torch.manual_seed(11)
        init = (torch.randn(layout.total) * 0.02).bfloat16()
        for n, e in layout.entries.items():
            if n.endswith("norm"):
                init[e.offset:e.offset + e.numel] = 1.0
        kw = dict(ops="fused", learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0, total_steps=10, lr_scheduler_type="constant",
                  gradient_checkpointing=ckpt)
        variants = {"resident": dict(comm="nccl" if world > 1 else "none", shard_parameters=False),
                    "z3_nccl": dict(comm="nccl" if world > 1 else "none", shard_parameters=True)}
        if world > 1:
            variants["z3_peer"] = dict(comm="fused", shard_parameters=True)      # gather by the copy engines
            variants["z3_peer_sm"] = dict(comm="fused", shard_parameters=True)   # gather by the pull kernel
            variants["z3_peer_mm"] = dict(comm="fused", shard_parameters=True)   # reduction by multimem.ld_reduce (if the fabric offers it)
        out = {}
        for name, v in variants.items():
            os.environ["B200_Z3_GATHER"] = "sm" if name == "z3_peer_sm" else "ce"
            os.environ["B200_MULTIMEM"] = "1" if name == "z3_peer_mm" else "0"
            L = Learner(spec, LearnerConfig(**kw, **v), device=device, flat_init=init.to(device))
            assert (L.z3 is not None) == v["shard_parameters"]
            if name.startswith("z3_peer"):
                assert L.z3.peer is not None and L.z3.peer.gather_mode == ("sm" if name == "z3_peer_sm" else "ce")
            trace = []
            for step in range(3):
                r = L.sft_step([batch(spec, device, 100 * step + 10 * mb + rank) for mb in range(2)])
                trace.append((r["loss"].item(), r["grad_norm"].item()))
            torch.cuda.synchronize()
            lib.check_status()
            out[name] = (trace, L.full_flat().float()[:layout.total].clone())
            if name == "z3_nccl":  # checkpoint round trip of the sharded state
                sd = {k: (t.clone() if torch.is_tensor(t) else t) for k, t in L.opt.state_dict().items()}
                L.opt.load_state_dict(sd)
                again = L.full_flat().float()[:layout.total]
                assert torch.equal(again, out[name][1])
            del L
            torch.cuda.empty_cache()
        ref_trace, ref_w = out["resident"]
        for name, (trace, w) in out.items():
            for (l0, n0), (l1, n1) in zip(ref_trace, trace):
                assert abs(l0 - l1) < 2e-2 * max(1.0, abs(l0)), (name, ref_trace, trace)
                assert abs(n0 - n1) < 3e-2 * max(1.0, abs(n0)), (name, ref_trace, trace)
            rel = ((w - ref_w).norm() / ref_w.norm()).item()
            assert rel < 2e-3, (name, rel)
    pdist.barrier()
    print(f"ZERO3_GPU_OK rank={rank}")


if __name__ == "__main__":
    main()
