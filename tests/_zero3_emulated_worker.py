"""Worker for the parameter-sharding test with the real model: gloo ranks on CPU, the fused path's driver over PyTorch restatements
of the kernels (``ops="emulated"``), parameters sharded over the ranks (each layer gathered before use, its gradients reduced
right after its backward); must follow one unsharded process that sees every rank's micro-batches."""

import os, sys, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from open_instruct_b200.learner import Learner, LearnerConfig
from open_instruct_b200.models import ModelSpec
from open_instruct_b200.models.spec import ParamLayout
from open_instruct_b200.parallel import dist as pdist
def batch(spec, seed):
    g = torch.Generator().manual_seed(seed); lens = [40, 70, 18]
    ids = torch.randint(1, spec.vocab_size, (sum(lens),), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens]); cu = torch.tensor([0, 40, 110, 128], dtype=torch.int32)
    labels = torch.roll(ids, -1); labels[cu[1:].long() - 1] = -100
    return {"input_ids": ids, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels}
rank, world, device = pdist.init_distributed()
spec = ModelSpec(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16)
kw = dict(learning_rate=1e-2, weight_decay=0.1, max_grad_norm=1.0, total_steps=10, lr_scheduler_type="constant", seed=4, dtype=torch.float32)
oracle = Learner(spec, LearnerConfig(ops="ref", comm="none", **kw), device=device, group=pdist.SOLO)
total = ParamLayout(spec).total
sh = Learner(spec, LearnerConfig(ops="emulated", shard_parameters=True, gradient_checkpointing=(os.environ.get("CKPT") == "1"), **kw), device=device,
             flat_init=oracle.model.flat.detach()[:total].clone())
assert sh.z3 is not None
for step in range(3):
    want = oracle.sft_step([batch(spec, 100 * step + 10 * mb + r) for r in range(world) for mb in range(2)])
    got = sh.sft_step([batch(spec, 100 * step + 10 * mb + rank) for mb in range(2)])
    assert abs(got["grad_norm"].item() - want["grad_norm"].item()) < 1e-3 * max(1.0, want["grad_norm"].item()), (step, got["grad_norm"], want["grad_norm"])
err = (sh.full_flat()[:total].float() - oracle.model.flat.detach()[:total]).abs().max().item()
assert err < 2e-4, err
pdist.barrier(); print(f"Z3_EMUL_OK rank={rank} err={err:.2e}")
