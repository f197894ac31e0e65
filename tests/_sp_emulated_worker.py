"""Worker for the sequence-parallel test on CPU: gloo ranks, the model's hand-driven forward / backward over PyTorch restatements
of the kernels (``ops="emulated"``), the four head <-> sequence exchanges done with all-gathers (``HostUlyssesContext``).  Every rank
runs the same packed batch through an ordinary model and through the sequence-parallel one that shares its weights: local
log-probs equal the matching chunk of the full ones, gradients summed over the ranks equal the single-rank gradient."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.models import ModelSpec  # noqa: E402
from open_instruct_b200.models.llama import LlamaModel  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402
from open_instruct_b200.parallel.ulysses import HostUlyssesContext  # noqa: E402


def main():
    rank, world, device = pdist.init_distributed()
    base = ModelSpec(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16)
    for ckpt, spec in ((False, base), (True, base), (False, base.replace(attention_bias=True, model_type="qwen2")),
                       (True, base.replace(qk_norm=True, model_type="qwen3")),
                       # OLMo-2 blocks: norm after the sub-layer, q/k norm over ALL heads (completed across the ranks by an all-reduce)
                       (False, base.replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo2")),
                       (True, base.replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo2"))):
        full = LlamaModel(spec, ops="emulated", seed=3, gradient_checkpointing=ckpt)
        with torch.no_grad():
            gen = torch.Generator().manual_seed(11)
            for name, v in full.p.items():
                if name.endswith(("bqkv", "q_norm", "k_norm")):
                    v.add_(torch.randn(v.shape, generator=gen) * 0.1)
        spm = LlamaModel(spec, ops="emulated", flat=full.flat, gradient_checkpointing=ckpt)
        spm.sp = HostUlyssesContext(spec, 256, device)
        g = torch.Generator().manual_seed(5)
        lens = [37, 75, 16]   # 128 tokens; document boundaries do not line up with the rank boundary
        T = sum(lens)
        ids = torch.randint(1, spec.vocab_size, (T,), generator=g)
        pos = torch.cat([torch.arange(n) for n in lens])
        cu = torch.tensor([0, 37, 112, 128], dtype=torch.int32)
        labels = torch.roll(ids, -1)
        labels[cu[1:].long() - 1] = -100
        wts = torch.rand(T, generator=g)
        lp_full, _ = full.token_logprobs(ids, pos, cu, labels)
        (-(lp_full * wts).sum()).backward()
        g_full = full.main_grad.clone()
        lo, hi = spm.sp.local_tokens(T)
        lp_loc, _ = spm.token_logprobs(ids, pos, cu, labels)
        assert lp_loc.shape[0] == T // world
        (-(lp_loc * wts[lo:hi]).sum()).backward()
        assert (lp_loc.detach() - lp_full.detach()[lo:hi]).abs().max().item() < 1e-5
        g_sp = spm.main_grad.clone()
        dist.all_reduce(g_sp)
        assert (g_sp - g_full).abs().max().item() < 1e-4 * max(1.0, g_full.abs().max().item()), (g_sp - g_full).abs().max().item()
    dist.barrier()
    print(f"SP_EMUL_OK rank={rank}")


if __name__ == "__main__":
    main()
