"""Worker for the sequence-parallel (Ulysses) test: two ranks under torchrun, one GPU each.

Every rank runs the same packed batch (a) through an ordinary single-GPU fused model and (b) through the
sequence-parallel model that shares its weights.  Checks: local log-probs equal the matching chunk of the full
log-probs, and the gradients summed over the two ranks equal the single-GPU gradient.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.llama import LlamaModel  # noqa: E402
from open_instruct_b200.ops import lib  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402
from open_instruct_b200.parallel.ulysses import UlyssesContext  # noqa: E402


def main():
    rank, world, device = pdist.init_distributed()
    base = get_spec("tiny128").replace(num_heads=4, num_kv_heads=2, hidden_size=512, intermediate_size=1024, num_layers=3)
    # plain Llama blocks with and without activation checkpointing, then the families with extras on the fused projection:
    # Qwen2-style q/k/v bias and Qwen3 / OLMo-2 style per-head q/k RMSNorm (applied to this rank's heads after the exchange)
    for ckpt, spec in ((False, base), (True, base), (False, base.replace(attention_bias=True, model_type="qwen2")),
                       (True, base.replace(qk_norm=True, model_type="qwen3"))):
        full = LlamaModel(spec, device=device, dtype=torch.bfloat16, ops="fused", seed=3, gradient_checkpointing=ckpt)
        if spec.attention_bias or spec.qk_norm:
            with torch.no_grad():  # biases start at zero and norm weights at one: move them so that they matter
                gen = torch.Generator(device=device).manual_seed(11)
                for name, v in full.p.items():
                    if name.endswith(("bqkv", "q_norm", "k_norm")):
                        v.add_((torch.randn(v.shape, device=device, generator=gen) * 0.1).to(v.dtype))
        spm = LlamaModel(spec, device=device, dtype=torch.bfloat16, ops="fused", flat=full.flat, gradient_checkpointing=ckpt)
        spm.sp = UlyssesContext(spec, 1024, device)
        g = torch.Generator().manual_seed(5)
        lens = [150, 300, 62]  # 512 tokens; document boundaries do not line up with the rank boundary
        T = sum(lens)
        ids = torch.randint(1, spec.vocab_size, (T,), generator=g).to(device)
        pos = torch.cat([torch.arange(n) for n in lens]).to(device)
        cu = torch.tensor([0, 150, 450, 512], dtype=torch.int32, device=device)
        labels = torch.roll(ids, -1)
        labels[cu[1:].long() - 1] = -100
        wts = torch.rand(T, generator=g).to(device)  # a non-uniform loss so that errors cannot cancel

        lp_full, _ = full.token_logprobs(ids, pos, cu, labels)
        (-(lp_full * wts).sum()).backward()
        g_full = full.main_grad.clone()

        lo, hi = spm.sp.local_tokens(T)
        lp_loc, _ = spm.token_logprobs(ids, pos, cu, labels)
        assert lp_loc.shape[0] == T // world
        (-(lp_loc * wts[lo:hi]).sum()).backward()
        torch.cuda.synchronize()
        lib.check_status()
        err = (lp_loc.detach() - lp_full.detach()[lo:hi]).abs().max().item()
        assert err < 5e-2, f"log-prob mismatch {err}"
        g_sp = spm.main_grad.clone()
        dist.all_reduce(g_sp)
        num = (g_sp - g_full).norm().item()
        den = g_full.norm().item()
        assert num / den < 2e-2, f"gradient mismatch: relative error {num / den}"
        # per-entry check on the attention weights, where the exchanges matter
        extra = (["l1.bqkv"] if spec.attention_bias else []) + (["l0.q_norm", "l2.k_norm"] if spec.qk_norm else [])
        for name in ["l0.wqkv", "l1.wo", "l2.w_down", "embed"] + extra:
            a, b = full.layout.view(g_sp, name), full.layout.view(g_full, name)
            rel = ((a - b).norm() / b.norm().clamp(min=1e-12)).item()
            assert rel < 3e-2, (name, rel)
        del full, spm
    dist.barrier()
    if rank == 0:
        print("SP_WORKER_OK")


if __name__ == "__main__":
    main()
