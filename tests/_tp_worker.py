"""Worker for the tensor-parallel rollout test (two ranks under torchrun, one GPU each).

Checks, on every rank: (1) the fused all-reduce + residual + RMSNorm kernel against a PyTorch fp32 reference of the same
op computed from both ranks' partials (exchanged with NCCL); (2) the TP=2 engine's final hidden states and greedy-ish
generations against an unsharded engine with the same weights; (3) a wait on a peer that never signals ends with the
timeout status instead of hanging (rank 1 simply does not launch the kernel for that epoch).
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.data_types import SamplingConfig  # noqa: E402
from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.llama import LlamaModel  # noqa: E402
from open_instruct_b200.ops import lib  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402
from open_instruct_b200.parallel.tp import TPContext, local_spec, shard_flat  # noqa: E402
from open_instruct_b200.rollout.engine import RolloutEngine  # noqa: E402


def main():
    rank, world, device = pdist.init_distributed()
    assert world == 2
    spec = get_spec("tiny128").replace(num_heads=4, num_kv_heads=2, hidden_size=512, intermediate_size=1024)
    D = spec.hidden_size
    tp = TPContext(D, 4096, device)

    # (1) kernel numerics, several sizes, with and without residual / weight
    g = torch.Generator(device=device).manual_seed(7 + rank)
    for B in (1, 5, 130, 1000):
        part = tp.out_buffer(B)
        part.copy_(torch.randn(B, D, device=device, generator=g).bfloat16())
        res = torch.randn(B, D, device=device, generator=torch.Generator(device=device).manual_seed(B)).bfloat16()
        w = (torch.rand(D, device=device, generator=torch.Generator(device=device).manual_seed(3)) + 0.5).bfloat16()
        both = [torch.empty_like(part) for _ in range(2)]
        dist.all_gather(both, part.clone())
        y, h = tp.reduce_norm(part, w, 1e-5, res=res)
        h_ref = (both[0].float() + both[1].float() + res.float())
        hb = h_ref.bfloat16()
        y_ref = hb.float() * torch.rsqrt(hb.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        torch.cuda.synchronize()
        lib.check_status()
        assert torch.equal(h, hb), (B, (h.float() - hb.float()).abs().max())
        assert torch.allclose(y.float(), y_ref, atol=2e-2, rtol=2e-2), (B, (y.float() - y_ref).abs().max())

    # (1b) row-parallel GEMM with the peer push fused into its epilogue, then the purely local reduction
    for T in (300, 1000):
        gx = torch.Generator(device=device).manual_seed(100 + rank)
        x = torch.randn(T, 384, device=device, generator=gx).bfloat16()
        w = (torch.randn(D, 384, device=device, generator=gx) * 0.05).bfloat16()
        res = torch.randn(T, D, device=device, generator=torch.Generator(device=device).manual_seed(T)).bfloat16()
        nw = (torch.rand(D, device=device, generator=torch.Generator(device=device).manual_seed(3)) + 0.5).bfloat16()
        part = tp.row_gemm(x, w)
        y, h = tp.reduce_norm(part, nw, 1e-5, res=res)
        torch.cuda.synchronize()
        lib.check_status()
        mine = (x.float() @ w.float().t()).bfloat16()
        both = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(both, mine)
        hb = (both[0].float() + both[1].float() + res.float()).bfloat16()
        assert (h.float() - hb.float()).abs().max() < 0.06, (T, (h.float() - hb.float()).abs().max())

    # (2) engine: TP=2 against the unsharded engine (prefill through the fused peer push as well as the default pull)
    os.environ["B200_TP_PUSH"] = "1"
    full = LlamaModel(spec, device=device, dtype=torch.bfloat16, ops="fused", seed=11).flat.detach()
    ref_eng = RolloutEngine(spec, device=device, num_blocks=64, flat=full.clone(), eos_token_ids=[], seed=5)
    ls = local_spec(spec, 2)
    tp_eng = RolloutEngine(ls, device=device, num_blocks=64, flat=shard_flat(full, spec, rank, 2), eos_token_ids=[], seed=5, tp=tp)
    prompts = [[(7 * i + j) % (spec.vocab_size - 1) + 1 for j in range(20 + 150 * i)] for i in range(3)]  # 20 + 170 + 320 > 256: pushed path
    cfg = SamplingConfig(temperature=0.01, top_p=1.0, max_tokens=12, n=1, seed=123)
    a = ref_eng.generate(prompts, cfg)
    b = tp_eng.generate(prompts, cfg)
    torch.cuda.synchronize()
    lib.check_status()
    same = sum(int(x.responses[0] == y.responses[0]) for x, y in zip(a, b))
    toks = [torch.tensor(y.responses[0], device=device) for y in b]
    other = [torch.empty_like(t) for t in toks]
    for t, o in zip(toks, other):
        lst = [torch.empty_like(t) for _ in range(2)]
        dist.all_gather(lst, t)
        assert torch.equal(lst[0], lst[1]), "TP ranks sampled different tokens"
    assert same >= 2, f"only {same}/3 generations match the unsharded engine"

    # (3) bounded wait: rank 1 does not arrive
    tp.peer_timeout_ms = 300
    if rank == 0:
        part = tp.out_buffer(4)
        part.zero_()
        tp.reduce_norm(part, None, 1e-5, res=None)
        torch.cuda.synchronize()
        st = int(lib.status_word(device).item())
        assert st != 0, "expected a peer timeout status"
        lib.status_word(device).zero_()
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK")


if __name__ == "__main__":
    main()
