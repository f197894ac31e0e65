"""Worker for the parameter-sharding test: gloo ranks on CPU drive ``Zero3State`` through the hook sequence the model
engine issues (two micro-batches per step, two steps) with synthetic gradients, and compare the gathered result with a
single-process resident optimizer fed the summed gradients."""

import os
import sys
import types

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402
from open_instruct_b200.parallel.zero import ZeroOptimizer, padded_numel  # noqa: E402
from open_instruct_b200.parallel.zero3 import Zero3State  # noqa: E402


def synthetic_grad(p: torch.Tensor, rank: int, mb: int) -> torch.Tensor:
    return 0.01 * (rank + 1) * p + 0.001 * (mb + 1)


def close(a, b):
    return torch.allclose(a, b, rtol=1e-5, atol=1e-6)  # after the first step the two sides differ by summation order


def main():
    rank, world, device = pdist.init_distributed()
    spec = get_spec("tiny").replace(num_layers=5, tie_word_embeddings=(os.environ.get("TIED", "0") == "1"))
    layout = ParamLayout(spec)
    L = spec.num_layers
    torch.manual_seed(0)
    full = torch.randn(layout.total)
    for e in layout.entries.values():  # alignment gaps are zero in a real model
        full[e.offset + e.numel:(e.offset + e.numel + 127) // 128 * 128] = 0
    hyper = dict(lr=1e-2, weight_decay=0.1, max_grad_norm=0.5)

    shard_degree = int(os.environ.get("SHARD_DEGREE", "0"))
    groups = {}
    if shard_degree:  # hybrid: shard groups of ``shard_degree`` ranks, replicated world / shard_degree times
        sg, rg = pdist.hsdp_groups(shard_degree)
        groups = dict(group=sg, replica_group=rg)
    z = Zero3State(layout, device, torch.float32, use_kernels=False, **hyper, **groups)
    assert z.world == (shard_degree or world)
    z.load_full(full)
    model = types.SimpleNamespace()
    z.attach(model)

    # oracle: one process, resident parameters, gradients summed over the ranks
    n = padded_numel(layout.total, 1)
    ref_flat = torch.zeros(n)
    ref_flat[:layout.total] = full
    oracle = ZeroOptimizer(ref_flat, layout.total, layout.decay_end, group=pdist.SOLO, comm="none", use_kernels=False, **hyper)

    head = "lm_head" if "lm_head" in layout.entries else "embed"
    for step in range(2):
        ref_grad = torch.zeros(n)
        rv, rg = layout.views(ref_flat), layout.views(ref_grad)
        for mb in range(2):
            z.fwd_begin()
            assert close(model.p["embed"], rv["embed"])
            for i in range(L):
                z.layer_fwd(i)
                for leaf in ("wqkv", "wo", "w_gate_up", "w_down", "attn_norm", "mlp_norm"):
                    assert close(model.p[f"l{i}.{leaf}"], rv[f"l{i}.{leaf}"]), (step, mb, i, leaf)
            z.head()
            assert close(model.p[head], rv[head])
            model.g[head] += synthetic_grad(model.p[head], rank, mb)
            model.g["final_norm"] += synthetic_grad(model.p["final_norm"], rank, mb)
            for i in reversed(range(L)):
                z.layer_bwd(i)
                for leaf in ("wqkv", "wo", "w_gate_up", "w_down", "attn_norm", "mlp_norm"):
                    assert close(model.p[f"l{i}.{leaf}"], rv[f"l{i}.{leaf}"]), (step, mb, i, leaf, "bwd")
                    gr = synthetic_grad(model.p[f"l{i}.{leaf}"], rank, mb)
                    if leaf.endswith("norm"):
                        model.g[f"l{i}.{leaf}"] += gr      # replicated tail: accumulates until the step
                    else:
                        model.g[f"l{i}.{leaf}"].copy_(gr)  # layer workspace: overwritten per micro-batch, reduced right away
                z.layer_bwd_done(i)
            model.g["embed"] += 0.5 * synthetic_grad(model.p["embed"], rank, mb)
            for r in range(world):  # what every rank contributed
                for name in layout.entries:
                    k = 1.0 + (0.5 if name == "embed" else 0.0) * (1 if head == "embed" else 0) - (0.5 if (name == "embed" and head != "embed") else 0.0)
                    rg[name] += k * synthetic_grad(rv[name], r, mb)
        # the backward reuses the two layers still resident after the forward, and the next micro-batch's forward the two
        # left by the backward; an optimizer step invalidates everything
        assert z.gather_count == (step + 1) * ((L + L - 2) + (L - 2 + L - 2)), z.gather_count
        norm = z.step(lr=1e-2, grad_scale=0.25)
        want_norm = oracle.step(ref_grad, lr=1e-2, grad_scale=0.25)
        assert torch.allclose(norm, want_norm, rtol=1e-5), (norm, want_norm)
        got = z.gather_full()
        assert torch.allclose(got, ref_flat[:layout.total], rtol=1e-5, atol=1e-6), (step, (got - ref_flat[:layout.total]).abs().max())
    sd = z.state_dict()
    z.load_state_dict(sd)
    pdist.barrier()
    print(f"ZERO3_OK rank={rank}")


if __name__ == "__main__":
    main()
