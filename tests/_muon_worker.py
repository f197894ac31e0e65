"""torchrun worker (gloo): Muon on WORLD ranks must equal Muon on one process, step for step, and both must equal a plain
PyTorch statement of the update written without the flat buffer."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.models.spec import ParamLayout  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402
from open_instruct_b200.parallel.muon import MuonOptimizer, muon_matrices, newton_schulz  # noqa: E402
from open_instruct_b200.parallel.zero import padded_numel  # noqa: E402


def main():
    rank, world, _ = pdist.init_distributed(backend="gloo")
    spec = get_spec("tiny128").replace(num_layers=2)
    layout = ParamLayout(spec)
    mats = muon_matrices(layout)
    assert len(mats) == 2 * 7  # q, k, v, o, gate, up, down per layer
    n = padded_numel(layout.total, world)
    g = torch.Generator().manual_seed(0)
    w0 = torch.randn(n, generator=g) * 0.05
    w0[layout.total:] = 0
    hyper = dict(lr=0.02, weight_decay=0.1, max_grad_norm=1.0, mu=0.9, nesterov=True, ns_steps=5)
    flat = w0.clone()
    opt = MuonOptimizer(flat, layout.total, layout.decay_end, mats, comm="none" if world == 1 else "nccl", use_kernels=False, **hyper)
    solo_flat = torch.zeros(padded_numel(layout.total, 1))
    solo_flat[: layout.total] = w0[: layout.total]
    solo = MuonOptimizer(solo_flat, layout.total, layout.decay_end, mats, group=pdist.SOLO, comm="none", use_kernels=False, **hyper)
    # plain statement: per-tensor masters and moments
    W = w0[: layout.total].clone()
    mom = torch.zeros_like(W)
    ex, ex2 = torch.zeros_like(W), torch.zeros_like(W)
    in_matrix = torch.zeros(layout.total, dtype=torch.bool)
    for s, r, c in mats:
        in_matrix[s:s + r * c] = True
    for step in range(1, 4):
        grads = [torch.randn(layout.total, generator=torch.Generator().manual_seed(100 * step + r)) for r in range(world)]
        mean = torch.stack(grads).sum(0) / world
        mine = torch.zeros(n)
        mine[: layout.total] = grads[rank]
        opt.step(mine, grad_scale=1.0 / world)
        sg = torch.zeros(solo_flat.numel())
        sg[: layout.total] = torch.stack(grads).sum(0)
        solo.step(sg, grad_scale=1.0 / world)
        # the plain statement
        gn = mean.double().norm().float()
        gcl = mean * torch.clamp(hyper["max_grad_norm"] / (gn + 1e-6), max=1.0)
        for s, r, c in mats:
            sl = slice(s, s + r * c)
            mom[sl] = hyper["mu"] * mom[sl] + gcl[sl]
            u = gcl[sl] + hyper["mu"] * mom[sl]
            O = newton_schulz(u.view(r, c), 5).reshape(-1)
            W[sl] = W[sl] * (1 - hyper["lr"] * hyper["weight_decay"]) - hyper["lr"] * max(1.0, r / c) ** 0.5 * O
        rest = ~in_matrix
        ex[rest] = 0.9 * ex[rest] + 0.1 * gcl[rest]
        ex2[rest] = 0.999 * ex2[rest] + 0.001 * gcl[rest] ** 2
        decay = torch.zeros(layout.total)
        decay[: layout.decay_end] = hyper["weight_decay"]
        upd = (ex / (1 - 0.9 ** step)) / ((ex2 / (1 - 0.999 ** step)).sqrt() + 1e-8)
        W[rest] = (W * (1 - hyper["lr"] * decay) - hyper["lr"] * upd)[rest]
        assert torch.allclose(solo_flat[: layout.total], W, atol=2e-5, rtol=1e-4), (step, (solo_flat[: layout.total] - W).abs().max())
        assert torch.allclose(flat[: layout.total], solo_flat[: layout.total], atol=2e-5, rtol=1e-4), (step, (flat[: layout.total] - solo_flat[: layout.total]).abs().max())
    # orthogonalisation really happened: the update of a matrix has roughly equal singular values
    s, r, c = mats[3]
    sv = torch.linalg.svdvals(newton_schulz(torch.randn(r, c), 5))
    assert sv.max() < 1.3 and 0.7 < sv.median() < 1.3 and (sv > 0.5).float().mean() > 0.85, sv  # the smallest few converge slowly
    print(f"MUON_OK rank {rank}", flush=True)
    if dist.is_initialized():
        dist.barrier()


if __name__ == "__main__":
    main()
