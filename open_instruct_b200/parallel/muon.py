"""Muon on the sharded flat parameter buffer.

The reference offers Muon next to AdamW in its olmo-core DPO trainer (``open_instruct/dpo.py:259-268``,
``open_instruct/dpo_utils.py:125-128``: ``optimizer_type``, ``optimizer_kwargs``).  Muon replaces AdamW's elementwise step for
the 2-D weight matrices of the decoder layers by an orthogonalised momentum step:

    m  <- mu * m + g                      (momentum; g is the clipped mean gradient)
    u  <- g + mu * m   (Nesterov) or m
    O  <- NewtonSchulz5(u)                (five iterations of X <- aX + (bA + cA^2)X, A = X X^T, on the normalised matrix)
    W  <- W * (1 - lr * wd) - lr * sqrt(max(1, rows / cols)) * O

Embeddings, the output head, norm weights and biases keep AdamW.

How it fits the sharded optimizer: states stay what ``ZeroOptimizer`` holds - this rank's contiguous slice of master
weights, ``m`` (momentum for matrix entries, Adam's first moment elsewhere) and ``v`` (unused for matrix entries).  Momentum is
elementwise, so it is updated on the slice.  Orthogonalisation needs whole matrices: the slices of ``u`` are all-gathered
(bf16, one collective), every rank runs Newton-Schulz for the matrices that INTERSECT its slice and applies the part of ``O``
that falls inside it.  A matrix cut by a slice boundary is orthogonalised by both neighbours (at most ``world - 1`` of some
230 matrices); the work per rank is otherwise proportional to its slice.  q / k / v and gate / up are separate matrices,
as in a checkpoint with unfused projections.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import ref
from .zero import ZeroOptimizer

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def muon_matrices(layout) -> list[tuple[int, int, int]]:
    """(flat offset, rows, cols) of every matrix Muon treats: the decoder layers' projections, unfused."""
    out = []
    for name, e in layout.entries.items():
        if "." not in name or name.split(".", 1)[1] not in ("wqkv", "wo", "w_gate_up", "w_down"):
            continue
        cols = e.shape[1]
        for _, r0, r1 in layout.hf_names(name):
            out.append((e.offset + r0 * cols, r1 - r0, cols))
    return sorted(out)


def newton_schulz(x: torch.Tensor, steps: int = 5, use_kernels: bool = False) -> torch.Tensor:
    """Approximate orthogonalisation of a 2-D matrix (the polar factor's direction), quintic Newton-Schulz iteration.
    Works on the wide orientation (rows <= cols) so that ``A = X X^T`` is the small square."""
    a, b, c = NS_COEFFS
    tall = x.shape[0] > x.shape[1]
    dt = torch.bfloat16 if x.is_cuda else torch.float32
    X = (x.t() if tall else x).to(dt).contiguous()
    X = X / (X.float().norm() + 1e-7).to(dt)
    kern = use_kernels and X.is_cuda and X.shape[0] % 8 == 0 and X.shape[1] % 8 == 0
    if kern:
        from ..ops import fused
    for _ in range(steps):
        if kern:
            A = fused.gemm(X, X)                  # X X^T  (second operand read as [N, K])
            B = b * A + c * fused.gemm(A, A)      # A is symmetric: A A^T = A^2
            X = a * X + fused.gemm(B, X, b_mn=True)  # B X   (second operand stored [K, N])
        else:
            A = X @ X.t()
            B = b * A + c * (A @ A)
            X = a * X + B @ X
    return X.t() if tall else X


class MuonOptimizer(ZeroOptimizer):
    """``ZeroOptimizer`` whose step is Muon for the ranges in ``matrices`` and AdamW for everything else.

    ``mu`` momentum, ``nesterov``, ``ns_steps`` Newton-Schulz iterations, ``adamw_lr_scale`` multiplies the learning rate of the
    AdamW-treated entries (1.0: same schedule).  Exchanges go through ``torch.distributed`` (``comm`` 'nccl' / 'none')."""

    def __init__(self, flat, total, decay_end, matrices, *, mu: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 adamw_lr_scale: float = 1.0, **kw):
        if kw.get("comm") == "fused":
            raise ValueError("Muon exchanges its momentum through torch.distributed: use comm='nccl' (or 'none' on one rank)")
        if kw.get("offload"):
            raise NotImplementedError("Muon with host-offloaded optimizer states is not built")
        super().__init__(flat, total, decay_end, **kw)
        self.matrices = [(s, r, c) for (s, r, c) in matrices if s < self.hi and s + r * c > self.lo]  # those touching my slice
        self.mu, self.nesterov, self.ns_steps, self.adamw_lr_scale = mu, nesterov, ns_steps, adamw_lr_scale
        self._ubuf = None

    def _adamw_ranges(self):
        """(start, end, weight decay) pieces of my slice (slice-local) outside every Muon matrix."""
        cuts = sorted((max(s, self.lo) - self.lo, min(s + r * c, self.hi) - self.lo) for (s, r, c) in self.matrices)
        out = []
        for a, b, wd in self._segments():
            pos = a
            for c0, c1 in cuts:
                if c1 <= pos or c0 >= b:
                    continue
                if c0 > pos:
                    out.append((pos, c0, wd))
                pos = max(pos, c1)
            if pos < b:
                out.append((pos, b, wd))
        return out

    @torch.no_grad()
    def step(self, grad: torch.Tensor, lr: float | None = None, grad_scale: float = 1.0, norm_sq: torch.Tensor | None = None) -> torch.Tensor:
        lr = self.lr if lr is None else lr
        self.step_count += 1
        gs = self._reduce_scatter(grad, grad_scale)
        if norm_sq is not None:
            self._norm_sq.copy_(norm_sq)
        else:
            self._norm_sq.copy_(gs.double().pow(2).sum().float().reshape(1))
            if self.world > 1:
                dist.all_reduce(self._norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        norm = self._norm_sq.sqrt() * grad_scale
        self.last_grad_norm = norm
        if self.max_grad_norm is not None and self.max_grad_norm > 0:
            self._gscale.copy_(torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0) * grad_scale)
        else:
            self._gscale.fill_(grad_scale)
        my_flat = self.flat[self.lo:self.hi]
        # ---- momentum on my slice of every matrix, then the direction u for all ranks
        if self._ubuf is None:
            self._ubuf = torch.zeros(self.shard * self.world, dtype=torch.bfloat16 if self.flat.is_cuda else torch.float32, device=self.device)
        u_mine = self._ubuf[self.lo:self.hi]
        for (s, r, c) in self.matrices:
            a, b = max(s, self.lo) - self.lo, min(s + r * c, self.hi) - self.lo
            g = gs[a:b] * self._gscale
            self.m[a:b].mul_(self.mu).add_(g)
            u_mine[a:b].copy_(g.add_(self.m[a:b], alpha=self.mu) if self.nesterov else self.m[a:b])
        if self.world > 1:
            if self._ubuf.is_cuda:
                dist.all_gather_into_tensor(self._ubuf, u_mine.clone(), group=self.group)
            else:
                parts = [torch.empty_like(u_mine) for _ in range(self.world)]
                dist.all_gather(parts, u_mine.contiguous(), group=self.group)
                self._ubuf.copy_(torch.cat(parts))
        # ---- orthogonalise every matrix that touches my slice; apply the part inside it
        for (s, r, c) in self.matrices:
            O = newton_schulz(self._ubuf[s:s + r * c].view(r, c), self.ns_steps, self.use_kernels).reshape(-1)
            g0, g1 = max(s, self.lo), min(s + r * c, self.hi)
            a, b = g0 - self.lo, g1 - self.lo
            M = self.master[a:b]
            if self.weight_decay:
                M.mul_(1.0 - lr * self.weight_decay)
            M.add_(O[g0 - s:g1 - s].to(M.dtype), alpha=-lr * max(1.0, r / c) ** 0.5)
            my_flat[a:b].copy_(M.to(my_flat.dtype))
        # ---- AdamW for the rest of my slice
        b1, b2 = self.betas
        for (a, b, wd) in self._adamw_ranges():
            ref.adamw_step(self.master[a:b], self.m[a:b], self.v[a:b], gs[a:b], lr * self.adamw_lr_scale, b1, b2, self.eps, wd,
                           self.step_count, gscale=self._gscale)
            my_flat[a:b].copy_(self.master[a:b].to(my_flat.dtype))
        if self.world == 1:
            gs.zero_()  # one rank: the slice IS the model's gradient buffer (AdamW's kernel zeroes it in passing; here nobody did)
        # ---- refreshed working copy to every rank
        if self.world > 1:
            if self.flat.is_cuda:
                dist.all_gather_into_tensor(self.flat, my_flat.clone(), group=self.group)
            else:
                parts = [torch.empty_like(my_flat) for _ in range(self.world)]
                dist.all_gather(parts, my_flat.contiguous(), group=self.group)
                self.flat.copy_(torch.cat(parts))
        return norm

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["optimizer_type"] = "muon"
        return sd
