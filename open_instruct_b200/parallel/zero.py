"""Sharded optimizer over the flat parameter buffer (the ZeRO learner).

What DeepSpeed ZeRO does for the reference (``open_instruct/utils.py:1419-1504``,
``configs/ds_configs/stage3_no_offloading_accelerate.conf``) is re-designed for 180 GB of HBM per
GPU and an NVSwitch fabric:

* fp32 master weights and both Adam moments are partitioned: rank r owns the contiguous slice
  ``[r * shard, (r + 1) * shard)`` of the flat buffer (ZeRO optimizer-state and master sharding);
* every rank keeps the full bf16 working copy resident (16 GB at 8B) instead of re-gathering
  each layer two or three times per micro-batch - the role DeepSpeed's hpZ secondary partition
  plays across nodes is played here by HBM capacity inside the node;
* gradients accumulate locally in one fp32 flat buffer across micro-batches (the wgrad GEMM
  epilogue adds into it) and cross NVLink ONCE per optimizer step: a reduce-scatter whose output
  feeds the partitioned AdamW, whose bf16 result is pushed to every peer's working copy.

Three communication back ends share this state machine:

``comm="none"``   single process.
``comm="nccl"``   ``reduce_scatter_tensor`` + ``all_gather_into_tensor`` (gloo: all_reduce + slice).  The
                  NCCL-only baseline.
``comm="fused"``  the gradient buffer and the bf16 working copy live in symmetric memory; one
                  kernel reduces the owner's slice straight out of every peer's buffer (P2P loads)
                  while accumulating the squared norm, and one kernel applies AdamW and stores the
                  refreshed bf16 values into every peer's working copy (P2P stores) - see
                  ``open_instruct_b200/parallel/symm.py``.
"""

from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from ..ops import ref
from . import dist as pdist

ALIGN = 1024  # shard sizes are multiples of this many elements


def shard_size_for(total: int, world: int) -> int:
    per = (total + world - 1) // world
    return (per + ALIGN - 1) // ALIGN * ALIGN


def padded_numel(total: int, world: int) -> int:
    """Size to allocate for the flat buffers so that they split evenly over ``world`` ranks."""
    return shard_size_for(total, world) * world


class ZeroOptimizer:
    """AdamW on this rank's slice of the flat parameters, with gradient clipping.

    ``flat``      bf16 (fused) or fp32 (ref) working parameters, ``padded_numel`` long.
    ``grad_fn``   callable returning the flat gradient accumulated since the last step.
    """

    def __init__(self, flat: torch.Tensor, total: int, decay_end: int, *, lr: float = 1e-5,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, max_grad_norm: float | None = None,
                 group=None, comm: str = "auto", use_kernels: bool | None = None, symm=None, offload: bool = False,
                 offload_chunk: int = 1 << 26, norm_weights: list | None = None, norm_extra_group=None):
        # ``norm_weights``: (start, end, weight) ranges of the flat buffer for the gradient norm, with ``norm_extra_group`` a
        # second group the squared norm is summed over.  Tensor parallelism uses it: the flat buffer is one rank's shard, the
        # norm must cover all shards (summed over the TP group) but count replicated entries once (weight 1 / tp).
        self.norm_weights, self.norm_extra_group = norm_weights, norm_extra_group
        # ``offload``: fp32 master / m / v shards live in pinned host memory and stream through two device staging
        # sets per optimizer step (H2D on one side stream, D2H on another, AdamW on the main stream) - the 12 bytes
        # per parameter leave the GPU, the price is 24 bytes per parameter over PCIe per step
        # (cf. DeepSpeed ``offload_optimizer``, ``open_instruct/dpo_tune_cache.py:76-114``).
        self.offload, self.offload_chunk = offload, offload_chunk
        self.flat = flat
        self.total = total
        self.decay_end = decay_end
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.group = group
        self.world = pdist.world_size(group)
        self.rank = pdist.rank(group)
        if comm == "auto":
            comm = "none" if self.world == 1 else "nccl"
        if comm == "none" and self.world > 1:
            raise ValueError("comm='none' needs a single process")
        self.comm = comm
        self.symm = symm
        if comm == "fused" and symm is None:
            raise ValueError("comm='fused' needs a SymmetricState (parallel.symm)")
        self.shard = shard_size_for(total, self.world)
        if flat.numel() != self.shard * self.world:
            raise ValueError(f"flat buffer must have padded_numel={self.shard * self.world} elements, got {flat.numel()}")
        self.lo = self.rank * self.shard
        self.hi = self.lo + self.shard
        self.device = flat.device
        self.use_kernels = (flat.is_cuda and flat.dtype == torch.bfloat16) if use_kernels is None else use_kernels
        with torch.no_grad():
            if offload:
                pin = flat.is_cuda
                self.master = torch.empty(self.shard, dtype=torch.float32, pin_memory=pin)
                self.master.copy_(flat.detach()[self.lo:self.hi])
                self.m = torch.zeros(self.shard, dtype=torch.float32, pin_memory=pin)
                self.v = torch.zeros(self.shard, dtype=torch.float32, pin_memory=pin)
            else:
                self.master = flat.detach()[self.lo:self.hi].to(torch.float32, copy=True)
                self.m = torch.zeros_like(self.master)
                self.v = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros(self.shard, dtype=torch.float32, device=flat.device) if self.world > 1 else None
        self._stage = None
        # B200_OVERLAP_GRADS=1: start reducing a layer's gradients as soon as the last micro-batch's backward has produced them.
        # Off by default.  Measured at 8B: on 2 GPUs the optimizer step shrinks from 66.9 to 38.8 ms but the backward slows by
        # as much (the step is power-capped and the reduce kernel's CTAs cannot share an SM with the weight-gradient GEMM's:
        # 136 x 256 + 255 x 192 registers exceed the file), step time unchanged; on 8 GPUs the per-layer reductions wait on the
        # slowest of eight backwards each time and the step got SLOWER (3307 ms, optimizer step 325 ms, against about 3200 / 180
        # without overlap).  The exchange after the backward costs 42 + 21 ms at 8 GPUs (0.86 / 0.85 of the link rate).
        self.overlap = os.environ.get("B200_OVERLAP_GRADS", "0") == "1"
        self.step_count = 0
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._gscale = torch.ones(1, dtype=torch.float32, device=self.device)
        self.last_grad_norm: torch.Tensor | None = None

    # ------------------------------------------------------------------ helpers
    def _segments(self):
        """(start, end, weight_decay) pieces of my shard, in shard-local coordinates."""
        segs = []
        lo, hi = self.lo, min(self.hi, self.total)
        if lo < min(hi, self.decay_end):
            segs.append((0, min(hi, self.decay_end) - lo, self.weight_decay))
        if hi > max(lo, self.decay_end):
            segs.append((max(lo, self.decay_end) - lo, hi - lo, 0.0))
        return segs

    def _reduce_scatter(self, grad: torch.Tensor, grad_scale: float) -> torch.Tensor:
        """Sum the flat gradient over ranks; returns this rank's fp32 slice."""
        if self.world == 1:
            return grad[self.lo:self.hi]
        if self.comm == "fused":
            return self.symm.reduce_scatter_grad(self.grad_shard, self._norm_sq)
        g = grad if grad.dtype == torch.float32 else grad.float()
        if g.is_cuda:
            dist.reduce_scatter_tensor(self.grad_shard, g, op=dist.ReduceOp.SUM, group=self.group)
        else:  # gloo has no reduce_scatter for all dtypes: all-reduce and slice
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
            self.grad_shard.copy_(g[self.lo:self.hi])
        return self.grad_shard

    def grads_ready(self, lo: int, hi: int) -> None:
        """The flat gradient range ``[lo, hi)`` has received its last contribution of this optimizer step (called by the
        model during the final micro-batch's backward, in the same order on every rank).  With the fused back end the
        owner starts reducing it right away on a side stream; the other back ends exchange everything in ``step``."""
        if self.comm == "fused" and self.world > 1 and self.overlap:
            self.symm.reduce_ready_range(lo, hi, self.grad_shard)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, grad: torch.Tensor, lr: float | None = None, grad_scale: float = 1.0,
             norm_sq: torch.Tensor | None = None) -> torch.Tensor:
        """One optimizer step from the accumulated flat gradient.

        ``grad_scale`` multiplies the summed gradient before clipping (1 / accumulation steps,
        1 / world for mean-reduced losses).  Returns the global gradient norm (device scalar,
        after ``grad_scale``, before clipping).  The caller zeroes its gradient buffer afterwards
        (``zero_grad`` below does it for the shard it owns; the full buffer is the model's).
        ``norm_sq`` (device scalar) replaces the squared gradient norm computed here: a caller that runs this
        optimizer over rank-local buffers (parameter sharding) supplies the global value.
        """
        lr = self.lr if lr is None else lr
        self.step_count += 1
        fused_comm = self.comm == "fused" and self.world > 1
        gs = self._reduce_scatter(grad, grad_scale)
        # ---- global grad norm (of the summed gradient times grad_scale)
        if norm_sq is not None:
            self._norm_sq.copy_(norm_sq)
        elif self.norm_weights is not None:
            self._norm_sq.zero_()
            part = torch.zeros_like(self._norm_sq)
            for (a, b, w) in self.norm_weights:
                a2, b2 = max(a, self.lo) - self.lo, min(b, self.hi) - self.lo
                if b2 <= a2:
                    continue
                if self.use_kernels and a2 % 4 == 0:
                    from ..ops import fused

                    fused.sumsq(gs[a2:b2], part)
                else:
                    part.copy_(gs[a2:b2].double().pow(2).sum().float().reshape(1))
                self._norm_sq.add_(part, alpha=w)
            if self.norm_extra_group is not None:
                dist.all_reduce(self._norm_sq, op=dist.ReduceOp.SUM, group=self.norm_extra_group)
        elif fused_comm:
            pass  # the reduce-scatter kernel already accumulated this rank's sum of squares
        elif self.use_kernels:
            from ..ops import fused

            fused.sumsq(gs, self._norm_sq)
        else:
            self._norm_sq.copy_(gs.double().pow(2).sum().float().reshape(1))
        if self.world > 1 and not fused_comm and norm_sq is None:
            dist.all_reduce(self._norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        norm = self._norm_sq.sqrt() * grad_scale
        self.last_grad_norm = norm
        if self.max_grad_norm is not None and self.max_grad_norm > 0:
            clip = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
            self._gscale.copy_(clip * grad_scale)
        else:
            self._gscale.fill_(grad_scale)
        # ---- AdamW on the shard (+ bf16 refresh of my slice of the working copy)
        b1, b2 = self.betas
        my_flat = self.flat[self.lo:self.hi]
        if self.offload:
            self._step_offloaded(gs, my_flat, lr, fused_comm)
        for (a, b, wd) in ([] if self.offload else self._segments()):
            if self.use_kernels:
                from ..ops import fused

                if fused_comm:
                    self.symm.adamw_allgather(self.master[a:b], self.m[a:b], self.v[a:b], gs[a:b], self.lo + a,
                                              gscale=self._gscale, lr=lr, beta1=b1, beta2=b2, eps=self.eps, wd=wd,
                                              step=self.step_count)
                else:
                    fused.adamw(self.master[a:b], self.m[a:b], self.v[a:b], gs[a:b], my_flat[a:b], lr=lr, beta1=b1,
                                beta2=b2, eps=self.eps, wd=wd, step=self.step_count, gscale=self._gscale,
                                zero_grad=True)
            else:
                ref.adamw_step(self.master[a:b], self.m[a:b], self.v[a:b], gs[a:b], lr, b1, b2, self.eps, wd,
                               self.step_count, gscale=self._gscale)
                my_flat[a:b].copy_(self.master[a:b].to(my_flat.dtype))
        # ---- refreshed working copy to every rank
        if self.world > 1:
            if fused_comm:
                self.symm.finish_step()
            elif self.flat.is_cuda:
                dist.all_gather_into_tensor(self.flat, my_flat, group=self.group)
            else:
                parts = [torch.empty_like(my_flat) for _ in range(self.world)]
                dist.all_gather(parts, my_flat.contiguous(), group=self.group)
                self.flat.copy_(torch.cat(parts))
        return norm

    def _adamw_piece(self, M, m, v, g, out16, goff: int, lr: float, wd: float, fused_comm: bool) -> None:
        b1, b2 = self.betas
        if self.use_kernels:
            from ..ops import fused

            if fused_comm:
                self.symm.adamw_allgather(M, m, v, g, goff, gscale=self._gscale, lr=lr, beta1=b1, beta2=b2, eps=self.eps, wd=wd,
                                          step=self.step_count)
            else:
                fused.adamw(M, m, v, g, out16, lr=lr, beta1=b1, beta2=b2, eps=self.eps, wd=wd, step=self.step_count,
                            gscale=self._gscale, zero_grad=True)
        else:
            ref.adamw_step(M, m, v, g, lr, b1, b2, self.eps, wd, self.step_count, gscale=self._gscale)
            out16.copy_(M.to(out16.dtype))

    def _step_offloaded(self, gs: torch.Tensor, my_flat: torch.Tensor, lr: float, fused_comm: bool) -> None:
        """AdamW over host-resident state, chunk by chunk through two staging sets."""
        CH = self.offload_chunk
        pieces = [(c0, min(b, c0 + CH), wd) for (a, b, wd) in self._segments() for c0 in range(a, b, CH)]
        if not self.flat.is_cuda:
            for c0, c1, wd in pieces:  # host-only run (tests): same arithmetic, no streams
                self._adamw_piece(self.master[c0:c1], self.m[c0:c1], self.v[c0:c1], gs[c0:c1], my_flat[c0:c1], self.lo + c0, lr, wd, fused_comm)
            return
        dev = self.device
        if self._stage is None:
            n = min(CH, self.shard)
            self._stage = [[torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3)] for _ in range(2)]
            self._h2d, self._d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            self._ev_in = [torch.cuda.Event() for _ in range(2)]
            self._ev_comp = [torch.cuda.Event() for _ in range(2)]
            self._ev_out = [torch.cuda.Event() for _ in range(2)]
        main = torch.cuda.current_stream(dev)
        host = (self.master, self.m, self.v)
        for i, (c0, c1, wd) in enumerate(pieces):
            k, n = i & 1, c1 - c0
            st = self._stage[k]
            with torch.cuda.stream(self._h2d):
                if i >= 2:
                    self._h2d.wait_event(self._ev_out[k])  # the chunk that used this set two rounds ago is back on the host
                else:
                    self._h2d.wait_stream(main)
                for d, h in zip(st, host):
                    d[:n].copy_(h[c0:c1], non_blocking=True)
                self._ev_in[k].record(self._h2d)
            main.wait_event(self._ev_in[k])
            self._adamw_piece(st[0][:n], st[1][:n], st[2][:n], gs[c0:c1], my_flat[c0:c1], self.lo + c0, lr, wd, fused_comm)
            self._ev_comp[k].record(main)
            with torch.cuda.stream(self._d2h):
                self._d2h.wait_event(self._ev_comp[k])
                for d, h in zip(st, host):
                    h[c0:c1].copy_(d[:n], non_blocking=True)
                self._ev_out[k].record(self._d2h)
        main.wait_stream(self._d2h)  # host state is complete before the step returns (checkpointing reads it)

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v, "rank": self.rank,
                "world": self.world, "shard": self.shard}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["shard"] != self.shard:
            raise ValueError("optimizer shard layout changed; reshard with ckpt.train_state.reshard_optimizer")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        with torch.no_grad():
            self.flat[self.lo:self.hi].copy_(self.master.to(self.flat.dtype))


# ---------------------------------------------------------------------- LR schedules
def lr_at(step: int, base_lr: float, total_steps: int, warmup_steps: int, kind: str = "linear",
          final_lr_ratio: float | None = None, num_cycles: float | None = None) -> float:
    """Learning rate for optimizer step ``step`` (0-based), HF ``get_scheduler`` semantics.

    ``linear`` with ``final_lr_ratio`` decays to ``base_lr * final_lr_ratio`` instead of zero
    (``open_instruct/finetune.py:354-363``).
    """
    if kind in ("constant",):
        return base_lr
    if step < warmup_steps:
        return base_lr * step / max(1, warmup_steps)
    if kind == "constant_with_warmup":
        return base_lr
    progress = (step - warmup_steps) / max(1, total_steps - warmup_steps)
    progress = min(max(progress, 0.0), 1.0)
    if kind == "linear":
        if final_lr_ratio is not None:
            return base_lr * (final_lr_ratio + (1.0 - final_lr_ratio) * (1.0 - progress))
        return base_lr * max(0.0, 1.0 - progress)
    if kind == "cosine":  # transformers' default: half a cosine wave
        return base_lr * max(0.0, 0.5 * (1.0 + math.cos(math.pi * (0.5 if num_cycles is None else num_cycles) * 2.0 * progress)))
    if kind == "cosine_with_restarts":  # transformers' default: one hard restart cycle
        if progress >= 1.0:
            return 0.0
        return base_lr * max(0.0, 0.5 * (1.0 + math.cos(math.pi * (((1 if num_cycles is None else num_cycles) * progress) % 1.0))))
    if kind == "polynomial":
        lr_end, power = 1e-7, 1.0
        return (base_lr - lr_end) * (1 - progress) ** power + lr_end
    raise ValueError(f"unknown lr_scheduler_type {kind}")
