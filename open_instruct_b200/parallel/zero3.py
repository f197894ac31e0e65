"""Parameter-sharded learner state (ZeRO stage 3) for models that do not fit one GPU resident.

The resident design of ``parallel/zero.py`` keeps the whole bf16 working copy and one fp32 gradient accumulator on every
GPU (24 GB at 8B; 420 GB at 70B).  This module shards both, the way DeepSpeed stage 3 does for the reference
(``configs/ds_configs/stage3_no_offloading_accelerate.conf``, ``open_instruct/utils.py:1419-1460``), but organised around
the flat parameter layout and the manual layer-by-layer engine instead of module hooks:

* the flat buffer is cut into *units*: the embedding, each decoder layer's four matrices (contiguous in the layout), the
  output head; every unit is split evenly over the ranks, rank r keeps slice r (bf16 working shard, fp32 master and
  moments, fp32 gradient shard).  The small no-decay tail (norm weights, biases) stays replicated;
* a decoder layer's parameters are gathered into one of TWO layer-sized workspaces right before the layer runs; the
  gather of the next layer (previous, in the backward) is issued on a communication stream as soon as the layer that used
  that workspace has been enqueued, so it overlaps the current layer's GEMMs.  The model's parameter views point into
  the workspaces, so the kernels never know the difference;
* the backward writes a layer's fp32 weight gradients into one of two layer-sized gradient workspaces; when the layer
  is done the workspace is reduce-scattered on the communication stream and added to the rank's gradient shard;
* the embedding and the output head are *pinned* units: gathered once per optimizer step (their values only change
  then), their gradients accumulate over the micro-batches and are reduce-scattered once per step - per micro-batch
  they cost nothing;
* the optimizer is ``ZeroOptimizer`` run over the rank-local buffers (so the fused AdamW kernel, the host offload of
  the states and the checkpoint format are shared with the resident design), fed with the global gradient norm.

``comm="nccl"`` uses ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` (gloo on CPU: ``all_gather`` /
``all_reduce``); ``comm="peer"`` keeps the bf16 shards and the gradient workspaces in symmetric memory and moves the
data with this package's own kernels (``ops/csrc/zero_comm.cu``): the gather PULLS the peers' shards with plain
loads - parameters are constant between optimizer steps, so it needs no handshake at all - and the reduction reads the
owner's slice out of every peer's workspace after a bounded flag barrier.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import dist as pdist
from .zero import ZeroOptimizer, padded_numel

ALIGN = 128  # shard sizes are multiples of this many elements (256 bytes in bf16: TMA bases stay aligned)


@dataclass
class Unit:
    name: str
    start: int      # first element in the global flat layout
    size: int       # elements in the global layout
    shard: int      # elements per rank (size rounded up)
    soff: int       # offset of this rank's slice in the rank-local buffers
    pinned: bool


def plan_units(layout, world: int) -> tuple[list[Unit], int]:
    """Cut ``layout`` into gather units.  Returns ``(units, n_shard)``: the rank-local buffers hold the units'
    slices back to back in ``[0, n_shard)`` and the replicated tail after them."""
    e, L = layout.entries, layout.spec.num_layers
    starts = [("embed", e["embed"].offset, True)] + [(f"l{i}", e[f"l{i}.wqkv"].offset, False) for i in range(L)]
    if "lm_head" in e:
        starts.append(("lm_head", e["lm_head"].offset, True))
    units, soff = [], 0
    for k, (name, a, pinned) in enumerate(starts):
        b = starts[k + 1][1] if k + 1 < len(starts) else layout.decay_end
        shard = ((b - a + world - 1) // world + ALIGN - 1) // ALIGN * ALIGN
        units.append(Unit(name, a, b - a, shard, soff, pinned))
        soff += shard
    return units, soff


class Zero3State:
    """Sharded parameters + gradients + optimizer of one rank; ``attach`` wires a ``LlamaModel`` to it."""

    def __init__(self, layout, device, dtype, group=None, comm: str = "auto", lr: float = 1e-5, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, max_grad_norm: float | None = None, use_kernels: bool | None = None,
                 offload: bool = False, peer_timeout_ms: int = 20000, replica_group=None):
        # ``group`` is the SHARD group (its ranks split every unit); ``replica_group`` holds the ranks of other shard
        # groups that own the same slices (hybrid sharding): their gradient shards are summed once per optimizer step.
        self.layout, self.device, self.dtype, self.group = layout, torch.device(device), dtype, group
        self.replica_group = replica_group
        self.replicas = pdist.world_size(replica_group) if replica_group is not None else 1
        self.world, self.rank = pdist.world_size(group), pdist.rank(group)
        cuda = self.device.type == "cuda"
        if comm == "auto":
            comm = "nccl"
        if comm not in ("nccl", "peer"):
            raise ValueError("comm must be 'nccl' or 'peer'")
        if comm == "peer" and (not cuda or self.world == 1):
            comm = "nccl"
        self.comm = comm
        self.units, self.n_shard = plan_units(layout, self.world)
        self.by_name = {u.name: u for u in self.units}
        self.layers = [u for u in self.units if not u.pinned]
        self.tail_n = layout.total - layout.decay_end
        self.n_local = self.n_shard + self.tail_n
        n_alloc = padded_numel(self.n_local, 1)
        ws = max(u.shard for u in self.layers) * self.world
        self.peer = None
        if comm == "peer":
            from .zero3_peer import PeerComm

            self.peer = PeerComm(n_alloc, ws, self.device, group, peer_timeout_ms)
            self.local16 = self.peer.shards
            self.gws = self.peer.grad_ws
        else:
            self.local16 = torch.zeros(n_alloc, dtype=dtype, device=self.device)
            self.gws = [torch.zeros(ws, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.grad_local = torch.zeros(n_alloc, dtype=torch.float32, device=self.device)
        self.pws = [torch.zeros(ws, dtype=dtype, device=self.device) for _ in range(2)]
        self.pin_p = {u.name: torch.zeros(u.shard * self.world, dtype=dtype, device=self.device) for u in self.units if u.pinned}
        self.pin_g = {u.name: torch.zeros(u.shard * self.world, dtype=torch.float32, device=self.device) for u in self.units if u.pinned}
        self._rs_tmp = torch.zeros(max(u.shard for u in self.units), dtype=torch.float32, device=self.device)
        self.resident: list[int | None] = [None, None]   # which layer each parameter workspace holds
        self.pinned_fresh = False
        self.gather_count = 0   # layer gathers issued (tests check the prefetch / reuse logic with it)
        # two communication streams: the gather of the next layer must not queue behind a gradient reduction
        self.cs = torch.cuda.Stream(self.device) if cuda else None   # gathers
        self.rs = torch.cuda.Stream(self.device) if cuda else None   # reductions
        self._ev_g = [torch.cuda.Event() for _ in range(2)] if cuda else None       # gather into slot k finished
        self._ev_r = [None, None]                                                  # reduce out of grad slot k finished
        self._ev_pin: dict[str, torch.cuda.Event] = {}
        self._opt_args = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                              use_kernels=use_kernels, offload=offload)
        self.opt: ZeroOptimizer | None = None
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ loading / exporting whole models
    def _my_slice(self, u: Unit) -> tuple[int, int]:
        """Global element range of this rank's slice of ``u`` (may be empty or short at the unit's end)."""
        a = u.start + self.rank * u.shard
        return a, max(a, min(a + u.shard, u.start + u.size))

    @torch.no_grad()
    def load_full(self, flat: torch.Tensor) -> None:
        """Take this rank's slices out of a full flat buffer (any device; every rank passes the same values)."""
        self.local16.zero_()
        for u in self.units:
            a, b = self._my_slice(u)
            self.local16[u.soff:u.soff + (b - a)].copy_(flat[a:b])
        self.local16[self.n_shard:self.n_local].copy_(flat[self.layout.decay_end:self.layout.total])
        self._after_weights_changed()
        self._make_optimizer()

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """N(0, std) matrices and unit norm weights without ever holding the whole model: every rank draws a unit from the
        same generator state and keeps its slice."""
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000003 + 17)
        self.local16.zero_()
        for u in self.units:
            a, b = self._my_slice(u)
            full = torch.randn(u.size, device=self.device, generator=gen, dtype=torch.float32) * std
            self.local16[u.soff:u.soff + (b - a)].copy_(full[a - u.start:b - u.start])
            del full
        tail = self.local16[self.n_shard:self.n_local]
        tail.zero_()
        for name, ent in self.layout.entries.items():
            if ent.offset >= self.layout.decay_end and name.endswith("norm"):
                o = ent.offset - self.layout.decay_end
                tail[o:o + ent.numel].fill_(1.0)
        self._after_weights_changed()
        self._make_optimizer()

    def _make_optimizer(self) -> None:
        a = self._opt_args
        if self.opt is not None:
            # new weights into the existing state (no second set of fp32 buffers, not even for a moment)
            with torch.no_grad():
                self.opt.master.copy_(self.local16[:self.opt.master.numel()])
                self.opt.m.zero_()
                self.opt.v.zero_()
            self.opt.step_count = 0
            return
        self.opt = ZeroOptimizer(self.local16, self.n_local, self.n_shard, lr=a["lr"], betas=a["betas"], eps=a["eps"],
                                 weight_decay=a["weight_decay"], max_grad_norm=a["max_grad_norm"], group=pdist.SOLO, comm="none",
                                 use_kernels=a["use_kernels"], offload=a["offload"])

    def _after_weights_changed(self) -> None:
        self.resident = [None, None]
        self.pinned_fresh = False
        if self.peer is not None:
            self.peer.barrier()  # nobody pulls a shard that its owner is still writing

    @torch.no_grad()
    def gather_full(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """The whole model in the global flat layout (checkpoints, weight sync to rollout engines)."""
        if out is None:
            out = torch.zeros(self.layout.total, dtype=self.dtype, device=self.device)
        tmp = torch.empty(max(u.shard for u in self.units) * self.world, dtype=self.dtype, device=self.device)
        for u in self.units:
            t = tmp[:u.shard * self.world]
            self._all_gather(t, u)
            out[u.start:u.start + u.size].copy_(t[:u.size])
        out[self.layout.decay_end:self.layout.total].copy_(self.local16[self.n_shard:self.n_local])
        return out

    # ------------------------------------------------------------------ collectives
    def _all_gather(self, out: torch.Tensor, u: Unit) -> None:
        mine = self.local16[u.soff:u.soff + u.shard]
        if self.world == 1:
            out.copy_(mine)
        elif self.peer is not None:
            self.peer.all_gather(out, u.soff, u.shard)
        elif out.is_cuda:
            dist.all_gather_into_tensor(out, mine, group=self.group)
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine.contiguous(), group=self.group)
            out.copy_(torch.cat(parts))

    def _reduce_scatter_add(self, ws: torch.Tensor, u: Unit, slot: int | None = None) -> None:
        """``grad_local[slice of u] += sum over ranks of ws[my slice]``."""
        dst = self.grad_local[u.soff:u.soff + u.shard]
        src = ws[:u.shard * self.world]
        if self.world == 1:
            dst.add_(src)
        elif self.peer is not None and slot is not None:
            self.peer.reduce_scatter_add(slot, u.shard, dst)
        else:
            tmp = self._rs_tmp[:u.shard]
            if src.is_cuda:
                dist.reduce_scatter_tensor(tmp, src, op=dist.ReduceOp.SUM, group=self.group)
            else:
                full = src.clone()
                dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                tmp.copy_(full[self.rank * u.shard:(self.rank + 1) * u.shard])
            dst.add_(tmp)

    # ------------------------------------------------------------------ model wiring
    def attach(self, model) -> None:
        """Point ``model.p`` / ``model.g`` at the workspaces and register this state for the per-layer hooks."""
        p, g = {}, {}
        tail16 = self.local16[self.n_shard:self.n_local]
        tailg = self.grad_local[self.n_shard:self.n_local]
        for name, ent in self.layout.entries.items():
            if ent.offset >= self.layout.decay_end:
                o = ent.offset - self.layout.decay_end
                p[name], g[name] = tail16[o:o + ent.numel].view(ent.shape), tailg[o:o + ent.numel].view(ent.shape)
                continue
            uname = name if name in ("embed", "lm_head") else name.split(".", 1)[0]
            u = self.by_name[uname]
            o = ent.offset - u.start
            if u.pinned:
                pw, gw = self.pin_p[uname], self.pin_g[uname]
            else:
                k = int(uname[1:]) & 1
                pw, gw = self.pws[k], self.gws[k]
            p[name], g[name] = pw[o:o + ent.numel].view(ent.shape), gw[o:o + ent.numel].view(ent.shape)
        model.p, model.g, model.zero3 = p, g, self

    def _main(self):
        return torch.cuda.current_stream(self.device)

    def _gather_layer(self, i: int) -> None:
        """Issue the gather of layer ``i`` into its workspace, after everything enqueued so far (the last user of that
        workspace is among it)."""
        k, u = i & 1, self.layers[i]
        self.gather_count += 1
        self.resident[k] = i
        if self.cs is None:
            self._all_gather(self.pws[k][:u.shard * self.world], u)
            return
        self.cs.wait_stream(self._main())
        with torch.cuda.stream(self.cs):
            self._all_gather(self.pws[k][:u.shard * self.world], u)
            self._ev_g[k].record(self.cs)

    def _want(self, i: int, nxt: int) -> None:
        k = i & 1
        if self.resident[k] != i:
            self._gather_layer(i)
        if self.cs is not None:
            self._main().wait_event(self._ev_g[k])
        if 0 <= nxt < len(self.layers) and self.resident[nxt & 1] != nxt:
            self._gather_layer(nxt)

    # ---- hooks called by the model engine
    def fwd_begin(self) -> None:
        """Before the embedding lookup: the pinned units are gathered if an optimizer step changed them."""
        if self.pinned_fresh:
            return
        for u in self.units:
            if not u.pinned:
                continue
            if self.cs is None:
                self._all_gather(self.pin_p[u.name], u)
            else:
                self.cs.wait_stream(self._main())
                with torch.cuda.stream(self.cs):
                    self._all_gather(self.pin_p[u.name], u)
                    self._ev_pin[u.name] = torch.cuda.Event()
                    self._ev_pin[u.name].record(self.cs)
        self.pinned_fresh = True
        if self.cs is not None:
            self._main().wait_event(self._ev_pin["embed"])

    def head(self) -> None:
        ev = self._ev_pin.pop("lm_head", None)
        if ev is not None:
            self._main().wait_event(ev)

    def layer_fwd(self, i: int) -> None:
        self._want(i, i + 1)

    def layer_bwd(self, i: int) -> None:
        self._want(i, i - 1)
        k = i & 1
        # the reduction that last read this gradient workspace has finished - on every rank: the peer transport closes each
        # reduction with a barrier.  The weight-gradient GEMMs then overwrite the workspace (no zeroing needed).
        if self._ev_r[k] is not None:
            self._main().wait_event(self._ev_r[k])
            self._ev_r[k] = None

    def layer_bwd_done(self, i: int) -> None:
        k, u = i & 1, self.layers[i]
        if self.cs is None:
            self._reduce_scatter_add(self.gws[k], u, slot=k)
            return
        self.rs.wait_stream(self._main())
        with torch.cuda.stream(self.rs):
            self._reduce_scatter_add(self.gws[k], u, slot=k)
            self._ev_r[k] = torch.cuda.Event()
            self._ev_r[k].record(self.rs)

    # ------------------------------------------------------------------ optimizer step
    @torch.no_grad()
    def step(self, lr: float | None = None, grad_scale: float = 1.0) -> torch.Tensor:
        """Reduce what is still local (pinned units, tail), global norm, clip, AdamW on the shards."""
        if self.cs is not None:
            self._main().wait_stream(self.cs)
            self._main().wait_stream(self.rs)
            self._ev_r = [None, None]
        if self.peer is not None:
            self.peer.barrier()  # every rank's layer reductions have read my workspaces; pinned gradients are complete
        for u in self.units:
            if u.pinned:
                self._reduce_scatter_add(self.pin_g[u.name], u)
                self.pin_g[u.name].zero_()
        tail = self.grad_local[self.n_shard:self.n_local]
        if self.world > 1:
            dist.all_reduce(tail, op=dist.ReduceOp.SUM, group=self.group)
        if self.replicas > 1:  # the other shard groups' contributions to my slices (and to the tail), once per step
            dist.all_reduce(self.grad_local[:self.n_local], op=dist.ReduceOp.SUM, group=self.replica_group)
        sharded = self.grad_local[:self.n_shard]
        if self.opt.use_kernels:
            from ..ops import fused

            fused.sumsq(sharded, self._norm_sq)
        else:
            self._norm_sq.copy_(sharded.double().pow(2).sum().float().reshape(1))
        if self.world > 1:
            dist.all_reduce(self._norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        self._norm_sq.add_(tail.double().pow(2).sum().float())  # replicated: counted once
        norm = self.opt.step(self.grad_local, lr=lr, grad_scale=grad_scale, norm_sq=self._norm_sq)
        if not self.opt.use_kernels:  # the fused AdamW zeroes the gradient it consumed
            self.grad_local.zero_()
        self._after_weights_changed()
        return norm

    # ------------------------------------------------------------------ checkpointing
    is_param_sharded = True

    @property
    def master(self) -> torch.Tensor:
        return self.opt.master

    @property
    def shard(self) -> int:
        return self.opt.shard

    def state_dict(self) -> dict:
        sd = self.opt.state_dict()
        sd.update(rank=self.rank, world=self.world, zero3=True, n_shard=self.n_shard)
        return sd

    def load_state_dict(self, sd: dict) -> None:
        if sd.get("world") != self.world or sd.get("n_shard") != self.n_shard:
            raise ValueError("parameter-sharded state was saved with another world size; load the full weights instead")
        sd = dict(sd, world=1, rank=0)
        self.opt.load_state_dict(sd)
        self._after_weights_changed()
