"""The learner: model + sharded optimizer + the per-step state machine shared by every trainer.

One ``Learner`` lives in each rank's process (one process per GPU).  SFT, DPO, reward-model and
GRPO trainers differ only in the loss they build from per-token log-probabilities or hidden
states; gradient accumulation, the once-per-step gradient exchange, clipping, the partitioned
AdamW and the bf16 refresh are here.  It stands where ``accelerator.prepare`` +
``deepspeed.initialize`` stand in the reference (``open_instruct/finetune.py:707-709``,
``open_instruct/grpo_fast.py:384-391``).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from .data.collate import IGNORE
from .models import LlamaModel, ModelSpec
from .parallel import dist as pdist
from .parallel.zero import ZeroOptimizer, lr_at, padded_numel
from .utils.common import nvtx_range


@dataclass
class LearnerConfig:
    ops: str = "auto"  # "fused" (sm_100a kernels), "ref" (PyTorch), "auto"; "emulated": the fused path's driver over PyTorch restatements of the kernels (tests)
    comm: str = "auto"  # "fused" (symmetric-memory kernels), "nccl", "none", "auto"
    learning_rate: float = 2e-5
    weight_decay: float = 0.0
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    max_grad_norm: float | None = None
    lr_scheduler_type: str = "linear"
    warmup_steps: int = 0
    total_steps: int = 1
    final_lr_ratio: float | None = None
    gradient_checkpointing: bool = False
    seed: int = 0
    dtype: torch.dtype | None = None
    offload_optimizer: bool = False   # fp32 master / moments in pinned host memory, streamed through the GPU per step
    sequence_parallel_size: int = 1   # Ulysses: every packed micro-batch is split over groups of this many consecutive ranks
    sp_max_tokens: int = 8192         # largest packed micro-batch (all ranks together) the exchange buffers hold
    # Parameter sharding (ZeRO stage 3): None = only when the resident design does not fit this GPU (``needs_sharding``)
    shard_parameters: bool | None = None
    # Hybrid sharding: parameters are split over groups of this many consecutive ranks and replicated across the groups
    # (gradient shards summed between the groups once per step).  None = one shard group spanning all ranks.
    shard_degree: int | None = None
    # Tensor parallelism of the training engine: groups of this many consecutive ranks split every layer (heads and MLP
    # channels); data parallelism and the optimizer sharding run across the groups.
    tensor_parallel_degree: int = 1
    # weight decay also on norm weights and biases (the reference's ``set_weight_decay_on_bias_and_norm=False``, which hands the
    # optimizer ungrouped parameters, ``open_instruct/grpo_fast.py:371-374``); default: those take none
    decay_bias_and_norm: bool = False
    load_balancing_weight: float = 0.0  # mixture of experts: weight of the router's load-balancing loss added to the SFT loss
    optimizer_type: str = "adamw"     # "adamw" | "muon" (orthogonalised momentum for the decoder layers' matrices, AdamW elsewhere)
    optimizer_kwargs: dict = field(default_factory=dict)  # Muon: mu, nesterov, ns_steps, adamw_lr_scale


def needs_sharding(total_params: int, world: int, hbm_bytes: int, offload_optimizer: bool = False) -> bool:
    """True when bf16 parameters + the fp32 gradient accumulator resident on every GPU, plus this rank's share of the fp32
    master weights and Adam moments, would take more than 70 % of the GPU's memory (the rest is for activations)."""
    world = max(world, 1)
    resident = 6 * total_params + (0 if offload_optimizer else 12 * total_params // world) + (4 * total_params // world if world > 1 else 0)
    return resident > 0.7 * hbm_bytes


class Learner:
    def __init__(self, spec: ModelSpec, cfg: LearnerConfig, device=None, group=None, flat_init: torch.Tensor | None = None):
        self.full_spec = spec
        self.tp = None
        if cfg.tensor_parallel_degree > 1:
            from .parallel.tp import TrainTP, local_spec

            if group is not None:
                raise ValueError("tensor parallelism builds its own groups from the default group")
            tp_group, group = pdist.tp_groups(cfg.tensor_parallel_degree)   # group: data-parallel ranks of my shard
            self.tp = TrainTP(tp_group)
            spec = local_spec(spec, cfg.tensor_parallel_degree)              # the model of this rank
        self.spec, self.cfg, self.group = spec, cfg, group
        self.rank, self.world = pdist.rank(group), pdist.world_size(group)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        ops = cfg.ops
        if ops == "auto":
            ops = "fused" if (self.device.type == "cuda" and spec.head_dim == 128 and not spec.post_norm and not spec.num_experts
                              and torch.cuda.get_device_capability(self.device)[0] == 10) else "ref"
        # "emulated": everything below takes the fused path's branches (fp32 main_grad, hand-driven backward) except the ones
        # that launch a kernel of this package (optimizer kernels, symmetric-memory exchange, the device status word)
        self.emulated = ops == "emulated"
        model_ops = ops
        if self.emulated:
            ops = "fused"
        self.ops = ops
        dtype = cfg.dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        comm = cfg.comm
        if comm == "auto":
            comm = "none" if self.world == 1 else ("fused" if (ops == "fused" and not self.emulated) else "nccl")
        if self.tp is not None:
            comm = "none" if self.world == 1 else "nccl"   # the data-parallel exchange of a TP shard goes through NCCL
            if cfg.shard_parameters or cfg.sequence_parallel_size > 1:
                raise NotImplementedError("tensor parallelism together with parameter sharding or sequence parallelism is not built")
            flat_init = self._tp_shard_of(flat_init, dtype, cfg.seed)
        self.comm = comm
        from .models.spec import ParamLayout

        layout = ParamLayout(spec)
        n = padded_numel(layout.total, self.world)
        self.symm = None
        self.z3 = None
        if cfg.optimizer_type not in ("adamw", "muon"):
            raise ValueError(f"unknown optimizer_type {cfg.optimizer_type!r}: 'adamw' or 'muon'")
        muon = cfg.optimizer_type == "muon"
        if muon:
            if self.tp is not None or cfg.shard_parameters or cfg.offload_optimizer:
                raise NotImplementedError("Muon runs with resident parameters and device-resident optimizer states (no tensor "
                                          "parallelism, parameter sharding or optimizer offload)")
            if comm == "fused":
                comm = "nccl" if self.world > 1 else "none"  # momentum is exchanged through torch.distributed
                self.comm = comm
        if cfg.decay_bias_and_norm and (cfg.shard_parameters or muon):
            raise NotImplementedError("weight decay on norm weights and biases is built for the resident AdamW only")
        shard = cfg.shard_parameters
        if shard is None and muon:
            shard = False
        if shard is None:
            shard = (ops == "fused" and not self.emulated and self.world > 1 and self.tp is None and
                     needs_sharding(layout.total, self.world, torch.cuda.get_device_properties(self.device).total_memory, cfg.offload_optimizer))
        if shard:
            if ops != "fused":
                raise NotImplementedError("parameter sharding runs on the fused (CUDA) path")
            from .parallel.zero3 import Zero3State

            self.model = LlamaModel(spec, device=self.device, dtype=dtype, ops=model_ops, sharded=True,
                                    gradient_checkpointing=cfg.gradient_checkpointing)
            shard_group, replica_group = group, None
            if cfg.shard_degree and cfg.shard_degree != self.world:
                shard_group, replica_group = pdist.hsdp_groups(cfg.shard_degree)
            self.z3 = Zero3State(layout, self.device, dtype, shard_group, replica_group=replica_group, comm="peer" if comm == "fused" else "nccl", lr=cfg.learning_rate,
                                 betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                 use_kernels=not self.emulated, offload=cfg.offload_optimizer)
            if flat_init is not None:
                self.z3.load_full(flat_init)
            else:
                self.z3.init_random(cfg.seed)
            self.z3.attach(self.model)
            self.opt = self.z3  # same checkpoint interface (state_dict / load_state_dict / master)
            self.global_step = 0
            self._accum = 0
            self.sp = 1
            self._setup_sequence_parallel(spec, cfg, group)
            return
        if comm == "fused":
            from .parallel.symm import SymmetricState

            self.symm = SymmetricState(n, self.device, group)
            flat = self.symm.params
        else:
            flat = torch.zeros(n, dtype=dtype, device=self.device)
        self.model = LlamaModel(spec, device=self.device, dtype=dtype, ops=model_ops, seed=cfg.seed, flat=flat,
                                gradient_checkpointing=cfg.gradient_checkpointing)
        if flat_init is not None:
            with torch.no_grad():
                self.model.flat[: flat_init.numel()].copy_(flat_init.to(dtype))
        else:
            self.model.init_weights(cfg.seed)
            if self.world > 1:  # identical start on every rank
                torch.distributed.broadcast(self.model.flat.detach(), src=0, group=group)
        if self.symm is not None:
            self.model.bind_main_grad(self.symm.grads)
        self.model.tp = self.tp
        if muon:
            from .parallel.muon import MuonOptimizer, muon_matrices

            self.opt = MuonOptimizer(self.model.flat.detach(), layout.total, layout.decay_end, muon_matrices(layout), lr=cfg.learning_rate,
                                     betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                     group=group, comm=comm, use_kernels=(ops == "fused" and not self.emulated), **dict(cfg.optimizer_kwargs or {}))
        else:
            self.opt = ZeroOptimizer(self.model.flat.detach(), layout.total, layout.total if cfg.decay_bias_and_norm else layout.decay_end, lr=cfg.learning_rate,
                                     betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay,
                                     max_grad_norm=cfg.max_grad_norm, group=group, comm=comm, symm=self.symm,
                                     use_kernels=(ops == "fused" and not self.emulated), offload=cfg.offload_optimizer,
                                     norm_weights=self.tp.norm_weights(layout) if self.tp is not None else None,
                                     norm_extra_group=self.tp.group if self.tp is not None else None)
        self.global_step = 0
        self._accum = 0
        self.sp = 1
        self._setup_sequence_parallel(spec, cfg, group)

    def _setup_sequence_parallel(self, spec, cfg, group) -> None:
        """Ulysses groups of ``sequence_parallel_size`` CONSECUTIVE ranks inside the data-parallel world (the reference's
        layout, ``open_instruct/grpo_fast.py:484-495``): the ranks of a group work on the same packed micro-batches, each on
        its chunk of the tokens; gradients are exchanged over the whole world as before (the partial sums of a group's ranks
        add up to the micro-batch's gradient), optimizer states and - with ``shard_parameters`` - parameters stay sharded
        over all ranks."""
        sp = cfg.sequence_parallel_size
        self.sp_group = None
        if sp <= 1:
            return
        if self.ops != "fused":
            raise NotImplementedError("sequence parallelism runs on the fused (CUDA) path")
        if self.world % sp:
            raise ValueError(f"sequence_parallel_size {sp} must divide the number of ranks {self.world}")
        if group is not None and sp != self.world:
            raise ValueError("sequence-parallel groups inside a custom process group are not supported")
        from .parallel.ulysses import HostUlyssesContext, UlyssesContext

        sp_group = group
        if sp != self.world:
            sp_group, _ = pdist.hsdp_groups(sp)  # consecutive ranks; collective: every rank builds every group
        self.sp = sp
        self.sp_group = sp_group
        self.model.sp = (HostUlyssesContext if self.emulated else UlyssesContext)(spec, cfg.sp_max_tokens, self.device, sp_group)

    def local_slice(self, t: torch.Tensor) -> torch.Tensor:
        """This rank's chunk of a per-token tensor of the packed micro-batch (identity without sequence parallelism)."""
        if self.sp == 1:
            return t
        lo, hi = self.model.sp.local_tokens(t.shape[-1])
        return t[..., lo:hi]

    # ------------------------------------------------------------------ pieces
    def lr(self, step: int | None = None) -> float:
        c = self.cfg
        return lr_at(self.global_step if step is None else step, c.learning_rate, c.total_steps, c.warmup_steps,
                     c.lr_scheduler_type, c.final_lr_ratio)

    def token_logprobs(self, batch: dict, temperature: float = 1.0, want_entropy: bool = False):
        with nvtx_range("forward"):
            return self.model.token_logprobs(batch["input_ids"], batch["position_ids"], batch["cu_seq_lens_q"],
                                             batch["labels_shifted"], temperature, want_entropy)

    def backward(self, loss: torch.Tensor, last: bool = False) -> None:
        """Backward of one micro-batch.  ``last=True`` says that no further micro-batch follows before
        ``optimizer_step``: every layer's gradients are then final as soon as this backward has passed the layer, and the
        sharded optimizer starts exchanging them under the rest of the backward pass (the overlap DeepSpeed's
        ``overlap_comm`` gives the reference, ``open_instruct/utils.py:1431-1460``).  Every rank must pass the same value."""
        hook = getattr(self.opt, "grads_ready", None) if (last and self.z3 is None and self.ops == "fused") else None
        self.model.grad_ready_hook = hook
        try:
            with nvtx_range("backward"):
                loss.backward()
        finally:
            self.model.grad_ready_hook = None
        self._accum += 1

    def optimizer_step(self, grad_scale: float | None = None) -> torch.Tensor:
        """Exchange + clip + AdamW + refresh.  ``grad_scale`` defaults to 1/(micro-batches * world):
        the mean over everything accumulated since the last step, DeepSpeed's convention."""
        if grad_scale is None:
            grad_scale = 1.0 / (max(self._accum, 1) * self.world)
        if self.z3 is not None:
            with nvtx_range("optimizer_step"):
                norm = self.z3.step(lr=self.lr(), grad_scale=grad_scale)
            self._accum = 0
            self.global_step += 1
            self._check_kernel_status()
            return norm
        grad = self.model.grad_flat()
        if grad is None:
            raise RuntimeError("optimizer_step called without any backward")
        if self.tp is not None:
            self.tp.sync_replicated_grads(self.model.layout.views(grad), self.spec)
        if grad.numel() < self.opt.flat.numel():  # ref path: autograd grad has the padded size already
            raise RuntimeError("gradient buffer smaller than the parameter buffer")
        with nvtx_range("optimizer_step"):
            norm = self.opt.step(grad, lr=self.lr(), grad_scale=grad_scale)
        if self.ops == "fused":
            if self.world > 1 or self.comm != "none" or self.emulated:
                self.model.main_grad.zero_()
            else:
                # single rank: AdamW zeroed the (only) shard in place, padding included
                pass
        else:
            self.model.flat.grad = None
        self._accum = 0
        self.global_step += 1
        self._check_kernel_status()
        return norm

    def _check_kernel_status(self) -> None:
        """Every optimizer step ends by reading the status word of the bounded device waits, so that a peer that never
        arrived (the reduce-scatter then summed unfinished buffers) raises here - before the next step runs and before a
        checkpoint of the diverged state can be written.  Ranks that wait on peers read it now (one small device
        synchronisation per optimizer step); a single rank only has its own pipeline waits and uses the non-blocking form."""
        if self.ops != "fused" or self.emulated:
            return
        from .ops import lib

        lib.check_status(sync=self.world > 1 or self.sp > 1 or self.tp is not None)

    # ------------------------------------------------------------------ whole-model views (loading, saving, weight sync)
    def _tp_shard_of(self, full: torch.Tensor | None, dtype, seed: int) -> torch.Tensor:
        """This rank's tensor-parallel shard of ``full`` (or of a fresh random initialisation drawn with ``seed``, identical
        on every rank)."""
        from .models.spec import ParamLayout
        from .parallel.tp import shard_flat

        if full is None:
            full = LlamaModel(self.full_spec, device=self.device, dtype=dtype, ops="ref", seed=seed).flat.detach()
        total = ParamLayout(self.full_spec).total
        return shard_flat(full[:total].to(self.device), self.full_spec, self.tp.rank, self.tp.world)

    @torch.no_grad()
    def load_full_weights(self, flat: torch.Tensor) -> None:
        """Install a complete flat parameter vector (global layout, any device) as the working copy and the fp32 master."""
        if self.tp is not None:
            flat = self._tp_shard_of(flat, self.model.flat.dtype, 0)
        if self.z3 is not None:
            self.z3.load_full(flat)
            return
        w = self.model.flat.detach()
        w[: flat.numel()].copy_(flat.to(w.dtype))
        self.opt.master.copy_(w[self.opt.lo:self.opt.hi].float())

    def load_hf(self, path: str, strict: bool = False) -> None:
        """Load a Hugging Face checkpoint folder.  With sharded parameters the tensors are staged in host memory and every
        rank keeps its slices only."""
        from .ckpt.hf_io import load_hf_checkpoint

        if self.z3 is None and self.tp is None:
            load_hf_checkpoint(path, self.model.flat.detach(), self.spec, strict=strict)
            self.opt.master.copy_(self.model.flat.detach()[self.opt.lo:self.opt.hi].float())
            return
        from .models.spec import ParamLayout

        stage = torch.zeros(ParamLayout(self.full_spec).total, dtype=self.z3.dtype if self.z3 is not None else self.model.flat.dtype)
        load_hf_checkpoint(path, stage, self.full_spec, strict=strict)
        self.load_full_weights(stage)

    @torch.no_grad()
    def full_flat(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """The complete bf16 parameter vector in the global layout: the resident working copy, or a gather of the shards
        (a collective: every rank calls it)."""
        if self.tp is not None:
            from .parallel.tp import unshard_flat

            mine = self.model.flat.detach()[: self.model.layout.total].contiguous()
            parts = [torch.empty_like(mine) for _ in range(self.tp.world)]
            torch.distributed.all_gather(parts, mine, group=self.tp.group)
            return unshard_flat(parts, self.full_spec, out)
        if self.z3 is None:
            return self.model.flat.detach()
        return self.z3.gather_full(out)

    # ------------------------------------------------------------------ residency (colocated learner + engine)
    def offload_to_cpu(self) -> int:
        """Move what only the optimizer step needs (fp32 master weights, moments, gradient shard, gradient accumulator) to
        pinned host memory, e.g. while a colocated rollout engine generates (cf. ``RayProcess.offload_to_cpu``,
        ``open_instruct/utils.py:1600-1648``).  Returns the bytes freed on the GPU.  A no-op for buffers that are in
        symmetric memory (they must stay mapped) or already on the host."""
        moved = 0
        self._parked = {}
        opt = self.z3.opt if self.z3 is not None else self.opt
        for name in ("master", "m", "v", "grad_shard"):
            t = getattr(opt, name, None)
            if t is not None and t.is_cuda:
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                host.copy_(t)
                self._parked[name] = host
                setattr(opt, name, host)  # keeps the attribute valid (state_dict works while parked)
                moved += t.numel() * t.element_size()
        if self.z3 is None and self.symm is None and self.model.main_grad is not None and self.model.main_grad.is_cuda and self._accum == 0:
            moved += self.model.main_grad.numel() * 4
            self.model.main_grad = None
            self.model.g = {}
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()
        return moved

    def backload_to_gpu(self) -> None:
        for name, host in getattr(self, "_parked", {}).items():
            setattr(self.z3.opt if self.z3 is not None else self.opt, name, host.to(self.device, non_blocking=True))
        self._parked = {}
        if self.ops == "fused" and self.symm is None and self.z3 is None:
            self.model.ensure_main_grad()

    # ------------------------------------------------------------------ SFT
    def sft_micro_step(self, batch: dict, reduce_loss: str = "mean", last: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """Forward + backward of one packed micro-batch.  Returns (loss, number of target tokens).

        ``mean``: mean CE over this micro-batch's target tokens (HF default, ``finetune.py:822-826``);
        ``sum`` : summed CE; the caller normalises by the global token count at the step.
        """
        logp, _ = self.token_logprobs(batch)  # sequence parallel: log-probs of this rank's chunk only
        n = (batch["labels_shifted"] != IGNORE).sum()  # target tokens of the whole micro-batch (every SP rank sees all labels)
        total = -logp.sum()
        # "mean": the sp ranks' partial sums add up in the gradient exchange, which then divides by the world size
        loss = total * self.sp / n.clamp(min=1) if reduce_loss == "mean" else total
        aux = getattr(self.model, "aux_loss", None)
        if aux is not None and self.cfg.load_balancing_weight:
            # mixture of experts: keep the router from collapsing onto few experts (``open_instruct/finetune.py:817-819``)
            loss = loss + self.cfg.load_balancing_weight * aux
            self.last_aux_loss = aux.detach()
        if self.sp > 1:
            n = self.local_slice(batch["labels_shifted"] != IGNORE).sum()
        # the fused path's ``aux_loss`` is a number: its backward pass adds the balancing loss's gradient itself, with this weight
        self.model.aux_loss_coef = float(self.cfg.load_balancing_weight or 0.0) if aux is not None else 0.0
        try:
            self.backward(loss, last=last)
        finally:
            self.model.aux_loss_coef = 0.0
        return loss.detach(), n

    def sft_step(self, micro_batches: list[dict], reduce_loss: str = "mean") -> dict:
        """One optimizer step over a list of packed micro-batches already on the device."""
        losses, toks = [], []
        for k, mb in enumerate(micro_batches):
            loss, n = self.sft_micro_step(mb, reduce_loss, last=(k == len(micro_batches) - 1))
            losses.append(loss)
            toks.append(n)
        loss_t = torch.stack(losses)
        tok_t = torch.stack(toks).sum()
        if reduce_loss == "sum":
            tot = tok_t.clone().float()
            pdist.all_reduce_(tot, group=self.group)
            norm = self.optimizer_step(grad_scale=None if False else float(1.0 / max(tot.item(), 1.0)))
            loss_out = loss_t.sum() / tok_t.clamp(min=1)
        else:
            norm = self.optimizer_step()
            loss_out = loss_t.mean()
        return {"loss": loss_out, "grad_norm": norm, "target_tokens": tok_t}
