"""Supervised fine-tuning entry point (the ``finetune`` API).

    python -m open_instruct_b200.finetune config.yaml [--flag value ...]
    torchrun --nproc-per-node 8 -m open_instruct_b200.finetune --model_name_or_path ... --packing ...

Flag surface and loop semantics follow the reference trainer (``open_instruct/finetune.py``:
``FlatArguments`` ``:76-351``, scheduler with ``final_lr_ratio`` ``:354-363``, loop ``:778-978``, checkpoints
``:966-990``), but nothing of accelerate / DeepSpeed is used: one process per GPU, the ``Learner`` runs
the fused sm_100a forward/backward, gradients are accumulated locally in fp32 and exchanged once per
optimizer step by the sharded optimizer (``parallel/zero.py``).

Batching: ``per_device_train_batch_size`` examples form one micro-batch, always padding-free (packed
with document boundaries); ``--packing`` additionally lets the loader fill micro-batches up to
``max_seq_length`` tokens.  Effective batch = per_device x world x gradient_accumulation_steps.
"""

from __future__ import annotations

import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Literal

import torch

from .ckpt.hf_io import load_hf_checkpoint, save_hf_checkpoint
from .ckpt.train_state import load_train_state, save_train_state
from .config.argparser import ArgumentParserPlus
from .data.collate import IGNORE, TensorDataCollatorWithFlattening, to_device
from .data.loader import HFDataLoader
from .data.tokenize import TOKENIZED_SFT_DATASET_KEYS, TokenizerConfig
from .learner import Learner, LearnerConfig
from .models import get_spec
from .parallel import dist as pdist
from .utils.common import (
    Tracker,
    clean_last_n_checkpoints,
    get_last_checkpoint_path,
    is_checkpoint_folder,
    set_seed,
    setup_logger,
)

logger = setup_logger(__name__)


@dataclass
class FlatArguments:
    """Everything the SFT run needs in one flat namespace (YAML keys = field names)."""

    exp_name: str = "finetune"
    do_not_randomize_output_dir: bool = False
    model_name_or_path: str | None = field(default=None, metadata={"help": "HF checkpoint directory or a preset name (e.g. llama3.1-8b) for random init"})
    config_name: str | None = field(default=None, metadata={"help": "Pretrained config name or path if not the same as model_name"})
    model_revision: str | None = None
    additional_model_arguments: dict | str | None = field(default_factory=dict, metadata={"help": "Overrides applied to the model spec (JSON)"})
    low_cpu_mem_usage: bool = False
    dataset_name: str | None = None
    dataset_mixer: dict | None = None
    dataset_mixer_list: list[str] = field(default_factory=lambda: ["allenai/tulu-3-sft-personas-algebra", "1.0"])
    dataset_mixer_list_splits: list[str] = field(default_factory=lambda: ["train"])
    dataset_transform_fn: list[str] = field(default_factory=lambda: ["sft_tulu_tokenize_and_truncate_v1", "sft_tulu_filter_v1"])
    dataset_target_columns: list[str] = field(default_factory=lambda: list(TOKENIZED_SFT_DATASET_KEYS))
    dataset_cache_mode: Literal["hf", "local"] = "local"
    dataset_local_cache_dir: str = "local_dataset_cache"
    dataset_config_hash: str | None = None
    dataset_skip_cache: bool = False
    dataset_mix_dir: str | None = None
    dataset_config_name: str | None = None
    max_train_samples: int | None = None
    preprocessing_num_workers: int | None = None
    max_seq_length: int | None = None
    overwrite_cache: bool = False
    clip_grad_norm: float = field(default=-1, metadata={"help": "Clip gradient norm; negative disables clipping"})
    gradient_accumulation_steps: int = 1
    learning_rate: float = 2e-5
    logging_steps: int | None = None
    lora_rank: int = 64
    lora_alpha: float = 16
    lora_dropout: float = 0.1
    lr_scheduler_type: str = "linear"
    num_train_epochs: int = 2
    output_dir: str = "output/"
    per_device_train_batch_size: int = 8
    use_lora: bool = False
    use_qlora: bool = False
    use_8bit_optimizer: bool = False
    warmup_ratio: float = 0.03
    final_lr_ratio: float | None = None
    weight_decay: float = 0.0
    timeout: int = 1800
    reduce_loss: Literal["mean", "sum"] = "mean"
    resume_from_checkpoint: str | None = None
    report_to: str | list[str] = "all"
    save_to_hub: str | None = None
    gradient_checkpointing: bool = False
    use_liger_kernel: bool = field(default=False, metadata={"help": "Accepted for recipe compatibility; the fused path always uses this package's kernels"})
    use_flash_attn: bool = field(default=True, metadata={"help": "Accepted for recipe compatibility"})
    max_train_steps: int | None = None
    seed: int = 42
    checkpointing_steps: str | None = field(default=None, metadata={"help": "An integer number of steps, or 'epoch'"})
    keep_last_n_checkpoints: int = 3
    fused_optimizer: bool = True
    load_balancing_loss: bool = False
    load_balancing_weight: float = 0.5
    clean_checkpoints_at_end: bool = True
    with_tracking: bool = False
    wandb_project_name: str = "open_instruct_internal"
    wandb_entity: str | None = None
    push_to_hub: bool = False
    hf_entity: str | None = None
    hf_repo_id: str | None = None
    hf_repo_revision: str | None = None
    hf_repo_url: str | None = None
    try_launch_beaker_eval_jobs: bool = False
    hf_metadata_dataset: str | None = None
    cache_dataset_only: bool = False
    try_auto_save_to_beaker: bool = False
    gs_bucket_path: str | None = None
    oe_eval_tasks: list[str] | None = None
    oe_eval_max_length: int = 4096
    sync_each_batch: bool = False
    packing: bool = field(default=False, metadata={"help": "Fill micro-batches up to max_seq_length tokens (padding-free either way)"})
    verbose: bool = False
    sequence_parallel_size: int = field(default=1, metadata={"help": "Ulysses sequence-parallel degree"})
    profiling: bool = field(default=False, metadata={"help": "torch.profiler trace of a few steps into <output_dir>/profiler"})
    tensor_parallel_degree: int = field(default=1, metadata={"help": "split every layer over groups of this many GPUs (data parallel across the groups)"})
    shard_parameters: bool | None = field(default=None, metadata={"help": "ZeRO-3 parameter sharding: gather each layer on use. Default: only when the resident design does not fit the GPU"})
    offload_optimizer: bool = field(default=False, metadata={"help": "keep fp32 master weights and Adam moments in pinned host memory"})
    # engine selection (not in the reference: there the back end is fixed by the launcher config)
    ops: Literal["auto", "fused", "ref", "emulated"] = "auto"
    comm_backend: Literal["auto", "fused", "nccl"] = "auto"
    fsdp_shard_degree: int | None = field(default=None, metadata={"help": "HSDP: shard optimizer state (and parameters) over groups of this many ranks, replicate across the groups"})
    zero_stage: int = field(default=3, metadata={"help": "Kept for recipe compatibility: optimizer states are always sharded, working params resident"})

    def __post_init__(self):
        if self.reduce_loss not in ("mean", "sum"):
            raise ValueError("reduce_loss must be 'mean' or 'sum'")
        if self.dataset_name is None and self.dataset_mixer is None and self.dataset_mixer_list is None:
            raise ValueError("Need either a dataset name, dataset mixer, or dataset mixer list.")
        if sum(x is not None for x in (self.dataset_name, self.dataset_mixer)) > 1:
            raise ValueError("Cannot provide two dataset selection mechanisms.")
        if self.use_qlora:
            self.use_lora = True  # QLoRA = LoRA adapters over an NF4-quantised frozen base
        if self.use_8bit_optimizer and not self.use_lora:
            # the reference, too, only builds its 8-bit optimizer next to QLoRA (``open_instruct/finetune.py:668-678``); the
            # full-parameter optimizer here is the sharded fp32 AdamW
            raise ValueError("use_8bit_optimizer applies to adapter training (use_lora / use_qlora): 8-bit moments for the adapters' AdamW")
        if isinstance(self.additional_model_arguments, str):
            self.additional_model_arguments = json.loads(self.additional_model_arguments)
        if self.sequence_parallel_size < 1:
            raise ValueError("sequence_parallel_size must be >= 1")


def build_spec(args: FlatArguments):
    name = args.config_name or args.model_name_or_path
    if name is None:
        raise ValueError("model_name_or_path (or config_name) is required")
    spec = get_spec(name)
    if args.additional_model_arguments:
        spec = spec.replace(**args.additional_model_arguments)
    return spec


def _micro_batches(loader_iter, accum: int):
    """Up to ``accum`` micro-batches for one optimizer step (fewer at the end of the epoch)."""
    out = []
    for _ in range(accum):
        try:
            out.append(next(loader_iter))
        except StopIteration:
            break
    return out


def main(args: FlatArguments, tc: TokenizerConfig) -> dict:
    rank, world, device = pdist.init_distributed(timeout_s=args.timeout)
    set_seed(args.seed)
    is_main = rank == 0
    if tc.tokenizer_name_or_path is None:
        tc.tokenizer_name_or_path = args.model_name_or_path
    tc.tokenizer_revision = tc.tokenizer_revision or args.model_revision
    if not args.do_not_randomize_output_dir and not os.path.basename(os.path.normpath(args.output_dir)).startswith(args.exp_name):
        pass  # output_dir is used as given: auto-resume needs a stable path

    # ------------------------------------------------------------------ data
    from .data.mixer import get_cached_dataset_tulu

    if args.dataset_mixer is not None:
        args.dataset_mixer_list = [str(x) for kv in args.dataset_mixer.items() for x in kv]
    elif args.dataset_name is not None:
        args.dataset_mixer_list = [args.dataset_name, "1.0"]
    transform_args = [{"max_seq_length": args.max_seq_length} if "truncate" in fn else {} for fn in args.dataset_transform_fn]
    if is_main:
        dataset = get_cached_dataset_tulu(args.dataset_mixer_list, args.dataset_mixer_list_splits, tc, args.dataset_transform_fn,
                                          transform_args, target_columns=args.dataset_target_columns,
                                          dataset_cache_mode=args.dataset_cache_mode, dataset_config_hash=args.dataset_config_hash,
                                          dataset_local_cache_dir=args.dataset_local_cache_dir, dataset_skip_cache=args.dataset_skip_cache)
    pdist.barrier()
    if not is_main:  # main process first: the others read the cache it wrote
        dataset = get_cached_dataset_tulu(args.dataset_mixer_list, args.dataset_mixer_list_splits, tc, args.dataset_transform_fn,
                                          transform_args, target_columns=args.dataset_target_columns,
                                          dataset_cache_mode=args.dataset_cache_mode, dataset_config_hash=args.dataset_config_hash,
                                          dataset_local_cache_dir=args.dataset_local_cache_dir, dataset_skip_cache=args.dataset_skip_cache)
    if args.cache_dataset_only:
        return {"cached": len(dataset)}
    dataset = dataset.shuffle(seed=args.seed)
    if args.max_train_samples is not None:
        dataset = dataset.select(range(min(args.max_train_samples, len(dataset))))
    tokenizer = tc.tokenizer

    # ------------------------------------------------------------------ model
    spec = build_spec(args)
    if len(tokenizer) > spec.vocab_size:
        spec = spec.replace(vocab_size=(len(tokenizer) + 7) // 8 * 8)  # grow the embedding to a multiple of 8
    spec = spec.replace(pad_token_id=tokenizer.pad_token_id, eos_token_id=tokenizer.eos_token_id, bos_token_id=tokenizer.bos_token_id)
    per_rank = args.per_device_train_batch_size
    collator = TensorDataCollatorWithFlattening(max_seq_length=args.max_seq_length if args.packing else None,
                                                pad_token_id=tokenizer.pad_token_id or 0, native=True)
    if args.packing:
        collator.max_seq_length = args.max_seq_length  # loader packs to this token budget; collator pads the row up to it
    sp = args.sequence_parallel_size
    if sp > 1:
        if world % sp or not args.packing or args.max_seq_length % sp:
            raise ValueError("sequence_parallel_size must divide the number of ranks, with --packing and max_seq_length divisible by it")
    tp = max(1, args.tensor_parallel_degree)
    if tp > 1 and (sp > 1 or world % tp):
        raise ValueError("tensor_parallel_degree must divide the number of ranks and excludes sequence parallelism")
    grp = sp * tp  # (one of them is 1)
    dp_rank, dp_world = rank // grp, world // grp  # the ranks of one sequence- or tensor-parallel group read the same micro-batches
    loader = HFDataLoader(dataset, batch_size=per_rank * dp_world, seed=args.seed, dp_rank=dp_rank, dp_world_size=dp_world,
                          collator=collator, drop_last=True)
    steps_per_epoch = math.ceil(len(loader) / args.gradient_accumulation_steps)
    max_steps = args.max_train_steps or args.num_train_epochs * steps_per_epoch
    num_epochs = math.ceil(max_steps / max(1, steps_per_epoch))
    warmup = int(max_steps * args.warmup_ratio)
    cfg = LearnerConfig(ops=args.ops, comm=args.comm_backend, learning_rate=args.learning_rate, weight_decay=args.weight_decay,
                        max_grad_norm=args.clip_grad_norm if args.clip_grad_norm > 0 else None,
                        lr_scheduler_type=args.lr_scheduler_type, warmup_steps=warmup, total_steps=max_steps,
                        final_lr_ratio=args.final_lr_ratio, gradient_checkpointing=args.gradient_checkpointing, seed=args.seed,
                        sequence_parallel_size=sp, sp_max_tokens=args.max_seq_length * max(1, per_rank) if sp > 1 else 0,
                        offload_optimizer=args.offload_optimizer, shard_parameters=args.shard_parameters,
                        tensor_parallel_degree=tp, shard_degree=args.fsdp_shard_degree,
                        load_balancing_weight=args.load_balancing_weight if args.load_balancing_loss else 0.0)
    if args.load_balancing_loss and not spec.num_experts:
        raise ValueError("load_balancing_loss applies to mixture-of-experts models (OLMoE); this model is dense")
    learner = Learner(spec, cfg, device=device)
    src = args.model_name_or_path
    if src and os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
        learner.load_hf(src)
    tracker = Tracker(args.output_dir, args.exp_name, {**asdict(args), **{f"tc_{k}": v for k, v in asdict(tc).items()}},
                      report_to=args.report_to if args.with_tracking else ("jsonl",), wandb_project=args.wandb_project_name,
                      wandb_entity=args.wandb_entity, enabled=is_main)

    lora = None
    if args.use_lora and learner.z3 is not None:
        raise NotImplementedError("LoRA adapters need the resident parameter copy; run with shard_parameters false")
    if args.use_lora:
        from .models.lora import LoRATrainer

        lora = LoRATrainer(learner, rank=args.lora_rank, alpha=args.lora_alpha, dropout=args.lora_dropout, lr=args.learning_rate,
                           weight_decay=args.weight_decay, quantize_base=args.use_qlora, eight_bit_optimizer=args.use_8bit_optimizer)
        logger.info("LoRA: %d trainable parameters (rank %d) on a frozen base", lora.adapters.num_parameters(), args.lora_rank)

    # ------------------------------------------------------------------ resume
    completed, start_epoch = 0, 0
    ckpt = get_last_checkpoint_path(args.output_dir, args.resume_from_checkpoint)
    if ckpt and is_checkpoint_folder(ckpt):
        st = load_train_state(ckpt, learner.opt)
        if lora is not None:
            lora.load_state(ckpt)  # adapters + their AdamW moments; raises when the checkpoint has none
        completed, start_epoch = st["completed_steps"], st["epoch"]
        learner.global_step = completed
        loader.load_state_dict(st["loader"])
        logger.info("resumed from %s at step %d", ckpt, completed)
    ckpt_every = args.checkpointing_steps
    ckpt_every = int(ckpt_every) if ckpt_every and str(ckpt_every).isdigit() else ckpt_every

    def save_ckpt(tag: str, epoch: int):
        d = os.path.join(args.output_dir, tag)
        save_train_state(d, learner.opt, {"completed_steps": completed, "epoch": epoch, "loader": loader.state_dict()},
                         before_complete=lora.save_state if lora is not None else None)
        if is_main:
            clean_last_n_checkpoints(args.output_dir, args.keep_last_n_checkpoints)

    # ------------------------------------------------------------------ loop
    from .utils.common import StepProfiler

    profiler = StepProfiler(args.profiling, args.output_dir, rank)
    total_tokens = torch.zeros((), dtype=torch.long, device=device)
    pred_tokens = torch.zeros((), dtype=torch.long, device=device)
    loss_acc = torch.zeros((), device=device)
    last_log, t_start = completed, time.time()
    logging_steps = args.logging_steps or 1
    final_metrics: dict = {}
    for epoch in range(start_epoch, num_epochs):
        if loader._epoch != epoch:
            loader.reshuffle(epoch)
        it = iter(loader)
        while completed < max_steps:
            mbs = _micro_batches(it, args.gradient_accumulation_steps)
            if not mbs:
                break
            mbs = [to_device(mb, device) for mb in mbs]
            out = lora.step(mbs, learner.lr(completed)) if lora is not None else learner.sft_step(mbs, args.reduce_loss)
            profiler.step()
            completed += 1
            loss_acc += out["loss"].detach()
            pred_tokens += out["target_tokens"]
            total_tokens += sum(int(mb["input_ids"].numel()) for mb in mbs)
            if completed % logging_steps == 0:
                vec = torch.stack([loss_acc / (completed - last_log), total_tokens.float(), pred_tokens.float()])
                vec_sum = vec.clone()
                pdist.all_reduce_(vec_sum)
                dt = time.time() - t_start
                final_metrics = {"train_loss": float(vec_sum[0]) / world, "learning_rate": learner.lr(completed - 1),
                                 "total_tokens": int(vec_sum[1]), "total_pred_tokens": int(vec_sum[2]),
                                 "per_device_tps": float(vec_sum[1]) / world / max(dt, 1e-9),
                                 "grad_norm": float(out["grad_norm"]), "epoch": epoch, "training_step": completed}
                if device.type == "cuda":
                    final_metrics["reserved_mem_GiB"] = torch.cuda.max_memory_reserved(device) / 2**30
                    final_metrics["allocated_mem_GiB"] = torch.cuda.max_memory_allocated(device) / 2**30
                tracker.log(final_metrics, completed)
                if is_main:
                    logger.info("step %d: loss %.4f lr %.3e tps/dev %.0f", completed, final_metrics["train_loss"],
                                final_metrics["learning_rate"], final_metrics["per_device_tps"])
                loss_acc.zero_()
                last_log = completed
            if isinstance(ckpt_every, int) and completed % ckpt_every == 0:
                save_ckpt(f"step_{completed}", epoch)
        if ckpt_every == "epoch":
            save_ckpt(f"epoch_{epoch}", epoch + 1)
        if completed >= max_steps:
            break

    profiler.close()
    # ------------------------------------------------------------------ final export
    pdist.barrier()
    full_weights = learner.full_flat()  # a gather when the parameters are sharded: every rank takes part
    if is_main:
        save_hf_checkpoint(full_weights, spec, args.output_dir, tokenizer=tokenizer)  # with LoRA: the merged model
        if lora is not None:
            lora.save(os.path.join(args.output_dir, "adapter"), args.model_name_or_path or "")
        if args.clean_checkpoints_at_end:
            clean_last_n_checkpoints(args.output_dir, 0)
    tracker.close()
    pdist.barrier()
    final_metrics["completed_steps"] = completed
    return final_metrics


def cli() -> None:
    """Command line: a YAML / JSON recipe and / or ``--key value`` flags."""
    main(*ArgumentParserPlus((FlatArguments, TokenizerConfig)).parse())


if __name__ == "__main__":
    cli()
