"""DPO with cached reference log-probs (the ``dpo_tune_cache`` API).

    python -m open_instruct_b200.dpo_tune_cache config.yaml [--flag value ...]

Phase A builds (or loads) the reference log-prob cache with the initial weights; phase B trains with
``args.forward_fn`` + ``dpo_utils.compute_loss``.  Control flow, metric names and the cache key follow
the reference (``open_instruct/dpo_tune_cache.py:117-750``); the engine is this package's ``Learner``
(sharded optimizer, fused kernels), so ``zero_stage`` / offload flags are accepted but the placement
of states is decided by the learner (states sharded, bf16 working copy resident).
"""

from __future__ import annotations

import math
import os
import time
from dataclasses import asdict

import torch

from .ckpt.hf_io import load_hf_checkpoint, save_hf_checkpoint
from .ckpt.train_state import load_train_state, save_train_state
from .config.argparser import ArgumentParserPlus
from .data.collate import TensorDataCollatorWithFlatteningDPO, to_device
from .data.loader import HFDataLoader
from .data.mixer import compute_config_hash, get_cached_dataset_tulu, load_dataset_configs
from .data.tokenize import TokenizerConfig
from .dpo_utils import (
    REFERENCE_LOGPROBS_CACHE_PATH,
    DPOExperimentConfig,
    DPOLossType,
    build_reference_logprobs_cache,
    compute_loss,
    compute_reference_cache_hash,
)
from .learner import Learner, LearnerConfig
from .models import get_spec
from .parallel import dist as pdist
from .utils.common import (
    MetricsTracker,
    Tracker,
    clean_last_n_checkpoints,
    get_last_checkpoint_path,
    is_checkpoint_folder,
    set_seed,
    setup_logger,
)
from .utils.model_dims import ModelDims

logger = setup_logger(__name__)


def build_deepspeed_config(zero_stage: int, offload_optimizer: bool = False, offload_param: bool = False,
                           zero_hpz_partition_size: int = 8) -> dict:
    """The placement the sharded learner applies, in DeepSpeed's vocabulary (for logging / recipe parity)."""
    return {
        "bf16": {"enabled": True},
        "zero_optimization": {
            "stage": zero_stage,
            "overlap_comm": True,
            "states": "sharded over data-parallel ranks",
            "working_params": "resident bf16 replica per GPU (role of hpZ secondary partition)",
            "zero_hpz_partition_size": zero_hpz_partition_size,
            "offload_optimizer": {"device": "cpu" if offload_optimizer else "none"},
            "offload_param": {"device": "cpu" if offload_param else "none"},
        },
        "gradient_exchange": "once per optimizer step (fp32 local accumulation)",
    }


def prepare(args: DPOExperimentConfig, tc: TokenizerConfig):
    """Everything both DPO drivers share: process group, cached preference dataset, model + sharded learner, data loader and
    the reference log-prob cache (phase A).  Returns a namespace; ``done`` holds the result when the flags asked for an early
    exit (``cache_dataset_only`` / ``cache_logprobs_only``)."""
    from types import SimpleNamespace

    rank, world, device = pdist.init_distributed(timeout_s=args.timeout)
    set_seed(args.seed)
    is_main = rank == 0
    if tc.tokenizer_name_or_path is None:
        tc.tokenizer_name_or_path = args.model_name_or_path
    if args.dataset_mixer is not None:
        args.mixer_list = [str(x) for kv in args.dataset_mixer.items() for x in kv]
    elif args.dataset_name is not None:
        args.mixer_list = [args.dataset_name, "1.0"]
    transform_args = [{"max_seq_length": args.max_seq_length}, {}][: len(args.transform_fn)]
    transform_args += [{}] * (len(args.transform_fn) - len(transform_args))

    def _load():
        return get_cached_dataset_tulu(args.mixer_list, args.mixer_list_splits, tc, args.transform_fn, transform_args,
                                       target_columns=args.target_columns, dataset_cache_mode=args.cache_mode,
                                       dataset_config_hash=args.config_hash, dataset_local_cache_dir=args.local_cache_dir,
                                       dataset_skip_cache=args.skip_cache)

    if is_main:
        dataset = _load()
    pdist.barrier()
    if not is_main:
        dataset = _load()
    if args.cache_dataset_only:
        return SimpleNamespace(done={"cached": len(dataset)})
    if args.max_train_samples is not None:
        dataset = dataset.select(range(min(args.max_train_samples, len(dataset))))
    if "index" in dataset.column_names:
        dataset = dataset.remove_columns(["index"])
    dataset = dataset.add_column("index", list(range(len(dataset))))
    tokenizer = tc.tokenizer

    # ------------------------------------------------------------------ model
    spec = get_spec(args.config_name or args.model_name_or_path)
    from .config.schemas import spec_with_rope_flags

    spec = spec_with_rope_flags(spec, args)   # --rope_scaling_factor: YaRN context extension
    if args.additional_model_arguments:
        spec = spec.replace(**args.additional_model_arguments)
    if len(tokenizer) > spec.vocab_size:
        spec = spec.replace(vocab_size=(len(tokenizer) + 7) // 8 * 8)
    spec = spec.replace(pad_token_id=tokenizer.pad_token_id, eos_token_id=tokenizer.eos_token_id, bos_token_id=tokenizer.bos_token_id)
    collator = TensorDataCollatorWithFlatteningDPO(max_seq_length=None, pad_token_id=tokenizer.pad_token_id or 0)
    if args.packing:
        collator.max_seq_length = args.max_seq_length
    # the ranks of one tensor-parallel group work on the same micro-batches: data is sharded over the groups
    tp = max(1, args.tensor_parallel_degree)
    if world % tp:
        raise ValueError(f"tensor_parallel_degree {tp} must divide the number of ranks {world}")
    data_rank, data_world = rank // tp, world // tp
    loader = HFDataLoader(dataset, batch_size=args.per_device_train_batch_size * data_world,
                          seed=args.data_loader_seed if args.data_loader_seed is not None else args.seed, dp_rank=data_rank,
                          dp_world_size=data_world, collator=collator, drop_last=True)
    steps_per_epoch = math.ceil(len(loader) / args.gradient_accumulation_steps)
    max_steps = args.max_train_steps or args.num_epochs * steps_per_epoch
    cfg = LearnerConfig(ops=args.ops, comm=args.comm_backend, learning_rate=args.learning_rate, weight_decay=args.weight_decay,
                        max_grad_norm=args.max_grad_norm, lr_scheduler_type=args.lr_scheduler_type,
                        warmup_steps=int(max_steps * args.warmup_ratio), total_steps=max_steps,
                        gradient_checkpointing=args.activation_memory_budget < 1 or args.gradient_checkpointing, seed=args.seed,
                        offload_optimizer=args.offload_optimizer, shard_parameters=args.shard_parameters,
                        tensor_parallel_degree=args.tensor_parallel_degree, shard_degree=args.fsdp_shard_degree,
                        optimizer_type=args.optimizer_type, optimizer_kwargs=dict(args.optimizer_kwargs or {}))
    learner = Learner(spec, cfg, device=device)
    src = args.model_name_or_path
    if src and os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
        learner.load_hf(src)
    dims = ModelDims.from_spec(spec)
    if is_main and args.zero_stage is not None:
        logger.info("placement: %s", build_deepspeed_config(args.zero_stage, args.offload_optimizer, args.offload_param,
                                                           args.zero_hpz_partition_size))

    # ------------------------------------------------------------------ phase A: reference cache
    lt = DPOLossType(args.loss_type)
    average = lt.is_average_loss
    forward_fn = args.forward_fn
    reference_cache = None
    if lt.needs_reference_model:
        dcs_hash = args.config_hash
        if dcs_hash is None:
            dcs = load_dataset_configs(args.mixer_list, args.mixer_list_splits, args.transform_fn, transform_args, args.target_columns)
            dcs_hash = compute_config_hash(dcs, tc)
        cache_hash = compute_reference_cache_hash(args, dcs_hash)
        cache_path = os.path.join(REFERENCE_LOGPROBS_CACHE_PATH, f"{cache_hash}.pt")
        cache_loader = HFDataLoader(dataset, batch_size=args.per_device_train_batch_size * data_world, seed=args.seed, dp_rank=data_rank,
                                    dp_world_size=data_world, collator=collator, drop_last=False)
        t0 = time.time()
        reference_cache = build_reference_logprobs_cache(learner, cache_loader, average, forward_fn, len(dataset), device,
                                                         cache_path, is_main)
        logger.info("reference cache ready in %.1fs (%s)", time.time() - t0, cache_path)
    done = {"cache_built": True} if args.cache_logprobs_only else None
    return SimpleNamespace(done=done, rank=rank, world=world, device=device, is_main=is_main, dataset=dataset, tokenizer=tokenizer, spec=spec,
                           loader=loader, learner=learner, dims=dims, lt=lt, average=average, forward_fn=forward_fn, reference_cache=reference_cache,
                           data_world=data_world, steps_per_epoch=steps_per_epoch, max_steps=max_steps)


def main(args: DPOExperimentConfig, tc: TokenizerConfig) -> dict:
    p = prepare(args, tc)
    if p.done is not None:
        return p.done
    rank, world, device, is_main, tokenizer, spec = p.rank, p.world, p.device, p.is_main, p.tokenizer, p.spec
    loader, learner, dims, lt, average, forward_fn = p.loader, p.learner, p.dims, p.lt, p.average, p.forward_fn
    reference_cache, data_world, max_steps = p.reference_cache, p.data_world, p.max_steps


    # ------------------------------------------------------------------ resume
    tracker = Tracker(args.output_dir, args.run_name or args.exp_name, asdict(args),
                      report_to=args.report_to if args.with_tracking else ("jsonl",), wandb_project=args.wandb_project,
                      wandb_entity=args.wandb_entity, enabled=is_main)
    # adapters (``use_lora``, ``open_instruct/dpo_tune_cache.py:360-376``): the base stays frozen - it is also the reference policy,
    # whose log-probs were cached above from the same weights - and AdamW runs on the low-rank pairs only
    lora = None
    if args.use_lora:
        if learner.z3 is not None or learner.tp is not None:
            raise NotImplementedError("LoRA adapters need the resident, unsplit parameter copy (no shard_parameters, no tensor parallelism)")
        from .models.lora import LoRATrainer

        lora = LoRATrainer(learner, rank=args.lora_rank, alpha=args.lora_alpha, dropout=args.lora_dropout, lr=args.learning_rate,
                           weight_decay=args.weight_decay)
        logger.info("LoRA: %d trainable parameters (rank %d) on a frozen base", lora.adapters.num_parameters(), args.lora_rank)
    completed, start_epoch = 0, 0
    ckpt = get_last_checkpoint_path(args.output_dir, args.resume_from_checkpoint)
    if ckpt and is_checkpoint_folder(ckpt):
        st = load_train_state(ckpt, learner.opt)
        if lora is not None:
            lora.load_state(ckpt)
        completed, start_epoch = st["completed_steps"], st["epoch"]
        learner.global_step = completed
        loader.load_state_dict(st["loader"])

    # ------------------------------------------------------------------ phase B: training
    from .utils.common import StepProfiler

    profiler = StepProfiler(args.profiling, args.output_dir, rank)
    metrics = MetricsTracker(device=device)
    t_start, tokens_seen, last = time.time(), 0, {}
    for epoch in range(start_epoch, args.num_epochs):
        if loader._epoch != epoch:
            loader.reshuffle(epoch)
        it = iter(loader)
        while completed < max_steps:
            mbs = []
            for _ in range(args.gradient_accumulation_steps):
                try:
                    mbs.append(next(it))
                except StopIteration:
                    break
            if not mbs:
                break
            step_t0 = time.time()
            lengths = []
            if lora is not None:
                lora.begin()
            for k, mb in enumerate(mbs):
                mb = to_device(mb, device)
                pc, pr, aux = forward_fn(learner, mb, average_log_prob=average)
                losses, c_rew, r_rew = compute_loss(args, mb, pc, pr, reference_cache,
                                                    (aux["chosen_tokens"], aux["rejected_tokens"]))
                loss = losses.mean()
                learner.backward(loss, last=(k == len(mbs) - 1) and lora is None)
                metrics.add("train_loss", loss.detach() / len(mbs))
                metrics.add("logps/chosen", pc.detach().mean() / len(mbs))
                metrics.add("logps/rejected", pr.detach().mean() / len(mbs))
                if lt.computes_reward_metrics:
                    metrics.add("rewards/chosen", c_rew.mean() / len(mbs))
                    metrics.add("rewards/rejected", r_rew.mean() / len(mbs))
                    metrics.add("rewards/average", (c_rew + r_rew).mean() / 2 / len(mbs))
                    metrics.add("rewards/accuracy", (c_rew > r_rew).float().mean() / len(mbs))
                    metrics.add("rewards/margin", (c_rew - r_rew).mean() / len(mbs))
                ntok = mb["chosen_input_ids"].numel() + mb["rejected_input_ids"].numel()
                metrics.add("token_count", float(ntok))
                for k in ("chosen", "rejected"):
                    cu = mb[f"{k}_cu_seq_lens_q"]
                    lengths += (cu[1:] - cu[:-1]).tolist()
            if lora is not None:
                norm = lora.finish(len(mbs), learner.lr(completed), args.max_grad_norm)
                learner.global_step = completed + 1
            else:
                norm = learner.optimizer_step()
            profiler.step()
            completed += 1
            if completed % args.logging_steps == 0:
                metrics.reduce_(average=True)
                vals = metrics.get_metrics_list()
                step_time = time.time() - step_t0
                tokens_step = vals.pop("token_count") * data_world
                tokens_seen += tokens_step
                last = {**vals, "learning_rate": learner.lr(completed - 1), "grad_norm": float(norm), "epoch": epoch,
                        "training_step": completed, "perf/tokens_per_second_step": tokens_step / max(step_time, 1e-9),
                        "perf/tokens_per_second_avg": tokens_seen / max(time.time() - t_start, 1e-9),
                        "perf/mfu_step": dims.approximate_learner_utilization(tokens_step, sum(x * x for x in lengths) * world / max(1, sum(lengths)),
                                                                              step_time, world, device_name=None)}
                tracker.log(last, completed)
                if is_main:
                    logger.info("step %d loss %.4f acc %.3f", completed, last["train_loss"], last.get("rewards/accuracy", float("nan")))
                metrics.zero_()
            if args.checkpointing_steps and completed % args.checkpointing_steps == 0:
                d = os.path.join(args.output_dir, f"step_{completed}")
                save_train_state(d, learner.opt, {"completed_steps": completed, "epoch": epoch, "loader": loader.state_dict()},
                                 before_complete=lora.save_state if lora is not None else None)
                if is_main:
                    clean_last_n_checkpoints(args.output_dir, args.keep_last_n_checkpoints)
        if completed >= max_steps:
            break
    pdist.barrier()
    full_weights = learner.full_flat()  # a gather when the parameters are sharded: every rank takes part
    if is_main:
        save_hf_checkpoint(full_weights, spec, args.output_dir, tokenizer=tokenizer)   # with adapters: the merged model
        if lora is not None:
            lora.save(os.path.join(args.output_dir, "adapter"), args.model_name_or_path)
    profiler.close()
    tracker.close()
    pdist.barrier()
    last["completed_steps"] = completed
    return last


def cli() -> None:
    """Command line: a YAML / JSON recipe and / or ``--key value`` flags."""
    main(*ArgumentParserPlus((DPOExperimentConfig, TokenizerConfig)).parse())


if __name__ == "__main__":
    cli()
