"""DPO driven by a ``Trainer`` with a train module and callbacks (the ``dpo`` API).

    python -m open_instruct_b200.dpo recipe.yaml [--flag value ...]

The reference has two DPO entry points that share one config dataclass: ``dpo_tune_cache.py`` (an accumulate / step loop)
and ``dpo.py`` (``open_instruct/dpo.py:141-342``: an olmo-core ``Trainer`` running a ``DPOTrainModule`` with callbacks,
HSDP + tensor parallelism).  This is the second one over this package's learner:

* the loss of a step is TOKEN-weighted over the rank's micro-batches (``train_modules.DPOTrainModule``), not a plain
  mean of micro-batch means as in ``dpo_tune_cache``;
* ``tensor_parallel_degree`` splits every layer over groups of that many ranks with a vocabulary-parallel log-prob head
  (``parallel/tp.py``); ``fsdp_shard_degree`` / ``shard_parameters`` shard the parameters (``parallel/zero3.py``);
* checkpointing, step timing, throughput / MFU and the optional profiler are callbacks (``trainer.py``);
* the final model is exported as a Hugging Face directory (a gather when parameters are sharded).

Dataset handling, the reference log-prob cache and its hash are the shared ``dpo_tune_cache.prepare``.
"""

from __future__ import annotations

import os
from dataclasses import asdict

from .ckpt.hf_io import save_hf_checkpoint
from .ckpt.train_state import load_train_state
from .config.argparser import ArgumentParserPlus
from .data.tokenize import TokenizerConfig
from .dpo_tune_cache import prepare
from .dpo_utils import DPOExperimentConfig
from .parallel import dist as pdist
from .train_modules import DPOTrainModule, num_tokens
from .trainer import CheckpointerCallback, PerfCallback, ProfilerCallback, StepTimingCallback, Trainer
from .utils.common import Tracker, get_last_checkpoint_path, is_checkpoint_folder, setup_logger

logger = setup_logger(__name__)


class _StepBatches:
    """Groups the loader's micro-batches into per-step lists of ``gradient_accumulation_steps`` and reshuffles per epoch."""

    def __init__(self, loader, accumulation: int):
        self.loader, self.accumulation = loader, max(1, accumulation)

    def __iter__(self):
        group = []
        for mb in self.loader:
            group.append(mb)
            if len(group) == self.accumulation:
                yield group
                group = []
        self.loader.reshuffle(self.loader._epoch + 1)


def main(args: DPOExperimentConfig, tc: TokenizerConfig) -> dict:
    if args.use_lora:   # as in the reference (``open_instruct/dpo.py:142-143``): adapters are the other trainer's business
        raise ValueError("LoRA is not supported by the callback-driven DPO trainer. Use dpo_tune_cache instead.")
    p = prepare(args, tc)
    if p.done is not None:
        return p.done
    learner = p.learner
    tracker = Tracker(args.output_dir, args.run_name or args.exp_name, asdict(args), report_to=args.report_to if args.with_tracking else ("jsonl",),
                      wandb_project=args.wandb_project, wandb_entity=args.wandb_entity, enabled=p.is_main)
    start = 0
    ckpt = get_last_checkpoint_path(args.output_dir, args.resume_from_checkpoint)
    if ckpt and is_checkpoint_folder(ckpt):
        st = load_train_state(ckpt, learner.opt)
        start = st["completed_steps"]
        learner.global_step = start
        if "loader" in st:
            p.loader.load_state_dict(st["loader"])
        logger.info("resumed from %s at step %d", ckpt, start)
    module = DPOTrainModule(learner, args, p.reference_cache, p.forward_fn, data_parallel_world=p.data_world)

    def tokens_of(batch):
        return sum(num_tokens(mb) for mb in batch)

    def seq_len_of(batch):
        lens = [int(x) for mb in batch for k in ("chosen", "rejected") for x in (mb[f"{k}_cu_seq_lens_q"][1:] - mb[f"{k}_cu_seq_lens_q"][:-1])]
        return sum(x * x for x in lens) / max(1, sum(lens))

    callbacks = [StepTimingCallback(), PerfCallback(p.dims, tokens_of, seq_len_of),
                 CheckpointerCallback(args.output_dir, args.checkpointing_steps, args.keep_last_n_checkpoints,
                                      extra_state=lambda: {"epoch": p.loader._epoch, "loader": p.loader.state_dict()}),
                 ProfilerCallback(args.profiling, args.output_dir)]
    trainer = Trainer(module, _StepBatches(p.loader, args.gradient_accumulation_steps), max_steps=p.max_steps, callbacks=callbacks, tracker=tracker,
                      save_folder=args.output_dir, metrics_collect_interval=args.logging_steps, dp_process_group=learner.group,
                      steps_per_epoch=p.steps_per_epoch, start_step=start)
    last = trainer.fit()
    pdist.barrier()
    full = learner.full_flat()  # a gather when the parameters are sharded or tensor-parallel: every rank takes part
    if p.is_main:
        save_hf_checkpoint(full, p.spec, args.output_dir, tokenizer=p.tokenizer)
    tracker.close()
    pdist.barrier()
    last["completed_steps"] = trainer.global_step
    return last


if __name__ == "__main__":
    main(*ArgumentParserPlus((DPOExperimentConfig, TokenizerConfig)).parse())
