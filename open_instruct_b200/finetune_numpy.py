"""SFT from pre-tokenised numpy shards: fixed-length packed windows, token-count batch sizes.

This is the counterpart of the reference's second SFT entry point (``open_instruct/olmo_core_finetune.py:137-363``):
it does not tokenise - it requires the output of ``data/numpy_dataset_conversion.py`` - and its batch is counted in
tokens: ``global_batch_size`` tokens per optimizer step, ``rank_microbatch_size`` tokens per forward/backward, both
multiples of ``sequence_length``.  The loss is the token-weighted sum over the whole global batch (every target token
weighs the same whatever micro-batch or rank it landed in).  Training state (optimizer shards, step, data position)
is saved every ``save_interval`` steps and picked up again from ``save_folder``; the final model is exported as a
Hugging Face directory.  The sharded-optimizer engine underneath is the same one the other trainers use.
"""

from __future__ import annotations

import math
import os
import time
from dataclasses import asdict, dataclass

import numpy as np
import torch

from .ckpt.hf_io import load_hf_checkpoint, save_hf_checkpoint
from .ckpt.train_state import load_train_state, save_train_state
from .data.collate import IGNORE, shift_labels
from .data.numpy_dataset_conversion import NumpyPackedFSLDataset
from .learner import Learner, LearnerConfig
from .models.spec import get_spec
from .parallel import dist as pdist
from .utils.common import Tracker, clean_last_n_checkpoints, get_last_checkpoint_path, is_checkpoint_folder, set_seed, setup_logger

logger = setup_logger(__name__)


@dataclass
class Args:
    model_name_or_path: str = "tiny"
    dataset_path: str = ""
    vocab_size: int | None = None          # of the tokenizer the shards were written with (defaults to the model's)
    sequence_length: int = 4096
    global_batch_size: int = 64 * 4096     # tokens per optimizer step over all ranks
    rank_microbatch_size: int = 4096       # tokens per forward/backward on one rank
    learning_rate: float = 8e-5
    weight_decay: float = 0.0
    warmup_ratio: float = 0.03
    lr_scheduler_type: str = "linear"
    max_grad_norm: float = 1.0
    num_epochs: int = 1
    max_train_steps: int | None = None
    seed: int = 33333
    save_folder: str = "output/sft_numpy"
    save_interval: int = 1000
    keep_last_n_checkpoints: int = 2
    ops: str = "auto"
    comm_backend: str = "fused"
    gradient_checkpointing: bool = False
    logging_steps: int = 1
    exp_name: str = "sft_numpy"
    # parallelism switches of the reference's entry point (``open_instruct/olmo_core_finetune.py:208-218``,
    # ``open_instruct/olmo_core_utils.py:151-181``)
    cp_degree: int | None = None           # context parallelism: every packed micro-batch is split over this many consecutive ranks
    cp_strategy: str = "ulysses"           # "ulysses" (built: heads <-> sequence exchange); "llama3" / "zig_zag" rings are refused
    shard_parameters: bool | None = None   # FSDP-style parameter sharding (None: only when the model does not fit resident)
    fsdp_shard_degree: int | None = None   # HSDP: shard over groups of this many ranks, replicate across the groups


def window_to_batch(windows) -> dict:
    """Concatenate windows into one packed micro-batch (documents keep their boundaries, window edges cut documents)."""
    ids = torch.from_numpy(np.concatenate([w.input_ids for w in windows]))
    mask = torch.from_numpy(np.concatenate([w.label_mask for w in windows]))
    cu, off = [0], 0
    for w in windows:
        cu += [off + int(c) for c in w.cu_seqlens[1:]]
        off += len(w.input_ids)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    starts = cu_t[:-1].long()
    lens = (cu_t[1:] - cu_t[:-1]).long()
    pos = torch.arange(ids.numel()) - torch.repeat_interleave(starts, lens)
    labels = torch.where(mask, ids, torch.full_like(ids, IGNORE))
    labels[starts] = IGNORE  # the first token of a document has no predecessor
    return {"input_ids": ids, "labels": labels, "labels_shifted": shift_labels_per_doc(labels, cu_t), "position_ids": pos,
            "cu_seq_lens_q": cu_t, "cu_seq_lens_k": cu_t, "max_length_q": int(lens.max()), "max_length_k": int(lens.max())}


def shift_labels_per_doc(labels: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
    """``out[t] = labels[t + 1]`` inside a document; the last position of every document is ignored."""
    out = shift_labels(labels)
    out[cu[1:].long() - 1] = IGNORE
    return out


def main(args: Args) -> dict:
    rank, world, device = pdist.init_distributed()
    set_seed(args.seed)
    spec = get_spec(args.model_name_or_path)
    L = args.sequence_length
    from .config.schemas import check_context_parallel

    cp = check_context_parallel(args.cp_degree, args.cp_strategy, world)
    dp_world, dp_rank = world // cp, rank // cp  # the ranks of one context-parallel group read the same windows
    if args.rank_microbatch_size % L or args.global_batch_size % (args.rank_microbatch_size * dp_world):
        raise ValueError("rank_microbatch_size must be a multiple of sequence_length, and global_batch_size of rank_microbatch_size x "
                         "data-parallel size (world size / cp_degree)")
    if cp > 1 and args.rank_microbatch_size % cp:
        raise ValueError("rank_microbatch_size must divide by cp_degree")
    ds = NumpyPackedFSLDataset(args.dataset_path, L, args.vocab_size or spec.vocab_size)
    win_per_step = args.global_batch_size // L
    win_per_micro = args.rank_microbatch_size // L
    micro_per_rank = win_per_step // (win_per_micro * dp_world)
    steps_per_epoch = len(ds) // win_per_step
    if steps_per_epoch == 0:
        raise ValueError(f"dataset has {len(ds)} windows of {L} tokens; one step needs {win_per_step}")
    max_steps = args.max_train_steps or steps_per_epoch * args.num_epochs
    ops = args.ops if args.ops != "auto" else ("fused" if device.type == "cuda" and spec.head_dim == 128 and not spec.post_norm and not spec.num_experts else "ref")
    cfg = LearnerConfig(ops=ops, comm=args.comm_backend if world > 1 else "none", learning_rate=args.learning_rate,
                        weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm, lr_scheduler_type=args.lr_scheduler_type,
                        warmup_steps=int(max_steps * args.warmup_ratio), total_steps=max_steps,
                        gradient_checkpointing=args.gradient_checkpointing, seed=args.seed, sequence_parallel_size=cp,
                        sp_max_tokens=args.rank_microbatch_size if cp > 1 else 0, shard_parameters=args.shard_parameters,
                        shard_degree=args.fsdp_shard_degree)
    learner = Learner(spec, cfg, device=device)
    src = args.model_name_or_path
    if os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
        learner.load_hf(src)
    tracker = Tracker(args.save_folder, args.exp_name, asdict(args), report_to=("jsonl",), enabled=rank == 0)
    step = 0
    ckpt = get_last_checkpoint_path(args.save_folder, None)
    if ckpt and is_checkpoint_folder(ckpt):
        step = load_train_state(ckpt, learner.opt)["completed_steps"]
        learner.global_step = step
    metrics: dict = {}
    t0, tokens_seen = time.time(), 0
    while step < max_steps:
        epoch, in_epoch = divmod(step, steps_per_epoch)
        order = np.random.default_rng(args.seed + epoch).permutation(len(ds))
        base = in_epoch * win_per_step
        mine = order[base + dp_rank * micro_per_rank * win_per_micro: base + (dp_rank + 1) * micro_per_rank * win_per_micro]
        mbs = []
        for m in range(micro_per_rank):
            b = window_to_batch([ds[int(i)] for i in mine[m * win_per_micro:(m + 1) * win_per_micro]])
            mbs.append({k: (v.to(device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in b.items()})
        out = learner.sft_step(mbs, "sum")
        step += 1
        tokens_seen += args.global_batch_size
        if step % args.logging_steps == 0:
            metrics = {"train_loss": float(out["loss"]), "grad_norm": float(out["grad_norm"]), "learning_rate": learner.lr(step - 1),
                       "tokens_per_second": tokens_seen / max(time.time() - t0, 1e-9), "training_step": step}
            tracker.log(metrics, step)
        if args.save_interval and step % args.save_interval == 0:
            save_train_state(os.path.join(args.save_folder, f"step_{step}"), learner.opt, {"completed_steps": step, "epoch": epoch, "loader": {}})
            if rank == 0:
                clean_last_n_checkpoints(args.save_folder, args.keep_last_n_checkpoints)
    pdist.barrier()
    full_weights = learner.full_flat()  # a gather when the parameters are sharded: every rank takes part
    if rank == 0:
        save_hf_checkpoint(full_weights, spec, os.path.join(args.save_folder, "hf"))
    tracker.close()
    pdist.barrier()
    metrics["completed_steps"] = step
    return metrics


if __name__ == "__main__":
    from .config.argparser import ArgumentParserPlus

    main(ArgumentParserPlus((Args,)).parse())
