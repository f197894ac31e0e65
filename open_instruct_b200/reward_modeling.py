"""Bradley-Terry reward-model training (the ``reward_modeling`` API) and its evaluation helper.

    python -m open_instruct_b200.reward_modeling --model_name_or_path ... --dataset_mixer_list data.jsonl 1.0

Behaviour follows ``open_instruct/reward_modeling.py`` (``Args`` ``:55-157``, scalar head initialised with
``std = 1/sqrt(hidden + 1)`` ``:306-308``, loss ``-logsigmoid(r_chosen - r_rejected)`` ``:351-360``, AdamW
``eps = 1e-5``) and ``get_reward`` (``open_instruct/model_utils.py:372-436``: the score is read at the last
non-pad token).  The backbone is the packed decoder of this package: chosen and rejected sequences
of the micro-batch are concatenated along the token axis, final hidden states come from the fused
forward, and only the last token of every document reaches the scalar head.
"""

from __future__ import annotations

import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Literal

import torch
import torch.nn.functional as F

from .ckpt.hf_io import load_hf_checkpoint, save_hf_checkpoint
from .config.argparser import ArgumentParserPlus
from .config.schemas import ModelConfig
from .data.collate import flatten_examples, to_device
from .data.loader import HFDataLoader
from .data.mixer import get_cached_dataset_tulu
from .data.tokenize import (
    CHOSEN_INPUT_IDS_KEY,
    REJECTED_INPUT_IDS_KEY,
    TOKENIZED_PREFERENCE_DATASET_KEYS,
    TokenizerConfig,
)
from .learner import Learner, LearnerConfig
from .models import get_spec
from .parallel import dist as pdist
from .utils.common import Tracker, set_seed, setup_logger

logger = setup_logger(__name__)


@dataclass
class Args:
    dataset_mixer_list: list[str] = field(default_factory=lambda: ["allenai/tulu-3-wildchat-reused-on-policy-8b", "1.0"])
    dataset_mixer_eval_list: list[str] = field(default_factory=list)
    dataset_mixer_list_splits: list[str] = field(default_factory=lambda: ["train"])
    dataset_mixer_eval_list_splits: list[str] = field(default_factory=list)
    dataset_transform_fn: list[str] = field(default_factory=lambda: ["preference_tokenize_v1", "preference_filter_v1"])
    dataset_target_columns: list[str] = field(default_factory=lambda: list(TOKENIZED_PREFERENCE_DATASET_KEYS))
    dataset_cache_mode: Literal["hf", "local"] = "local"
    dataset_local_cache_dir: str = "local_dataset_cache"
    dataset_config_hash: str | None = None
    dataset_config_eval_hash: str | None = None
    dataset_skip_cache: bool = False
    max_token_length: int = 512
    max_prompt_token_length: int = 256
    cache_dataset_only: bool = False
    exp_name: str = "reward_modeling"
    seed: int = 1
    run_name: str | None = None
    eps: float = 1e-5
    learning_rate: float = 2e-5
    lr_scheduler_type: Literal["linear", "cosine", "cosine_with_restarts", "polynomial", "constant", "constant_with_warmup"] = "linear"
    warm_up_steps: int = 0
    num_train_epochs: int = 1
    gradient_accumulation_steps: int = 8
    per_device_train_batch_size: int | None = 1
    per_device_eval_batch_size: int | None = 1
    total_episodes: int | None = None
    world_size: int | None = None
    micro_batch_size: int | None = None
    local_batch_size: int | None = None
    batch_size: int | None = None
    num_training_steps: int | None = None
    num_evals: int = 1
    eval_freq: int | None = None
    with_tracking: bool = False
    wandb_project_name: str = "open_instruct_internal"
    wandb_entity: str | None = None
    push_to_hub: bool = False
    hf_entity: str | None = None
    hf_repo_id: str | None = None
    hf_repo_revision: str | None = None
    hf_repo_url: str | None = None
    output_dir: str = "output"
    gs_bucket_path: str | None = None
    ops: str = "auto"
    comm_backend: str = "auto"


def layer_init(weight: torch.Tensor, std: float) -> torch.Tensor:
    torch.nn.init.normal_(weight, std=std)
    return weight


class RewardHead:
    """Scalar head ``score.weight`` [1, hidden] (replicated on every rank, fp32, own AdamW)."""

    def __init__(self, hidden: int, device, lr: float, eps: float, seed: int):
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(1, hidden, generator=g) * (1.0 / math.sqrt(hidden + 1))
        self.weight = w.to(device).requires_grad_(True)
        self.opt = torch.optim.AdamW([self.weight], lr=lr, eps=eps, weight_decay=0.0)

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        return (h.float() @ self.weight.t()).squeeze(-1)

    def step(self, lr: float, scale: float, group=None) -> None:
        if self.weight.grad is not None:
            pdist.all_reduce_(self.weight.grad, group=group)
            self.weight.grad.mul_(scale)
            for g in self.opt.param_groups:
                g["lr"] = lr
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)


def save_reward_model(flat: torch.Tensor, score_weight: torch.Tensor, spec, out_dir: str, tokenizer=None, dtype=torch.bfloat16) -> None:
    """A folder ``AutoModelForSequenceClassification.from_pretrained`` reads: the backbone under its usual names, the scalar
    head as ``score.weight`` in the same weight files, no ``lm_head``, the family's ``...ForSequenceClassification``
    architecture and ``num_labels = 1`` (what the reference saves, ``open_instruct/reward_modeling.py:395-410``)."""
    arch = spec.to_hf_config()["architectures"][0].replace("ForCausalLM", "ForSequenceClassification")
    extra = {"architectures": [arch], "num_labels": 1, "id2label": {"0": "LABEL_0"}, "label2id": {"LABEL_0": 0}}
    if spec.pad_token_id is None and tokenizer is not None and getattr(tokenizer, "pad_token_id", None) is not None:
        extra["pad_token_id"] = tokenizer.pad_token_id  # HF reads the score at the last non-pad token
    save_hf_checkpoint(flat, spec, out_dir, tokenizer=tokenizer, dtype=dtype, extra_config=extra,
                       extra_tensors={"score.weight": score_weight.reshape(1, -1)}, skip={"lm_head.weight"})


def load_score_weight(model_dir: str) -> torch.Tensor | None:
    """``score.weight`` of a reward-model folder (inside the weight files; the separate ``score_head.safetensors`` of earlier
    exports is still read), or None."""
    from safetensors import safe_open

    from .ckpt.hf_io import _open_shards

    try:
        handles, where = _open_shards(model_dir)
    except FileNotFoundError:
        handles, where = {}, {}
    if "score.weight" in where:
        return handles[where["score.weight"]].get_tensor("score.weight")
    old = os.path.join(model_dir, "score_head.safetensors")
    if os.path.exists(old):
        with safe_open(old, framework="pt", device="cpu") as f:
            return f.get_tensor("score.weight")
    return None


def pack_preference_batch(rows: list[dict]) -> dict:
    """Chosen documents first, then rejected, as one packed batch."""
    ids = [r[CHOSEN_INPUT_IDS_KEY] for r in rows] + [r[REJECTED_INPUT_IDS_KEY] for r in rows]
    batch = flatten_examples(ids)
    batch["num_pairs"] = len(rows)
    if "index" in rows[0]:
        batch["index"] = torch.tensor([int(r["index"]) for r in rows])
    return batch


def get_reward(learner: Learner, head: RewardHead, batch: dict) -> torch.Tensor:
    """Scalar reward of every document of a packed batch, read at its last token."""
    h = learner.model.hidden_states(batch["input_ids"], batch["position_ids"], batch["cu_seq_lens_q"])
    last = batch["cu_seq_lens_q"][1:].long() - 1
    return head(h[last])


def reward_loss(rewards: torch.Tensor, num_pairs: int):
    chosen, rejected = rewards[:num_pairs], rewards[num_pairs : 2 * num_pairs]
    loss = -F.logsigmoid(chosen - rejected).mean()
    acc = (chosen > rejected).float().mean()
    return loss, acc, chosen, rejected


@torch.no_grad()
def evaluate(learner: Learner, head: RewardHead, loader, device, max_batches: int | None = None) -> dict:
    """Accuracy / loss / mean scores over a preference set (``open_instruct/reward_modeling_eval.py:33``)."""
    tot = {"loss": 0.0, "accuracy": 0.0, "chosen": 0.0, "rejected": 0.0, "n": 0}
    for i, batch in enumerate(loader):
        if max_batches is not None and i >= max_batches:
            break
        batch = to_device(batch, device)
        loss, acc, c, r = reward_loss(get_reward(learner, head, batch), batch["num_pairs"])
        n = batch["num_pairs"]
        tot["loss"] += loss.item() * n
        tot["accuracy"] += acc.item() * n
        tot["chosen"] += c.sum().item()
        tot["rejected"] += r.sum().item()
        tot["n"] += n
    n = max(tot["n"], 1)
    return {"eval/rm/loss": tot["loss"] / n, "eval/rm/accuracy": tot["accuracy"] / n, "eval/rm/chosen_rewards": tot["chosen"] / n,
            "eval/rm/rejected_rewards": tot["rejected"] / n, "eval/rm/reward_margin": (tot["chosen"] - tot["rejected"]) / n}


def main(args: Args, tc: TokenizerConfig, model_config: ModelConfig) -> dict:
    rank, world, device = pdist.init_distributed()
    set_seed(args.seed)
    is_main = rank == 0
    if tc.tokenizer_name_or_path is None:
        tc.tokenizer_name_or_path = model_config.model_name_or_path
    transform_args = [{}, {"max_token_length": args.max_token_length, "max_prompt_token_length": args.max_prompt_token_length}]
    transform_args = transform_args[: len(args.dataset_transform_fn)]

    def _load(mix, splits, h):
        return get_cached_dataset_tulu(mix, splits, tc, args.dataset_transform_fn, transform_args,
                                       target_columns=args.dataset_target_columns, dataset_cache_mode=args.dataset_cache_mode,
                                       dataset_config_hash=h, dataset_local_cache_dir=args.dataset_local_cache_dir,
                                       dataset_skip_cache=args.dataset_skip_cache)

    if is_main:
        train = _load(args.dataset_mixer_list, args.dataset_mixer_list_splits, args.dataset_config_hash)
    pdist.barrier()
    if not is_main:
        train = _load(args.dataset_mixer_list, args.dataset_mixer_list_splits, args.dataset_config_hash)
    eval_ds = None
    if args.dataset_mixer_eval_list:
        eval_ds = _load(args.dataset_mixer_eval_list, args.dataset_mixer_eval_list_splits or ["train"], args.dataset_config_eval_hash)
    if args.cache_dataset_only:
        return {"cached": len(train)}
    tokenizer = tc.tokenizer
    # derived batch sizes, as the reference computes them
    args.world_size = world
    args.micro_batch_size = args.per_device_train_batch_size * world
    args.local_batch_size = args.per_device_train_batch_size * args.gradient_accumulation_steps
    args.batch_size = args.local_batch_size * world
    if args.total_episodes is None:
        args.total_episodes = args.num_train_epochs * len(train)
    args.num_training_steps = max(1, args.total_episodes // args.batch_size)
    args.eval_freq = args.eval_freq or max(1, args.num_training_steps // max(1, args.num_evals))

    spec = get_spec(model_config.config_name or model_config.model_name_or_path)
    from .config.schemas import spec_with_rope_flags

    spec = spec_with_rope_flags(spec, model_config)   # --rope_scaling_factor: YaRN context extension
    if len(tokenizer) > spec.vocab_size:
        spec = spec.replace(vocab_size=(len(tokenizer) + 7) // 8 * 8)
    cfg = LearnerConfig(ops=args.ops, comm=args.comm_backend, learning_rate=args.learning_rate, eps=args.eps,
                        lr_scheduler_type=args.lr_scheduler_type, warmup_steps=args.warm_up_steps,
                        total_steps=args.num_training_steps, gradient_checkpointing=model_config.gradient_checkpointing, seed=args.seed)
    learner = Learner(spec, cfg, device=device)
    src = model_config.model_name_or_path
    if src and os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
        learner.load_hf(src)
    head = RewardHead(spec.hidden_size, device, args.learning_rate, args.eps, args.seed)
    if src and os.path.isdir(src):
        w0 = load_score_weight(src)  # continuing from a reward model: its head comes along with the backbone
        if w0 is not None:
            with torch.no_grad():
                head.weight.copy_(w0.reshape(1, -1).to(head.weight))
    loader = HFDataLoader(train, batch_size=args.micro_batch_size, seed=args.seed, dp_rank=rank, dp_world_size=world,
                          collator=pack_preference_batch, automatic_reshuffle=True)
    eval_loader = None
    if eval_ds is not None:
        eval_loader = HFDataLoader(eval_ds, batch_size=(args.per_device_eval_batch_size or 1) * world, seed=args.seed, dp_rank=rank,
                                   dp_world_size=world, collator=pack_preference_batch, drop_last=False)
    tracker = Tracker(args.output_dir, args.run_name or args.exp_name, asdict(args),
                      report_to=("tensorboard", "wandb") if args.with_tracking else ("jsonl",),
                      wandb_project=args.wandb_project_name, wandb_entity=args.wandb_entity, enabled=is_main)
    it = iter(loader)
    last = {}
    t0 = time.time()
    for step in range(1, args.num_training_steps + 1):
        losses, accs, cs, rs = [], [], [], []
        for _ in range(args.gradient_accumulation_steps):
            try:
                batch = next(it)
            except StopIteration:
                it = iter(loader)
                batch = next(it)
            batch = to_device(batch, device)
            loss, acc, c, r = reward_loss(get_reward(learner, head, batch), batch["num_pairs"])
            learner.backward(loss)
            losses.append(loss.detach()); accs.append(acc); cs.append(c.mean().detach()); rs.append(r.mean().detach())
        lr = learner.lr()
        scale = 1.0 / (args.gradient_accumulation_steps * world)
        head.step(lr, scale)
        norm = learner.optimizer_step()
        vec = torch.stack([torch.stack(losses).mean(), torch.stack(accs).mean(), torch.stack(cs).mean(), torch.stack(rs).mean()])
        pdist.all_reduce_(vec)
        vec /= world
        last = {"train/rm/loss": vec[0].item(), "train/rm/accuracy": vec[1].item(), "train/rm/chosen_rewards": vec[2].item(),
                "train/rm/rejected_rewards": vec[3].item(), "train/rm/reward_margin": (vec[2] - vec[3]).item(), "train/rm/lr": lr,
                "episode": step * args.batch_size, "grad_norm": float(norm)}
        if eval_loader is not None and (step % args.eval_freq == 0 or step == args.num_training_steps):
            last.update(evaluate(learner, head, eval_loader, device))
        tracker.log(last, step)
        if is_main:
            logger.info("step %d loss %.4f acc %.3f", step, last["train/rm/loss"], last["train/rm/accuracy"])
    pdist.barrier()
    full_weights = learner.full_flat()  # a gather when the parameters are sharded: every rank takes part
    if is_main:
        save_reward_model(full_weights, head.weight, spec, args.output_dir, tokenizer)
    tracker.close()
    pdist.barrier()
    last["seconds"] = time.time() - t0
    return last


def cli() -> None:
    """Command line: a YAML / JSON recipe and / or ``--key value`` flags."""
    main(*ArgumentParserPlus((Args, TokenizerConfig, ModelConfig)).parse())


if __name__ == "__main__":
    cli()
