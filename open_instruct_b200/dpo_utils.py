"""DPO family: configuration, losses, policy forwards over packed batches, reference-logprob cache.

Loss definitions follow the reference (``open_instruct/dpo_utils.py``: ``dpo_loss`` ``:523-563``, ``wpo_loss``
``:566-613``, ``simpo_loss`` ``:617-642``, ``compute_loss`` ``:645-686``), as does the cache protocol
(``build_reference_logprobs_cache`` ``:405-520``, hash ``:362-383``).  What differs is the forward: there is
no padded path and no ``[T, V]`` fp32 logits - chosen and rejected sides are concatenated along the
packed token axis, the model returns per-token log-probs straight from the bf16 logits kernel, and
per-sequence sums/means are a segment reduction.
"""

from __future__ import annotations

import enum
import hashlib
import json
import logging
import os
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from .config.schemas import (
    CheckpointConfig,
    DatasetMixConfig,
    EvalConfig,
    ExperimentConfig,
    HubConfig,
    LoggingConfig,
    LoRAConfig,
    ModelConfig,
    TrainingConfig,
)
from .data.collate import concatenated_inputs, get_batch_logps
from .data.tokenize import TOKENIZED_PREFERENCE_DATASET_KEYS
from .parallel import dist as pdist

logger = logging.getLogger(__name__)


class DPOLossType(str, enum.Enum):
    dpo = "dpo"
    dpo_norm = "dpo_norm"
    simpo = "simpo"
    wpo = "wpo"

    @property
    def is_average_loss(self) -> bool:
        """Length-normalised variants compare mean (not summed) token log-probs."""
        return self in (DPOLossType.dpo_norm, DPOLossType.simpo)

    @property
    def needs_reference_model(self) -> bool:
        return self in (DPOLossType.dpo, DPOLossType.dpo_norm, DPOLossType.wpo)

    @property
    def computes_reward_metrics(self) -> bool:
        return self in (DPOLossType.dpo, DPOLossType.dpo_norm)


@dataclass
class DPOConfig:
    beta: float = 5.0
    loss_type: DPOLossType = DPOLossType.dpo_norm
    gamma_beta_ratio: float = 0.3
    label_smoothing: float = 0.0
    load_balancing_loss: bool = False
    load_balancing_weight: float = 0.001
    concatenated_forward: bool = True
    packing: bool = False


@dataclass
class DPOTrainingConfig(TrainingConfig):
    use_8bit_optimizer: bool = False
    dpo_use_paged_optimizer: bool = False
    optimizer_type: str = "adamw"
    optimizer_kwargs: dict | str = field(default_factory=dict)
    tensor_parallel_degree: int = 1
    context_parallel_degree: int = 1
    cache_logprobs_only: bool = False
    fsdp_shard_degree: int | None = None
    fsdp_num_replicas: int | None = None


REFERENCE_LOGPROBS_CACHE_PATH = os.environ.get("REFERENCE_LOGPROBS_CACHE_PATH", "reference_logprobs_cache")


@dataclass
class DPOExperimentConfig(ExperimentConfig, ModelConfig, DPOConfig, DPOTrainingConfig, DatasetMixConfig, LoRAConfig,
                          LoggingConfig, HubConfig, CheckpointConfig, EvalConfig):
    exp_name: str = "dpo"
    transform_fn: list[str] = field(default_factory=lambda: ["preference_tulu_tokenize_and_truncate_v1", "preference_tulu_filter_v1"])
    target_columns: list[str] = field(default_factory=lambda: list(TOKENIZED_PREFERENCE_DATASET_KEYS))
    do_not_randomize_output_dir: bool = False
    send_slack_alerts: bool = False
    additional_model_arguments: dict | str | None = field(default_factory=dict)
    sync_each_batch: bool = False
    dataset_name: str | None = None
    dataset_mixer: dict | None = None
    dataset_mix_dir: str | None = None
    dataset_config_name: str | None = None
    max_train_samples: int | None = None
    preprocessing_num_workers: int | None = None
    overwrite_cache: bool = False
    use_qlora: bool = False
    timeout: int = 1800
    save_to_hub: str | None = None
    use_liger_kernel: bool = False
    profiling: bool = False
    hf_metadata_dataset: str | None = None
    zero_stage: int | None = None
    offload_optimizer: bool = False
    shard_parameters: bool | None = None  # gather-on-use parameter sharding; None = only when the model does not fit resident
    offload_param: bool = False
    zero_hpz_partition_size: int = 8
    ops: str = "auto"
    comm_backend: str = "auto"

    @property
    def forward_fn(self):
        return concatenated_forward if self.concatenated_forward else separate_forward

    def __post_init__(self):
        if isinstance(self.loss_type, str):
            self.loss_type = DPOLossType(self.loss_type)
        if self.dataset_name is None and self.dataset_mixer is None and not self.mixer_list:
            raise ValueError("Need either a dataset name, dataset mixer, or a training file.")
        if self.dataset_name is not None and (self.dataset_mixer is not None or self.mixer_list):
            raise ValueError("Cannot provide two dataset selection mechanisms.")
        if self.try_launch_beaker_eval_jobs and not self.push_to_hub:
            raise ValueError("Cannot launch Beaker evaluation jobs without pushing to the Hub.")
        if isinstance(self.additional_model_arguments, str):
            self.additional_model_arguments = json.loads(self.additional_model_arguments)
        if isinstance(self.optimizer_kwargs, str):
            self.optimizer_kwargs = json.loads(self.optimizer_kwargs) if self.optimizer_kwargs.startswith("{") else {}
        if self.zero_stage is not None:
            if self.zero_stage not in (0, 1, 2, 3):
                raise ValueError(f"zero_stage must be 0, 1, 2, or 3, got {self.zero_stage}")
            if self.offload_param and self.zero_stage != 3:
                raise ValueError("offload_param can only be used with zero_stage 3")
        if self.offload_param:
            raise ValueError("offload_param is not built: with shard_parameters every GPU keeps 1/N of the bf16 weights (17.5 GB for a 70B "
                             "model on 8 GPUs), which fits; use offload_optimizer to move the 12 bytes/parameter of optimizer state to host memory")
        if self.context_parallel_degree > 1:
            raise NotImplementedError("context parallelism is not supported with DPO: the preference trainer sums log-probs per sequence on one rank")
        if self.use_qlora or self.use_8bit_optimizer:
            raise ValueError("quantised training paths are not part of this framework")
        from .config.schemas import check_context_parallel, check_model_config

        check_model_config(self)
        if check_context_parallel(self.cp_degree, self.cp_strategy) > 1:
            raise ValueError("cp_degree > 1: the preference trainer sums log-probs per sequence on one rank and has no context-parallel "
                             "path; use tensor_parallel_degree or shard_parameters for long pairs (SFT and GRPO support sequence parallelism)")
        if self.load_balancing_loss:
            raise ValueError("load_balancing_loss is wired into SFT (finetune) for mixture-of-experts models; the preference trainers do not add it")


# ---------------------------------------------------------------------------------- losses
def dpo_loss(policy_chosen_logps, policy_rejected_logps, reference_chosen_logps, reference_rejected_logps, beta: float,
             reference_free: bool = False, label_smoothing: float = 0.0):
    """Sigmoid DPO (conservative variant when ``label_smoothing`` > 0).  Returns (losses, chosen_rewards, rejected_rewards)."""
    pi = policy_chosen_logps - policy_rejected_logps
    ref = torch.zeros_like(pi) if reference_free else reference_chosen_logps - reference_rejected_logps
    z = pi - ref
    losses = -F.logsigmoid(beta * z) * (1 - label_smoothing) - F.logsigmoid(-beta * z) * label_smoothing
    chosen_rewards = beta * (policy_chosen_logps - reference_chosen_logps).detach()
    rejected_rewards = beta * (policy_rejected_logps - reference_rejected_logps).detach()
    return losses, chosen_rewards, rejected_rewards


def wpo_loss(policy_chosen_logps, policy_rejected_logps, reference_chosen_logps, reference_rejected_logps, beta: float,
             label_smoothing: float = 0.0, chosen_loss_mask=None, rejected_loss_mask=None):
    """Weighted preference optimisation: DPO scaled by how on-policy the pair is,
    weight = clamp(exp(mean chosen logp + mean rejected logp), max 1), detached."""
    z = (policy_chosen_logps - policy_rejected_logps) - (reference_chosen_logps - reference_rejected_logps)
    nc = chosen_loss_mask.sum(-1).clamp(min=1) if chosen_loss_mask is not None else 1.0
    nr = rejected_loss_mask.sum(-1).clamp(min=1) if rejected_loss_mask is not None else 1.0
    weights = torch.clamp(torch.exp(policy_chosen_logps / nc + policy_rejected_logps / nr), max=1).detach()
    losses = (-F.logsigmoid(beta * z) * (1 - label_smoothing) - F.logsigmoid(-beta * z) * label_smoothing) * weights
    chosen_rewards = beta * (policy_chosen_logps - reference_chosen_logps).detach()
    rejected_rewards = beta * (policy_rejected_logps - reference_rejected_logps).detach()
    return losses, chosen_rewards, rejected_rewards


def simpo_loss(policy_chosen_logps, policy_rejected_logps, beta: float, gamma_beta_ratio: float, label_smoothing: float = 0.0):
    """Reference-free, length-normalised, with a target margin gamma = beta * gamma_beta_ratio."""
    z = (policy_chosen_logps - policy_rejected_logps) - gamma_beta_ratio
    losses = -F.logsigmoid(beta * z) * (1 - label_smoothing) - F.logsigmoid(-beta * z) * label_smoothing
    return losses, beta * policy_chosen_logps.detach(), beta * policy_rejected_logps.detach()


def compute_loss(args: DPOConfig, batch: dict, policy_chosen_logps, policy_rejected_logps, reference_cache=None,
                 token_counts: tuple | None = None):
    """Dispatch on ``args.loss_type``; reference log-probs come from the cache by dataset ``index``."""
    lt = DPOLossType(args.loss_type) if not isinstance(args.loss_type, DPOLossType) else args.loss_type
    ref_c = ref_r = None
    if lt.needs_reference_model:
        if reference_cache is None:
            raise ValueError(f"loss_type {lt.value} needs cached reference log-probs")
        idx = batch["index"]
        ref_c, ref_r = reference_cache["chosen_logps"][idx], reference_cache["rejected_logps"][idx]
    if lt in (DPOLossType.dpo, DPOLossType.dpo_norm):
        return dpo_loss(policy_chosen_logps, policy_rejected_logps, ref_c, ref_r, args.beta, label_smoothing=args.label_smoothing)
    if lt == DPOLossType.simpo:
        return simpo_loss(policy_chosen_logps, policy_rejected_logps, args.beta, args.gamma_beta_ratio, args.label_smoothing)
    if lt == DPOLossType.wpo:
        nc, nr = token_counts if token_counts is not None else (None, None)
        cm = torch.ones(len(nc), 1, device=policy_chosen_logps.device) * nc[:, None] if nc is not None else None
        rm = torch.ones(len(nr), 1, device=policy_chosen_logps.device) * nr[:, None] if nr is not None else None
        return wpo_loss(policy_chosen_logps, policy_rejected_logps, ref_c, ref_r, args.beta, args.label_smoothing, cm, rm)
    raise ValueError(f"unknown loss type {lt}")


# ---------------------------------------------------------------------------------- forwards
def concatenated_forward(learner, batch: dict, average_log_prob: bool = False):
    """One packed forward over chosen‖rejected.  Returns (chosen_logps, rejected_logps, aux) per pair."""
    packed, n_chosen = concatenated_inputs(batch)
    logp, _ = learner.token_logprobs(packed)
    per_doc = get_batch_logps(logp, packed["labels_shifted"], packed["cu_seq_lens_q"], average_log_prob)
    n_pairs = batch["index"].numel() if "index" in batch else n_chosen
    # a padded tail document (when rows are padded to a fixed length) sits after the real ones
    chosen = per_doc[:n_pairs]
    rejected = per_doc[n_chosen : n_chosen + n_pairs]
    counts = get_batch_logps(torch.ones_like(logp), packed["labels_shifted"], packed["cu_seq_lens_q"], False)
    aux = {"chosen_tokens": counts[:n_pairs], "rejected_tokens": counts[n_chosen : n_chosen + n_pairs]}
    return chosen, rejected, aux


def separate_forward(learner, batch: dict, average_log_prob: bool = False):
    """Two forwards (chosen, then rejected): halves peak activation memory at the cost of latency."""
    outs, aux = [], {}
    for side in ("chosen", "rejected"):
        sub = {k[len(side) + 1:]: v for k, v in batch.items() if k.startswith(side + "_")}
        logp, _ = learner.token_logprobs(sub)
        n_pairs = batch["index"].numel() if "index" in batch else sub["cu_seq_lens_q"].numel() - 1
        outs.append(get_batch_logps(logp, sub["labels_shifted"], sub["cu_seq_lens_q"], average_log_prob)[:n_pairs])
        aux[f"{side}_tokens"] = get_batch_logps(torch.ones_like(logp), sub["labels_shifted"], sub["cu_seq_lens_q"], False)[:n_pairs]
    return outs[0], outs[1], aux


# ---------------------------------------------------------------------------------- reference cache
class TensorCache:
    """Named 1-D tensors indexed by dataset index; atomic save (tmp + rename)
    (``open_instruct/model_utils.py:92-115``)."""

    def __init__(self, tensors: dict[str, torch.Tensor]):
        self.tensors = tensors

    def __getitem__(self, key: str) -> torch.Tensor:
        return self.tensors[key]

    def to_disk(self, path) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(path.suffix + ".tmp")
        torch.save({k: v.cpu() for k, v in self.tensors.items()}, tmp)
        os.replace(tmp, path)

    @classmethod
    def from_disk(cls, path, device=None) -> "TensorCache":
        data = torch.load(path, weights_only=True, map_location="cpu")
        return cls({k: v.to(device) if device is not None else v for k, v in data.items()})


def compute_reference_cache_hash(args: DPOExperimentConfig, dataset_config_hash: str) -> str:
    blob = {"concatenated_forward": args.concatenated_forward, "dataset_config_hash": dataset_config_hash,
            "loss_type": str(DPOLossType(args.loss_type).value), "max_train_samples": args.max_train_samples,
            "model_name_or_path": args.model_name_or_path, "model_revision": args.model_revision, "packing": args.packing,
            "use_lora": args.use_lora, "use_qlora": args.use_qlora}
    return hashlib.sha256(json.dumps(blob, sort_keys=True).encode()).hexdigest()[:16]


def build_reference_logprobs_cache(learner, dataloader, average_log_prob: bool, forward_fn, full_dataset_size: int, device,
                                   cache_path, is_main_process: bool) -> TensorCache:
    """Reference log-probs of every pair, computed once with the initial weights and cached on disk.

    Each rank fills the entries of the rows it sees into dense ``[dataset_size]`` fp32 vectors
    initialised to -inf; a MAX all-reduce merges them; any index still at -inf is an error.
    """
    cache_path = Path(cache_path)
    if cache_path.exists():
        logger.info("loading reference logprobs cache from %s", cache_path)
        return TensorCache.from_disk(cache_path, device=device)
    if is_main_process:
        cache_path.parent.mkdir(parents=True, exist_ok=True)
        probe = cache_path.parent / f".write_test_{cache_path.stem}"
        try:
            probe.touch()
            probe.unlink()
        except OSError as e:
            raise RuntimeError(f"Cannot write to cache directory {cache_path.parent}: {e}. "
                               "Set REFERENCE_LOGPROBS_CACHE_PATH to a writable location.") from e
    pdist.barrier()
    chosen = torch.full((full_dataset_size,), float("-inf"), dtype=torch.float32, device=device)
    rejected = torch.full((full_dataset_size,), float("-inf"), dtype=torch.float32, device=device)
    from .data.collate import to_device

    with torch.no_grad():
        for batch in dataloader:
            batch = to_device(batch, device)
            c, r, _ = forward_fn(learner, batch, average_log_prob=average_log_prob)
            if batch.get("is_padding", False):
                continue
            chosen[batch["index"]] = c.float()
            rejected[batch["index"]] = r.float()
    if pdist.is_dist():
        torch.distributed.all_reduce(chosen, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(rejected, op=torch.distributed.ReduceOp.MAX)
    missing = torch.unique(torch.cat([torch.where(chosen == float("-inf"))[0], torch.where(rejected == float("-inf"))[0]]))
    if missing.numel():
        raise RuntimeError(f"Missing {missing.numel()} indices during reference logprobs caching. First 10: {missing[:10].tolist()}")
    cache = TensorCache({"chosen_logps": chosen, "rejected_logps": rejected})
    if is_main_process:
        cache.to_disk(cache_path)
    pdist.barrier()
    return cache
