"""GRPO configuration and loss mathematics.

Definitions follow the reference (``open_instruct/grpo_utils.py``): truncated-importance-sampling
correction rho with token / sequence / TV masking (``:372-463``), ``resolve_old_logprob`` (``:475-501``),
DAPO and CISPO policy losses with the four KL estimators (``:504-538``, ``open_instruct/model_utils.py:793-818``),
token-count normalisation across ranks (``:651-671``), pass@k (``:34-66``).  All functions are pure
tensor code on ``[B, T]`` or packed ``[T]`` tensors; the per-token log-probs they consume come from
the fused log-prob kernel on the B200 path.
"""

from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Literal

import numpy as np
import torch

from .config.schemas import ExperimentConfig
from .parallel import dist as pdist
from .utils.common import INVALID_LOGPROB


class GRPOLossType(str, enum.Enum):
    dapo = "dapo"
    cispo = "cispo"


@dataclass
class GRPOExperimentConfig(ExperimentConfig):
    exp_name: str = "grpo"
    # optimizer
    learning_rate: float = 2e-5
    lr_scheduler_type: str = "linear"
    warm_up_steps: int = 0
    warmup_ratio: float = 0.0
    weight_decay: float = 0.0
    set_weight_decay_on_bias_and_norm: bool = True
    fused_optimizer: bool = True
    max_grad_norm: float = 1.0
    # batch sizes
    per_device_train_batch_size: int = 1
    total_episodes: int = 100000
    world_size: int | None = None
    num_training_steps: int | None = None
    local_eval_every: int = 100
    eval_on_step_0: bool = False  # also evaluate (and save, with save_freq > 0) at the first training step
    save_freq: int = 200
    verify_weight_sync: bool = False  # debug: after every sync compare weight checksums of the learner and every engine rank
    save_final_model: bool = True  # benchmarks switch the final Hugging Face export off
    backend_timeout: int = 120
    model_dtype: str = "bfloat16"
    # algorithm
    num_epochs: int = 1
    num_mini_batches: int = 1
    beta: float = 0.05
    clip_lower: float = 0.2
    clip_higher: float = 0.272
    use_rho_correction: bool = True
    rho_clamp_lower_bound: float = 0.0
    rho_clamp_upper_bound: float = 2.0
    rho_mask_lower_bound: float = 0.0
    rho_mask_upper_bound: float = 0.0
    rho_mask_sequence_level: bool = False
    rho_mask_tv_divergence: bool = False
    kl_estimator: Literal[0, 1, 2, 3] = 2
    loss_denominator: str = "token"
    alpha: float = 0.6
    ref_policy_update_freq: int | None = None
    load_ref_policy: bool = True
    loss_fn: GRPOLossType = GRPOLossType.dapo
    record_entropy: bool = False
    use_vllm_logprobs: bool = False
    # the sampling temperature lives in StreamingDataLoaderConfig; main() copies it here for the learner's log-prob passes
    temperature: float = field(default=1.0, init=False)
    # process topology
    single_gpu_mode: bool = False
    num_learners_per_node: list[int] = field(default_factory=lambda: [1])
    num_nodes: int = 1
    sequence_parallel_size: int = 1
    deepspeed_stage: int = 0
    deepspeed_zpg: int = 8
    deepspeed_offload_param: bool = False
    deepspeed_offload_optimizer: bool = False
    shard_parameters: bool | None = None  # gather-on-use parameter sharding of the learner; None = only when the model does not fit resident
    deepspeed_checkpoint_load_universal: bool = False
    gather_whole_model: bool = True
    fsdp_shard_degree: int | None = None
    fsdp_num_replicas: int | None = None
    enable_queue_dashboard: bool = True
    queue_dashboard_port: int | None = None
    # tracking / saving
    verbose: bool = False
    with_tracking: bool = False
    wandb_project_name: str = "open_instruct_internal"
    wandb_entity: str | None = None
    push_to_hub: bool = False
    hf_entity: str | None = None
    hf_repo_id: str | None = None
    hf_repo_revision: str | None = None
    hf_repo_url: str | None = None
    output_dir: str = "output"
    cache_dataset_only: bool = False
    keep_last_n_checkpoints: int = 3
    checkpoint_state_freq: int = 200
    checkpoint_state_dir: str | None = None
    gs_checkpoint_state_dir: str | None = None
    try_launch_beaker_eval_jobs_on_weka: bool = False
    try_auto_save_to_beaker: bool = False
    gs_bucket_path: str | None = None
    oe_eval_tasks: list[str] | None = None
    oe_eval_max_length: int = 4096
    oe_eval_beaker_image: str | None = None
    oe_eval_gpu_multiplier: int | None = None
    eval_priority: Literal["low", "normal", "high", "urgent"] = "normal"
    eval_workspace: str = "ai2/tulu-3-results"
    send_slack_alerts: bool = False
    eval_pass_at_k: int = 1
    eval_top_p: float | None = None
    ops: str = "auto"
    comm_backend: str = "auto"

    def __post_init__(self):
        if isinstance(self.loss_fn, str):
            self.loss_fn = GRPOLossType(self.loss_fn)
        if self.loss_denominator != "token":
            try:
                if float(self.loss_denominator) <= 0:
                    raise ValueError
            except ValueError:
                raise ValueError(f"loss_denominator must be 'token' or a positive number, got {self.loss_denominator!r}") from None
        if self.num_mini_batches < 1 or self.num_epochs < 1:
            raise ValueError("num_mini_batches and num_epochs must be >= 1")
        if self.eval_on_step_0 and self.local_eval_every <= 0:
            raise ValueError("`eval_on_step_0` requires `local_eval_every` > 0. Set `local_eval_every` to a positive value or "
                             "disable `eval_on_step_0`.")
        if self.sequence_parallel_size < 1:
            raise ValueError("sequence_parallel_size must be >= 1")
        if self.deepspeed_offload_param:
            raise ValueError("deepspeed_offload_param is not built: with shard_parameters every GPU keeps 1/N of the bf16 weights, which fits "
                             "in GPU memory; use deepspeed_offload_optimizer to move the optimizer states to host memory")
        # (the reference needs deepspeed_stage 3 for sequence parallelism, ``open_instruct/grpo_utils.py:275-276``; here it
        # works with resident and with sharded parameters alike)
        if self.use_vllm_logprobs and self.use_rho_correction:
            # rho == 1 by construction when the engine's log-probs ARE the old log-probs
            self.use_rho_correction = False
        if self.checkpoint_state_dir is not None and self.checkpoint_state_freq <= 0:
            raise ValueError("checkpoint_state_freq must be positive when checkpoint_state_dir is set")
        if not (0.0 <= self.alpha <= 1.0):
            raise ValueError("alpha (reference polyak coefficient) must lie in [0, 1]")


# ---------------------------------------------------------------------------------- small helpers
def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis: int | None = None, denominator: float | None = None) -> torch.Tensor:
    """Mean of ``values`` where ``mask`` (``open_instruct/rl_utils.py:426-448``).

    ``values`` may carry leading dimensions the mask does not have (e.g. four KL estimators stacked over one mask): the
    result keeps them.  ``axis=None``: one mean over all masked elements.  ``axis=k``: a masked mean along mask dimension
    ``k`` for every row, then the plain mean of those (sample-level averaging).  An empty mask (or empty row) gives 0, not
    NaN.  With ``denominator`` the masked SUM is divided by it instead (token-normalised losses)."""
    m = mask.to(values.dtype)
    extra = values.ndim - m.ndim
    if axis is None:
        dims = tuple(range(extra, values.ndim))
    else:
        dims = axis + extra if axis >= 0 else axis
    num = (values * m).sum(dim=dims)
    if denominator is not None:
        res = num / denominator if denominator > 0 else torch.zeros_like(num)
    else:
        den = m.sum(dim=axis) if axis is not None else m.sum()
        res = torch.where(den > 0, num / den.clamp(min=1e-30), torch.zeros_like(num))
    return res.flatten(extra).mean(-1) if res.ndim > extra else res


def estimate_kl(ref_logprobs_diff: torch.Tensor, ratio: torch.Tensor) -> torch.Tensor:
    """Four estimators of KL(pi || ref) stacked on dim 0, d = log pi - log ref:
    0: d, 1: d^2/2, 2: expm1(-d) + d (non-negative, low variance), 3: ratio * d."""
    d = ref_logprobs_diff
    return torch.stack([d, d.pow(2) / 2, torch.expm1(-d) + d, ratio * d])


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    z = logits.float()
    lse = torch.logsumexp(z, -1)
    return lse - (torch.softmax(z, -1) * z).sum(-1)


def mask_logprobs(vllm_logprobs: torch.Tensor, response_mask: torch.Tensor) -> torch.Tensor:
    out = torch.masked_fill(vllm_logprobs, ~response_mask, INVALID_LOGPROB)
    return torch.nan_to_num(out, nan=INVALID_LOGPROB)


def compute_vllm_local_debug_metrics(local_logprobs, vllm_logprobs, response_mask) -> dict[str, float]:
    """How far the rollout engine's log-probs are from the learner's for the same tokens."""
    with torch.no_grad():
        valid = response_mask & ~torch.isnan(vllm_logprobs)
        n = valid.sum()
        diff = torch.masked_fill((local_logprobs - vllm_logprobs).abs(), ~valid, 0.0)
        mean = diff.sum() / n if n > 0 else torch.tensor(0.0)
        mx = diff.max() if n > 0 else torch.tensor(0.0)
        std = diff[valid].std() if n > 1 else torch.tensor(0.0)
        rkl = torch.masked_fill(torch.exp(vllm_logprobs) * (vllm_logprobs - local_logprobs), ~valid, 0.0)
        rkl = rkl.sum() / n if n > 0 else torch.tensor(0.0)
    return {"debug/vllm_vs_local_logprob_diff_mean": float(mean), "debug/vllm_vs_local_logprob_diff_max": float(mx),
            "debug/vllm_vs_local_logprob_diff_std": float(std), "debug/vllm_local_reverse_kl": float(rkl)}


# ---------------------------------------------------------------------------------- rho correction
@dataclass
class RhoCorrection:
    weights: torch.Tensor  # multiplied into the policy loss as a stop-gradient weight
    metrics: dict[str, torch.Tensor]
    histogram_metrics: dict[str, torch.Tensor] = field(default_factory=dict)


def _drop_masks(rho, response_mask, lower: float, upper: float):
    low = (rho < lower) & response_mask if lower > 0.0 else torch.zeros_like(response_mask)
    high = (rho > upper) & response_mask if upper > 0.0 else torch.zeros_like(response_mask)
    return low, high


def _sequence_level_mean(values, response_mask, segment_ids: torch.Tensor | None = None):
    """Per-sequence masked mean broadcast back to tokens.  Rows are sequences for ``[B, T]`` input;
    for packed input pass ``segment_ids`` (sample id per token, 0 = not a response token)."""
    valid = response_mask.to(values.dtype)
    if segment_ids is None:
        s = (values * valid).sum(-1, keepdim=True)
        c = valid.sum(-1, keepdim=True).clamp_min(1.0)
        return (s / c).expand_as(values)
    flat_v, flat_m, seg = values.reshape(-1), valid.reshape(-1), segment_ids.reshape(-1).long()
    n = int(seg.max().item()) + 1 if seg.numel() else 1
    s = torch.zeros(n, dtype=values.dtype, device=values.device).scatter_add_(0, seg, flat_v * flat_m)
    c = torch.zeros(n, dtype=values.dtype, device=values.device).scatter_add_(0, seg, flat_m).clamp_min(1.0)
    return (s / c)[seg].reshape(values.shape)


def compute_rho_correction(old_logprob, vllm_logprobs, response_mask, advantages, config: GRPOExperimentConfig,
                           segment_ids: torch.Tensor | None = None) -> RhoCorrection:
    """rho = pi_train_old / pi_infer_old on response tokens: clamp (truncated importance sampling)
    and optionally drop tokens / sequences whose rho (or TV divergence) is out of range."""
    diff = torch.where(response_mask, (old_logprob - vllm_logprobs).clamp(-10.0, 10.0), torch.zeros_like(old_logprob))
    rho = torch.exp(diff)
    hist = {"val/rho_hist": rho[response_mask].detach().float()}
    if not config.use_rho_correction:
        return RhoCorrection(torch.ones_like(rho), {}, hist)
    rho_eff = torch.exp(_sequence_level_mean(diff, response_mask, segment_ids)) if config.rho_mask_sequence_level else rho
    if config.rho_mask_tv_divergence:
        tv_seq = _sequence_level_mean(torch.abs(rho - 1.0), response_mask, segment_ids)
        low, high = _drop_masks(tv_seq, response_mask, config.rho_mask_lower_bound, config.rho_mask_upper_bound)
        grows = torch.sign(diff) * advantages > 0  # only tokens that push the divergence further
        low, high = low & grows, high & grows
    else:
        low, high = _drop_masks(rho_eff, response_mask, config.rho_mask_lower_bound, config.rho_mask_upper_bound)
    keep = response_mask & ~low & ~high
    clamped = rho_eff
    if config.rho_clamp_lower_bound > 0.0:
        clamped = torch.clamp(clamped, min=config.rho_clamp_lower_bound)
    if config.rho_clamp_upper_bound > 0.0:
        clamped = torch.clamp(clamped, max=config.rho_clamp_upper_bound)
    weights = torch.where(keep, clamped, torch.zeros_like(clamped))
    metrics = {"val/rho_drop_frac": (low | high).float(), "val/rho_drop_low_frac": low.float(), "val/rho_drop_high_frac": high.float(),
               "val/rho_weight": weights.float(), "val/rho_clipfrac": (clamped != rho_eff).float()}
    return RhoCorrection(weights, metrics, hist)


def resolve_old_logprob(cache: list, sample_idx: int, epoch_idx: int, num_mini_batches: int, use_vllm_logprobs: bool,
                        vllm_logprobs, new_logprobs):
    """Old log-probs of a micro-batch: precomputed when there are several mini-batches, else set
    lazily on the first epoch from the engine's log-probs or the detached current ones
    (so that on the very first pass ratio == 1 while the gradient still flows)."""
    if num_mini_batches > 1:
        out = cache[sample_idx]
    else:
        with torch.no_grad():
            if epoch_idx == 0:
                cache[sample_idx] = vllm_logprobs if use_vllm_logprobs else new_logprobs.detach()
            out = cache[sample_idx]
    if out is None:
        raise RuntimeError("old log-probs were not precomputed for this micro-batch")
    return out


def compute_grpo_loss(new_logprobs, ratio, advantages, ref_logprobs, config: GRPOExperimentConfig, rho_weights):
    """Per-token (policy loss, clip indicator, KL estimate)."""
    if config.loss_fn == GRPOLossType.dapo:
        unclipped = -advantages * ratio
        clipped = -advantages * torch.clamp(ratio, 1.0 - config.clip_lower, 1.0 + config.clip_higher)
        clipfrac = (clipped > unclipped).float()
        pg = torch.max(unclipped, clipped)
    elif config.loss_fn == GRPOLossType.cispo:
        clipfrac = (ratio > 1.0 + config.clip_higher).float()
        pg = -advantages * torch.clamp(ratio.detach(), max=1.0 + config.clip_higher) * new_logprobs
    else:
        raise ValueError(f"Invalid loss function: {config.loss_fn}")
    pg = pg * rho_weights
    clipfrac = clipfrac * (rho_weights != 0).float()
    if ref_logprobs is not None:
        d = (new_logprobs - ref_logprobs).clamp(-40.0, 40.0)
        kl = estimate_kl(d, ratio)[config.kl_estimator]
    else:
        kl = torch.zeros_like(pg)
    return pg, clipfrac, kl


def calculate_token_counts(accumulation_steps: int, response_masks: list[torch.Tensor], device, group=None) -> dict[int, float]:
    """Response-token count of every accumulation group, summed over data-parallel ranks: the
    denominator of the ``loss_denominator == "token"`` normalisation."""
    counts = {}
    n = len(response_masks)
    starts = list(range(0, n, accumulation_steps))
    vec = torch.zeros(len(starts), dtype=torch.float32, device=device)
    for gi, s in enumerate(starts):
        for m in response_masks[s : s + accumulation_steps]:
            vec[gi] += m.sum().float()
    pdist.all_reduce_(vec, group=group)
    for gi, s in enumerate(starts):
        counts[s] = float(vec[gi].item())
    return counts


def compute_pass_at_k_metrics(scores: list[float], prompt_ids: list, k: int, max_possible_score: float) -> dict[str, float]:
    """Unbiased pass@k per prompt group, averaged over groups (a sample passes at the maximum score)."""
    groups: dict = {}
    for s, pid in zip(scores, prompt_ids):
        groups.setdefault(pid, []).append(s)
    vals = []
    for g in groups.values():
        n, c = len(g), sum(1 for s in g if s >= max_possible_score)
        if n < k:
            continue
        vals.append(1.0 if n - c < k else 1.0 - math.comb(n - c, k) / math.comb(n, k))
    return {f"eval/pass_at_{k}": float(np.mean(vals)) if vals else 0.0}
