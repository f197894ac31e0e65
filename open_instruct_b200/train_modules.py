"""Train modules: what one batch does in the callback-driven trainers (``dpo.py``, ``grpo.py``).

``DPOTrainModule.train_batch`` follows the reference's olmo-core DPO module (``open_instruct/olmo_core_train_modules.py:224-317``):
the rank's batch is cut into micro-batches, every micro-batch's loss is weighted by its share of the batch's real
(non-padding) tokens before the backward pass, and the metrics are token-weighted ratios reduced over the data-parallel
group in ONE collective together with their denominators.  ``GRPOTrainModule`` runs the GRPO step of this package on the
rank's packed data (``open_instruct/olmo_core_train_modules.py:430-635``).
"""

from __future__ import annotations

import torch

from .data.collate import to_device
from .dpo_utils import DPOLossType, compute_loss
from .parallel import dist as pdist
from .trainer import TrainModule


def num_tokens(mb: dict) -> int:
    """Real tokens of a packed preference micro-batch (chosen + rejected; packed rows carry no padding)."""
    return int(mb["chosen_input_ids"].numel() + mb["rejected_input_ids"].numel())


def num_sequences(mb: dict) -> int:
    return int(mb["chosen_cu_seq_lens_q"].numel() - 1) + int(mb["rejected_cu_seq_lens_q"].numel() - 1)


class DPOTrainModule(TrainModule):
    def __init__(self, learner, dpo_config, reference_cache, forward_fn, data_parallel_world: int | None = None):
        super().__init__(learner)
        self.cfg, self.cache, self.forward_fn = dpo_config, reference_cache, forward_fn
        self.loss_type = DPOLossType(dpo_config.loss_type)
        self.dp_world = data_parallel_world or learner.world

    def train_batch(self, batch, dry_run: bool = False) -> None:
        """``batch``: the rank's micro-batches for this step (list of packed preference batches on any device)."""
        L = self.learner
        micro = batch if isinstance(batch, (list, tuple)) else [batch]
        micro = [to_device(mb, L.device) for mb in micro]
        counts = [num_tokens(mb) for mb in micro]
        total = max(sum(counts), 1)
        names = ["loss", "chosen_logps", "rejected_logps"] + (["chosen_rewards", "rejected_rewards", "accuracy"] if self.loss_type.computes_reward_metrics else [])
        sums = {k: torch.zeros((), device=L.device) for k in names}
        average = self.loss_type.is_average_loss
        for k, mb in enumerate(micro):
            pc, pr, aux = self.forward_fn(L, mb, average_log_prob=average)
            losses, c_rew, r_rew = compute_loss(self.cfg, mb, pc, pr, self.cache, (aux["chosen_tokens"], aux["rejected_tokens"]))
            loss = losses.mean()
            w = counts[k] / total
            if not dry_run:
                L.backward(loss * w, last=(k == len(micro) - 1))
            with torch.no_grad():
                sums["loss"] += loss.detach() * counts[k]
                sums["chosen_logps"] += pc.detach().mean() * counts[k]
                sums["rejected_logps"] += pr.detach().mean() * counts[k]
                if self.loss_type.computes_reward_metrics:
                    sums["chosen_rewards"] += c_rew.mean() * counts[k]
                    sums["rejected_rewards"] += r_rew.mean() * counts[k]
                    sums["accuracy"] += (c_rew > r_rew).float().mean() * counts[k]
        if dry_run:
            return
        # numerators and the shared denominator in one all-reduce over the data-parallel group (ranks of one tensor-parallel
        # group saw the same batch: reducing over the data-parallel group counts every batch once)
        vec = torch.stack([torch.tensor(float(total), device=L.device), *[sums[k] for k in names]])
        pdist.all_reduce_(vec, group=L.group)
        tok = vec[0].clamp(min=1.0)
        out = {k: float(vec[i + 1] / tok) for i, k in enumerate(names)}
        self.record_metric("train_loss", out["loss"], None)
        self.record_metric("logps/chosen", out["chosen_logps"], None)
        self.record_metric("logps/rejected", out["rejected_logps"], None)
        if self.loss_type.computes_reward_metrics:
            self.record_metric("rewards/chosen", out["chosen_rewards"], None)
            self.record_metric("rewards/rejected", out["rejected_rewards"], None)
            self.record_metric("rewards/average", (out["chosen_rewards"] + out["rejected_rewards"]) / 2, None)
            self.record_metric("rewards/accuracy", out["accuracy"], None)
            self.record_metric("rewards/margin", out["chosen_rewards"] - out["rejected_rewards"], None)
        self.record_metric("train/token_count", float(vec[0]), None)
        self.record_metric("train/sequences_per_rank", float(sum(num_sequences(mb) for mb in micro)), "mean")

    def optim_step(self) -> torch.Tensor:
        # the micro-batch weights already sum to one on every rank: only the mean over data-parallel ranks is left
        norm = self.learner.optimizer_step(grad_scale=1.0 / self.learner.world)
        self.record_metric("optim/grad_norm", norm, None)
        self.record_metric("learning_rate", self.learner.lr(max(0, self.learner.global_step - 1)), None)
        return norm


class GRPOTrainModule(TrainModule):
    """One GRPO training step on this rank's packed rollouts (all epochs and mini-batches; the optimizer steps happen inside,
    one per accumulation group)."""

    def __init__(self, learner, args, ref_learner=None, group=None):
        super().__init__(learner)
        self.args, self.ref, self.group = args, ref_learner, group
        self.last: dict = {}

    def train_batch(self, batch, dry_run: bool = False) -> None:
        from .grpo_fast import grpo_train_step

        self.last = grpo_train_step(self.learner, batch, self.args, self.ref, self.group)
        w = self.last.get("num_response_tokens", 0.0)
        for k, v in self.last.items():
            if isinstance(v, (int, float)):
                self.record_metric(k, v, "sum" if k == "num_response_tokens" else "mean")
        self.record_metric("train/response_tokens", w, "sum")

    def optim_step(self):  # done inside ``grpo_train_step``, per accumulation group
        return None
