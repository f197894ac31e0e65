"""Callbacks of the callback-driven GRPO entry point (``grpo.py``).

Counterparts of ``open_instruct/grpo_callbacks.py``: weight sync into the rollout engines after every step
(``VLLMWeightSyncCallback``, ``:138-176``), polyak update of the reference policy (``RefPolicyUpdateCallback``, ``:179-226``),
evaluation rollouts (``EvalCallback``, ``:255-313``), model / state checkpoints carrying the data-preparation state
(``DataPreparationActorCheckpointCallback``, ``:229-252``) and per-step logging.  They act on a ``grpo_fast.GRPORun``, which owns the
actors; the trainer that calls them runs in the driver process.
"""

from __future__ import annotations

from .trainer import Callback, TrainModule


class DriverGRPOModule(TrainModule):
    """Train module of the DRIVER: one call dispatches this step's packed data to every learner actor and waits for their
    GRPO steps.  The optimizer steps happen inside the learner actors."""

    def __init__(self, run):
        self.run, self.learner = run, _DeviceOnly()

    def train_batch(self, batch, dry_run: bool = False) -> None:
        step = self.trainer.global_step
        metrics = self.run.train_step(step)
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.record_metric(k, v, None)

    def optim_step(self):
        return None


class _DeviceOnly:
    """The driver holds no model; the trainer only asks a train module's learner for the device of its metric vector."""

    import torch as _torch

    device = _torch.device("cpu")


class StepSource:
    """The trainer's "data loader" in the driver: the data itself travels from the data-preparation actor to the learner
    actors inside ``GRPORun.train_step``; this only counts steps."""

    def __init__(self, first: int, last: int):
        self.first, self.last = first, last

    def __iter__(self):
        return iter(range(self.first, self.last + 1))


class VLLMWeightSyncCallback(Callback):
    def __init__(self, run):
        self.run = run

    def post_step(self) -> None:
        t = self.run.sync_step(self.trainer.global_step)
        self.trainer.record_metric("time/weight_sync", t, None)


class RefPolicyUpdateCallback(Callback):
    """ref <- alpha * policy + (1 - alpha) * ref every ``ref_policy_update_freq`` steps, on every learner rank."""

    def __init__(self, run):
        self.run = run

    def post_step(self) -> None:
        a = self.run.args
        if a.load_ref_policy and a.ref_policy_update_freq and self.trainer.global_step % a.ref_policy_update_freq == 0:
            self.run.call_all(self.run.learners, "update_ref_policy")


class EvalCallback(Callback):
    def __init__(self, run):
        self.run = run

    def post_step(self) -> None:
        self.run.evaluate(self.trainer.global_step)
        for k, v in self.run.last.items():
            if k.startswith("eval/") and isinstance(v, (int, float)):
                self.trainer.record_metric(k, v, None)


class DataPreparationActorCheckpointCallback(Callback):
    """Model exports every ``save_freq`` steps and resumable state (optimizer shards + the data-preparation actor's position
    and RNG) every ``checkpoint_state_freq`` steps."""

    def __init__(self, run):
        self.run = run

    def post_step(self) -> None:
        self.run.checkpoint(self.trainer.global_step)

    def post_train(self) -> None:
        if self.run.args.save_final_model:
            self.run.save_model()


class StepLogCallback(Callback):
    def __init__(self, run):
        self.run = run

    def post_step(self) -> None:
        self.run.log_step(self.trainer.global_step)
