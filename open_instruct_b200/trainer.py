"""Step-driven trainer with callbacks and train modules (the structure of the reference's second trainer generation).

The reference's ``dpo.py`` / ``grpo.py`` / ``olmo_core_finetune.py`` hand a ``TrainModule`` (what one batch does) and a list
of ``Callback`` objects (what happens around a step) to a ``Trainer`` that owns the loop
(``open_instruct/dpo.py:141-342``, ``open_instruct/grpo_callbacks.py``, ``open_instruct/olmo_core_callbacks.py``).  This file
is that structure over this package's ``Learner``:

* ``TrainModule.train_batch(batch)`` runs forward + backward over the batch's micro-batches and leaves gradients
  accumulated; ``optim_step()`` does the exchange, clipping, AdamW and bf16 refresh.
* ``Trainer.fit()`` pulls batches, calls the module and the callbacks (``pre_train``, ``pre_step``, ``post_step``,
  ``post_train``), gathers the metrics recorded during the step and hands them to the tracker.
* metrics recorded with ``reduce_type="mean" | "sum" | "max"`` are reduced over the ranks in ONE small collective per
  logging step; ``None`` means the value is already global.
"""

from __future__ import annotations

import os
import time
from typing import Any, Iterable

import torch

from .parallel import dist as pdist


class Callback:
    """Hooks around the training loop; ``self.trainer`` is set when the callback is attached."""

    trainer: "Trainer" = None  # type: ignore[assignment]

    def pre_train(self) -> None: ...
    def pre_step(self, batch: Any) -> None: ...
    def post_step(self) -> None: ...
    def post_checkpoint_saved(self, path: str) -> None: ...
    def post_train(self) -> None: ...
    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, sd: dict) -> None: ...


class TrainModule:
    """What one batch does.  Subclasses implement ``train_batch``; the optimizer step is the learner's."""

    trainer: "Trainer" = None  # type: ignore[assignment]

    def __init__(self, learner):
        self.learner = learner

    def train_batch(self, batch: Any, dry_run: bool = False) -> None:
        raise NotImplementedError

    def optim_step(self) -> torch.Tensor:
        norm = self.learner.optimizer_step()
        self.record_metric("optim/grad_norm", norm, None)
        self.record_metric("optim/lr", self.learner.lr(max(0, self.learner.global_step - 1)), None)
        return norm

    def record_metric(self, name: str, value, reduce_type: str | None = "mean") -> None:
        if self.trainer is not None:
            self.trainer.record_metric(name, value, reduce_type)

    def state_dict(self) -> dict:
        return self.learner.opt.state_dict()


class Trainer:
    def __init__(self, train_module: TrainModule, data_loader: Iterable, *, max_steps: int, callbacks: list[Callback] | None = None,
                 tracker=None, save_folder: str | None = None, metrics_collect_interval: int = 1, dp_process_group=None,
                 steps_per_epoch: int | None = None, start_step: int = 0):
        self.train_module, self.data_loader = train_module, data_loader
        self.max_steps, self.global_step = max_steps, start_step
        self.callbacks = list(callbacks or [])
        self.tracker, self.save_folder = tracker, save_folder
        self.metrics_collect_interval = max(1, metrics_collect_interval)
        self.dp_process_group = dp_process_group
        self.steps_per_epoch = steps_per_epoch
        self.device = train_module.learner.device
        self._metrics: dict[str, tuple[Any, str | None]] = {}
        self.last_metrics: dict[str, float] = {}
        self.stop_requested = False
        train_module.trainer = self
        for cb in self.callbacks:
            cb.trainer = self

    # ------------------------------------------------------------------ metrics
    def record_metric(self, name: str, value, reduce_type: str | None = "mean") -> None:
        if reduce_type not in (None, "mean", "sum", "max"):
            raise ValueError(f"unknown reduce_type {reduce_type!r}")
        self._metrics[name] = (value, reduce_type)

    def _collect_metrics(self) -> dict[str, float]:
        """One collective for everything recorded since the last collection (a MAX pass only when someone asked for it)."""
        names = list(self._metrics)
        vals = torch.tensor([float(self._metrics[n][0]) for n in names], dtype=torch.float64, device=self.device)
        kinds = [self._metrics[n][1] for n in names]
        world = pdist.world_size()
        if world > 1 and any(k is not None for k in kinds):
            summed = vals.clone()
            pdist.all_reduce_(summed)
            maxed = None
            if "max" in kinds:
                maxed = vals.clone()
                pdist.all_reduce_(maxed, op=torch.distributed.ReduceOp.MAX)
            for i, k in enumerate(kinds):
                if k == "sum":
                    vals[i] = summed[i]
                elif k == "mean":
                    vals[i] = summed[i] / world
                elif k == "max":
                    vals[i] = maxed[i]
        self._metrics.clear()
        return {n: float(v) for n, v in zip(names, vals.tolist())}

    # ------------------------------------------------------------------ loop
    def fit(self) -> dict[str, float]:
        for cb in self.callbacks:
            cb.pre_train()
        it = iter(self.data_loader)
        while self.global_step < self.max_steps and not self.stop_requested:
            try:
                batch = next(it)
            except StopIteration:
                it = iter(self.data_loader)  # next epoch (a loader that reshuffles does so in __iter__)
                try:
                    batch = next(it)
                except StopIteration:
                    break
            self.global_step += 1
            for cb in self.callbacks:
                cb.pre_step(batch)
            self.train_module.train_batch(batch)
            self.train_module.optim_step()
            for cb in self.callbacks:
                cb.post_step()
            if self.global_step % self.metrics_collect_interval == 0 or self.global_step == self.max_steps:
                self.last_metrics = self._collect_metrics()
                self.last_metrics["training_step"] = self.global_step
                if self.tracker is not None:
                    self.tracker.log(self.last_metrics, self.global_step)
        for cb in self.callbacks:
            cb.post_train()
        return self.last_metrics


# ------------------------------------------------------------------------------------------------ general callbacks
class StepTimingCallback(Callback):
    """Wall time of every step and of the wait for its batch (``open_instruct/grpo_callbacks.py:67-135``)."""

    def pre_train(self) -> None:
        self._t_end = time.perf_counter()

    def pre_step(self, batch) -> None:
        self._t0 = time.perf_counter()
        self.trainer.record_metric("time/trainer_waiting_for_data", self._t0 - self._t_end, "max")

    def post_step(self) -> None:
        self._t_end = time.perf_counter()
        self.trainer.record_metric("time/training", self._t_end - self._t0, "max")


class PerfCallback(Callback):
    """Tokens per second and model FLOPs utilisation from the analytic model dimensions
    (``open_instruct/olmo_core_callbacks.py:122-233``)."""

    def __init__(self, dims, tokens_of_batch, seq_len_of_batch=None):
        self.dims, self.tokens_of_batch, self.seq_len_of_batch = dims, tokens_of_batch, seq_len_of_batch
        self.total_tokens = 0

    def pre_train(self) -> None:
        self._t_start = time.perf_counter()

    def pre_step(self, batch) -> None:
        self._t0 = time.perf_counter()
        self._tokens = int(self.tokens_of_batch(batch))
        self._seq = float(self.seq_len_of_batch(batch)) if self.seq_len_of_batch else 0.0

    def post_step(self) -> None:
        dt = max(time.perf_counter() - self._t0, 1e-9)
        world = pdist.world_size()
        self.total_tokens += self._tokens * world
        self.trainer.record_metric("perf/tokens_per_second_step", self._tokens / dt, "sum")
        self.trainer.record_metric("perf/tokens_per_second_avg", self.total_tokens / max(time.perf_counter() - self._t_start, 1e-9), None)
        if self._seq and self.trainer.device.type == "cuda":
            self.trainer.record_metric("perf/mfu_step", self.dims.approximate_learner_utilization(self._tokens * world, self._seq, dt, world), None)


class CheckpointerCallback(Callback):
    """Training state every ``save_interval`` steps, the last ``max_checkpoints`` kept
    (``open_instruct/olmo_core_utils.py:244-263``)."""

    def __init__(self, save_folder: str, save_interval: int, max_checkpoints: int = 3, extra_state=None):
        self.save_folder, self.save_interval, self.max_checkpoints, self.extra_state = save_folder, save_interval, max_checkpoints, extra_state

    def post_step(self) -> None:
        step = self.trainer.global_step
        if not self.save_interval or step % self.save_interval:
            return
        from .ckpt.train_state import save_train_state
        from .utils.common import clean_last_n_checkpoints

        d = os.path.join(self.save_folder, f"step_{step}")
        state = {"completed_steps": step, "callbacks": {type(cb).__name__: cb.state_dict() for cb in self.trainer.callbacks}}
        if self.extra_state is not None:
            state.update(self.extra_state())
        save_train_state(d, self.trainer.train_module.learner.opt, state)
        if pdist.rank() == 0:
            clean_last_n_checkpoints(self.save_folder, self.max_checkpoints)
        for cb in self.trainer.callbacks:
            cb.post_checkpoint_saved(d)


class ProfilerCallback(Callback):
    """``torch.profiler`` over a window of steps (``open_instruct/dpo.py:87-90``: skip 5, wait 1, warm up 2, record 3)."""

    def __init__(self, enabled: bool, out_dir: str):
        from .utils.common import StepProfiler

        self._p = StepProfiler(enabled, out_dir, pdist.rank())

    def post_step(self) -> None:
        self._p.step()

    def post_train(self) -> None:
        self._p.close()
