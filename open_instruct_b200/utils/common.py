"""Small shared utilities: metrics vector, checkpoint-directory bookkeeping, timers, retry,
experiment tracking, seeding.

Counterparts in the reference: ``MetricsTracker`` (``open_instruct/utils.py:142-175``),
``get_last_checkpoint_path`` / ``clean_last_n_checkpoints`` (``:789-835``), ``retry_on_exception``
(``:1300-1333``), ``Timer`` (``open_instruct/rl_utils.py:162-180``), logger set-up
(``open_instruct/logger_utils.py:18-39``), runtime leak checks (``utils.py:1717-1779``).
"""

from __future__ import annotations

import functools
import json
import logging
import os
import random
import re
import shutil
import threading
import time
from contextlib import ContextDecorator
from dataclasses import dataclass

import numpy as np
import torch

INVALID_LOGPROB = 1.0  # filler for positions without a valid log-prob (never enters a masked mean)


def setup_logger(name: str | None = None, rank: int = 0) -> logging.Logger:
    """INFO on rank 0, WARNING elsewhere; one stream handler."""
    root = logging.getLogger()
    if not root.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s - %(name)s:%(lineno)d - %(levelname)s - %(message)s"))
        root.addHandler(h)
    root.setLevel(logging.INFO if rank == 0 else logging.WARNING)
    return logging.getLogger(name)


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class MetricsTracker:
    """Named scalars in one preallocated device vector so a log step costs ONE all-reduce."""

    def __init__(self, max_metrics: int = 64, device="cpu"):
        self.metrics = torch.zeros(max_metrics, dtype=torch.float32, device=device)
        self.names2idx: dict[str, int] = {}
        self.current_idx = 0

    def _slot(self, name: str) -> int:
        if name not in self.names2idx:
            if self.current_idx >= self.metrics.numel():
                raise ValueError(f"exceeded the number of metric slots ({self.metrics.numel()})")
            self.names2idx[name] = self.current_idx
            self.current_idx += 1
        return self.names2idx[name]

    def __setitem__(self, name: str, value) -> None:
        self.metrics[self._slot(name)] = value

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.metrics[self.names2idx[name]]

    def add(self, name: str, value) -> None:
        self.metrics[self._slot(name)] += value

    def get_metrics_list(self) -> dict[str, float]:
        vals = self.metrics.tolist()
        return {n: vals[i] for n, i in self.names2idx.items()}

    def reduce_(self, group=None, average: bool = True) -> "MetricsTracker":
        from ..parallel import dist as pdist

        st = None
        if self.metrics.is_cuda and self.metrics.numel() <= 512 and pdist.is_dist():
            from ..parallel.symm import metrics_state

            st = metrics_state(group)
        if st is not None:
            st.allreduce_vector_(self.metrics)   # one kernel over symmetric memory
        else:
            pdist.all_reduce_(self.metrics, group=group)
        if average:
            self.metrics /= pdist.world_size(group)
        return self

    def zero_(self) -> None:
        self.metrics.zero_()


class Timer(ContextDecorator):
    """Wall-clock timer usable as context manager or decorator; logs unless ``noop``."""

    def __init__(self, description: str, noop: bool = False, logger: logging.Logger | None = None):
        self.description, self.noop = description, noop
        self.logger = logger or logging.getLogger(__name__)
        self.duration = 0.0

    def __enter__(self):
        self.start = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.duration = time.perf_counter() - self.start
        if not self.noop:
            self.logger.info("%s: %.3f seconds", self.description, self.duration)
        return False


class DeviceTimer:
    """CUDA-event timer on the current stream; ``elapsed_ms_max`` reduces as max over ranks."""

    def __init__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        return False

    def elapsed_ms(self) -> float:
        self.e1.synchronize()
        return self.e0.elapsed_time(self.e1)

    def elapsed_ms_max(self) -> float:
        from ..parallel import dist as pdist

        return pdist.max_over_ranks(self.elapsed_ms())


def retry_on_exception(max_attempts: int = 4, delay: float = 1.0, backoff: float = 2.0):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            wait = delay
            for attempt in range(max_attempts):
                try:
                    return fn(*a, **kw)
                except Exception:  # noqa: BLE001
                    if attempt == max_attempts - 1:
                        raise
                    time.sleep(wait)
                    wait *= backoff
        return wrapper
    return deco


# ---------------------------------------------------------------------------------- checkpoint directories
_STEP_RE = re.compile(r"^(step|epoch)_(\d+)$")


def _ckpt_dirs(output_dir: str) -> list[tuple[int, int, str]]:
    """(kind order, number, path) of complete checkpoints: ``step_N`` / ``epoch_N`` holding COMPLETED."""
    out = []
    if not os.path.isdir(output_dir):
        return out
    for name in os.listdir(output_dir):
        m = _STEP_RE.match(name)
        p = os.path.join(output_dir, name)
        if m and os.path.isdir(p) and os.path.exists(os.path.join(p, "COMPLETED")):
            out.append((int(m.group(2)), name, p))
    return sorted(out, key=lambda t: os.path.getmtime(t[2]))


def get_last_checkpoint(output_dir: str, incomplete: bool = False) -> str | None:
    """Newest checkpoint folder (only ones with the COMPLETED marker unless ``incomplete``)."""
    if incomplete:
        cands = [os.path.join(output_dir, n) for n in os.listdir(output_dir) if _STEP_RE.match(n)] if os.path.isdir(output_dir) else []
        return max(cands, key=os.path.getmtime) if cands else None
    dirs = _ckpt_dirs(output_dir)
    return dirs[-1][2] if dirs else None


def get_last_checkpoint_path(output_dir: str, resume_from_checkpoint: str | None = None, overwrite_output_dir: bool = False) -> str | None:
    """Explicit path wins; else the newest complete checkpoint under ``output_dir`` (auto-resume)."""
    if resume_from_checkpoint:
        return resume_from_checkpoint
    if os.path.isdir(output_dir) and not overwrite_output_dir:
        return get_last_checkpoint(output_dir)
    return None


def clean_last_n_checkpoints(output_dir: str, keep_last_n_checkpoints: int) -> None:
    """Delete all but the newest ``keep_last_n_checkpoints`` complete checkpoints (-1 keeps all)."""
    if keep_last_n_checkpoints < 0:
        return
    dirs = _ckpt_dirs(output_dir)
    for _, _, p in dirs[: max(0, len(dirs) - keep_last_n_checkpoints)]:
        shutil.rmtree(p, ignore_errors=True)


def is_checkpoint_folder(path: str) -> bool:
    return bool(_STEP_RE.match(os.path.basename(os.path.normpath(path)))) and os.path.isdir(path)


# ---------------------------------------------------------------------------------- tracking
class Tracker:
    """Scalar logging to JSONL always, to TensorBoard / wandb when asked and importable (offline-safe)."""

    def __init__(self, output_dir: str, run_name: str, config: dict | None = None, report_to=("jsonl",),
                 wandb_project: str | None = None, wandb_entity: str | None = None, enabled: bool = True):
        self.enabled = enabled
        self.writers = []
        if not enabled:
            return
        os.makedirs(output_dir, exist_ok=True)
        self._fh = open(os.path.join(output_dir, "metrics.jsonl"), "a")
        if config is not None:
            with open(os.path.join(output_dir, "run_config.json"), "w") as fh:
                json.dump(config, fh, indent=2, default=str)
        report = [report_to] if isinstance(report_to, str) else list(report_to or [])
        if "tensorboard" in report or "all" in report:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self.writers.append(("tb", SummaryWriter(os.path.join(output_dir, "tb", run_name))))
            except Exception:  # noqa: BLE001
                pass
        if "wandb" in report:
            try:
                import wandb

                os.environ.setdefault("WANDB_MODE", "offline")
                wandb.init(project=wandb_project, entity=wandb_entity, name=run_name, config=config, dir=output_dir)
                self.writers.append(("wandb", wandb))
            except Exception:  # noqa: BLE001
                pass

    def log(self, metrics: dict, step: int) -> None:
        if not self.enabled:
            return
        rec = {"step": step, **{k: (float(v) if isinstance(v, (int, float, np.floating, torch.Tensor)) else v) for k, v in metrics.items()}}
        self._fh.write(json.dumps(rec, default=str) + "\n")
        self._fh.flush()
        for kind, w in self.writers:
            if kind == "tb":
                for k, v in metrics.items():
                    if isinstance(v, (int, float)):
                        w.add_scalar(k, v, step)
            elif kind == "wandb":
                w.log(metrics, step=step)

    def close(self) -> None:
        if not self.enabled:
            return
        self._fh.close()
        for kind, w in self.writers:
            if kind == "tb":
                w.close()
            elif kind == "wandb":
                w.finish()


def check_runtime_leaks(baseline_threads: set | None = None) -> dict:
    """Threads and child processes still alive (tests assert this is empty after teardown)."""
    import multiprocessing

    threads = [t.name for t in threading.enumerate() if t is not threading.main_thread() and t.is_alive()
               and not t.daemon and (baseline_threads is None or t.name not in baseline_threads)]
    children = [p.pid for p in multiprocessing.active_children()]
    return {"threads": threads, "processes": children}


def warn_if_low_disk_space(path: str, threshold: float = 0.9) -> bool:
    try:
        usage = shutil.disk_usage(path if os.path.exists(path) else os.path.dirname(os.path.abspath(path)) or ".")
    except OSError:
        return False
    if usage.used / usage.total >= threshold:
        logging.getLogger(__name__).warning("disk usage near capacity: %.1f%% of %.0f GiB used at %s",
                                            100 * usage.used / usage.total, usage.total / 2**30, path)
        return True
    return False


class nvtx_range(ContextDecorator):
    """NVTX range around a phase of the step (visible in Nsight timelines); a no-op without CUDA or when
    ``B200_NVTX=0``."""

    def __init__(self, name: str):
        self.name = name
        self.on = os.environ.get("B200_NVTX", "1") == "1"

    def __enter__(self):
        import torch

        self.on = self.on and torch.cuda.is_available()
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            import torch

            torch.cuda.nvtx.range_pop()
        return False


class StepProfiler:
    """``--profiling``: torch.profiler over a few training steps (skip 5, wait 1, warm up 2, record 3, with memory), the
    schedule the reference's profiler callback uses (``open_instruct/dpo.py:87-90``).  Call ``step()`` once per
    optimizer step; the Chrome trace lands in ``<output_dir>/profiler``."""

    def __init__(self, enabled: bool, output_dir: str, rank: int = 0):
        self.prof = None
        if enabled:
            import torch
            from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            self.prof = profile(activities=acts, schedule=schedule(skip_first=5, wait=1, warmup=2, active=3, repeat=1), profile_memory=True,
                                on_trace_ready=tensorboard_trace_handler(os.path.join(output_dir, "profiler"), worker_name=f"rank{rank}"))
            self.prof.__enter__()

    def step(self) -> None:
        if self.prof is not None:
            self.prof.step()

    def close(self) -> None:
        if self.prof is not None:
            self.prof.__exit__(None, None, None)
            self.prof = None
