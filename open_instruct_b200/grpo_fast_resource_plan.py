"""What a GRPO run needs from the machine before any actor starts, and a readable account of what is missing.

Topology (``open_instruct/grpo_fast_resource_plan.py:27-57``): one learner process per learner GPU with
``CPU_PER_LEARNER_GPU`` host cores each; unless ``single_gpu_mode`` shares the learner's GPU, every rollout engine
takes ``tensor_parallel_size`` GPUs and as many cores; the data-preparation actor and the actor manager take
2 and 1 cores.  ``detect_resources()`` reads what this host offers (NVML when present, else ``torch.cuda``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

CPU_PER_LEARNER_GPU = 10
DATA_PREPARATION_ACTOR_NUM_CPUS = 2
ACTOR_MANAGER_NUM_CPUS = 1


def _fmt(x: float) -> str:
    x = float(x)
    return str(int(x)) if x.is_integer() else f"{x:g}"


def format_resource_snapshot(resources: dict | None) -> str:
    if not resources:
        return "{}"
    return "{" + ", ".join(f"{k}={_fmt(v) if isinstance(v, (int, float)) else v}" for k, v in sorted(resources.items())) + "}"


@dataclass
class ResourcePlan:
    learner_bundles: list[dict] = field(default_factory=list)
    learner_gpus: float = 0.0
    learner_cpus: float = 0.0
    engine_gpus: float = 0.0
    engine_cpus: float = 0.0
    data_prep_cpus: float = float(DATA_PREPARATION_ACTOR_NUM_CPUS)
    actor_manager_cpus: float = float(ACTOR_MANAGER_NUM_CPUS)

    @property
    def min_gpus(self) -> float:
        return self.learner_gpus + self.engine_gpus

    @property
    def min_cpus(self) -> float:
        return self.learner_cpus + self.engine_cpus + self.data_prep_cpus + self.actor_manager_cpus

    def describe(self) -> str:
        return "\n".join([
            f"Learner group: bundles={self.learner_bundles}, totals=(GPU={_fmt(self.learner_gpus)}, CPU={_fmt(self.learner_cpus)})",
            f"Separate rollout engines: totals=(GPU={_fmt(self.engine_gpus)}, CPU={_fmt(self.engine_cpus)})",
            f"Minimum full topology: (GPU={_fmt(self.min_gpus)}, CPU={_fmt(self.min_cpus)}; includes data preparation "
            f"CPU={_fmt(self.data_prep_cpus)}, actor manager CPU={_fmt(self.actor_manager_cpus)})",
        ])

    def shortfalls(self, available: dict) -> list[str]:
        out = []
        for kind, learner, full in (("GPU", self.learner_gpus, self.min_gpus), ("CPU", self.learner_cpus, self.min_cpus)):
            have = float(available.get(kind, 0.0))
            if have < learner:
                out.append(f"learner group requires {kind}={_fmt(learner)} but this host offers {kind}={_fmt(have)}")
            elif have < full:
                out.append(f"full topology requires at least {kind}={_fmt(full)} but this host offers {kind}={_fmt(have)}")
        return out


def build_plan(num_learners_per_node: list[int], single_gpu_mode: bool, num_engines: int, tensor_parallel_size: int) -> ResourcePlan:
    bundles = [{"GPU": n, "CPU": n * CPU_PER_LEARNER_GPU} for n in num_learners_per_node]
    eng = 0.0 if single_gpu_mode else float(num_engines * tensor_parallel_size)
    return ResourcePlan(bundles, float(sum(b["GPU"] for b in bundles)), float(sum(b["CPU"] for b in bundles)), eng, eng)


def detect_resources() -> dict:
    gpus = 0
    try:
        import torch

        gpus = torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        pass
    return {"GPU": float(gpus), "CPU": float(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count() or 1)}


def check_or_raise(plan: ResourcePlan, available: dict | None = None, strict_cpu: bool = False) -> list[str]:
    """Raise on a GPU shortfall (the run cannot start); CPU shortfalls are returned as warnings unless ``strict_cpu``."""
    available = available if available is not None else detect_resources()
    msgs = plan.shortfalls(available)
    fatal = [m for m in msgs if "GPU=" in m or strict_cpu]
    if fatal:
        raise RuntimeError("not enough resources for this GRPO topology:\n  " + "\n  ".join(fatal) + "\n" + plan.describe()
                           + "\navailable: " + format_resource_snapshot(available))
    return msgs
