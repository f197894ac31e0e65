"""Plain containers exchanged between the GRPO processes (driver, data preparation, rollout
engines, learners).  Field names follow ``open_instruct/data_types.py`` so recipes, traces and tests
that inspect them keep working; every class is picklable with the standard library.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class TokenStatistics:
    num_prompt_tokens: int = 0
    num_response_tokens: int = 0
    generation_time: float = 0.0
    earliest_start_time: float | None = None


@dataclass
class ToolCallStats:
    tool_name: str
    success: bool
    runtime: float


@dataclass
class RequestInfo:
    num_calls: list[int] = field(default_factory=list)
    timeouts: list[int] = field(default_factory=list)
    tool_errors: list[str] = field(default_factory=list)
    tool_outputs: list[str] = field(default_factory=list)
    tool_runtimes: list[float] = field(default_factory=list)
    tool_calleds: list[bool] = field(default_factory=list)
    tool_call_stats: list[list[ToolCallStats]] = field(default_factory=list)
    rollout_states: list[dict] = field(default_factory=list)


@dataclass
class EnvConfigEntry:
    env_name: str
    kwargs: dict = field(default_factory=dict)


@dataclass
class EnvConfig:
    max_steps: int = 8
    env_configs: list[EnvConfigEntry] = field(default_factory=list)


@dataclass
class SamplingConfig:
    temperature: float = 1.0
    top_p: float = 1.0
    max_tokens: int = 256
    n: int = 1
    stop: list[str] | None = None
    seed: int | None = None
    logprobs: int | None = 1
    min_tokens: int = 0
    include_stop_str_in_output: bool = True


@dataclass
class PromptRequest:
    prompt: list[int]
    generation_config: SamplingConfig
    index: int
    prompt_id: str
    is_eval: bool = False
    active_tools: list[str] | None = None
    env_config: EnvConfig | None = None
    raw_query: str | None = None
    ground_truth: Any = None
    dataset: Any = None
    epoch_number: int = 0
    training_step: int | None = None


@dataclass
class GenerationResult:
    responses: list[list[int]]
    finish_reasons: list[str]
    masks: list[list[int]]
    request_info: RequestInfo
    index: int | None = None
    prompt_id: str | None = None
    epoch_number: int | None = None
    token_statistics: TokenStatistics | None = None
    start_time: float | None = None
    logprobs: list[list[float]] | None = None
    reward_scores: list[float] | None = None
    reward_metrics: dict[str, Any] | None = None
    model_step: int | None = None
    is_eval: bool = False
    queries: list[list[int]] | None = None
    decoded_responses: list[str] | None = None
    ground_truth: Any = None
    dataset: Any = None
    raw_query: str | None = None


@dataclass
class CollatedBatchData:
    """Per-rank training data of one step: lists with one tensor per micro-batch."""

    query_responses: list[torch.Tensor]
    attention_masks: list[torch.Tensor]
    position_ids: list[torch.Tensor]
    advantages: list[torch.Tensor]
    response_masks: list[torch.Tensor]
    vllm_logprobs: list[torch.Tensor]
    cu_seqlens: list[torch.Tensor] | None = None

    def __len__(self) -> int:
        return len(self.query_responses)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return CollatedBatchData(**{k: (v[idx] if v is not None else None) for k, v in self.__dict__.items()})
        return {k: (v[idx] if v is not None else None) for k, v in self.__dict__.items()}

    def to(self, device, non_blocking: bool = True) -> "CollatedBatchData":
        mv = lambda lst: None if lst is None else [t.to(device, non_blocking=non_blocking) for t in lst]
        return CollatedBatchData(**{k: mv(v) for k, v in self.__dict__.items()})

    def pin_memory(self) -> "CollatedBatchData":
        if not torch.cuda.is_available():
            return self
        pm = lambda lst: None if lst is None else [t.pin_memory() for t in lst]
        return CollatedBatchData(**{k: pm(v) for k, v in self.__dict__.items()})


@dataclass
class Batch:
    """Column-wise container of prompts with list-like indexing: ``b[3]``, ``b[2:5]``, ``b[[1, 4]]`` all give a
    ``Batch`` (cf. ``open_instruct/model_utils.py:118-174``).  Optional columns stay ``None``."""

    queries: list
    ground_truths: list
    datasets: list
    raw_queries: list | None = None
    decoded_responses: list | None = None
    indices: list | None = None
    scores: list | None = None
    active_tools: list | None = None
    model_steps: list = field(default_factory=list)

    def __len__(self) -> int:
        return len(self.queries)

    def __getitem__(self, key) -> "Batch":
        if isinstance(key, slice):
            pick = lambda col: col[key]
        elif isinstance(key, int):
            pick = lambda col: [col[key]]
        else:
            pick = lambda col: [col[i] for i in key]
        cols = {}
        for name, col in self.__dict__.items():
            cols[name] = None if col is None else (pick(col) if (col or name != "model_steps") else [])
        return Batch(**cols)


class ShutdownSentinel:
    """Put on a queue to tell its consumer to stop."""
