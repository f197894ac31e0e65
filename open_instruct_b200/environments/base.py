"""Environment and tool interfaces for multi-turn rollouts.

Same contracts as the reference (``open_instruct/environments/base.py:29-119``,
``open_instruct/environments/tools/utils.py:384-433``): an ``RLEnvironment`` is reset per rollout, stepped
with parsed tool calls and returns a ``StepResult`` (observation text, reward, done); ``RolloutState``
accumulates per-turn rewards for the reward aggregator; a ``Tool`` is a stateless environment with
one callable and an OpenAI-style function schema.
"""

from __future__ import annotations

import abc
import dataclasses
import inspect
import time
from typing import Any


@dataclasses.dataclass
class ToolCall:
    name: str
    args: dict[str, Any]
    id: str | None = None


@dataclasses.dataclass
class StepResult:
    observation: str
    reward: float = 0.0
    done: bool = False
    info: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class ToolOutput:
    output: str
    called: bool = True
    error: str = ""
    timeout: bool = False
    runtime: float = 0.0


@dataclasses.dataclass
class RolloutState:
    rewards: list[float] = dataclasses.field(default_factory=list)
    step_count: int = 0
    done: bool = False
    info: dict = dataclasses.field(default_factory=dict)

    def record(self, result: StepResult) -> None:
        self.rewards.append(float(result.reward))
        self.step_count += 1
        self.done = self.done or result.done

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


class RLEnvironment(abc.ABC):
    """Stateful environment acted upon through named tool calls."""

    config_name: str = "env"
    max_steps: int = 16

    @classmethod
    def get_tool_definitions(cls) -> list[dict]:
        return []

    @abc.abstractmethod
    def reset(self, **task) -> StepResult: ...

    @abc.abstractmethod
    def step(self, call: ToolCall) -> StepResult: ...

    def state(self) -> dict:
        return {}

    def close(self) -> None:
        pass


class TextRLEnvironment(RLEnvironment):
    """Environment that reads the model's raw text turn instead of structured calls."""

    def step(self, call: ToolCall) -> StepResult:
        return self.text_step(call.args.get("text", ""))

    @abc.abstractmethod
    def text_step(self, text: str) -> StepResult: ...


class Tool(RLEnvironment):
    """Stateless tool: ``execute(**args) -> ToolOutput``; the schema is derived from the signature."""

    config_name = "tool"
    description = ""

    def reset(self, **task) -> StepResult:
        return StepResult("")

    @abc.abstractmethod
    def execute(self, **kwargs) -> ToolOutput: ...

    def step(self, call: ToolCall) -> StepResult:
        t0 = time.perf_counter()
        try:
            out = self.execute(**call.args)
        except TypeError as e:
            out = ToolOutput("", called=False, error=f"bad arguments for {self.config_name}: {e}")
        except Exception as e:  # noqa: BLE001
            out = ToolOutput("", called=True, error=f"{type(e).__name__}: {e}")
        out.runtime = time.perf_counter() - t0
        return StepResult(out.output if not out.error else f"{out.output}\n{out.error}".strip(), 0.0, False,
                          {"tool_output": out})

    @classmethod
    def get_tool_definitions(cls) -> list[dict]:
        sig = inspect.signature(cls.execute)
        props, required = {}, []
        for name, p in sig.parameters.items():
            if name in ("self", "kwargs"):
                continue
            typ = {int: "integer", float: "number", bool: "boolean"}.get(p.annotation, "string")
            props[name] = {"type": typ}
            if p.default is inspect.Parameter.empty:
                required.append(name)
        return [{"type": "function", "function": {"name": cls.config_name, "description": cls.description or (cls.__doc__ or "").strip(),
                                                  "parameters": {"type": "object", "properties": props, "required": required}}}]
