"""Multi-turn rollouts with tools and environments on top of the continuous-batching engine.

The reference runs one coroutine per sample that alternates ``completions.create`` calls with tool
execution (``open_instruct/vllm_utils.py:949-1166``).  Here a sample is a ``ToolSession`` state machine:
every model turn is an ordinary engine request; when a turn ends, the text is parsed for tool calls,
the calls are stepped on environments borrowed from the pools, the observation is tokenised and
appended with loss-mask 0 (model tokens carry mask 1, ``vllm_utils.py:169-214``), and the remaining
token budget decides whether another turn is submitted (``:242-268``).  Per-turn rewards are collected
in a ``RolloutState`` for the reward aggregator.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..data_types import SamplingConfig, ToolCallStats
from ..environments.base import RolloutState, TextRLEnvironment, ToolCall


@dataclass
class ToolSession:
    prompt: list[int]
    sampling: SamplingConfig
    seed: int
    max_steps: int
    max_tool_calls: int
    tokens: list[int] = field(default_factory=list)      # everything after the prompt
    masks: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    state: RolloutState = field(default_factory=RolloutState)
    num_calls: int = 0
    timeout: bool = False
    tool_error: str = ""
    tool_output: str = ""
    tool_runtime: float = 0.0
    tool_called: bool = False
    call_stats: list[ToolCallStats] = field(default_factory=list)
    finish_reason: str | None = None
    turns: int = 0
    envs: dict = field(default_factory=dict)              # name -> borrowed environment

    def budget(self) -> int:
        return self.sampling.max_tokens - len(self.tokens)

    def next_request(self) -> tuple[list[int], SamplingConfig]:
        cfg = SamplingConfig(temperature=self.sampling.temperature, top_p=self.sampling.top_p, max_tokens=self.budget(), n=1,
                             stop=self.sampling.stop, seed=self.seed + 7919 * self.turns, min_tokens=0)
        return self.prompt + self.tokens, cfg


class ToolRunner:
    """Owns pools + parser + tokenizer; advances sessions after each model turn."""

    def __init__(self, pools: dict, parser, tokenizer, max_steps: int = 8, max_tool_calls: int = 5, text_env: str | None = None):
        self.pools, self.parser, self.tok = pools, parser, tokenizer
        self.max_steps, self.max_tool_calls = max_steps, max_tool_calls
        self.text_env = text_env  # name of a TextRLEnvironment that sees every turn's raw text

    def stop_strings(self) -> list[str]:
        return list(self.parser.stop_sequences)

    def new_session(self, prompt: list[int], sampling: SamplingConfig, seed: int, task: dict | None = None) -> ToolSession:
        stops = list(dict.fromkeys((sampling.stop or []) + self.stop_strings()))
        cfg = SamplingConfig(**{**sampling.__dict__, "stop": stops or None, "n": 1})
        s = ToolSession(list(prompt), cfg, seed, self.max_steps, self.max_tool_calls)
        if self.text_env is not None:
            env = self.pools[self.text_env].acquire()
            s.envs[self.text_env] = env
            first = env.reset(**(task or {}))
            if first.observation:
                obs = self.tok.encode("\n" + first.observation + "\n", add_special_tokens=False)
                s.prompt = s.prompt + obs
        return s

    def _env_for(self, s: ToolSession, name: str, task: dict | None):
        if name in s.envs:
            return s.envs[name]
        for pool_name, pool in self.pools.items():
            defs = [d["function"]["name"] for d in pool.tool_definitions()] or [pool_name]
            if name == pool_name or name in defs:
                env = pool.acquire()
                env.reset(**(task or {}))
                for n in set(defs + [pool_name]):
                    s.envs[n] = env
                s.envs.setdefault("__owned__", []).append((pool, env))
                return env
        return None

    def on_turn(self, s: ToolSession, new_tokens: list[int], new_logprobs: list[float], finish_reason: str, task: dict | None = None) -> bool:
        """Record a model turn; run tools.  Returns True when another model turn should be submitted."""
        s.tokens += new_tokens
        s.masks += [1] * len(new_tokens)
        s.logprobs += new_logprobs
        s.turns += 1
        text = self.tok.decode(new_tokens, skip_special_tokens=False)
        outputs: list[str] = []
        done = False
        if self.text_env is not None:
            res = s.envs[self.text_env].text_step(text)
            s.state.record(res)
            outputs.append(res.observation)
            done = res.done
        else:
            calls = self.parser.get_tool_calls(text)
            if not calls:
                s.finish_reason = finish_reason
                return False
            for call in calls:
                if s.num_calls >= s.max_tool_calls:
                    outputs.append("Max tool calls exceeded.")
                    done = True
                    break
                env = self._env_for(s, call.name, task)
                if env is None:
                    outputs.append(f"Unknown tool: {call.name}")
                    s.tool_error = s.tool_error or f"unknown tool {call.name}"
                    continue
                t0 = time.perf_counter()
                res = env.step(ToolCall(call.name, call.args))
                dt = time.perf_counter() - t0
                s.num_calls += 1
                s.tool_called = True
                s.tool_runtime += dt
                s.state.record(res)
                to = res.info.get("tool_output")
                err = to.error if to is not None else ""
                s.timeout = s.timeout or bool(to is not None and to.timeout)
                s.tool_error = s.tool_error or err
                s.tool_output += res.observation
                s.call_stats.append(ToolCallStats(call.name, not err, dt))
                outputs.append(res.observation)
                done = done or res.done
        obs_ids = self.tok.encode(self.parser.format_tool_outputs(outputs) if self.text_env is None else "\n" + "\n".join(outputs) + "\n",
                                  add_special_tokens=False)
        room = s.budget()
        if room <= 0:
            s.finish_reason = "length"
            return False
        obs_ids = obs_ids[:room]
        s.tokens += obs_ids
        s.masks += [0] * len(obs_ids)
        s.logprobs += [0.0] * len(obs_ids)
        if done or s.turns >= s.max_steps or s.budget() <= 0:
            s.finish_reason = "stop" if done else "length"
            return False
        return True

    def close_session(self, s: ToolSession) -> None:
        for pool, env in s.envs.pop("__owned__", []):
            pool.release(env)
        if self.text_env is not None and self.text_env in s.envs:
            self.pools[self.text_env].release(s.envs[self.text_env])
        s.envs.clear()
