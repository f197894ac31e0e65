"""Tool / environment configuration and HTTP helper.

``EnvsConfig`` carries the CLI surface of the reference (``open_instruct/environments/tools/utils.py:34-107``):
which tools and environments are active, their per-tool JSON configs, the parser, pool size and
limits.  ``make_api_request`` retries on 429 / 5xx with exponential backoff (``:233-312``).
"""

from __future__ import annotations

import json
import time
from dataclasses import dataclass, field


@dataclass
class EnvsConfig:
    tools: list[str] | None = None
    tool_call_names: list[str] | None = None
    tool_configs: list[str] = field(default_factory=list)
    tool_parser_type: str = "legacy"
    max_tool_calls: int = 5
    max_steps: int = 8
    only_reward_good_outputs: bool = False
    pool_size: int | None = None
    tool_timeout: float = 60.0
    pass_tools_to_chat_template: bool = True
    envs: list[str] | None = None
    env_configs: list[str] = field(default_factory=list)

    def __post_init__(self):
        self.tools = self.tools or []
        self.envs = self.envs or []
        if self.tool_call_names is None:
            self.tool_call_names = list(self.tools)
        if len(self.tool_call_names) != len(self.tools):
            raise ValueError("tool_call_names must have one entry per tool")
        if self.tool_configs and len(self.tool_configs) != len(self.tools):
            raise ValueError("tool_configs must have one JSON object per tool")
        self.parsed_tool_configs = [json.loads(c) if isinstance(c, str) else dict(c) for c in self.tool_configs] or [{} for _ in self.tools]
        self.parsed_env_configs = [json.loads(c) if isinstance(c, str) else dict(c) for c in self.env_configs] or [{} for _ in self.envs]
        if self.max_tool_calls < 0 or self.max_steps < 1:
            raise ValueError("max_tool_calls must be >= 0 and max_steps >= 1")

    @property
    def enabled(self) -> bool:
        return bool(self.tools or self.envs)


def make_api_request(url: str, payload: dict | None = None, method: str = "POST", timeout: float = 30.0, max_retries: int = 3,
                     backoff: float = 0.5, headers: dict | None = None, session=None) -> dict:
    """JSON request with retry on 429 / 5xx / connection errors.  Returns ``{"data": ..., "error": str}``."""
    import requests

    sess = session or requests
    err = ""
    for attempt in range(max_retries + 1):
        try:
            r = sess.request(method, url, json=payload, timeout=timeout, headers=headers)
            if r.status_code == 429 or r.status_code >= 500:
                err = f"HTTP {r.status_code}"
            elif r.status_code >= 400:
                return {"data": None, "error": f"HTTP {r.status_code}: {r.text[:200]}"}
            else:
                return {"data": r.json(), "error": ""}
        except Exception as e:  # noqa: BLE001
            err = f"{type(e).__name__}: {e}"
        if attempt < max_retries:
            time.sleep(backoff * 2 ** attempt)
    return {"data": None, "error": err}
