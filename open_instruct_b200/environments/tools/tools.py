"""Concrete tools and the tool / environment registry.

``TOOL_REGISTRY`` maps config names to classes as in the reference
(``open_instruct/environments/tools/tools.py:647-662``): ``python``, ``jina_browse``, ``s2_search``,
``serper_search``, ``crawl4ai_browse``, ``dr_agent_mcp``, ``generic_mcp``, ``counter``, ``guess_number``,
``generic_sandbox``, ``wordle``.  Network tools are thin HTTP clients over ``make_api_request`` (endpoint
and key from the tool config or the environment); ``python`` runs code in a local subprocess when
no ``api_endpoint`` is configured.
"""

from __future__ import annotations

import os
import subprocess
import sys
import tempfile

from ..base import Tool, ToolOutput
from ..examples import CounterEnv, GuessNumberEnv, WordleTextEnv
from .utils import make_api_request


class PythonCodeTool(Tool):
    """Execute Python code and return stdout / stderr."""

    config_name = "python"
    description = "Executes Python code and returns what it prints."

    def __init__(self, api_endpoint: str | None = None, timeout: float = 10.0, **_):
        self.api_endpoint, self.timeout = api_endpoint, timeout

    def execute(self, code: str = "", text: str | None = None) -> ToolOutput:
        code = code or text or ""
        if not code.strip():
            return ToolOutput("", called=False, error="empty code")
        if self.api_endpoint:
            res = make_api_request(self.api_endpoint, {"code": code, "timeout": self.timeout}, timeout=self.timeout + 5)
            if res["error"]:
                return ToolOutput("", error=res["error"], timeout="timeout" in res["error"].lower())
            d = res["data"]
            return ToolOutput(d.get("output", ""), error=d.get("error") or "")
        with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as fh:
            fh.write(code)
            path = fh.name
        try:
            p = subprocess.run([sys.executable, "-I", path], capture_output=True, text=True, timeout=self.timeout)
            return ToolOutput(p.stdout, error=p.stderr.strip()[-2000:] if p.returncode else "")
        except subprocess.TimeoutExpired:
            return ToolOutput("", error=f"timed out after {self.timeout}s", timeout=True)
        finally:
            os.unlink(path)


class _HttpTool(Tool):
    env_key = ""
    default_endpoint = ""

    def __init__(self, api_endpoint: str | None = None, api_key: str | None = None, timeout: float = 30.0, **extra):
        self.api_endpoint = api_endpoint or self.default_endpoint
        self.api_key = api_key or os.environ.get(self.env_key, "")
        self.timeout, self.extra = timeout, extra

    def _headers(self) -> dict:
        return {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}

    def _format(self, data) -> str:
        return str(data)[:8000]

    def _payload(self, **kw) -> dict:
        return kw

    def execute(self, query: str = "", text: str | None = None, url: str | None = None) -> ToolOutput:
        arg = query or text or url or ""
        if not arg:
            return ToolOutput("", called=False, error="empty argument")
        res = make_api_request(self.api_endpoint, self._payload(query=arg), timeout=self.timeout, headers=self._headers())
        if res["error"]:
            return ToolOutput("", error=res["error"], timeout="timeout" in res["error"].lower())
        return ToolOutput(self._format(res["data"]))


class SerperSearchTool(_HttpTool):
    """Web search through the Serper API."""

    config_name, env_key, default_endpoint = "serper_search", "SERPER_API_KEY", "https://google.serper.dev/search"

    def _headers(self):
        return {"X-API-KEY": self.api_key}

    def _payload(self, query):
        return {"q": query, "num": self.extra.get("num_results", 5)}

    def _format(self, data):
        return "\n\n".join(f"{r.get('title', '')}\n{r.get('link', '')}\n{r.get('snippet', '')}" for r in data.get("organic", []))[:8000]


class S2SearchTool(_HttpTool):
    """Semantic Scholar snippet search."""

    config_name, env_key = "s2_search", "S2_API_KEY"
    default_endpoint = "https://api.semanticscholar.org/graph/v1/snippet/search"

    def _headers(self):
        return {"x-api-key": self.api_key} if self.api_key else {}

    def _format(self, data):
        return "\n\n".join(d.get("snippet", {}).get("text", "") for d in data.get("data", []))[:8000]


class JinaBrowseTool(_HttpTool):
    """Fetch a web page as markdown through Jina Reader."""

    config_name, env_key, default_endpoint = "jina_browse", "JINA_API_KEY", "https://r.jina.ai/"

    def _payload(self, query):
        return {"url": query}

    def _format(self, data):
        return str(data.get("data", {}).get("content", data))[:8000]


class Crawl4AIBrowseTool(_HttpTool):
    """Fetch a web page through a Crawl4AI server."""

    config_name, env_key, default_endpoint = "crawl4ai_browse", "CRAWL4AI_API_KEY", "http://127.0.0.1:11235/crawl"

    def _payload(self, query):
        return {"urls": [query]}


class GenericMCPTool(Tool):
    """Call a tool of an MCP server over its streamable-HTTP JSON-RPC endpoint."""

    config_name = "generic_mcp"

    def __init__(self, server_url: str = "http://127.0.0.1:8000/mcp", tool_name: str = "", timeout: float = 30.0, **_):
        self.server_url, self.tool_name, self.timeout = server_url, tool_name, timeout
        self._id = 0

    def execute(self, **kwargs) -> ToolOutput:
        self._id += 1
        name = kwargs.pop("tool_name", None) or self.tool_name
        res = make_api_request(self.server_url, {"jsonrpc": "2.0", "id": self._id, "method": "tools/call",
                                                 "params": {"name": name, "arguments": kwargs}}, timeout=self.timeout,
                               headers={"Accept": "application/json, text/event-stream"})
        if res["error"]:
            return ToolOutput("", error=res["error"])
        body = res["data"] or {}
        if "error" in body:
            return ToolOutput("", error=str(body["error"]))
        content = body.get("result", {}).get("content", [])
        return ToolOutput("\n".join(c.get("text", "") for c in content if isinstance(c, dict)))


class DrAgentMCPTool(GenericMCPTool):
    config_name = "dr_agent_mcp"


def _sandbox_factory(**kw):
    from ..generic_sandbox import GenericSandboxEnv

    return GenericSandboxEnv(**kw)


TOOL_REGISTRY = {
    "python": PythonCodeTool,
    "jina_browse": JinaBrowseTool,
    "s2_search": S2SearchTool,
    "serper_search": SerperSearchTool,
    "crawl4ai_browse": Crawl4AIBrowseTool,
    "dr_agent_mcp": DrAgentMCPTool,
    "generic_mcp": GenericMCPTool,
    "counter": CounterEnv,
    "guess_number": GuessNumberEnv,
    "generic_sandbox": _sandbox_factory,
    "wordle": WordleTextEnv,
}


def build_pools(envs_config, default_pool_size: int) -> dict:
    """One ``EnvironmentPool`` per configured tool / environment, keyed by its call name."""
    from ..pool import EnvironmentPool

    pools = {}
    size = envs_config.pool_size or default_pool_size
    for name, call_name, cfg in zip(envs_config.tools, envs_config.tool_call_names, envs_config.parsed_tool_configs):
        if name not in TOOL_REGISTRY:
            raise ValueError(f"unknown tool {name}; known: {sorted(TOOL_REGISTRY)}")
        pools[call_name] = EnvironmentPool(lambda n=name, c=cfg: TOOL_REGISTRY[n](**c), size)
    for name, cfg in zip(envs_config.envs, envs_config.parsed_env_configs):
        if name not in TOOL_REGISTRY:
            raise ValueError(f"unknown environment {name}; known: {sorted(TOOL_REGISTRY)}")
        pools[name] = EnvironmentPool(lambda n=name, c=cfg: TOOL_REGISTRY[n](**c), size)
    return pools
