"""Tool-call parsers: turn a model's text turn into ``ToolCall``s.

Formats (cf. ``open_instruct/environments/tools/parsers.py:225-264``):
  legacy        ``<tool_name>free text argument</tool_name>`` (one positional argument)
  dr_tulu       ``<call_tool name="search">query</call_tool>``
  hermes        ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``      (vllm_hermes / olmo3)
  llama3_json   a bare JSON object ``{"name": ..., "parameters": {...}}``          (vllm_llama3_json)
  qwen3_xml     ``<tool_call><function=NAME><parameter=K>V</parameter>...</function></tool_call>``
Each parser also knows how to render a tool result back into the conversation.
"""

from __future__ import annotations

import json
import re
from abc import ABC, abstractmethod

from ..base import ToolCall


class ToolParser(ABC):
    stop_sequences: list[str] = []

    @abstractmethod
    def get_tool_calls(self, text: str) -> list[ToolCall]: ...

    def format_tool_outputs(self, outputs: list[str]) -> str:
        return "".join(f"<output>\n{o}\n</output>\n" for o in outputs)


class LegacyToolParser(ToolParser):
    def __init__(self, tool_names: list[str], arg_names: dict[str, str] | None = None):
        self.tool_names = list(tool_names)
        self.arg_names = arg_names or {}
        self.stop_sequences = [f"</{n}>" for n in self.tool_names]
        self._re = {n: re.compile(rf"<{re.escape(n)}>(.*?)</{re.escape(n)}>", re.DOTALL) for n in self.tool_names}

    def get_tool_calls(self, text: str) -> list[ToolCall]:
        found = []
        for n, rx in self._re.items():
            for m in rx.finditer(text):
                found.append((m.start(), ToolCall(n, {self.arg_names.get(n, "text"): m.group(1).strip()})))
        return [c for _, c in sorted(found, key=lambda t: t[0])]


class DRTuluToolParser(ToolParser):
    stop_sequences = ["</call_tool>"]
    _re = re.compile(r'<call_tool\s+name="([^"]+)"\s*>(.*?)</call_tool>', re.DOTALL)

    def get_tool_calls(self, text: str) -> list[ToolCall]:
        return [ToolCall(m.group(1), {"text": m.group(2).strip()}) for m in self._re.finditer(text)]

    def format_tool_outputs(self, outputs):
        return "".join(f"<tool_output>\n{o}\n</tool_output>\n" for o in outputs)


class HermesToolParser(ToolParser):
    stop_sequences = ["</tool_call>"]
    _re = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)

    def get_tool_calls(self, text: str) -> list[ToolCall]:
        calls = []
        for m in self._re.finditer(text):
            try:
                obj = json.loads(m.group(1))
                args = obj.get("arguments", obj.get("parameters", {}))
                if isinstance(args, str):
                    args = json.loads(args)
                calls.append(ToolCall(obj["name"], dict(args)))
            except (json.JSONDecodeError, KeyError, TypeError, ValueError):
                continue
        return calls

    def format_tool_outputs(self, outputs):
        return "".join(f"<tool_response>\n{o}\n</tool_response>\n" for o in outputs)


class Llama3JsonToolParser(ToolParser):
    stop_sequences = ["<|eom_id|>"]

    def get_tool_calls(self, text: str) -> list[ToolCall]:
        calls, dec, i = [], json.JSONDecoder(), 0
        while (j := text.find("{", i)) >= 0:
            try:
                obj, end = dec.raw_decode(text[j:])
            except json.JSONDecodeError:
                i = j + 1
                continue
            i = j + end
            if isinstance(obj, dict) and "name" in obj and isinstance(obj.get("parameters", obj.get("arguments")), dict):
                calls.append(ToolCall(obj["name"], dict(obj.get("parameters", obj.get("arguments")))))
        return calls


class Qwen3XmlToolParser(ToolParser):
    stop_sequences = ["</tool_call>"]
    _fn = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.DOTALL)
    _par = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.DOTALL)

    def get_tool_calls(self, text: str) -> list[ToolCall]:
        calls = []
        for m in self._fn.finditer(text):
            args = {}
            for p in self._par.finditer(m.group(2)):
                v = p.group(2).strip()
                try:
                    args[p.group(1)] = json.loads(v)
                except json.JSONDecodeError:
                    args[p.group(1)] = v
            calls.append(ToolCall(m.group(1), args))
        return calls

    def format_tool_outputs(self, outputs):
        return "".join(f"<tool_response>\n{o}\n</tool_response>\n" for o in outputs)


PARSERS = {"legacy": LegacyToolParser, "dr_tulu": DRTuluToolParser, "vllm_hermes": HermesToolParser, "vllm_olmo3": HermesToolParser,
           "vllm_llama3_json": Llama3JsonToolParser, "vllm_qwen3_xml": Qwen3XmlToolParser}


def create_tool_parser(name: str, tool_names: list[str] | None = None, **kw) -> ToolParser:
    if name not in PARSERS:
        raise ValueError(f"unknown tool parser {name}; choose from {sorted(PARSERS)}")
    cls = PARSERS[name]
    return cls(tool_names or [], **kw) if cls is LegacyToolParser else cls()
