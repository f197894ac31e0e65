"""Keep LLM-judge requests inside the judge model's context window.

Same surface as ``open_instruct/context_window_checker.py``: ``check_context_window_limit``, ``will_exceed_context_window``,
``truncate_messages_to_fit_context`` (system messages are kept, the rest is cut from the end), ``truncate_str_for_prompt_template``.
Token counts come from a Hugging Face tokenizer when ``model_name`` names a loadable one (cached), else from a conservative
character heuristic (one token per 3 characters); role formatting costs 4 tokens per system message and 3 per other message
plus 3 for the reply priming, as in the reference.
"""

from __future__ import annotations

import functools
import logging

logger = logging.getLogger(__name__)


@functools.lru_cache(maxsize=8)
def _tokenizer(model_name: str):
    name = model_name.replace("hosted_vllm/", "")
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(name, local_files_only=True)
    except Exception:  # noqa: BLE001 - unknown or remote-only model: heuristic
        return None


class _Counter:
    def __init__(self, model_name: str):
        self.tok = _tokenizer(model_name)

    def count(self, text: str) -> int:
        return len(self.tok.encode(text, add_special_tokens=False)) if self.tok is not None else (len(text) + 2) // 3

    def cut(self, text: str, n: int) -> str:
        if n <= 0:
            return ""
        if self.tok is not None:
            ids = self.tok.encode(text, add_special_tokens=False)
            return text if len(ids) <= n else self.tok.decode(ids[:n])
        return text[: n * 3]


def _message_tokens(c: _Counter, m: dict) -> int:
    return c.count(m.get("content", "") or "") + (4 if m.get("role") == "system" else 3)


def check_context_window_limit(messages: list[dict], max_completion_tokens: int, model_name: str, max_context_length: int = 8192,
                               safety_margin: int = 100) -> bool:
    """True when prompt + completion budget + margin fit the window."""
    c = _Counter(model_name)
    total = sum(_message_tokens(c, m) for m in messages) + 3
    fits = total + max_completion_tokens + safety_margin <= max_context_length
    if not fits:
        logger.warning("judge request needs %d + %d tokens, window is %d", total, max_completion_tokens, max_context_length)
    return fits


def will_exceed_context_window(messages, max_completion_tokens, model_name, max_context_length: int = 8192, safety_margin: int = 100) -> bool:
    return not check_context_window_limit(messages, max_completion_tokens, model_name, max_context_length, safety_margin)


def truncate_messages_to_fit_context(messages: list[dict], max_completion_tokens: int, model_name: str, max_context_length: int = 8192,
                                     safety_margin: int = 100) -> list[dict]:
    c = _Counter(model_name)
    available = max_context_length - max_completion_tokens - safety_margin - 3
    system = [m for m in messages if m.get("role") == "system"]
    rest = [m for m in messages if m.get("role") != "system"]
    available -= sum(_message_tokens(c, m) for m in system)
    out = []
    for m in rest:
        need = _message_tokens(c, m)
        if need <= available:
            out.append(m)
            available -= need
            continue
        room = available - 3
        if room > 0:
            out.append({**m, "content": c.cut(m.get("content", "") or "", room)})
        break
    return system + out


def truncate_str_for_prompt_template(unformatted_str: str, prompt_template: str, max_completion_tokens: int, model_name: str,
                                     max_context_length: int = 8192, safety_margin: int = 100, placeholder: str = "{output}") -> str:
    c = _Counter(model_name)
    template_tokens = c.count(prompt_template.replace(placeholder, ""))
    room = max_context_length - max_completion_tokens - safety_margin - template_tokens - 6
    return c.cut(unformatted_str, max(0, room))
