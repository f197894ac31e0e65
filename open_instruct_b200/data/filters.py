"""Row filters for chat datasets before they enter a training mix.

The reference keeps these as one script per filter under ``scripts/data/filtering_and_updates/`` (``filter_chinese.py``,
``filter_cutoff_date.py``, ``filter_dataset_by_keywords.py``, ``filter_special_tokens.py``, ``filter_ngram_repetitions.py``,
``filter_cots.py``, ``filter_wildchat.py``).  Here they are functions over a row (a dict with a ``messages`` list) that compose,
plus one command:

    python -m open_instruct_b200.data.filters --input in.jsonl --output out.jsonl \\
        --filters cjk,cutoff,identity,repetition --rewrite special_tokens [--filter_user_turns] [--cjk_threshold 0.05]

A *filter* answers "drop this row?" with a reason string (or None to keep); a *rewrite* returns the row changed.  By default
only assistant turns are inspected (a user may write anything; what the model is trained to SAY is what matters),
``filter_user_turns`` widens that.  The report (``<output>.report.json``) counts drops per reason.
"""

from __future__ import annotations

import argparse
import json
import re
from collections import Counter

# ------------------------------------------------------------------------------------------------ text predicates
_CJK = re.compile(r"[一-鿿]")


def cjk_ratio(text: str) -> float:
    """Share of the characters that are CJK unified ideographs."""
    return len(_CJK.findall(text)) / max(1, len(text))


_CUTOFF = re.compile(
    r"(?i)\b(?:as of my (?:last|latest|most recent) (?:update|training|knowledge)"
    r"|(?:my )?(?:knowledge|training)(?: data)? (?:cut[- ]?off|cutoff)"
    r"|my (?:training )?(?:data|knowledge) (?:only )?(?:goes|extends|runs) (?:up )?(?:to|until)"
    r"|i (?:was|am) (?:last )?(?:trained|updated) (?:on data )?(?:up )?(?:to|until|through|in) (?:early |late |mid-?)?(?:\w+ )?(?:19|20)\d\d"
    r"|i (?:do not|don't|cannot|can't) (?:have|access|browse) (?:access to )?(?:real[- ]time|current|up[- ]to[- ]date) (?:information|data|events))")


def mentions_cutoff(text: str) -> bool:
    """The text talks about the speaker's own knowledge cutoff or lack of current information."""
    return bool(_CUTOFF.search(text))


_IDENTITY = re.compile(
    r"(?i)\b(?:i am|i'm|as) (?:an? )?(?:ai )?(?:language )?(?:model |assistant )?(?:called |named |known as )?(?:chatgpt|gpt-?[345][\w.-]*|claude|gemini|bard|llama|mistral|deepseek|qwen|grok|copilot)\b"
    r"|\b(?:developed|created|trained|built|made) by (?:openai|anthropic|google(?: deepmind)?|meta(?: ai)?|microsoft|mistral ai|deepseek|alibaba|xai)\b"
    r"|\bopenai'?s? (?:use|usage|content) polic(?:y|ies)\b")


def claims_other_identity(text: str) -> bool:
    """The speaker names itself as another lab's assistant or cites that lab's policies."""
    return bool(_IDENTITY.search(text))


_SENTENCE_END = re.compile(r"[.!?\n]+")
_CODEISH = re.compile(r"[=+*/^{}\[\]<>|&~#$\\]|\b(?:def|return|import|for|while|if|else)\b")


def repetition_reason(text: str, min_words: int = 6, max_repeats: int = 4, consecutive: int = 3) -> str | None:
    """Degenerate looping: the same sentence-like span (at least ``min_words`` words, not code or formulas) occurs more than
    ``max_repeats`` times, or ``consecutive`` times in a row; or one paragraph makes up most of a long text by repetition."""
    spans = [" ".join(s.split()).lower() for s in _SENTENCE_END.split(text)]
    spans = [s for s in spans if len(s.split()) >= min_words and len(_CODEISH.findall(s)) * 8 < len(s)]
    counts = Counter(spans)
    if counts:
        s, n = counts.most_common(1)[0]
        if n > max_repeats:
            return f"sentence repeated {n}x: {s[:60]!r}"
    run, prev = 1, None
    for s in spans:
        run = run + 1 if s == prev else 1
        prev = s
        if run >= consecutive:
            return f"sentence {run}x in a row: {s[:60]!r}"
    paras = [" ".join(p.split()).lower() for p in text.split("\n\n") if len(p.split()) >= min_words]
    if len(paras) >= 4:
        p, n = Counter(paras).most_common(1)[0]
        if n >= 3 and n * 2 >= len(paras):
            return f"paragraph repeated {n}x of {len(paras)}"
    return None


# control tokens that must not reach the tokenizer as literal text inside a message: rewritten to a visible, inert spelling
SPECIAL_TOKEN_REWRITES = {
    "<|endoftext|>": "<_endoftext_>", "<|im_start|>": "<_im_start_>", "<|im_end|>": "<_im_end_>", "<|eot_id|>": "<_eot_id_>",
    "<|start_header_id|>": "<_start_header_id_>", "<|end_header_id|>": "<_end_header_id_>", "<|begin_of_text|>": "<_begin_of_text_>",
    "<|end_of_text|>": "<_end_of_text_>", "<|user|>": "<_user_>", "<|assistant|>": "<_assistant_>", "<|system|>": "<_system_>",
    "<|pad|>": "<_pad_>",
}


def neutralise_special_tokens(text: str, extra: dict | None = None) -> str:
    for tok, safe in {**SPECIAL_TOKEN_REWRITES, **(extra or {})}.items():
        text = text.replace(tok, safe)
    return text


_THINK_ANSWER = re.compile(r"^\s*<think>[\s\S]*?</think>\s*<answer>[\s\S]*?</answer>\s*$")
_THINK = re.compile(r"^\s*<think>[\s\S]*?</think>[\s\S]*$")


def reasoning_format(text: str) -> str:
    """'think_answer' (``<think>..</think><answer>..</answer>``), 'think' (``<think>..</think>`` then free text) or 'plain'."""
    return "think_answer" if _THINK_ANSWER.match(text) else ("think" if _THINK.match(text) else "plain")


def add_answer_tags(text: str) -> str:
    """``<think>r</think>a`` -> ``<think>r</think><answer>a</answer>`` (other formats unchanged)."""
    if reasoning_format(text) != "think":
        return text
    head, tail = text.split("</think>", 1)
    return f"{head}</think><answer>{tail.strip()}</answer>"


def remove_answer_tags(text: str) -> str:
    if reasoning_format(text) != "think_answer":
        return text
    head, tail = text.split("</think>", 1)
    return head + "</think>" + re.sub(r"^\s*<answer>([\s\S]*?)</answer>\s*$", r"\1", tail)


# ------------------------------------------------------------------------------------------------ row level
def _turns(row: dict, column: str, user_too: bool):
    for m in row.get(column) or []:
        if isinstance(m, dict) and isinstance(m.get("content"), str) and (user_too or m.get("role") == "assistant"):
            yield m


def drop_reason(row: dict, filters: list[str], column: str = "messages", filter_user_turns: bool = False, cjk_threshold: float = 0.05,
                keep_formats: tuple = ()) -> str | None:
    """First reason to drop ``row`` among ``filters`` (names: cjk, cutoff, identity, repetition, format, toxic, redacted,
    non_english), or None."""
    for m in _turns(row, column, filter_user_turns):
        t = m["content"]
        if "cjk" in filters and cjk_ratio(t) >= cjk_threshold and _CJK.search(t):
            return "cjk"
        if "cutoff" in filters and mentions_cutoff(t):
            return "cutoff"
        if "identity" in filters and claims_other_identity(t):
            return "identity"
        if "repetition" in filters and repetition_reason(t):
            return "repetition"
        if "format" in filters and m.get("role") == "assistant" and reasoning_format(t) not in keep_formats:
            return "format"
    # conversation-level annotations (the WildChat columns)
    if "toxic" in filters and row.get("toxic"):
        return "toxic"
    if "redacted" in filters and row.get("redacted"):
        return "redacted"
    if "non_english" in filters and str(row.get("language") or "english").lower() != "english":
        return "non_english"
    return None


def rewrite_row(row: dict, rewrites: list[str], column: str = "messages") -> dict:
    """Apply ``rewrites`` (names: special_tokens, add_answer, remove_answer) to every turn's text (all roles for
    special_tokens, assistant turns for the answer tags)."""
    if not rewrites:
        return row
    out = dict(row)
    msgs = []
    for m in row.get(column) or []:
        m = dict(m)
        if isinstance(m.get("content"), str):
            if "special_tokens" in rewrites:
                m["content"] = neutralise_special_tokens(m["content"])
            if m.get("role") == "assistant":
                if "add_answer" in rewrites:
                    m["content"] = add_answer_tags(m["content"])
                if "remove_answer" in rewrites:
                    m["content"] = remove_answer_tags(m["content"])
        msgs.append(m)
    out[column] = msgs
    return out


def apply(rows, filters: list[str], rewrites: list[str] | None = None, **kw):
    """(kept rows, Counter of drop reasons)."""
    kept, why = [], Counter()
    column = kw.get("column", "messages")
    for row in rows:
        r = drop_reason(row, filters, **kw)
        if r:
            why[r] += 1
        else:
            kept.append(rewrite_row(row, rewrites or [], column))
    return kept, why


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", required=True, help="a .jsonl / .json / .parquet file or a dataset name the data layer loads")
    ap.add_argument("--output", required=True, help=".jsonl to write")
    ap.add_argument("--split", default="train")
    ap.add_argument("--column", default="messages")
    ap.add_argument("--filters", default="", help="comma list: cjk,cutoff,identity,repetition,format,toxic,redacted,non_english")
    ap.add_argument("--rewrite", default="", help="comma list: special_tokens,add_answer,remove_answer")
    ap.add_argument("--filter_user_turns", action="store_true")
    ap.add_argument("--cjk_threshold", type=float, default=0.05)
    ap.add_argument("--keep_formats", default="think_answer,think", help="with the format filter: formats of assistant turns to keep")
    a = ap.parse_args(argv)
    from .mixer import _load_any

    rows = list(_load_any(a.input, a.split, None))
    kept, why = apply(rows, [f for f in a.filters.split(",") if f], [r for r in a.rewrite.split(",") if r], column=a.column,
                      filter_user_turns=a.filter_user_turns, cjk_threshold=a.cjk_threshold, keep_formats=tuple(a.keep_formats.split(",")))
    with open(a.output, "w") as fh:
        for r in kept:
            fh.write(json.dumps(r, ensure_ascii=False) + "\n")
    rep = {"input_rows": len(rows), "kept": len(kept), "dropped": dict(why)}
    with open(a.output + ".report.json", "w") as fh:
        json.dump(rep, fh, indent=1)
    print(json.dumps(rep))
    return rep


if __name__ == "__main__":
    main()
