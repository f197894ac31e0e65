"""Instruction-following constraint checkers (IFEval family).

Two entry styles, as in the reference (``open_instruct/if_functions.py``, ``open_instruct/IFEvalG/``):
``IF_FUNCTIONS_MAP[name](text, **kwargs) -> bool`` for the single-constraint datasets and
``check_instruction("group:name", text, kwargs) -> bool`` for IFEval-style ids.  Each checker is a
pure function of the response text.
"""

from __future__ import annotations

import json
import re


def _words(text: str) -> list[str]:
    return re.findall(r"\b\w+\b", text)


def _sentences(text: str) -> list[str]:
    return [s for s in re.split(r"(?<=[.!?])\s+", text.strip()) if s]


def _paragraphs(text: str, sep: str = r"\n\s*\n") -> list[str]:
    return [p for p in re.split(sep, text.strip()) if p.strip()]


def _compare(n: int, relation: str | None, target: int, slack: int | None = None) -> bool:
    """``slack`` is the tolerance of the "around" quantifier (a tenth of the target, at least one, by default)."""
    rel = (relation or "at least").lower()
    if rel == "around":
        return abs(n - target) <= (max(round(0.1 * target), 1) if slack is None else slack)
    if rel in ("at least", ">=", "more than or equal"):
        return n >= target
    if rel in ("at most", "<=", "less than or equal"):
        return n <= target
    if rel in ("less than", "<"):
        return n < target
    if rel in ("more than", ">"):
        return n > target
    if rel in ("exactly", "==", "equal"):
        return n == target
    return False  # an unknown quantifier satisfies nothing


# ------------------------------------------------------------------ single-constraint functions
def verify_keywords(text: str, keyword_list: list[str]) -> bool:
    low = text.lower()
    return all(k.lower() in low for k in keyword_list)


def verify_keyword_frequency(text: str, word: str, N: int) -> bool:
    return len(re.findall(r"\b" + re.escape(word.lower()) + r"\b", text.lower())) == N


def validate_forbidden_words(text: str, forbidden_words: list[str]) -> bool:
    low = text.lower()
    return not any(re.search(r"\b" + re.escape(w.lower()) + r"\b", low) for w in forbidden_words)


def verify_letter_frequency(text: str, letter: str, N: int) -> bool:
    return text.count(letter) == N


def validate_response_language(text: str, language: str) -> bool:
    try:
        import langdetect

        return langdetect.detect(text) == language
    except Exception:  # noqa: BLE001 - detector missing or undecidable text: do not punish
        return True


def verify_paragraph_count(text: str, N: int) -> bool:
    return len([p for p in re.split(r"\s?\*\*\*\s?", text) if p.strip()]) == N


def validate_word_constraint(text: str, N: int, quantifier: str) -> bool:
    return _compare(len(text.strip().split()), quantifier, N)


def verify_sentence_constraint(text: str, N: int, quantifier: str) -> bool:
    return _compare(len(_sentences(text)), quantifier, N, slack=1)


def validate_paragraphs(text: str, N: int, first_word: str, i: int) -> bool:
    paras = [p.strip() for p in text.split("\n\n") if p.strip()]
    return len(paras) == N and 1 <= i <= len(paras) and paras[i - 1].lower().startswith(first_word.lower())


def verify_postscript(text: str, postscript_marker: str) -> bool:
    idx = text.find(postscript_marker)
    return idx >= 0 and len(text[idx + len(postscript_marker):].strip()) > 0


def validate_placeholders(text: str, N: int) -> bool:
    return len(re.findall(r"\[(.*?)\]", text)) >= N


def verify_bullet_points(text: str, N: int) -> bool:
    return len([ln for ln in text.split("\n") if ln.strip().startswith(("*", "-"))]) == N


def validate_title(text: str) -> bool:
    return re.search(r"<<(.+?)>>", text) is not None


def validate_choice(text: str, options: list[str]) -> bool:
    return any(text.strip() == o or o in text for o in options)


def validate_highlighted_sections(text: str, N: int) -> bool:
    return len(re.findall(r"\*[^\n\*]+\*", text)) >= N


def validate_sections(text: str, N: int, section_splitter: str) -> bool:
    parts = text.split(section_splitter)
    if parts and parts[0].strip() == "":
        parts = parts[1:]
    return len(parts) == N


def validate_json_format(text: str) -> bool:
    t = text.strip()
    t = re.sub(r"^```(?:json|JSON)?", "", t).strip()
    t = re.sub(r"```$", "", t).strip()
    try:
        json.loads(t)
        return True
    except ValueError:
        return False


def validate_repeat_prompt(text: str, original_prompt: str) -> bool:
    return text.strip().lower().startswith(original_prompt.strip().lower())


def validate_two_responses(text: str) -> bool:
    parts = text.split("******")
    return len(parts) == 2 and parts[0].strip() != parts[1].strip() and all(p.strip() for p in parts)


def validate_uppercase(text: str) -> bool:
    return text == text.upper()


def validate_lowercase(text: str) -> bool:
    return text == text.lower()


def validate_frequency_capital_words(text: str, N: int, quantifier: str) -> bool:
    return _compare(len(re.findall(r"\b[A-Z]+\b", text)), quantifier, N)


def validate_end(text: str, end_phrase: str) -> bool:
    return text.strip().endswith(end_phrase.strip())


def validate_quotation(text: str) -> bool:
    t = text.strip()
    return len(t) > 1 and t[0] == '"' and t[-1] == '"'


def validate_no_commas(text: str) -> bool:
    return "," not in text


IF_FUNCTIONS_MAP = {
    "verify_keywords": verify_keywords,
    "verify_keyword_frequency": verify_keyword_frequency,
    "validate_forbidden_words": validate_forbidden_words,
    "verify_letter_frequency": verify_letter_frequency,
    "validate_response_language": validate_response_language,
    "verify_paragraph_count": verify_paragraph_count,
    "validate_word_constraint": validate_word_constraint,
    "verify_sentence_constraint": verify_sentence_constraint,
    "validate_paragraphs": validate_paragraphs,
    "verify_postscript": verify_postscript,
    "validate_placeholders": validate_placeholders,
    "verify_bullet_points": verify_bullet_points,
    "validate_title": validate_title,
    "validate_choice": validate_choice,
    "validate_highlighted_sections": validate_highlighted_sections,
    "validate_sections": validate_sections,
    "validate_json_format": validate_json_format,
    "validate_repeat_prompt": validate_repeat_prompt,
    "validate_two_responses": validate_two_responses,
    "validate_uppercase": validate_uppercase,
    "validate_lowercase": validate_lowercase,
    "validate_frequency_capital_words": validate_frequency_capital_words,
    "validate_end": validate_end,
    "validate_quotation": validate_quotation,
    "validate_no_commas": validate_no_commas,
}


# ------------------------------------------------------------------ IFEval instruction ids
# The ``group:name`` constraint set (all ids of ``open_instruct/IFEvalG/instructions_registry.py``) lives in ``ifevalg.py``;
# an unknown id raises there instead of scoring zero.
from .ifevalg import INSTRUCTION_CHECKERS, UnknownInstruction, check_instruction, check_instruction_loose  # noqa: E402,F401
