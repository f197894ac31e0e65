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
def check_instruction(instruction_id: str, text: str, kw: dict) -> bool:
    """IFEval-style ids (``group:name``) mapped onto the checkers above."""
    kw = {k: v for k, v in (kw or {}).items() if v is not None}
    name = instruction_id.split(":")[-1]
    try:
        if name == "existence":
            return verify_keywords(text, kw["keywords"])
        if name == "frequency":
            return _compare(len(re.findall(r"\b" + re.escape(kw["keyword"].lower()) + r"\b", text.lower())), kw.get("relation"), kw["frequency"])
        if name == "forbidden_words":
            return validate_forbidden_words(text, kw["forbidden_words"])
        if name == "letter_frequency":
            return _compare(text.lower().count(kw["letter"].lower()), kw.get("let_relation"), kw["let_frequency"])
        if name == "response_language":
            return validate_response_language(text, kw["language"])
        if name == "number_sentences":
            return _compare(len(_sentences(text)), kw.get("relation"), kw["num_sentences"])
        if name == "number_paragraphs":
            return verify_paragraph_count(text, kw["num_paragraphs"])
        if name == "number_words":
            return _compare(len(_words(text)), kw.get("relation"), kw["num_words"])
        if name == "nth_paragraph_first_word":
            return validate_paragraphs(text, kw["num_paragraphs"], kw["first_word"], kw["nth_paragraph"])
        if name == "postscript":
            return verify_postscript(text, kw.get("postscript_marker", "P.S."))
        if name == "number_placeholders":
            return validate_placeholders(text, kw["num_placeholders"])
        if name == "number_bullet_lists":
            return verify_bullet_points(text, kw["num_bullets"])
        if name == "constrained_response":
            return validate_choice(text, ["My answer is yes.", "My answer is no.", "My answer is maybe."])
        if name == "number_highlighted_sections":
            return validate_highlighted_sections(text, kw["num_highlights"])
        if name == "multiple_sections":
            return validate_sections(text, kw["num_sections"], kw.get("section_spliter", "Section"))
        if name == "json_format":
            return validate_json_format(text)
        if name == "title":
            return validate_title(text)
        if name == "two_responses":
            return validate_two_responses(text)
        if name == "repeat_prompt":
            return validate_repeat_prompt(text, kw["prompt_to_repeat"])
        if name == "end_checker":
            return validate_end(text, kw["end_phrase"])
        if name == "capital_word_frequency":
            return validate_frequency_capital_words(text, kw["capital_frequency"], kw.get("capital_relation"))
        if name == "english_capital":
            return validate_uppercase(text)
        if name == "english_lowercase":
            return validate_lowercase(text)
        if name == "no_comma":
            return validate_no_commas(text)
        if name == "quotation":
            return validate_quotation(text)
    except (KeyError, TypeError, ValueError):
        return False
    return False
