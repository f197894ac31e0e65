"""IFEval-G: the generalised instruction-following constraint set, keyed by ``group:name`` ids.

Covers every id of the reference's registry (``open_instruct/IFEvalG/instructions_registry.py:54-121``: the 25 original
IFEval constraints and the 29 added ones - copying, per-sentence first / last words, bigram wrapping, counting, palindromes
...).  A checker is a plain function ``(response_text, kwargs) -> bool``; the registry is a dict, so a dataset that names a
constraint this file does not know raises ``UnknownInstruction`` instead of silently scoring zero.

Text handling is self-contained (no nltk / langdetect in this image):

* ``split_sentences``  rule-based splitter in the spirit of the reference's (``IFEvalG/instructions_util.py:1600-1640``):
  periods inside abbreviations, initials, decimals, web addresses and ellipses do not end a sentence; closing quotes stay
  with their sentence.
* ``word_tokens``      Treebank-like tokens: words (contractions split as ``do`` + ``n't``), numbers, each punctuation mark
  on its own - what the reference takes from ``nltk.word_tokenize``.
* ``detect_language``  script ranges for the non-Latin languages of the benchmark and stop-word voting for the Latin ones.
"""

from __future__ import annotations

import json
import re

COMPARISON = ("less than", "at least")


class UnknownInstruction(KeyError):
    """The dataset names a constraint id that has no checker."""


# ------------------------------------------------------------------------------------------------ text utilities
_ABBREV = {"mr", "mrs", "ms", "dr", "prof", "sr", "jr", "st", "mt", "vs", "etc", "inc", "ltd", "co", "corp", "capt", "cpt", "lt",
           "gen", "col", "sen", "rep", "gov", "e.g", "i.e", "no", "fig", "dept", "univ", "approx", "est", "ph.d", "u.s", "u.k", "a.m", "p.m"}
_STARTERS = {"mr", "mrs", "ms", "dr", "prof", "capt", "cpt", "lt", "he", "she", "it", "they", "their", "our", "we", "but", "however",
             "that", "this", "wherever", "the", "a", "an", "in", "on", "i", "you", "there", "what", "when", "why", "how"}
_SITE = re.compile(r"\.(com|net|org|io|gov|edu|me|ai|co)\b", re.I)


def split_sentences(text: str) -> list[str]:
    """Sentences of ``text`` (terminal punctuation kept).  Line breaks count as spaces."""
    t = " " + text.replace("\n", " ") + "  "
    t = _SITE.sub(lambda m: "<prd>" + m.group(1), t)
    t = re.sub(r"(\d)\.(\d)", r"\1<prd>\2", t)
    t = re.sub(r"\.{2,}", lambda m: "<prd>" * len(m.group(0)) + "<stop>", t)

    def protect(m: re.Match) -> str:
        word, nxt = m.group(1), m.group(2)
        low = word.lower().rstrip(".")
        is_abbrev = low in _ABBREV or re.fullmatch(r"(?:[A-Za-z]\.)+[A-Za-z]", word) is not None or len(word) == 1
        if not is_abbrev:
            return m.group(0)
        kept = word.replace(".", "<prd>") + "<prd>"
        # an acronym or suffix followed by a typical sentence opener does end the sentence ("... in the U.S. He left")
        if nxt and nxt[0].isupper() and nxt.lower() in _STARTERS and low not in {"mr", "mrs", "ms", "dr", "prof", "st", "mt", "capt", "cpt", "lt"} and len(word) > 1:
            kept += "<stop>"
        return kept + " " + nxt if nxt else kept

    t = re.sub(r"\b((?:[A-Za-z]\.)*[A-Za-z]+)\.(?:\s+(\w+))?", protect, t)
    for closer in ('"', "”"):
        for mark in ".!?":
            t = t.replace(mark + closer, closer + mark)
    for mark in ".?!":
        t = t.replace(mark, mark + "<stop>")
    t = t.replace("<prd>", ".")
    out = [s.strip() for s in t.split("<stop>")]
    if out and not out[-1]:
        out = out[:-1]
    return out


_TOKEN = re.compile(r"n't\b|'(?:s|re|ve|d|ll|m)\b|\d+(?:[.,]\d+)*|\w+(?:-\w+)*|\.\.\.|[^\w\s]", re.I)


def word_tokens(text: str) -> list[str]:
    """Words, numbers and punctuation marks as separate tokens; ``don't`` -> ``do`` + ``n't``, ``it's`` -> ``it`` + ``'s``."""
    out = []
    for chunk in text.split():
        m = re.fullmatch(r"(\w+)(n't)(\W*)", chunk, re.I)
        if m:
            out += [m.group(1), m.group(2)] + _TOKEN.findall(m.group(3))
            continue
        out += _TOKEN.findall(chunk)
    return out


def count_words(text: str) -> int:
    return len(re.findall(r"\w+", text))


_SCRIPTS = {"ko": r"[가-힯]", "ja": r"[぀-ヿ]", "zh": r"[一-鿿]", "ar": r"[؀-ۿ]", "fa": r"[؀-ۿ]",
            "ur": r"[؀-ۿ]", "hi": r"[ऀ-ॿ]", "mr": r"[ऀ-ॿ]", "ne": r"[ऀ-ॿ]", "bn": r"[ঀ-৿]",
            "pa": r"[਀-੿]", "gu": r"[઀-૿]", "ta": r"[஀-௿]", "te": r"[ఀ-౿]", "kn": r"[ಀ-೿]",
            "th": r"[฀-๿]", "ru": r"[Ѐ-ӿ]", "uk": r"[Ѐ-ӿ]", "bg": r"[Ѐ-ӿ]", "el": r"[Ͱ-Ͽ]",
            "he": r"[֐-׿]"}
_STOPWORDS = {
    "en": "the and is are of to in that it with for was this have not you be on as at by an or from but they which",
    "es": "el la los las de que y en un una es por con para no se su al lo como pero sus le ya este porque",
    "fr": "le la les de des et en un une est que qui dans pour pas sur au avec ce il elle nous vous sont mais",
    "de": "der die das und ist nicht ein eine zu den mit von auf für im dem es sich auch als wie aber oder wir",
    "it": "il lo la gli le di che e un una in per non con sono del della ma come anche più si questo",
    "pt": "o a os as de que e em um uma para com não por se mais como mas foi ao dos das isso está também",
    "nl": "de het een en van is dat niet op te in voor met zijn er maar ook als aan dit wat bij naar",
    "sv": "och det att en är som på för med har inte av den till jag ett om men var så vi kan",
    "da": "og det at en er som på for med har ikke af den til jeg et om men var så vi kan også",
    "fi": "ja on ei että se oli mutta tai kun niin myös hän ovat tämä joka vain kuin jos sitä",
    "pl": "i w nie na to się że z do jest jak ale po co tak za od przez dla czy być",
    "vi": "và là của có không được trong một cho với này người những để các đã khi như",
    "sw": "na ya kwa wa ni la katika za kuwa hii hiyo pia lakini au kama sana watu yake",
    "tr": "ve bir bu için ile da de çok ama gibi daha en kadar olan olarak var ne ben sen",
}


def detect_language(text: str) -> str | None:
    """ISO 639-1 code of the dominant language, or None when nothing can be said."""
    letters = re.findall(r"[^\W\d_]", text)
    if not letters:
        return None
    best, share = None, 0.0
    for code, pat in _SCRIPTS.items():
        s = len(re.findall(pat, text)) / len(letters)
        if s > share:
            best, share = code, s
    if share > 0.5:
        return best  # languages that share a script (ru/uk/bg, ar/fa/ur, hi/mr/ne) resolve to the first of the family
    words = re.findall(r"[^\W\d_]+", text.lower())
    votes = {code: sum(w in set(sw.split()) for w in words) for code, sw in _STOPWORDS.items()}
    code = max(votes, key=votes.get)
    return code if votes[code] > 0 else None


_SAME_SCRIPT = [{"ru", "uk", "bg"}, {"ar", "fa", "ur"}, {"hi", "mr", "ne"}]


def _relation(n: int, relation: str | None, target: int) -> bool:
    rel = relation or "at least"
    if rel == "less than":
        return n < target
    if rel == "at least":
        return n >= target
    raise ValueError(f"unsupported relation {rel!r} (expected one of {COMPARISON})")


def _split_paragraphs(text: str, pattern: str):
    """Paragraphs around ``pattern``; None when an empty paragraph sits between two dividers (an empty first or last piece
    is only a leading / trailing divider and is dropped)."""
    parts = re.split(pattern, text)
    out = []
    for i, p in enumerate(parts):
        if not p.strip():
            if i in (0, len(parts) - 1):
                continue
            return None
        out.append(p)
    return out


# ------------------------------------------------------------------------------------------------ the original 25
def keywords_existence(text, kw):
    return all(re.search(k, text, flags=re.IGNORECASE) for k in kw["keywords"])


def keywords_frequency(text, kw):
    return _relation(len(re.findall(kw["keyword"], text, flags=re.IGNORECASE)), kw.get("relation"), kw["frequency"])


def keywords_forbidden(text, kw):
    return not any(re.search(r"\b" + w + r"\b", text, flags=re.IGNORECASE) for w in kw["forbidden_words"])


def letter_frequency(text, kw):
    return _relation(text.lower().count(kw["letter"].lower()), kw.get("let_relation"), kw["let_frequency"])


def response_language(text, kw):
    want = kw["language"]
    got = detect_language(text)
    if got is None:
        return True  # undetectable text is not held against the response (the reference does the same on detector errors)
    return got == want or any(got in fam and want in fam for fam in _SAME_SCRIPT)


def number_sentences(text, kw):
    return _relation(len(split_sentences(text)), kw.get("relation"), kw["num_sentences"])


def number_paragraphs(text, kw):
    parts = _split_paragraphs(text, r"\s?\*\*\*\s?")
    return parts is not None and len(parts) == kw["num_paragraphs"]


def number_words(text, kw):
    return _relation(count_words(text), kw.get("relation"), kw["num_words"])


def nth_paragraph_first_word(text, kw):
    paragraphs = re.split(r"\n\n", text)
    n = len(paragraphs)
    for p in paragraphs:
        if not p.strip():
            n -= 1
    nth = kw["nth_paragraph"]
    if nth > n or nth < 1:
        return False
    paragraph = paragraphs[nth - 1].strip()
    if not paragraph:
        return False
    first = re.sub(r"[^\w]+$", "", re.sub(r"^[^\w]+", "", paragraph.split()[0].strip().lstrip("'\""))).lower()
    first = "".join(c for c in first if c not in ".,?!'\"")
    return n == kw["num_paragraphs"] and first == kw["first_word"].lower()


def number_placeholders(text, kw):
    return len(re.findall(r"\[.*?\]", text)) >= kw["num_placeholders"]


def postscript(text, kw):
    marker = kw.get("postscript_marker", "P.S.")
    low = text.lower()
    if marker == "P.P.S":
        pat = r"\s*p\.\s?p\.\s?s.*$"
    elif marker == "P.S.":
        pat = r"\s*p\.\s?s\..*$"
    else:
        pat = r"\s*" + marker.lower() + r".*$"
    return bool(re.findall(pat, low, flags=re.MULTILINE))


def number_bullets(text, kw):
    n = len(re.findall(r"^\s*\*[^\*].*$", text, flags=re.MULTILINE)) + len(re.findall(r"^\s*-.*$", text, flags=re.MULTILINE))
    return n == kw["num_bullets"]


def constrained_response(text, kw):
    return any(opt in text.strip() for opt in ("My answer is yes.", "My answer is no.", "My answer is maybe."))


def highlighted_sections(text, kw):
    n = sum(1 for h in re.findall(r"\*[^\n\*]*\*", text) if h.strip("*").strip())
    n += sum(1 for h in re.findall(r"\*\*[^\n\*]*\*\*", text) if h.removeprefix("**").removesuffix("**").strip())
    return n >= kw["num_highlights"]


def multiple_sections(text, kw):
    splitter = kw.get("section_spliter", "Section")
    return len(re.split(r"\s?" + splitter + r"\s?\d+\s?", text)) - 1 >= kw["num_sections"]


def json_format(text, kw):
    v = text.strip().removeprefix("```json").removeprefix("```Json").removeprefix("```JSON").removeprefix("```").removesuffix("```").strip()
    try:
        json.loads(v)
    except ValueError:
        return False
    return True


def title(text, kw):
    return any(t.lstrip("<").rstrip(">").strip() for t in re.findall(r"<<[^\n]+>>", text))


def two_responses(text, kw):
    valid = []
    parts = text.split("******")
    for i, r in enumerate(parts):
        if not r.strip():
            if i not in (0, len(parts) - 1):
                return False
        else:
            valid.append(r)
    return len(valid) == 2 and valid[0].strip() != valid[1].strip()


def repeat_prompt(text, kw):
    return text.strip().lower().startswith(kw["prompt_to_repeat"].strip().lower())


def end_checker(text, kw):
    return text.strip().strip('"').lower().endswith(kw["end_phrase"].strip().lower())


def capital_word_frequency(text, kw):
    n = sum(1 for w in word_tokens(text) if w.isupper())
    return _relation(n, kw.get("capital_relation"), kw["capital_frequency"])


def english_capital(text, kw):
    return text.isupper() and detect_language(text) in ("en", None)


def english_lowercase(text, kw):
    return text.islower() and detect_language(text) in ("en", None)


def no_comma(text, kw):
    return "," not in text


def quotation(text, kw):
    t = text.strip()
    return len(t) > 1 and t[0] == '"' and t[-1] == '"'


# ------------------------------------------------------------------------------------------------ the added constraints
def repeat_phrase(text, kw):
    """The phrase appears exactly ``small_n`` times, each time with exactly one word replaced."""
    ref = kw["phrase"].strip().split()
    found = re.findall(rf"{re.escape(ref[0])} .*? {re.escape(ref[-1])}", text)
    if len(found) != kw["small_n"]:
        return False
    for f in found:
        got = f.split()
        if len(got) != len(ref) or sum(a != b for a, b in zip(got, ref)) != 1:
            return False
    return True


def copy_exact(text, kw):
    return text.strip().lower() == kw["prompt_to_repeat"].strip().lower()


def copy_span_idx(text, kw):
    return text.strip().lower() == kw["prompt_to_repeat"][kw["n_start"]:kw["n_end"]].strip().lower()


def sentence_hyphens(text, kw):
    """Sentences joined by hyphens with no space around the joints."""
    gold = split_sentences(text.replace("-", " "))
    return all(s.strip() == s and s == g for s, g in zip(text.split("-"), gold))


def no_adjacent_consecutive(text, kw):
    w = text.split()
    return not any(ord(b[0].lower()) - ord(a[0].lower()) == 1 for a, b in zip(w, w[1:]))


def square_brackets(text, kw):
    return all(w.startswith("[") and w.endswith("]") for w in text.split())


def word_once(text, kw):
    return len(re.findall(kw["keyword"].strip(), text, flags=re.IGNORECASE)) == 1


def word_count_different_numbers(text, kw):
    return _relation(len(re.findall(kw["keyword"].strip(), text, flags=re.IGNORECASE)), kw.get("relation"), kw["frequency"])


def exclude_word_harder(text, kw):
    return f" {kw['keyword'].strip()} " not in text


def paragraphs_divider(text, kw):
    parts = _split_paragraphs(text, r"\s?\*\*\*\s?")
    return parts is not None and len(parts) == 2


def paragraphs_blank_line(text, kw):
    parts = _split_paragraphs(text, r"\n\n")
    return parts is not None and len(parts) == 2


def _one(v):
    return (v if isinstance(v, str) else v[0]).strip()


def first_word_sent(text, kw):
    want = _one(kw["first_word"]).lower()
    sents = split_sentences(text)
    return all(s.strip() and s.split()[0].strip().lower() == want for s in sents)


def first_word_answer(text, kw):
    return bool(text.split()) and text.split()[0].strip().lower() == kw["first_word"].strip().lower()


def _bare(word: str) -> str:
    return re.sub(r"[^\w\s]", "", word.strip())


def last_word_sent(text, kw):
    want = _one(kw["last_word"]).lower()
    return all(s.strip() and _bare(s.split()[-1]).lower() == want for s in split_sentences(text))


def last_word_answer(text, kw):
    return bool(text.split()) and _bare(text.split()[-1]).lower() == kw["last_word"].strip().lower()


def bigram_wrapping(text, kw):
    w = text.split()
    return all(w[i].startswith("<<") and w[i + 1].endswith(">>") for i in range(0, len(w) - 1, 2))


def copying_multiple(text, kw):
    parts = text.split("******")
    want = kw["prompt_to_repeat"].strip().lower()
    return len(parts) == kw["N"] and all(p.strip().lower() == want for p in parts)


def punctuation_dot(text, kw):
    return "." not in text


def punctuation_exclamation(text, kw):
    return "!" not in text


def lowercase_counting(text, kw):
    return len(re.findall(r"\b[a-z]+\b", text)) <= kw["N"]


def letter_counting(text, kw):
    n = len(re.findall(r"[a-zA-Z]", text))
    rel = kw.get("relation")
    return n >= kw["N"] if rel == "at least" else (n < kw["N"] if rel == "less than" else False)


def counting_composition(text, kw):
    """Three ``***``-separated paragraphs of ``n_sent`` sentences with ``n_words`` tokens each."""
    parts = re.split(r"\s?\*\*\*\s?", text)
    n = len(parts)
    for i, p in enumerate(parts):
        if not p.strip():
            if i in (0, len(parts) - 1):
                n -= 1
            else:
                return False
        sents = split_sentences(p)
        if len(sents) != kw["n_sent"] or any(len(word_tokens(s)) != kw["n_words"] for s in sents):
            return False
    return n == 3


def count_unique(text, kw):
    w = word_tokens(text)
    return len(w) == len(set(w))


def count_increment_word(text, kw):
    return (len(re.findall(kw["keyword1"].strip(), text, flags=re.IGNORECASE)) == 1
            and len(re.findall(kw["keyword2"].strip(), text, flags=re.IGNORECASE)) == 2)


def palindrome(text, kw):
    return any(w == w[::-1] for w in text.split())


def keyword_specific_position(text, kw):
    sents = split_sentences(text)
    if len(sents) < kw["n"]:
        return False
    w = word_tokens(sents[kw["n"] - 1])
    return len(w) >= kw["m"] and w[kw["m"] - 1] == _one(kw["keyword"])


def start_end(text, kw):
    w = word_tokens(text)
    return len(w) >= 2 and w[0].lower() == w[-1].lower()


INSTRUCTION_CHECKERS = {
    "keywords:existence": keywords_existence,
    "keywords:frequency": keywords_frequency,
    "keywords:forbidden_words": keywords_forbidden,
    "keywords:letter_frequency": letter_frequency,
    "language:response_language": response_language,
    "length_constraints:number_sentences": number_sentences,
    "length_constraints:number_paragraphs": number_paragraphs,
    "length_constraints:number_words": number_words,
    "length_constraints:nth_paragraph_first_word": nth_paragraph_first_word,
    "detectable_content:number_placeholders": number_placeholders,
    "detectable_content:postscript": postscript,
    "detectable_format:number_bullet_lists": number_bullets,
    "detectable_format:constrained_response": constrained_response,
    "detectable_format:number_highlighted_sections": highlighted_sections,
    "detectable_format:multiple_sections": multiple_sections,
    "detectable_format:json_format": json_format,
    "detectable_format:title": title,
    "combination:two_responses": two_responses,
    "combination:repeat_prompt": repeat_prompt,
    "startend:end_checker": end_checker,
    "change_case:capital_word_frequency": capital_word_frequency,
    "change_case:english_capital": english_capital,
    "change_case:english_lowercase": english_lowercase,
    "punctuation:no_comma": no_comma,
    "startend:quotation": quotation,
    # ---- added constraints
    "copy:repeat_phrase": repeat_phrase,
    "copy:copy": copy_exact,
    "new:copy_span_idx": copy_span_idx,
    "detectable_format:sentence_hyphens": sentence_hyphens,
    "keywords:no_adjacent_consecutive": no_adjacent_consecutive,
    "detectable_format:square_brackets": square_brackets,
    "keywords:word_once": word_once,
    "keywords:word_count_different_numbers": word_count_different_numbers,
    "keywords:exclude_word_harder": exclude_word_harder,
    "paragraphs:paragraphs": paragraphs_divider,
    "paragraphs:paragraphs2": paragraphs_blank_line,
    "first_word:first_word_sent": first_word_sent,
    "first_word:first_word_answer": first_word_answer,
    "last_word:last_word_sent": last_word_sent,
    "last_word:last_word_answer": last_word_answer,
    "detectable_format:bigram_wrapping": bigram_wrapping,
    "copy:copying_simple": copy_exact,
    "copy:copying_multiple": copying_multiple,
    "punctuation:punctuation_dot": punctuation_dot,
    "punctuation:punctuation_exclamation": punctuation_exclamation,
    "count:lowercase_counting": lowercase_counting,
    "letters:letter_counting": letter_counting,
    "letters:letter_counting2": letter_frequency,
    "count:counting_composition": counting_composition,
    "count:count_unique": count_unique,
    "count:count_increment_word": count_increment_word,
    "keywords:palindrome": palindrome,
    "keywords:keyword_specific_position": keyword_specific_position,
    "keywords:start_end": start_end,
}


def check_instruction(instruction_id: str, text: str, kwargs: dict | None) -> bool:
    """True when ``text`` satisfies the constraint.  Arguments that are None are dropped (datasets store one kwargs dict
    per constraint with the unused keys nulled).  An unknown id raises ``UnknownInstruction``; a constraint whose
    arguments are missing or malformed counts as not satisfied; an empty response satisfies nothing."""
    fn = INSTRUCTION_CHECKERS.get(instruction_id)
    if fn is None:
        raise UnknownInstruction(f"no checker for instruction id {instruction_id!r}; known ids: {sorted(INSTRUCTION_CHECKERS)}")
    if not text or not text.strip():
        return False
    kw = {k: v for k, v in (kwargs or {}).items() if v is not None}
    try:
        return bool(fn(text, kw))
    except (KeyError, TypeError, ValueError, IndexError, re.error):
        return False


def check_instruction_loose(instruction_id: str, text: str, kwargs: dict | None) -> bool:
    """The benchmark's "loose" scoring: the constraint holds for the response or for one of its usual variants (first or
    last line dropped, markdown asterisks removed)."""
    lines = text.split("\n")
    variants = [text, "\n".join(lines[1:]).strip(), "\n".join(lines[:-1]).strip(), "\n".join(lines[1:-1]).strip()]
    variants += [v.replace("*", "") for v in list(variants)]
    return any(v.strip() and check_instruction(instruction_id, v, kwargs) for v in variants)
