"""Answer extraction and normalisation for math verifiers.

Implements the conventions the reference relies on (``open_instruct/math_utils.py``): last ``\\boxed{}``
extraction, Minerva-style final-answer normalisation, Hendrycks-MATH string canonicalisation, and a
sympy equivalence check with a timeout-free, exception-safe wrapper.
"""

from __future__ import annotations

import re


def last_boxed_only_string(text: str) -> str | None:
    """The last ``\\boxed{...}`` (or ``\\fbox{...}``) span of ``text``, braces balanced; None if absent."""
    idx = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if idx < 0:
        return None
    if text[idx:].startswith("\\boxed "):
        return "\\boxed " + text[idx + len("\\boxed "):].split("$")[0]
    depth, start = 0, None
    for i in range(idx, len(text)):
        ch = text[i]
        if ch == "{":
            depth += 1
            if start is None:
                start = i
        elif ch == "}":
            depth -= 1
            if depth == 0 and start is not None:
                return text[idx:i + 1]
    return None


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    for left in ("\\boxed{", "\\fbox{"):
        if s.startswith(left) and s.endswith("}"):
            return s[len(left):-1]
    raise ValueError(f"not a boxed expression: {s[:40]!r}")


def get_unnormalized_answer(text: str) -> str:
    """Minerva format: 'Final Answer: The final answer is X. I hope it is correct.'"""
    m = re.search(r"Final Answer: The final answer is(.*?)\. I hope it is correct\.", text + "I hope it is correct.", re.DOTALL)
    return m.group(1).strip() if m else "[invalidanswer]"


_SUBSTITUTIONS = [("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), (r"\ ", ""), (" ", ""), ("mbox", "text"),
                  (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}")]
_REMOVED = ["square", "ways", "integers", "dollars", "mph", "inches", "ft", "hours", "km", "units", "\\ldots", "sue", "points",
            "feet", "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges", "students",
            "childrentickets", "multiples", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}",
            "\\text{}", r"\mathrm{th}", r"^\circ", r"^{\circ}", r"\;", r",\!", "{,}", '"', "\\dots"]


def normalize_final_answer(final_answer: str) -> str:
    """Minerva normalisation: strip units and text wrappers, canonicalise fractions / roots / commas."""
    final_answer = final_answer.split("=")[-1]
    for before, after in _SUBSTITUTIONS:
        final_answer = final_answer.replace(before, after)
    for expr in _REMOVED:
        final_answer = final_answer.replace(expr, "")
    final_answer = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", r"$\3$", final_answer)
    for cmd in ("text", "textbf", "overline", "boxed"):
        final_answer = re.sub(r"(\\%s\{)(.*?)(\})" % cmd, r"\2", final_answer)
    final_answer = re.sub(r"(frac)([^{])(.)", r"frac{\2}{\3}", final_answer)
    final_answer = re.sub(r"(sqrt)([^{])", r"sqrt{\2}", final_answer)
    final_answer = final_answer.replace("$", "")
    if final_answer.replace(",", "").isdigit():
        final_answer = final_answer.replace(",", "")
    return final_answer


def _fix_fracs(s: str) -> str:
    parts = s.split("\\frac")
    out = parts[0]
    for p in parts[1:]:
        out += "\\frac"
        if p and p[0] == "{":
            out += p
            continue
        if len(p) < 2:
            return s
        a, b = p[0], p[1]
        rest = p[2:]
        out += "{" + a + "}" + (b + rest if b == "{" else "{" + b + "}" + rest)
    return out


def _fix_a_slash_b(s: str) -> str:
    parts = s.split("/")
    if len(parts) != 2:
        return s
    try:
        a, b = int(parts[0]), int(parts[1])
        return f"\\frac{{{a}}}{{{b}}}" if s == f"{a}/{b}" else s
    except ValueError:
        return s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def strip_string(s: str) -> str:
    """Hendrycks-MATH canonical form used for exact string comparison."""
    s = s.replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "")
    if "\\text{ " in s:
        s = s.split("\\text{ ")[0]
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if not s:
        return s
    if s[0] == ".":
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s).replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    return _fix_a_slash_b(s)


def hendrycks_is_equiv(a: str | None, b: str | None) -> bool:
    if a is None or b is None:
        return a is None and b is None
    try:
        return strip_string(a) == strip_string(b)
    except Exception:  # noqa: BLE001
        return a == b


def is_equiv(x1: str, x2: str) -> bool:
    """Symbolic equality of two LaTeX expressions through sympy (False on any parse failure)."""
    try:
        import sympy
        from sympy.parsing.latex import parse_latex
    except Exception:  # noqa: BLE001 - sympy or its LaTeX parser is not installed
        return False
    try:
        p1, p2 = parse_latex(x1), parse_latex(x2)
        diff = p1 - p2
        return bool(sympy.simplify(diff) == 0)
    except Exception:  # noqa: BLE001
        return False
