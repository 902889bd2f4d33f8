"""Mathematical answer grading: extraction of the final ``\\boxed{}`` answer, textual normalisation (units, currency,
LaTeX wrappers, thousands separators), then equality by number (relative tolerance, percent forms), by tuple/interval
element-wise, and by symbolic difference when both sides parse (cosmos_rl/tools/eval_utils/grader.py)."""
from __future__ import annotations

import re
from typing import List, Optional

_UNIT_WORDS = ("degrees", "degree", "cm", "centimeters", "meters", "meter", "mph", "units", "unit", "square", "sq",
               "inches", "inch", "feet", "foot", "dollars", "dollar", "cents", "cent", "hours", "hour", "minutes",
               "minute", "seconds", "second", "days", "day", "percent", "points", "point")


def extract_boxed(text: str) -> Optional[str]:
    """Contents of the last ``\\boxed{...}`` / ``\\fbox{...}`` with balanced braces; None when there is none."""
    best = None
    for m in re.finditer(r"\\(?:boxed|fbox)\s*\{", text):
        depth, i = 1, m.end()
        while i < len(text) and depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        if depth == 0:
            best = text[m.end(): i - 1]
    return best


def _strip_wrappers(s: str) -> str:
    prev = None
    while prev != s:
        prev = s
        s = re.sub(r"\\(?:text|textbf|mathrm|mathbf|mbox|mathit)\s*\{([^{}]*)\}", r"\1", s)
    return s


def normalize_answer(ans: str) -> str:
    s = str(ans).strip()
    s = s.split("=")[-1] if re.fullmatch(r"[A-Za-z]\w*\s*=\s*[^=]+", s) else s          # "x = 5" -> "5"
    s = _strip_wrappers(s)
    s = s.replace("\\$", "").replace("$", "").replace("\\%", "%").replace("\\!", "").replace("\\,", "").replace("\\ ", " ")
    s = s.replace("\\left", "").replace("\\right", "").replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac")
    s = s.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    s = re.sub(r"\\(?:quad|qquad|;|:)", " ", s)
    for w in _UNIT_WORDS:
        s = re.sub(rf"(?<=[\d\s}}]){w}\b\.?", "", s)
    s = re.sub(r"(\d),(?=\d{3}\b)", r"\1", s)                                           # 1,234 -> 1234
    s = re.sub(r"\\frac\s*(\d)\s*(\d)", r"\\frac{\1}{\2}", s)                           # \frac12 -> \frac{1}{2}
    s = re.sub(r"\\sqrt\s*(\w)", r"\\sqrt{\1}", s)
    s = s.strip().rstrip(".").strip()
    if s.startswith("{") and s.endswith("}") and s.count("{") == 1:
        s = s[1:-1]
    return re.sub(r"\s+", "", s)


def _to_number(s: str) -> Optional[float]:
    pct = s.endswith("%")
    t = s[:-1] if pct else s
    m = re.fullmatch(r"(-?)\\frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", t)
    try:
        if m:
            v = float(m.group(2)) / float(m.group(3)) * (-1 if m.group(1) else 1)
        elif re.fullmatch(r"-?[\d.]+/-?[\d.]+", t):
            a, b = t.split("/")
            v = float(a) / float(b)
        else:
            v = float(t)
    except (ValueError, ZeroDivisionError):
        return None
    return v / 100.0 if pct else v


def _split_top(s: str) -> List[str]:
    parts, depth, cur = [], 0, ""
    for ch in s:
        depth += {"(": 1, "[": 1, "{": 1, ")": -1, "]": -1, "}": -1}.get(ch, 0)
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    return parts + [cur]


def _latex_to_expr(s: str) -> str:
    prev = None
    while prev != s:
        prev = s
        s = re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", s)
        s = re.sub(r"\\sqrt\{([^{}]*)\}", r"sqrt(\1)", s)
    s = s.replace("\\pi", "pi").replace("\\cdot", "*").replace("\\times", "*").replace("^", "**")
    s = s.replace("{", "(").replace("}", ")")
    return re.sub(r"(\d)([a-zA-Z(])", r"\1*\2", s)


def _symbolic_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr
        ea, eb = parse_expr(_latex_to_expr(a)), parse_expr(_latex_to_expr(b))
        return bool(sympy.simplify(ea - eb) == 0)
    except Exception:  # noqa: BLE001  (anything unparsable is simply not symbolically equal)
        return False


def math_equal(prediction: str, reference: str, rel_tol: float = 1e-4, allow_percent: bool = True) -> bool:
    a, b = normalize_answer(prediction), normalize_answer(reference)
    if a == b or a.lower() == b.lower():
        return True
    na, nb = _to_number(a), _to_number(b)
    if na is not None and nb is not None:
        cands = [nb] + ([nb / 100.0, nb * 100.0] if allow_percent else [])
        return any(abs(na - c) <= rel_tol * max(1.0, abs(c)) for c in cands)
    if a[:1] in "([" and b[:1] in "([" and a[-1:] in ")]" and b[-1:] in ")]":
        if a[0] != b[0] or a[-1] != b[-1]:
            return False                                   # open vs closed interval
        pa, pb = _split_top(a[1:-1]), _split_top(b[1:-1])
        return len(pa) == len(pb) and all(math_equal(x, y, rel_tol, False) for x, y in zip(pa, pb))
    if len(a) > 64 or len(b) > 64:
        return False
    return _symbolic_equal(a, b)


# ---- names of the reference's grader that data set scripts import (cosmos_rl/tools/eval_utils/grader.py:448-540)
def math_answer_cleaning(answer: str) -> str:
    return normalize_answer(str(answer))


def is_equal_after_calculation(extracted_answer: str, gold: str) -> bool:
    """Equal as numbers once fractions and arithmetic are evaluated."""
    a, b = _to_number(normalize_answer(str(extracted_answer))), _to_number(normalize_answer(str(gold)))
    if a is None or b is None:
        return _symbolic_equal(str(extracted_answer), str(gold))
    return abs(a - b) <= 1e-6 * max(1.0, abs(b))


def round_number(answer: str) -> str:
    """Numbers below 0.01 in magnitude are kept to two significant figures (so 0.00123456 compares as 0.0012)."""
    try:
        v = float(answer)
    except (TypeError, ValueError):
        return answer
    if v != 0 and abs(v) < 0.01:
        return f"{v:.2g}"
    return answer
