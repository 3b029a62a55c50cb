"""Answer extraction, normalisation and grading for math rewards (GSM8K / MATH style).

Grading is layered like tunix/utils/math_utils.py:603-690: exact match of normalised strings, then numeric
equality of anything that parses as a number / fraction / percentage / mixed number, then element-wise
comparison of tuples and interval endpoints. The reference's last layer is a sympy equivalence check; sympy
is an optional import here: when it is missing that layer is skipped and such pairs grade as different.
"""
from __future__ import annotations

import re
from fractions import Fraction
from typing import Optional


def last_boxed_only_string(s: str) -> Optional[str]:
    """The last `\\boxed{...}` / `\\fbox{...}` group (balanced braces), or None."""
    idx = max(s.rfind("\\boxed"), s.rfind("\\fbox"))
    if idx < 0:
        return None
    i = s.find("{", idx)
    if i < 0:
        rest = s[idx:].split()          # "\boxed 5"
        return " ".join(rest[:2]) if len(rest) >= 2 else None
    depth = 0
    for j in range(i, len(s)):
        if s[j] == "{":
            depth += 1
        elif s[j] == "}":
            depth -= 1
            if depth == 0:
                return s[idx:j + 1]
    return None


def remove_boxed(s: Optional[str]) -> Optional[str]:
    if s is None:
        return None
    for left in ("\\boxed{", "\\fbox{"):
        if s.startswith(left) and s.endswith("}"):
            return s[len(left):-1]
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    return None


def extract_boxed_answer(solution: str) -> Optional[str]:
    return remove_boxed(last_boxed_only_string(solution))


def extract_answer(passage: str) -> Optional[str]:
    """Boxed answer if present, else what follows '####' (GSM8K) or 'answer is'."""
    if "\\boxed" in passage or "\\fbox" in passage:
        return extract_boxed_answer(passage)
    m = re.search(r"####\s*(.+)", passage)
    if m:
        return m.group(1).strip()
    m = re.search(r"answer is[:\s]*\$?([^\n$]+?)\$?[.\s]*$", passage.strip(), re.IGNORECASE)
    return m.group(1).strip() if m else None


_UNITS = ("degrees", "degree", "cm", "centimeters", "meters", "meter", "mph", "units", "unit", "inches", "inch", "feet", "foot",
          "minutes", "minute", "hours", "hour", "seconds", "second", "dollars", "dollar", "cents", "cent", "square", "sq")


def _fix_fracs(s: str) -> str:
    s = re.sub(r"\\[dt]frac", r"\\frac", s)
    s = re.sub(r"\\frac\s*(\d)\s*(\d)", r"\\frac{\1}{\2}", s)                     # \frac12 -> \frac{1}{2}
    s = re.sub(r"\\frac\s*(\d)\s*\{", r"\\frac{\1}{", s)
    return s


def _strip_string(s: str) -> str:
    s = s.replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    s = s.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "").replace("$", "").replace("\\%", "%").replace("\\ ", " ")
    s = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", s)
    s = re.sub(r"\\mbox\{\s*([^}]*)\}", r"\1", s)
    s = _fix_fracs(s)
    s = re.sub(r"\\sqrt\s*(\w)", r"\\sqrt{\1}", s)
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if "=" in s and len(s.split("=")[0]) <= 2:                                     # "x = 5"
        s = s.split("=", 1)[1]
    for u in _UNITS:
        s = re.sub(rf"(?<=\d)\s*\\?{u}\b(\^\{{?\d\}}?)?", "", s)
    s = s.replace(" ", "")
    s = re.sub(r"^\\frac\{(-?\d+)\}\{(-?\d+)\}$", r"\1/\2", s)
    if s.endswith(".") and s[:-1].replace(".", "").isdigit():
        s = s[:-1]
    return s


def mathd_normalize_answer(answer: Optional[str]) -> Optional[str]:
    if answer is None:
        return None
    answer = answer.strip()
    m = re.search(r"^\\text\{(?P<text>.+?)\}$", answer)
    if m:
        answer = m.group("text").strip()
    try:
        return _strip_string(answer)
    except Exception:
        return answer


def _strip_commas(s: str) -> str:
    while True:
        t = re.sub(r"(\d)(,)(\d\d\d)(?!\d)", r"\1\3", s)
        if t == s:
            return s
        s = t


def _to_number(s: str) -> Optional[Fraction]:
    """Fraction value of plain numbers, `a/b`, `\\frac{a}{b}`, percentages and mixed numbers `1 2/3`; else None."""
    s = _strip_commas(s.strip().replace("\\%", "%").replace("$", "").replace("\\$", ""))
    scale = Fraction(1)
    if s.endswith("%"):
        s, scale = s[:-1], Fraction(1, 100)
    m = re.fullmatch(r"(-?)\s*(\d+)\s+(\d+)\s*/\s*(\d+)", s)
    try:
        if m:
            v = Fraction(int(m.group(2))) + Fraction(int(m.group(3)), int(m.group(4)))
            return (-v if m.group(1) else v) * scale
        m = re.fullmatch(r"(-?)\\?d?frac\{(-?\d+)\}\{(-?\d+)\}", s.replace(" ", ""))
        if m:
            v = Fraction(int(m.group(2)), int(m.group(3)))
            return (-v if m.group(1) else v) * scale
        s2 = s.replace(" ", "")
        if re.fullmatch(r"-?\d+/-?\d+", s2):
            a, b = s2.split("/")
            return Fraction(int(a), int(b)) * scale
        if re.fullmatch(r"-?(\d+\.?\d*|\.\d+)([eE]-?\d+)?", s2):
            return Fraction(s2) * scale
    except (ZeroDivisionError, ValueError):
        return None
    return None


def _normalize(expr: Optional[str]) -> Optional[str]:
    if expr is None:
        return None
    expr = mathd_normalize_answer(expr) or ""
    expr = _strip_commas(expr.replace("\\%", "%").replace("\\$", "").replace("$", ""))
    for w in ("million", "billion", "trillion"):
        m = re.fullmatch(rf"(-?\d+\.?\d*){w}", expr)
        if m:
            expr = str(Fraction(m.group(1)) * {"million": 10 ** 6, "billion": 10 ** 9, "trillion": 10 ** 12}[w])
    expr = expr.replace("\\cdot", "*").replace("\\times", "*").replace("\\le", "<=").replace("\\ge", ">=")
    if expr.startswith("{") and expr.endswith("}") and expr.count("{") == 1:
        expr = expr[1:-1]
    return expr.lower()


def split_tuple(expr: str) -> list:
    """`(1, 2]` -> ['1', '2'] (also bare comma lists); a scalar becomes a one-element list."""
    expr = _strip_commas(expr)
    if len(expr) >= 2 and expr[0] in "([" and expr[-1] in ")]" and all(c not in expr[1:-1] for c in "()[]"):
        return [e.strip() for e in expr[1:-1].split(",")]
    return [expr]


def _elements_equal(a: str, b: str) -> bool:
    if a == b:
        return True
    na, nb = _to_number(a), _to_number(b)
    if na is not None and nb is not None:
        return na == nb
    return are_equal_under_sympy(a, b)


def are_equal_under_sympy(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing import sympy_parser
    except Exception:
        return False
    if any(len(x) > 200 or re.search(r"[a-zA-Z]{4,}", x) for x in (a, b)):
        return False
    try:
        tr = sympy_parser.standard_transformations + (sympy_parser.implicit_multiplication_application,)
        diff = sympy_parser.parse_expr(f"({a})-({b})".replace("^", "**"), transformations=tr)
        return sympy.simplify(diff) == 0
    except Exception:
        return False


def grade_answer_mathd(given_answer: str, ground_truth: str) -> bool:
    return mathd_normalize_answer(given_answer) == mathd_normalize_answer(ground_truth)


def grade_answer_sympy(given_answer: str, ground_truth: str) -> bool:
    gt, gv = _normalize(ground_truth), _normalize(given_answer)
    if gt is None or gv is None or not gv:
        return False
    if gt == gv:
        return True
    ge, ve = split_tuple(gt), split_tuple(gv)
    if len(ge) > 1 and (gt[0] != gv[0] or gt[-1] != gv[-1]):       # interval brackets must agree
        return False
    if len(ge) != len(ve):
        return False
    return all(_elements_equal(x, y) for x, y in zip(ge, ve))


def grade_answer(given_answer: Optional[str], ground_truth: Optional[str]) -> bool:
    if given_answer is None or ground_truth is None:
        return False
    na, nb = _to_number(given_answer), _to_number(ground_truth)     # before spaces go: "1 1/2" is a mixed number
    if na is not None and nb is not None:
        return na == nb
    return grade_answer_mathd(given_answer, ground_truth) or grade_answer_sympy(given_answer, ground_truth)
