"""Answer-accuracy rewards (trl/rewards/accuracy_rewards.py:28-350).

The reference parses LaTeX with ``math_verify``; when that package is importable it is used here too.
Otherwise a built-in normaliser handles the common cases: ``\\boxed{...}``, ``$...$``, ``\\frac{a}{b}``,
decimals, percentages, thousands separators and plain strings.  As in the reference, a gold answer that
cannot be parsed yields ``None`` (the sample is skipped by the trainers) and extra columns can be logged
through ``log_extra``.
"""
from __future__ import annotations

import math
import re
from fractions import Fraction

try:  # pragma: no cover - optional
    from math_verify import LatexExtractionConfig, NormalizationConfig, parse as _mv_parse, verify as _mv_verify

    _HAS_MV = True
except Exception:
    _HAS_MV = False


def _last_boxed(text: str):
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth, k = 0, j
    while k < len(text):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
        k += 1
    return None


_FRAC = re.compile(r"\\d?frac\s*\{([^{}]+)\}\s*\{([^{}]+)\}")


def _normalise(expr: str):
    """-> Fraction for numeric answers, else a canonical string; None if empty."""
    s = expr.strip().strip("$").strip()
    s = re.sub(r"\\left|\\right|\\!|\\,|\;|\\ |\s+", "", s)
    s = re.sub(r"\\text\{([^{}]*)\}", r"\1", s).rstrip(".")
    if not s:
        return None
    t = s.replace(",", "")
    pct = t.endswith("\\%") or t.endswith("%")
    t = t.rstrip("%").rstrip("\\")
    m = _FRAC.fullmatch(t.lstrip("-"))
    try:
        if m:
            v = Fraction(m.group(1)) / Fraction(m.group(2))
            v = -v if t.startswith("-") else v
        elif re.fullmatch(r"-?\d+/\d+", t):
            v = Fraction(t)
        else:
            v = Fraction(t)
        return v / 100 if pct else v
    except (ValueError, ZeroDivisionError):
        return s.lower()


def _extract(text: str, require_marker: bool):
    b = _last_boxed(text)
    if b is not None:
        return _normalise(b)
    m = re.findall(r"\$([^$]+)\$", text)
    if m:
        return _normalise(m[-1])
    return None if require_marker else _normalise(text)


def _verify_builtin(content: str, gold: str):
    g = _extract(gold, require_marker=False)
    if g is None:
        return None
    if isinstance(g, str) and _last_boxed(gold) is None and "$" not in gold and not re.search(r"[\d\\^_=+*/<>]", gold):
        return None  # plain words: nothing a math parser would extract, the sample is skipped
    a = _extract(content, require_marker=True)
    if a is None:
        return 0.0
    if isinstance(g, Fraction) and isinstance(a, Fraction):
        return float(g == a or math.isclose(float(g), float(a), rel_tol=1e-9, abs_tol=1e-12))
    return float(str(g) == str(a))


def accuracy_reward(completions: list, solution: list[str], log_extra=None, **kwargs) -> list:
    """1.0 if the (last boxed / math-mode) answer of the completion equals the gold solution, 0.0 if not,
    ``None`` if the gold solution cannot be parsed."""
    contents = [c[0]["content"] if isinstance(c, list) else c for c in completions]
    rewards = []
    for content, sol in zip(contents, solution):
        if _HAS_MV:
            gold = _mv_parse(sol)
            if len(gold) == 0:
                rewards.append(None)
                continue
            ans = _mv_parse(content, extraction_config=[LatexExtractionConfig(
                normalization_config=NormalizationConfig(units=True), boxed_match_priority=0,
                try_extract_without_anchor=False)], extraction_mode="first_match")
            try:
                rewards.append(float(_mv_verify(gold, ans)))
            except Exception:
                rewards.append(None)
        else:
            rewards.append(_verify_builtin(content, sol))
    if log_extra is not None:
        log_extra("gold_answer", list(solution))
    return rewards


def reasoning_accuracy_reward(completions: list, solution: list[str], reasoning_delimiters=None, **kwargs) -> list:
    """Accuracy on the text after the reasoning block (default delimiter ``</think>``); 0.0 when the
    delimiter is missing, i.e. the reasoning was never closed."""
    delims = reasoning_delimiters or ["</think>"]
    contents = [c[0]["content"] if isinstance(c, list) else c for c in completions]
    finals, closed = [], []
    for text in contents:
        cut = None
        for d in delims:
            i = text.rfind(d)
            if i >= 0:
                cut = max(cut or 0, i + len(d))
        closed.append(cut is not None)
        finals.append(text[cut:] if cut is not None else "")
    base = accuracy_reward([[{"content": f}] for f in finals], solution)
    return [r if r is None else (r if ok else 0.0) for r, ok in zip(base, closed)]


class _CosineScaledReward:
    __name__ = "cosine_scaled_reward"

    def __init__(self, max_len, min_value_wrong, max_value_wrong, min_value_correct, max_value_correct):
        self.max_len = max_len
        self.min_value_wrong, self.max_value_wrong = min_value_wrong, max_value_wrong
        self.min_value_correct, self.max_value_correct = min_value_correct, max_value_correct

    def __call__(self, completions, solution, completion_ids, **kwargs):
        out = []
        for ok, ids in zip(accuracy_reward(completions, solution), completion_ids):
            if ok is None:
                out.append(None)
                continue
            c = math.cos(min(len(ids) / self.max_len, 1.0) * math.pi)
            lo, hi = (self.min_value_correct, self.max_value_correct) if ok else (self.max_value_wrong, self.min_value_wrong)
            out.append(float(lo + 0.5 * (hi - lo) * (1.0 + c)))
        return out


def get_cosine_scaled_reward(max_len: int = 1000, min_value_wrong: float = -1.0, max_value_wrong: float = -0.5,
                             min_value_correct: float = 0.5, max_value_correct: float = 1.0):
    """Length-aware accuracy: short correct answers score highest, short wrong answers lowest."""
    return _CosineScaledReward(max_len, min_value_wrong, max_value_wrong, min_value_correct, max_value_correct)
