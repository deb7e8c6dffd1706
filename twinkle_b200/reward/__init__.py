"""Rule-based rewards.

Parity: reference ``src/twinkle/reward/*.py`` — ``Reward.__call__(trajectories,
ground_truths) -> List[float]`` with GSM8K accuracy/format, generic math and
format rewards, an F1 reward and Countdown.
"""
from __future__ import annotations

import re
from collections import Counter
from typing import Any, Dict, List, Optional, Sequence


def _completion_text(traj) -> str:
    if isinstance(traj, str):
        return traj
    msgs = traj.get('messages', []) if isinstance(traj, dict) else []
    for m in reversed(msgs):
        if m.get('role') == 'assistant':
            c = m.get('content')
            return c if isinstance(c, str) else ' '.join(p.get('text', '') for p in c if isinstance(p, dict))
    return ''


_NUM = re.compile(r'-?\d[\d,]*\.?\d*')


def _norm_number(s: str) -> Optional[str]:
    m = _NUM.findall(s.replace('$', ''))
    if not m:
        return None
    v = m[-1].replace(',', '').rstrip('.')
    try:
        f = float(v)
        return str(int(f)) if f == int(f) else str(f)
    except ValueError:
        return None


def extract_boxed(text: str) -> Optional[str]:
    i = text.rfind('\\boxed{')
    if i < 0:
        return None
    depth, j = 0, i + 6
    for k in range(j, len(text)):
        if text[k] == '{':
            depth += 1
        elif text[k] == '}':
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
    return None


def safe_arithmetic(expr: str) -> float:
    """Value of an expression made of numbers, ``+ - * /``, unary minus and parentheses; anything else (names, calls,
    powers, attribute access) raises ``ValueError``. Model output is never handed to ``eval``."""
    import ast
    import operator as op
    ops = {ast.Add: op.add, ast.Sub: op.sub, ast.Mult: op.mul, ast.Div: op.truediv}

    def ev(n):
        if isinstance(n, ast.Expression):
            return ev(n.body)
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)) and not isinstance(n.value, bool):
            return float(n.value)
        if isinstance(n, ast.BinOp) and type(n.op) in ops:
            return ops[type(n.op)](ev(n.left), ev(n.right))
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, (ast.USub, ast.UAdd)):
            v = ev(n.operand)
            return -v if isinstance(n.op, ast.USub) else v
        raise ValueError(f'not plain arithmetic: {ast.dump(n)[:60]}')

    if len(expr) > 200:
        raise ValueError('expression too long')
    try:
        return ev(ast.parse(expr.strip(), mode='eval'))
    except (SyntaxError, ZeroDivisionError, RecursionError) as e:
        raise ValueError(str(e)) from None


class Reward:

    def __call__(self, trajectories: Sequence[Any], ground_truths: Optional[Sequence[Any]] = None, **kwargs) -> List[float]:  # pragma: no cover
        raise NotImplementedError


class GSM8KAccuracyReward(Reward):
    """1.0 when the last number after ``####`` (or the last number at all)
    equals the reference answer."""

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t, gt in zip(trajectories, ground_truths or [None] * len(trajectories)):
            text = _completion_text(t)
            tail = text.split('####')[-1] if '####' in text else (extract_boxed(text) or text)
            pred = _norm_number(tail)
            ref = _norm_number(str(gt).split('####')[-1]) if gt is not None else None
            out.append(1.0 if pred is not None and pred == ref else 0.0)
        return out


class GSM8KFormatReward(Reward):

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        return [1.0 if re.search(r'####\s*-?[\d,\.]+\s*$', _completion_text(t).strip()) else 0.0 for t in trajectories]


class FormatReward(Reward):
    """``<think>…</think>`` followed by ``<answer>…</answer>`` (or a custom regex)."""

    def __init__(self, pattern: str = r'^\s*<think>.*?</think>\s*<answer>.*?</answer>\s*$'):
        self.pattern = re.compile(pattern, re.S)

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        return [1.0 if self.pattern.match(_completion_text(t)) else 0.0 for t in trajectories]


class MathReward(Reward):
    """Boxed-answer exact match after light normalisation."""

    @staticmethod
    def _norm(s: str) -> str:
        s = s.strip().strip('$').replace(' ', '').replace('\\!', '').replace('dfrac', 'frac').replace('\\left', '').replace('\\right', '')
        n = _norm_number(s) if re.fullmatch(r'-?[\d,\.]+', s) else None
        return n if n is not None else s

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t, gt in zip(trajectories, ground_truths or []):
            pred = extract_boxed(_completion_text(t))
            ref = extract_boxed(str(gt)) or str(gt)
            out.append(1.0 if pred is not None and self._norm(pred) == self._norm(ref) else 0.0)
        return out


class F1Reward(Reward):

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t, gt in zip(trajectories, ground_truths or []):
            p, r = _completion_text(t).lower().split(), str(gt).lower().split()
            common = sum((Counter(p) & Counter(r)).values())
            if not common:
                out.append(0.0)
                continue
            pr, rc = common / len(p), common / len(r)
            out.append(2 * pr * rc / (pr + rc))
        return out


class CountdownReward(Reward):
    """Equation uses each given number once and evaluates to the target."""

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t, gt in zip(trajectories, ground_truths or []):
            m = re.search(r'<answer>(.*?)</answer>', _completion_text(t), re.S)
            ok = 0.0
            if m and isinstance(gt, dict):
                eq = m.group(1).strip().split('=')[0]
                if re.fullmatch(r'[\d\s\+\-\*/\(\)\.]+', eq):
                    nums = sorted(int(x) for x in re.findall(r'\d+', eq))
                    try:
                        if nums == sorted(gt['nums']) and abs(safe_arithmetic(eq) - gt['target']) < 1e-6:
                            ok = 1.0
                    except Exception:
                        ok = 0.0
            out.append(ok)
        return out


class OlympiadBenchReward(MathReward):
    pass


# ------------------------------------------------------------------------------------------------- graded math rewards
def _truth_of(traj, gts, i: int, key: str = 'ground_truth', default: Any = ''):
    """Ground truth for trajectory ``i``: the ``ground_truths`` argument when given, else ``user_data[key]`` (dict or a
    list of ``(key, value)`` pairs, the layout dataset rows use)."""
    if gts is not None and key == 'ground_truth':
        return gts[i]
    from ..data_format import user_data_get
    ud = traj.get('user_data') if isinstance(traj, dict) else None
    return user_data_get(ud, key, default)


def all_boxed(text: str) -> List[str]:
    """Contents of every ``\\boxed{…}`` in order (nested braces respected)."""
    out, i = [], 0
    while True:
        i = text.find('\\boxed{', i)
        if i < 0:
            return out
        depth, start = 0, i + 6
        for k in range(start, len(text)):
            if text[k] == '{':
                depth += 1
            elif text[k] == '}':
                depth -= 1
                if depth == 0:
                    out.append(text[start + 1:k])
                    break
        i = start


def normalize_math_answer(ans: str) -> str:
    """Canonical text of a short math answer: LaTeX wrappers (``\\text{}``, ``\\left``/``\\right``, ``$``, ``\\,`` …),
    units after ``\\text``, trailing periods and spaces removed; ``\\frac{a}{b}`` and ``a/b`` of integers → decimal
    string; ``\\dfrac``/``\\tfrac`` = ``\\frac``; thousands separators dropped."""
    a = str(ans).strip().strip('$').strip()
    a = re.sub(r'\\(?:text|mathrm|textbf|mathbf)\{([^{}]*)\}', r'\1', a)
    a = re.sub(r'\\(?:left|right|,|;|!|quad|qquad|displaystyle)', '', a)
    a = a.replace('\\dfrac', '\\frac').replace('\\tfrac', '\\frac').replace('\\%', '%').replace('^\\circ', '').replace('°', '')
    a = a.replace(' ', '').rstrip('.')
    m = re.fullmatch(r'(-?)\\frac\{(-?\d+)\}\{(-?\d+)\}', a) or re.fullmatch(r'(-?)(\d+)/(\d+)', a)
    if m and int(m.group(3)) != 0:
        v = int(m.group(2)) / int(m.group(3)) * (-1 if m.group(1) else 1)
        return repr(round(v, 10)).rstrip('0').rstrip('.') if v != int(v) else str(int(v))
    if re.fullmatch(r'-?\d{1,3}(?:,\d{3})+(?:\.\d+)?', a):
        a = a.replace(',', '')
    if re.fullmatch(r'-?\d+\.\d+', a):
        a = a.rstrip('0').rstrip('.')
    return a.lower()


def split_answers(gt: str) -> List[str]:
    """Top-level comma split: ``"(1,2),(3,4)"`` → ``["(1,2)", "(3,4)"]``."""
    parts, cur, depth = [], [], 0
    for ch in str(gt):
        if ch in '([{':
            depth += 1
        elif ch in ')]}':
            depth -= 1
        if ch == ',' and depth == 0:
            if cur:
                parts.append(''.join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    if cur:
        parts.append(''.join(cur).strip())
    return [p for p in parts if p]


def numeric_match(pred: str, gt: str, rel_tol: float = 0.01, abs_tol: float = 1e-4) -> bool:
    try:
        p, g = float(pred), float(gt)
    except (ValueError, OverflowError):
        return False
    if abs(p - g) < abs_tol:
        return True
    return abs(p) < rel_tol if g == 0 else abs(p - g) / abs(g) < rel_tol


def numeric_similarity(pred: str, gt: str, abs_tol: float = 1e-4) -> float:
    """1 for equal values, ``exp(−5·relative error)`` otherwise, 0 for non-numbers."""
    try:
        p, g = float(pred), float(gt)
    except (ValueError, OverflowError):
        return 0.0
    if abs(p - g) < abs_tol:
        return 1.0
    if g == 0:
        return 1.0 if abs(p) < 0.01 else 0.0
    import math
    return math.exp(-5 * abs(p - g) / abs(g))


class OlympiadBenchAccuracyReward(Reward):
    """1.0 for a matching final ``\\boxed`` answer (text-equal after normalisation, or numerically within 1 %); a wrong
    but numerically close answer earns ``0.99·exp(−5·rel.err)``. With ``user_data['is_multiple_answer']`` the score is the
    share of reference answers found among all boxed answers. Reference: ``reward/olympiad_bench.py:241-289``."""

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for i, t in enumerate(trajectories):
            boxed = all_boxed(_completion_text(t))
            gt = str(_truth_of(t, ground_truths, i) or '')
            gt = extract_boxed(gt) or gt
            if not boxed or not gt:
                out.append(0.0)
                continue
            refs = [normalize_math_answer(g) for g in split_answers(gt)]
            if not _truth_of(t, None, i, 'is_multiple_answer', False):
                pred, ref = normalize_math_answer(boxed[-1]), refs[0] if refs else ''
                out.append(1.0 if pred == ref or pred == normalize_math_answer(gt) or numeric_match(pred, ref) else 0.99 * numeric_similarity(pred, ref))
            else:
                preds = [normalize_math_answer(p) for b in boxed for p in (split_answers(b) or [b])]
                hit = sum(1 for r in refs if any(p == r or numeric_match(p, r) for p in preds))
                out.append(hit / len(refs) if refs else 0.0)
        return out


class OlympiadBenchFormatReward(Reward):
    """0.4 for having a boxed answer, +0.3 when the last one starts within the final 200 characters, +0.3 when all
    boxed answers agree, −0.3 when more than two different ones appear; clamped to [0, 1]."""

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t in trajectories:
            text = _completion_text(t)
            boxed, score = all_boxed(text), 0.0
            if boxed:
                score = 0.4
                if len(text) - text.rfind('\\boxed{') < 200:
                    score += 0.3
                distinct = {normalize_math_answer(b) for b in boxed}
                score += 0.3 if len(distinct) == 1 else (-0.3 if len(distinct) > 2 else 0.0)
            out.append(max(0.0, min(1.0, score)))
        return out


class OlympiadBenchQualityReward(Reward):
    """``0.4·reasoning + 0.3·length + 0.3·non-repetition``. Reasoning: a quarter each for ≥ 3 single ``=`` signs, ≥ 5
    operators, step/connective words, and a conclusion word followed by the boxed answer in the last 500 characters.
    Length: ramps up to 1 at 300 characters, stays 1 to 1500, eases down to 0.5 at 3000 and 0.25 at 6000. Repetition:
    mean share of distinct 50-character windows (stride 25) and distinct word 4-grams."""

    _STEPS = re.compile(r'第[一二三四五六七八九十\d]+步|step\s*\d+|首先|其次|然后|最后|因此|所以|\b(?:first|then|finally|therefore|hence)\b', re.I)
    _CONCLUDE = re.compile(r'(?:所以|因此|答案|故|得|thus|therefore|answer).*\\boxed', re.I | re.S)

    def reasoning(self, text: str) -> float:
        s = 0.25 * (len(re.findall(r'(?<![=!<>])=(?!=)', text)) >= 3)
        s += 0.25 * (len(re.findall(r'[+\-*/^]|\\frac|\\sqrt', text)) >= 5)
        s += 0.25 * bool(self._STEPS.search(text))
        s += 0.25 * bool(self._CONCLUDE.search(text[-500:]))
        return float(s)

    @staticmethod
    def length(n: int) -> float:
        import math
        if n < 100:
            return 0.3 * n / 100
        if n < 300:
            return 0.3 + 0.7 * (n - 100) / 200
        if n <= 1500:
            return 1.0
        if n <= 3000:
            return 0.5 + 0.5 * math.cos((n - 1500) / 1500 * math.pi / 2)
        return 0.5 * (1 - 0.5 * min((n - 3000) / 3000, 1.0))

    @staticmethod
    def non_repetition(text: str) -> float:
        if len(text) < 100:
            return 1.0
        windows = [text[i:i + 50] for i in range(0, len(text) - 50, 25)]
        w = len(set(windows)) / len(windows) if windows else 1.0
        words = text.split()
        grams = [' '.join(words[i:i + 4]) for i in range(len(words) - 3)]
        g = len(set(grams)) / len(grams) if grams else 1.0
        return (w + g) / 2

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for t in trajectories:
            text = _completion_text(t)
            out.append(0.4 * self.reasoning(text) + 0.3 * self.length(len(text)) + 0.3 * self.non_repetition(text))
        return out


class MultiModalAccuracyReward(Reward):
    """Visual question answering (CLEVR-style): the text inside ``<answer>…</answer>`` against the ground truth —
    equal ignoring case and surrounding space, numerically equal, or (for a ``solution`` that itself carries
    ``<answer>`` tags) equal to that tag's content. Reference: ``reward/mm_reward.py:8-70`` (its optional symbolic
    check through ``math_verify`` is replaced by the numeric comparison; that package is not available)."""

    @staticmethod
    def extract_answer(text: str) -> str:
        m = re.search(r'<answer>\s*(.*?)\s*</answer>', text or '', re.S)
        return m.group(1).strip() if m else ''

    def __call__(self, trajectories, ground_truths=None, **kwargs):
        out = []
        for i, t in enumerate(trajectories):
            pred = self.extract_answer(_completion_text(t))
            gt = str(_truth_of(t, ground_truths, i) or '')
            sol = str(_truth_of(t, None, i, 'solution', '') or '')
            refs = [r for r in (self.extract_answer(gt) or gt, self.extract_answer(sol) or sol) if r]
            ok = bool(pred) and any(pred.lower() == r.strip().lower() or numeric_match(normalize_math_answer(pred), normalize_math_answer(r), 1e-6, 1e-9)
                                    for r in refs)
            out.append(1.0 if ok else 0.0)
        return out


reward_mapping = {c.__name__: c for c in (GSM8KAccuracyReward, GSM8KFormatReward, FormatReward, MathReward, F1Reward,
                                          CountdownReward, OlympiadBenchReward, OlympiadBenchAccuracyReward, OlympiadBenchFormatReward,
                                          OlympiadBenchQualityReward, MultiModalAccuracyReward)}
__all__ = ['Reward', 'reward_mapping', 'safe_arithmetic', 'all_boxed', 'normalize_math_answer', 'split_answers', 'numeric_match', 'numeric_similarity'] + list(reward_mapping)
