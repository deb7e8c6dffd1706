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
                        if nums == sorted(gt['nums']) and abs(eval(eq, {'__builtins__': {}}) - gt['target']) < 1e-6:
                            ok = 1.0
                    except Exception:
                        ok = 0.0
            out.append(ok)
        return out


class OlympiadBenchReward(MathReward):
    pass


reward_mapping = {c.__name__: c for c in (GSM8KAccuracyReward, GSM8KFormatReward, FormatReward, MathReward, F1Reward,
                                          CountdownReward, OlympiadBenchReward)}
__all__ = ['Reward', 'reward_mapping'] + list(reward_mapping)
