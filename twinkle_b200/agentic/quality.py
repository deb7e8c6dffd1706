"""Router sampler, answer-overlap rewards and trajectory quality filters.

What it covers: reference ``src/twinkle_agentic/sampler/router_sampler.py``, ``reward/f1.py`` and the rule-based
members of ``preprocessor/`` (dedup, refusal, dead-loop, token-soup, hard limits, score threshold, PII, message
sanity / normalisation).  These are ``DataFilter`` objects (``keep(row) -> bool``).  The steps that rewrite rows, call a
language model or score rounds from log-probabilities live in ``preprocess.py`` and ``pii.py``.
"""
from __future__ import annotations

import hashlib
import math
import re
from collections import Counter
from typing import Any, Callable, Dict, List, Optional, Sequence

from ..data_format.sampling import SampleResponse, SamplingParams
from ..data_format.types import Trajectory
from ..preprocessor import DataFilter
from ..reward import Reward


# ------------------------------------------------------------------------------------------------- router sampler
class RouterSampler:
    """Samples from a cheap policy first and re-samples a sequence with a fallback (a larger policy or a chat API)
    when the cheap draw looks unreliable: mean token log-prob below ``min_mean_logp`` or mean top-k entropy above
    ``max_entropy``."""

    def __init__(self, primary, fallback, min_mean_logp: float = -1.5, max_entropy: float = 2.5, topk: int = 5):
        self.primary, self.fallback = primary, fallback
        self.min_mean_logp, self.max_entropy, self.topk = min_mean_logp, max_entropy, topk
        self.routed = 0

    @property
    def template(self):
        return getattr(self.primary, 'template', None)

    def set_template(self, *a, **kw):
        self.primary.set_template(*a, **kw)
        if hasattr(self.fallback, 'set_template'):
            self.fallback.set_template(*a, **kw)

    @staticmethod
    def entropy_from_topk(topk_logprobs) -> float:
        ents = []
        for row in topk_logprobs or []:
            ps = [math.exp(lp) for _, lp in row]
            rest = max(0.0, 1.0 - sum(ps))
            ent = -sum(p * math.log(p) for p in ps if p > 0) - (rest * math.log(rest) if rest > 1e-9 else 0.0)
            ents.append(ent)
        return sum(ents) / len(ents) if ents else 0.0

    def should_route(self, seq) -> bool:
        if seq.logprobs and sum(seq.logprobs) / max(len(seq.logprobs), 1) < self.min_mean_logp:
            return True
        return bool(seq.topk_logprobs) and self.entropy_from_topk(seq.topk_logprobs) > self.max_entropy

    def sample(self, inputs, sampling_params: Optional[SamplingParams] = None, **kwargs) -> List[SampleResponse]:
        sp = sampling_params or SamplingParams()
        if getattr(sp, 'logprobs', None) in (None, 0):
            sp = SamplingParams.from_dict({**sp.to_dict(), 'logprobs': self.topk})
        resps = self.primary.sample(inputs, sp, **kwargs)
        if callable(resps):
            resps = resps()
        redo = [i for i, r in enumerate(resps) if any(self.should_route(s) for s in r.sequences)]
        if redo:
            self.routed += len(redo)
            again = self.fallback.sample([inputs[i] for i in redo], sampling_params, **kwargs)
            if callable(again):
                again = again()
            for i, r in zip(redo, again):
                resps[i] = r
        return resps


# ------------------------------------------------------------------------------------------------------- rewards
_ANSWER = re.compile(r'<answer>(.*?)</answer>', re.S | re.I)


def _final_answer(text: str, pattern=None) -> str:
    m = list((pattern or _ANSWER).finditer(text or ''))
    if m:
        return m[-1].group(1).strip()
    boxed = re.findall(r'\\boxed\{([^{}]*)\}', text or '')
    if boxed:
        return boxed[-1].strip()
    lines = [l for l in (text or '').strip().splitlines() if l.strip()]
    return lines[-1].strip() if lines else ''


def _norm_tokens(s: str) -> List[str]:
    s = re.sub(r'\b(a|an|the)\b', ' ', s.lower())
    s = re.sub(r'[^\w\s]', ' ', s)
    return [re.sub(r'(ing|ed|es|s)$', '', t) if len(t) > 3 else t for t in s.split()]


def f1_score(prediction: str, gold: str) -> float:
    p, g = _norm_tokens(prediction), _norm_tokens(gold)
    if not p or not g:
        return float(p == g)
    common = sum((Counter(p) & Counter(g)).values())
    if common == 0:
        return 0.0
    pr, rc = common / len(p), common / len(g)
    return 2 * pr * rc / (pr + rc)


def _last_assistant(traj: Dict[str, Any]) -> str:
    for m in reversed(traj.get('messages', [])):
        if m.get('role') == 'assistant' and isinstance(m.get('content'), str):
            return m['content']
    return ''


def _gold(traj: Dict[str, Any], gt) -> str:
    if gt is not None:
        return str(gt)
    ud = traj.get('user_data')
    if isinstance(ud, dict):
        for k in ('ground_truth', 'answer', 'solution'):
            if k in ud:
                return str(ud[k])
    return ''


class F1Reward(Reward):
    """Token-level F1 between the final answer of the last assistant turn and the reference (best over a list)."""

    def __init__(self, answer_pattern=None):
        self.pattern = re.compile(answer_pattern, re.S) if isinstance(answer_pattern, str) else answer_pattern

    def __call__(self, trajectories, ground_truths=None, **kwargs) -> List[float]:
        out = []
        for t, gt in zip(trajectories, ground_truths or [None] * len(trajectories)):
            pred = _final_answer(_last_assistant(t), self.pattern)
            golds = gt if isinstance(gt, (list, tuple)) else [_gold(t, gt)]
            out.append(max((f1_score(pred, str(g)) for g in golds), default=0.0))
        return out


class CoTReward(Reward):
    """1.0 when the turn shows reasoning before the answer (a think block or ≥ 2 sentences ahead of ``<answer>``)."""

    def __call__(self, trajectories, ground_truths=None, **kwargs) -> List[float]:
        out = []
        for t in trajectories:
            text = _last_assistant(t)
            m = _ANSWER.search(text)
            before = text[:m.start()] if m else ''
            ok = bool(m) and ('</think>' in before or len(re.findall(r'[.!?]\s', before)) >= 2)
            out.append(1.0 if ok else 0.0)
        return out


class ToolExploreReward(Reward):
    """Rewards distinct, successful tool use on trajectories whose answer is already good (F1 ≥ threshold)."""

    def __init__(self, f1_threshold: float = 0.5, answer_pattern=None, bonus_per_tool: float = 0.1, cap: float = 0.3):
        self.f1, self.threshold, self.bonus, self.cap = F1Reward(answer_pattern), f1_threshold, bonus_per_tool, cap

    def __call__(self, trajectories, ground_truths=None, **kwargs) -> List[float]:
        base = self.f1(trajectories, ground_truths)
        out = []
        for t, b in zip(trajectories, base):
            if b < self.threshold:
                out.append(0.0)
                continue
            ok_ids = {m.get('tool_call_id') for m in t.get('messages', []) if m.get('role') == 'tool' and not str(m.get('content', '')).startswith('Error')}
            names = {c.get('tool_name') for m in t.get('messages', []) for c in (m.get('tool_calls') or []) if c.get('id') in ok_ids}
            out.append(min(self.cap, self.bonus * len(names)))
        return out


# ------------------------------------------------------------------------------------------------------- filters
def _text(traj: Dict[str, Any], roles=('assistant', )) -> str:
    return '\n'.join(m['content'] for m in traj.get('messages', []) if m.get('role') in roles and isinstance(m.get('content'), str))


class DedupFilter(DataFilter):
    """Drops exact and near duplicates (same set of hashed word 5-grams up to ``threshold`` Jaccard)."""

    def __init__(self, threshold: float = 0.9, roles=('user', 'assistant')):
        self.threshold, self.roles, self._seen_exact, self._sigs = threshold, roles, set(), []

    def _sig(self, text: str) -> frozenset:
        w = text.lower().split()
        grams = [' '.join(w[i:i + 5]) for i in range(max(len(w) - 4, 1))]
        hs = sorted(int(hashlib.md5(g.encode()).hexdigest()[:8], 16) for g in grams)
        return frozenset(hs[:64])  # bottom-k sketch

    def keep(self, row) -> bool:
        text = _text(row, self.roles)
        h = hashlib.sha1(text.encode()).hexdigest()
        if h in self._seen_exact:
            return False
        sig = self._sig(text)
        for s in self._sigs:
            inter = len(sig & s)
            if inter and inter / len(sig | s) >= self.threshold:
                return False
        self._seen_exact.add(h)
        self._sigs.append(sig)
        return True


class RefuseFilter(DataFilter):
    PATTERNS = re.compile(r"\b(i can(?:'|no)t (?:help|assist|comply)|i'm sorry,? but|as an ai(?: language model)?|i am unable to|i won't be able to)\b", re.I)

    def keep(self, row) -> bool:
        return not self.PATTERNS.search(_text(row)[:600])


class DeadLoopFilter(DataFilter):
    """Drops trajectories that repeat themselves: a line repeated ≥ ``max_repeat`` times, the same tool call issued
    ≥ ``max_repeat`` times in a row, or a long suffix made of one repeated n-gram."""

    def __init__(self, max_repeat: int = 4):
        self.max_repeat = max_repeat

    def keep(self, row) -> bool:
        lines = [l.strip() for l in _text(row).splitlines() if len(l.strip()) > 10]
        if lines and max(Counter(lines).values()) >= self.max_repeat:
            return False
        calls = [(c.get('tool_name'), str(c.get('arguments'))) for m in row.get('messages', []) for c in (m.get('tool_calls') or [])]
        run = 1
        for a, b in zip(calls, calls[1:]):
            run = run + 1 if a == b else 1
            if run >= self.max_repeat:
                return False
        words = _text(row).split()[-200:]
        for n in (1, 2, 3, 4):
            if len(words) >= n * self.max_repeat * 2:
                tail = words[-n * self.max_repeat * 2:]
                if all(tail[i] == tail[i % n] for i in range(len(tail))):
                    return False
        return True


class TokenSoupFilter(DataFilter):
    """Drops degenerate text: too few distinct words, too many non-word characters, or extremely long 'words'."""

    def __init__(self, min_distinct_ratio: float = 0.15, max_symbol_ratio: float = 0.4, max_word_len: int = 80):
        self.min_distinct, self.max_symbol, self.max_word_len = min_distinct_ratio, max_symbol_ratio, max_word_len

    def keep(self, row) -> bool:
        text = _text(row)
        if not text:
            return True
        words = text.split()
        if len(words) >= 50 and len(set(words)) / len(words) < self.min_distinct:
            return False
        sym = sum(1 for ch in text if not (ch.isalnum() or ch.isspace()))
        if sym / len(text) > self.max_symbol:
            return False
        return not any(len(w) > self.max_word_len and '://' not in w for w in words)


class HardFilter(DataFilter):
    """Structural limits: turn count, characters, presence of an assistant turn, optional required/forbidden regexes."""

    def __init__(self, max_messages: int = 200, max_chars: int = 200000, min_assistant_chars: int = 1, require: Optional[str] = None, forbid: Optional[str] = None):
        self.max_messages, self.max_chars, self.min_assistant = max_messages, max_chars, min_assistant_chars
        self.require, self.forbid = (re.compile(require, re.S) if require else None), (re.compile(forbid, re.S) if forbid else None)

    def keep(self, row) -> bool:
        msgs = row.get('messages', [])
        if not msgs or len(msgs) > self.max_messages:
            return False
        total = sum(len(m.get('content', '')) for m in msgs if isinstance(m.get('content', ''), str))
        a = _text(row)
        if total > self.max_chars or len(a) < self.min_assistant:
            return False
        if self.require and not self.require.search(a):
            return False
        return not (self.forbid and self.forbid.search(a))


class ScoreFilter(DataFilter):
    """Keeps rows whose score — ``user_data[key]`` or ``score_fn(row)`` (an LLM judge, a reward model, …) — reaches ``min_score``."""

    def __init__(self, min_score: float, key: str = 'score', score_fn: Optional[Callable[[Dict[str, Any]], float]] = None):
        self.min_score, self.key, self.score_fn = min_score, key, score_fn

    def keep(self, row) -> bool:
        if self.score_fn is not None:
            return float(self.score_fn(row)) >= self.min_score
        ud = row.get('user_data')
        return isinstance(ud, dict) and float(ud.get(self.key, float('-inf'))) >= self.min_score


class PIIFilter(DataFilter):
    """Regex detector for e-mail addresses, phone numbers, payment-card-like digit runs and IPv4 addresses; either drops
    the row or masks the spans in place (``mask=True``)."""

    PATTERNS = {
        'email': re.compile(r'\b[\w.+-]+@[\w-]+\.[\w.-]+\b'),
        'phone': re.compile(r'(?<!\d)(?:\+?\d{1,3}[ -]?)?(?:\(?\d{3}\)?[ -]?)\d{3}[ -]?\d{4}(?!\d)'),
        'card': re.compile(r'(?<!\d)(?:\d[ -]?){13,16}(?!\d)'),
        'ipv4': re.compile(r'(?<!\d)(?:\d{1,3}\.){3}\d{1,3}(?!\d)'),
    }

    def __init__(self, mask: bool = False):
        self.mask = mask

    def keep(self, row) -> bool:
        hit = False
        for m in row.get('messages', []):
            c = m.get('content')
            if not isinstance(c, str):
                continue
            for name, pat in self.PATTERNS.items():
                if pat.search(c):
                    hit = True
                    if self.mask:
                        c = pat.sub(f'<{name}>', c)
            if self.mask:
                m['content'] = c
        return True if self.mask else not hit


class MessageSanityFilter(DataFilter):
    """Role order and tool-call bookkeeping: starts with system/user, no two user turns in a row without an assistant
    turn between them, every tool message answers an earlier tool call, ends on an assistant turn."""

    def keep(self, row) -> bool:
        msgs = row.get('messages', [])
        if not msgs or msgs[0].get('role') not in ('system', 'user'):
            return False
        open_calls, prev = set(), None
        for m in msgs:
            r = m.get('role')
            if r not in ('system', 'user', 'assistant', 'tool'):
                return False
            if r == 'user' and prev == 'user':
                return False
            if r == 'assistant':
                open_calls |= {c.get('id') for c in (m.get('tool_calls') or [])}
            if r == 'tool':
                tid = m.get('tool_call_id')
                if tid and tid not in open_calls:
                    return False
            prev = r
        return msgs[-1].get('role') == 'assistant'


def normalize_messages(traj: Trajectory) -> Trajectory:
    """Canonical form: string contents, roles lower-cased, ``function``-style tool calls mapped to ``tool_name`` /
    ``arguments``, empty system prompts dropped, consecutive same-role text turns merged."""
    out: List[Dict[str, Any]] = []
    for m in traj.get('messages', []):
        m = dict(m)
        m['role'] = str(m.get('role', '')).lower()
        c = m.get('content')
        if isinstance(c, list):
            m['content'] = ''.join(p.get('text', '') for p in c if isinstance(p, dict))
        elif c is None:
            m['content'] = ''
        calls = []
        for tc in m.get('tool_calls') or []:
            fn = tc.get('function') or {}
            calls.append({'id': tc.get('id', ''), 'type': 'function', 'tool_name': tc.get('tool_name') or fn.get('name'),
                          'arguments': tc.get('arguments', fn.get('arguments', {}))})
        if calls:
            m['tool_calls'] = calls
        if m['role'] == 'system' and not m['content'].strip():
            continue
        if out and out[-1]['role'] == m['role'] and m['role'] in ('user', 'assistant') and not calls and not out[-1].get('tool_calls'):
            out[-1]['content'] += '\n' + m['content']
            continue
        out.append(m)
    res = dict(traj)
    res['messages'] = out
    return res
