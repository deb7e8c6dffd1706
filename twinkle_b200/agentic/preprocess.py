"""Trajectory-quality pipeline steps that return ``(kept, dropped)``: text clean-up mappers, character/token-count
filters, a model-family allow list, a heuristic intent classifier, LLM back ends (OpenAI-compatible HTTP or an
in-process sampler) and per-round difficulty scorers built on prompt log-probabilities.

Parity: reference ``src/twinkle_agentic/preprocessor/{__init__,data_juicer,model_filter,intent_classifier,llm_backend,
score_filter,message_normalizer}.py``. The reference delegates the text operators to the ``data_juicer`` package and
tokenisation to a hub tokenizer; neither is available offline, so the operators are restated here on the standard library
and the token counter is pluggable (a tokenizer object, a callable, or a whitespace/CJK-aware fallback)."""
from __future__ import annotations

import json
import math
import os
import re
import time
import unicodedata
from abc import ABC, abstractmethod
from collections import Counter
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Protocol, Sequence, Set, Tuple

from ..preprocessor import Preprocessor
from ..utils.logger import get_logger
from .quality import normalize_messages

logger = get_logger()

Rows = List[Dict[str, Any]]
Step = Tuple[Rows, Rows]


def _content_text(msg: Dict[str, Any]) -> str:
    c = msg.get('content')
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        return ''.join(p.get('text', '') for p in c if isinstance(p, dict))
    return ''


def _role_text(row: Dict[str, Any], role: str) -> str:
    return ' '.join(_content_text(m) for m in (row.get('messages') or []) if isinstance(m, dict) and m.get('role') == role)


def _map_role_text(rows: Rows, role: str, fn: Callable[[str], str]) -> None:
    """Apply ``fn`` to every string content of ``role``; list-of-parts contents are left untouched."""
    for row in rows:
        for m in row.get('messages') or []:
            if isinstance(m, dict) and m.get('role') == role and isinstance(m.get('content'), str):
                m['content'] = fn(m['content'])


def _split(rows: Rows, keep: Sequence[bool], reason: str) -> Step:
    kept, dropped = [], []
    for r, k in zip(rows, keep):
        (kept if k else dropped).append(r if k else dict(r, drop_reason=reason))
    return kept, dropped


# ----------------------------------------------------------------------------------------------- text operators
_MOJIBAKE = {'â€™': '’', 'â€œ': '“', 'â€\x9d': '”', 'â€“': '–', 'â€”': '—', 'â€¦': '…', 'Ã©': 'é', 'Ã¨': 'è', 'Ã¼': 'ü', 'Ã¶': 'ö',
             'Ã¤': 'ä', 'Ã±': 'ñ', 'Â\xa0': ' ', 'Â·': '·'}


class FixUnicodeFilter(Preprocessor):
    """Mapper: repairs common UTF-8-read-as-Latin-1 sequences, removes control characters other than tab/newline and
    normalises to ``normalization`` (NFC by default). Drops nothing."""

    def __init__(self, normalization: str = 'NFC', role: str = 'assistant'):
        if normalization.upper() not in ('NFC', 'NFKC', 'NFD', 'NFKD'):
            raise ValueError(f'unknown normalisation form {normalization!r}')
        self.normalization, self.role = normalization.upper(), role

    def fix(self, text: str) -> str:
        if 'Ã' in text or 'â€' in text or 'Â' in text:
            try:  # whole-string round trip succeeds when the text is uniformly mis-decoded
                text = text.encode('latin-1').decode('utf-8')
            except (UnicodeEncodeError, UnicodeDecodeError):
                for bad, good in _MOJIBAKE.items():
                    text = text.replace(bad, good)
        text = ''.join(ch for ch in text if ch in '\t\n\r' or unicodedata.category(ch) not in ('Cc', 'Cf') or ch == '‍')
        return unicodedata.normalize(self.normalization, text)

    def __call__(self, rows: Rows) -> Step:
        rows = list(rows)
        _map_role_text(rows, self.role, self.fix)
        return rows, []


_SENT_SPLIT = re.compile(r'(?<=[.!?。！？；;\n])')


class RemoveRepeatSentencesFilter(Preprocessor):
    """Mapper: removes a sentence that already appeared earlier in the same message (comparison optionally lower-cased
    and with punctuation/space ignored). Sentences shorter than ``min_repeat_sentence_length`` characters are kept, so
    short answers such as "Yes." survive. Drops nothing."""

    def __init__(self, lowercase: bool = False, ignore_special_character: bool = True, min_repeat_sentence_length: int = 2,
                 role: str = 'assistant'):
        self.lowercase, self.ignore, self.min_len, self.role = lowercase, ignore_special_character, min_repeat_sentence_length, role

    def _key(self, s: str) -> str:
        s = s.strip()
        if self.lowercase:
            s = s.lower()
        if self.ignore:
            s = ''.join(ch for ch in s if ch.isalnum())
        return s

    def dedup(self, text: str) -> str:
        out_lines = []
        seen: Set[str] = set()
        for line in text.split('\n'):
            kept = []
            for sent in _SENT_SPLIT.split(line):
                if not sent:
                    continue
                k = self._key(sent)
                if len(k) >= self.min_len and k in seen:
                    continue
                if len(k) >= self.min_len:
                    seen.add(k)
                kept.append(sent)
            out_lines.append(''.join(kept))
        return '\n'.join(out_lines)

    def __call__(self, rows: Rows) -> Step:
        rows = list(rows)
        _map_role_text(rows, self.role, self.dedup)
        return rows, []


def special_char_ratio(text: str) -> float:
    """Share of characters that are neither letters, digits (any script) nor white space."""
    if not text:
        return 0.0
    return sum(1 for ch in text if not (ch.isalnum() or ch.isspace())) / len(text)


class SpecialCharsFilter(Preprocessor):
    """Drops rows whose ``role`` text has more than ``max_ratio`` special characters; rows without such text pass."""

    def __init__(self, max_ratio: float = 0.25, role: str = 'assistant'):
        self.max_ratio, self.role = max_ratio, role

    def __call__(self, rows: Rows) -> Step:
        rows = list(rows)
        texts = [_role_text(r, self.role) for r in rows]
        return _split(rows, [not t.strip() or special_char_ratio(t) <= self.max_ratio for t in texts], 'special_chars_ratio')


_FALLBACK_TOKEN = re.compile(r'[一-鿿぀-ヿ가-힯]|[A-Za-z0-9_]+|[^\sA-Za-z0-9_]')


def count_tokens(text: str, tokenizer: Any = None) -> int:
    """Token count through ``tokenizer`` (callable returning ids or a mapping with ``input_ids``, or an object with
    ``encode``); without one, words / CJK characters / punctuation marks are counted."""
    if tokenizer is None:
        return len(_FALLBACK_TOKEN.findall(text))
    if hasattr(tokenizer, 'encode'):
        try:
            return len(tokenizer.encode(text, add_special_tokens=False))
        except TypeError:
            return len(tokenizer.encode(text))
    out = tokenizer(text)
    if isinstance(out, dict) or hasattr(out, 'keys'):
        out = out['input_ids']
    return len(out)


class TokenNumFilter(Preprocessor):
    """Keeps rows whose ``role`` text has between ``min_num`` and ``max_num`` tokens (inclusive)."""

    def __init__(self, tokenizer: Any = None, min_num: int = 10, max_num: int = 8192, role: str = 'assistant'):
        self.tokenizer, self.min_num, self.max_num, self.role = tokenizer, min_num, max_num, role

    def __call__(self, rows: Rows) -> Step:
        rows = list(rows)
        n = [count_tokens(_role_text(r, self.role), self.tokenizer) for r in rows]
        return _split(rows, [self.min_num <= k <= self.max_num for k in n], 'token_count_out_of_range')


# ------------------------------------------------------------------------------------------------ model allow list
_DEFAULT_FAMILIES = (r'minimax/minimax-m[23][\d.]*', r'opengvlab/internvl[\d._]+-2\d{2}b', r'qwen/qwen3[\d.]*-[123]\d{2}b(?:-a\d+b)?',
                     r'qwen/qwen3-coder', r'xiaomimimo/mimo-v[\d.]+', r'(?:zhipuai|z-ai)/glm-[56][\d.]*', r'deepseek-ai/deepseek-(?:r1|v[34])',
                     r'moonshotai/kimi', r'stepfun-ai/step')


class ModelFilter(Preprocessor):
    """Keeps rows whose ``field`` (the id of the model that produced the row) belongs to an allowed family; each pattern
    is a prefix, any ``-Variant.Suffix`` tail is accepted, matching ignores case."""

    def __init__(self, patterns: Optional[Sequence[str]] = None, field: str = 'model_id'):
        pats = _DEFAULT_FAMILIES if patterns is None else tuple(patterns)
        self.field = field
        self._re = re.compile('|'.join(f'(?:{p}[-\\w.]*)' for p in pats), re.I) if pats else None

    def __call__(self, rows: Rows) -> Step:
        rows = list(rows)
        return _split(rows, [bool(self._re and self._re.fullmatch(str(r.get(self.field) or ''))) for r in rows], 'model_not_allowed')


class MessageNormalizer(Preprocessor):
    """Mapper: brings every row's messages to the canonical form of :func:`normalize_messages`; rows whose messages
    are not a list are dropped."""

    def __call__(self, rows: Rows) -> Step:
        kept, dropped = [], []
        for r in rows:
            if isinstance(r.get('messages'), list):
                kept.append(normalize_messages(r))
            else:
                dropped.append(dict(r, drop_reason='no_messages'))
        return kept, dropped


# ------------------------------------------------------------------------------------------------ intent classifier
INTENT_TOOL_CALL, INTENT_CODE, INTENT_MATH = 'tool_call', 'code', 'math'
INTENT_COMPLEX_LOGIC, INTENT_REASONING, INTENT_USER_DISSATISFACTION, INTENT_OTHER = 'complex_logic', 'reasoning', 'user_dissatisfaction', 'other'

_FENCE = re.compile(r'```[\s\S]{10,}?```')
_CODE_TOKEN = re.compile(r'\b(?:def|class|import|from|function|const|let|var|return|public|private|static|void|struct|enum|interface|'
                         r'namespace|package|lambda|async|await|yield|catch|throw|fn|func)\s|#include\b|console\.log|println|'
                         r'[A-Za-z_]\w*\([^)\n]*\)\s*\{|=>\s*\{|->\s*[A-Za-z_]\w*')
_MATH_TOKEN = re.compile(
    r'\$\$.+?\$\$|\$[^$\n]+?\$|\\\[.+?\\\]|\\(?:frac|sum|int|lim|sqrt|boxed|cdot|times|leq|geq|neq|approx|infty|pi|alpha|beta|theta|'
    r'lambda|sigma|partial|nabla|mathbb|prod|to)\b|[×÷±∑∏∫√∂∇∞∈⊂⊆≤≥≠≈≡⇒⇔]|[α-ωΔΘΛΣΦΨΩ]|[⁰¹²³⁴-⁹₀-₉]|'
    r'\d+\s*[×÷*/+\-]\s*\d+\s*=\s*\d+|\b[a-zA-Z]\s*=\s*-?\d+\b|\w\^\{[^}]+\}|\w_\{[^}]+\}|'
    r'方程|不等式|导数|积分|极限|矩阵|向量|概率|方差|数列|质数|因数|倍数|面积|体积|周长|半径|三角形|平方|立方|根号|对数|'
    r'\b(?:integral|derivative|polynomial|equation|inequality|matrix|vector|determinant|eigenvalue|logarithm|theorem|lemma|proof|'
    r'probability|variance|median|factorial|radius|diameter|perimeter|hypotenuse|cosine|sine|tangent|coefficient)\b', re.S | re.I)
_LOGIC_TOKEN = re.compile(
    r'首先.{4,}?其次|第一.{4,}?第二|一方面.{4,}?另一方面|如果.{2,30}?那么|假设.{2,30}?则|因为.{2,40}?所以|由于.{2,40}?因此|综上|总而言之|'
    r'由此可[得见知]|优缺点|利弊|权衡|相比之下|约束条件|'
    r'\b(?:first(?:ly)?|second(?:ly)?|third(?:ly)?|finally|furthermore|moreover|in addition|on (?:the )?one hand|on the other hand|'
    r'as a result|consequently|therefore|hence|thus|accordingly|in (?:conclusion|summary)|to (?:summarize|conclude)|overall|'
    r'pros and cons|trade-?offs?|case \d|scenario \d)\b|\bif .{5,30}? then\b', re.S | re.I)
_UNHAPPY = re.compile(
    r'不对|不正确|不准确|不靠谱|太差|太烂|重新(?:回答|做|来|算|生成)|再(?:答|来|做|算|试)一(?:次|遍|下)|错了|错误|又错|搞错|答非所问|跑题|'
    r'胡说|瞎编|莫名其妙|失望|没听懂|理解错|我(?:说|问)的不是|浪费时间|垃圾|'
    r'\b(?:wrong|incorrect|useless|terrible|awful|horrible|stupid|ridiculous|misleading|disappointing|disappointed|unacceptable|'
    r'unhelpful|inaccurate|nonsense|garbage|gibberish|redo|try again|start over|off[- ]topic|frustrat\w+)\b|'
    r'\bnot (?:correct|right|helpful|useful|accurate|relevant|what i (?:asked|wanted|meant|need))\b|'
    r"(?:doesn'?t|does not|didn'?t|did not) (?:make sense|work|help|answer)|makes? no sense|waste of time|"
    r"you (?:misunderstood|don'?t understand|missed (?:the|my) point)|that'?s (?:not what|wrong|incorrect)|are you (?:serious|kidding)", re.I)
_THINK = re.compile(r'<think>([\s\S]*?)</think>')


def _owning_round(messages: Sequence[Dict[str, Any]], idx: int) -> Optional[int]:
    """Index of the assistant turn that a signal at ``idx`` belongs to: the turn itself, or the next assistant turn
    after a user message; signals in system/tool messages belong to no round."""
    role = messages[idx].get('role')
    if role == 'assistant':
        return idx
    if role == 'user':
        for j in range(idx + 1, len(messages)):
            if isinstance(messages[j], dict) and messages[j].get('role') == 'assistant':
                return j
    return None


class IntentDetector:
    """``detector(messages)`` → sorted indices of the assistant turns (key rounds) that show ``intent``. A
    ``definitive`` detector that fires ends the classifier's pipeline (hard signals such as real tool calls)."""
    intent: str = ''
    definitive: bool = False

    def __call__(self, messages: List[Dict[str, Any]]) -> List[int]:
        raise NotImplementedError


class _CountDetector(IntentDetector):
    pattern: 're.Pattern'
    roles: Tuple[str, ...] = ('user', 'assistant')

    def __init__(self, threshold: int):
        self.threshold = threshold

    def match(self, text: str) -> bool:
        return sum(1 for _ in self.pattern.finditer(text)) >= self.threshold

    def __call__(self, messages):
        rounds = set()
        for i, m in enumerate(messages):
            if not isinstance(m, dict) or m.get('role') not in self.roles:
                continue
            text = _content_text(m)
            if text and self.match(text):
                j = _owning_round(messages, i)
                if j is not None:
                    rounds.add(j)
        return sorted(rounds)


class ToolCallDetector(IntentDetector):
    intent, definitive = INTENT_TOOL_CALL, True

    def __call__(self, messages):
        return [i for i, m in enumerate(messages) if isinstance(m, dict) and m.get('role') == 'assistant' and m.get('tool_calls')]


class CodeDetector(_CountDetector):
    intent, pattern = INTENT_CODE, _CODE_TOKEN

    def __init__(self, threshold: int = 3):
        super().__init__(threshold)

    def match(self, text):
        return bool(_FENCE.search(text)) or super().match(text)


class MathDetector(_CountDetector):
    intent, pattern = INTENT_MATH, _MATH_TOKEN

    def __init__(self, threshold: int = 4):
        super().__init__(threshold)


class ComplexLogicDetector(_CountDetector):
    intent, pattern, roles = INTENT_COMPLEX_LOGIC, _LOGIC_TOKEN, ('assistant', )

    def __init__(self, threshold: int = 6):
        super().__init__(threshold)


class ReasoningDetector(IntentDetector):
    """Assistant turns with an explicit chain of thought: ``reasoning_content`` or a ``<think>`` block of at least
    ``min_chars`` characters."""
    intent = INTENT_REASONING

    def __init__(self, min_chars: int = 200):
        self.min_chars = min_chars

    def __call__(self, messages):
        out = []
        for i, m in enumerate(messages):
            if not isinstance(m, dict) or m.get('role') != 'assistant':
                continue
            rc = m.get('reasoning_content')
            if isinstance(rc, str) and len(rc.strip()) >= self.min_chars:
                out.append(i)
                continue
            t = _THINK.search(_content_text(m))
            if t and len(t.group(1).strip()) >= self.min_chars:
                out.append(i)
        return out


class UserDissatisfactionDetector(IntentDetector):
    """A user complaint is a reaction, so it counts only after an assistant turn; the key round is the assistant's
    next attempt."""
    intent = INTENT_USER_DISSATISFACTION

    def __call__(self, messages):
        seen, rounds = False, set()
        for i, m in enumerate(messages):
            if not isinstance(m, dict):
                continue
            if m.get('role') == 'assistant':
                seen = True
            elif m.get('role') == 'user' and seen and _UNHAPPY.search(_content_text(m)):
                j = _owning_round(messages, i)
                if j is not None:
                    rounds.add(j)
        return sorted(rounds)


class IntentClassifier(Preprocessor):
    """Annotates each row with its primary intent (``row[intent_field]``) and, in ``user_data``, ``key_rounds`` (sorted
    assistant indices) and ``intents`` (``{index: intent}``). Detectors run in order; an earlier detector's verdict on
    a round is never overridden. Rows without any key round are dropped unless ``drop_no_key_rounds=False`` (they then
    get the intent ``other``). Heuristics only — no model call."""

    def __init__(self, detectors: Optional[List[IntentDetector]] = None, intent_field: str = 'intent', drop_no_key_rounds: bool = True):
        self.detectors = list(detectors) if detectors is not None else [ToolCallDetector(), CodeDetector(), MathDetector(),
                                                                         ComplexLogicDetector(), ReasoningDetector(),
                                                                         UserDissatisfactionDetector()]
        self.intent_field, self.drop_no_key_rounds = intent_field, drop_no_key_rounds

    def detect(self, messages: List[Dict[str, Any]]) -> Dict[int, str]:
        found: Dict[int, str] = {}
        for det in self.detectors:
            rounds = det(messages)
            for i in rounds:
                found.setdefault(i, det.intent)
            if rounds and det.definitive:
                break
        return found

    def __call__(self, rows: Rows) -> Step:
        from ..data_format import user_data_set
        kept, dropped = [], []
        for row in rows:
            row = dict(row)
            msgs = row.get('messages')
            found = self.detect(msgs) if isinstance(msgs, list) and msgs else {}
            if found:
                ud = user_data_set(row.get('user_data') if row.get('user_data') is not None else [], 'key_rounds', sorted(found))
                row['user_data'] = user_data_set(ud, 'intents', {str(k): v for k, v in found.items()})
                row[self.intent_field] = Counter(found.values()).most_common(1)[0][0]
            elif self.drop_no_key_rounds:
                dropped.append(dict(row, drop_reason='no_key_rounds'))
                continue
            else:
                row[self.intent_field] = INTENT_OTHER
            kept.append(row)
        logger.info(f'[IntentClassifier] {dict(Counter(r[self.intent_field] for r in kept))}')
        return kept, dropped


# ------------------------------------------------------------------------------------------------------ LLM back ends
def split_think(text: str) -> Tuple[str, str]:
    """``(answer, reasoning)`` of a completion that may open with a ``<think>…</think>`` block."""
    if '</think>' in text:
        head, tail = text.split('</think>', 1)
        return tail.strip(), head.split('<think>')[-1].strip()
    return text, ''


class LLMBackend(ABC):
    """What the model-backed pipeline steps need from a language model: chat completions, log-probabilities of given
    tokens without generation, and (optionally) sentence embeddings."""

    @abstractmethod
    def chat(self, messages: List[Dict[str, Any]], *, temperature: float = 0.0, max_tokens: int = 16, n: int = 1) -> List[Dict[str, str]]:
        """``n`` choices, each ``{'content', 'reasoning_content'}``; an empty list on failure."""

    def chat_batch(self, messages_list: List[List[Dict[str, Any]]], *, temperature: float = 0.0, max_tokens: int = 16,
                   n: int = 1) -> List[List[Dict[str, str]]]:
        return [self.chat(m, temperature=temperature, max_tokens=max_tokens, n=n) for m in messages_list]

    @abstractmethod
    def prompt_logprobs(self, messages: List[Dict[str, Any]]) -> Optional[List]:
        """Per-token log-probabilities of the templated conversation (first entry ``None``), or ``None`` on failure."""

    @abstractmethod
    def prompt_logprobs_ids(self, input_ids_list: List[List[int]]) -> List[List]:
        """The same for raw token-id prompts (no chat template), one list per prompt."""

    def embeddings(self, texts: List[str]):
        raise NotImplementedError(f'{type(self).__name__} has no embedding endpoint')


class OpenAIBackend(LLMBackend):
    """Any OpenAI-compatible HTTP server (this framework's gateway included). ``post(url, json) -> dict`` can be
    injected; the default uses ``requests``. Batched chat fans out over ``max_workers`` threads."""

    def __init__(self, base_url: str, model: str, api_key: Optional[str] = None, timeout: float = 120.0, max_workers: int = 8,
                 embed_model: Optional[str] = None, post: Optional[Callable[[str, Dict[str, Any]], Dict[str, Any]]] = None):
        root = base_url.rstrip('/')
        self.root = root if root.endswith('/v1') else root + '/v1'
        self.model, self.embed_model, self.timeout, self.max_workers = model, embed_model or model, timeout, max_workers
        self._headers = {'Authorization': f'Bearer {api_key}'} if api_key else {}
        self._post = post or self._http_post

    def _http_post(self, url: str, body: Dict[str, Any]) -> Dict[str, Any]:
        import requests
        r = requests.post(url, json=body, headers=self._headers, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def chat(self, messages, *, temperature=0.0, max_tokens=16, n=1):
        try:
            data = self._post(self.root + '/chat/completions', {'model': self.model, 'messages': messages, 'temperature': temperature,
                                                                 'max_tokens': max_tokens, 'n': n})
        except Exception as e:  # a judge that is down must not kill a long pipeline run
            logger.warning(f'[OpenAIBackend] chat failed: {e}')
            return []
        out = []
        for c in data.get('choices', []):
            m = c.get('message') or {}
            content, reasoning = m.get('content') or '', m.get('reasoning_content') or ''
            if not reasoning:
                content, reasoning = split_think(content)
            out.append({'content': content, 'reasoning_content': reasoning})
        return out

    def chat_batch(self, messages_list, *, temperature=0.0, max_tokens=16, n=1):
        if len(messages_list) <= 1 or self.max_workers <= 1:
            return super().chat_batch(messages_list, temperature=temperature, max_tokens=max_tokens, n=n)
        with ThreadPoolExecutor(self.max_workers) as ex:
            return list(ex.map(lambda m: self.chat(m, temperature=temperature, max_tokens=max_tokens, n=n), messages_list))

    def prompt_logprobs(self, messages):
        try:
            data = self._post(self.root + '/chat/completions', {'model': self.model, 'messages': messages, 'max_tokens': 0, 'prompt_logprobs': 1})
        except Exception:
            return None
        return data.get('prompt_logprobs') or ((data.get('choices') or [{}])[0].get('prompt_logprobs'))

    def prompt_logprobs_ids(self, input_ids_list):
        out = []
        for ids in input_ids_list:
            data = self._post(self.root + '/completions', {'model': self.model, 'prompt': list(ids), 'max_tokens': 0, 'echo': True,
                                                           'prompt_logprobs': 1})
            ch = data.get('choices') or []
            out.append(ch[0]['prompt_logprobs'] if ch and 'prompt_logprobs' in ch[0] else data['prompt_logprobs'])
        return out

    def embeddings(self, texts):
        import numpy as np
        data = self._post(self.root + '/embeddings', {'model': self.embed_model, 'input': list(texts)}).get('data', [])
        return np.asarray([d['embedding'] for d in sorted(data, key=lambda d: d.get('index', 0))], dtype=np.float32)


class SamplerBackend(LLMBackend):
    """An in-process sampler of this framework (template already set) — no HTTP. ``max_tokens=0`` with
    ``prompt_logprobs`` is the sampler's score-only mode. Embeddings go to ``embed_backend`` when one is given."""

    def __init__(self, sampler, embed_backend: Optional[LLMBackend] = None, adapter_name: Optional[str] = None):
        self.sampler, self.embed_backend, self.adapter_name = sampler, embed_backend, adapter_name

    def _sample(self, inputs, params):
        from ..data_format import SamplingParams
        kw = {'adapter_name': self.adapter_name} if self.adapter_name else {}
        return self.sampler.sample(inputs, SamplingParams(**params), **kw)

    @staticmethod
    def _choices(resp) -> List[Dict[str, str]]:
        out = []
        for seq in getattr(resp, 'sequences', None) or resp.get('sequences', []):
            text = (getattr(seq, 'decoded', None) if not isinstance(seq, dict) else seq.get('decoded')) or ''
            content, reasoning = split_think(text)
            out.append({'content': content, 'reasoning_content': reasoning})
        return out

    def chat(self, messages, *, temperature=0.0, max_tokens=16, n=1):
        res = self.chat_batch([messages], temperature=temperature, max_tokens=max_tokens, n=n)
        return res[0] if res else []

    def chat_batch(self, messages_list, *, temperature=0.0, max_tokens=16, n=1):
        if not messages_list:
            return []
        try:
            resps = self._sample([{'messages': m} for m in messages_list], dict(temperature=temperature, max_tokens=max_tokens, num_samples=n))
        except Exception as e:
            logger.warning(f'[SamplerBackend] chat failed: {e}')
            return [[] for _ in messages_list]
        return [self._choices(r) for r in resps]

    def prompt_logprobs(self, messages):
        try:
            resps = self._sample([{'messages': messages}], dict(max_tokens=0, prompt_logprobs=1))
        except Exception as e:
            logger.warning(f'[SamplerBackend] prompt_logprobs failed: {e}')
            return None
        r = resps[0] if resps else None
        return None if r is None else (getattr(r, 'prompt_logprobs', None) if not isinstance(r, dict) else r.get('prompt_logprobs'))

    def prompt_logprobs_ids(self, input_ids_list):
        if not input_ids_list:
            raise ValueError('prompt_logprobs_ids needs at least one prompt')
        resps = self._sample([{'input_ids': list(ids)} for ids in input_ids_list], dict(max_tokens=0, prompt_logprobs=1))
        return [getattr(r, 'prompt_logprobs', None) if not isinstance(r, dict) else r.get('prompt_logprobs') for r in resps]

    def embeddings(self, texts):
        if self.embed_backend is None:
            return super().embeddings(texts)
        return self.embed_backend.embeddings(texts)


# ------------------------------------------------------------------------------------------- per-round difficulty scores
def _lp_value(entry: Any, token_id: Optional[int]) -> Optional[float]:
    """Log-probability of ``token_id`` from one prompt-logprob entry. Accepted shapes: a float; ``None``; a mapping
    ``{token_id: float | {'logprob': float}}`` (ids as int or str); a list of ``(token_id, logprob)`` pairs."""
    if entry is None:
        return None
    if isinstance(entry, (int, float)):
        return float(entry)
    if isinstance(entry, dict):
        if 'logprob' in entry:
            return float(entry['logprob'])
        v = entry.get(token_id, entry.get(str(token_id))) if token_id is not None else None
        if v is None and len(entry) == 1:
            v = next(iter(entry.values()))
        if isinstance(v, dict):
            v = v.get('logprob')
        return None if v is None else float(v)
    if isinstance(entry, (list, tuple)):
        for pair in entry:
            if isinstance(pair, (list, tuple)) and len(pair) == 2 and (token_id is None or int(pair[0]) == token_id):
                return float(pair[1])
    return None


def response_logprob_deltas(cond_lp: Sequence, asst_lp: Sequence, cond_ids: Sequence[int], asst_ids: Sequence[int],
                            n_prompt: int) -> List[Tuple[int, float]]:
    """``(token id, log p(token | prompt, prefix) − log p(token | prefix))`` per response position: how much the
    prompt helps each token. ``cond_lp`` covers prompt ⊕ response, ``asst_lp`` the response alone."""
    out = []
    for i in range(min(len(asst_lp or ()), len(asst_ids or ()))):
        ci = n_prompt + i
        if ci >= len(cond_lp or ()):
            break
        a = _lp_value(asst_lp[i], asst_ids[i])
        c = _lp_value(cond_lp[ci], cond_ids[ci] if ci < len(cond_ids) else None)
        if a is not None and c is not None:
            out.append((int(asst_ids[i]), c - a))
    return out


def chr_min_distinct(cond_lp, asst_lp, cond_ids, asst_ids, n_prompt, exclude_ids: Optional[Set[int]] = None) -> Optional[float]:
    """Share of distinct response token ids whose *smallest* delta over their occurrences is positive — i.e. tokens the
    prompt helps every time they appear. Low = the prompt explains little of the answer = a hard, informative sample."""
    by_tok: Dict[int, float] = {}
    for tid, d in response_logprob_deltas(cond_lp, asst_lp, cond_ids, asst_ids, n_prompt):
        if exclude_ids and tid in exclude_ids:
            continue
        by_tok[tid] = min(d, by_tok.get(tid, float('inf')))
    if not by_tok:
        return None
    return sum(1 for d in by_tok.values() if d > 0) / len(by_tok)


def ifd_family(cond_lp, asst_lp, cond_ids, asst_ids, n_prompt) -> Dict[str, Any]:
    """Instruction-following difficulty ``exp(−mean delta)`` (= conditioned perplexity ÷ unconditioned perplexity; high
    = the prompt helps little) and the selective variants over the 50 % / 75 % of tokens with the largest |delta|."""
    deltas = [d for _, d in response_logprob_deltas(cond_lp, asst_lp, cond_ids, asst_ids, n_prompt)]
    if not deltas:
        return {}
    n = len(deltas)
    mean = sum(deltas) / n
    out = {'n_tokens': n, 'mean_delta': mean, 'ifd': math.exp(-mean)}
    ranked = sorted(deltas, key=abs, reverse=True)
    for pct in (50, 75):
        sub = ranked[:max(1, int(round(n * pct / 100)))]
        out[f's_ifd_{pct}'] = math.exp(-sum(sub) / len(sub))
    return out


@dataclass
class RoundContext:
    """One candidate assistant turn handed to the scorers."""
    row_idx: int
    rnd_idx: int
    asst_idx: int
    row: Dict[str, Any]
    intent: Optional[str]
    messages: List[Dict[str, Any]]
    context_messages: List[Dict[str, Any]]
    cond_ids: List[int]
    n_prompt: int
    asst_ids: List[int]
    asst_text: str
    user_prompt: str
    features: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ScoreResult:
    score: Optional[float] = None
    passed: bool = True
    extras: Dict[str, Any] = field(default_factory=dict)


class Scorer(Protocol):
    name: str
    requires_logprobs: bool

    def score(self, contexts: List[RoundContext]) -> List[ScoreResult]:
        ...


class ChrMinScorer:
    """Keeps rounds whose :func:`chr_min_distinct` is below ``threshold`` (unscorable rounds pass)."""
    name, requires_logprobs = 'chr_min', True

    def __init__(self, threshold: float = 0.47):
        self.threshold = float(threshold)

    def score(self, contexts):
        out = []
        for c in contexts:
            s = chr_min_distinct(c.features.get('cond_lp'), c.features.get('asst_lp'), c.cond_ids, c.asst_ids, c.n_prompt)
            out.append(ScoreResult(s, s is None or s < self.threshold, {'threshold': self.threshold}))
        return out


class SIFDScorer:
    """Records IFD / S-IFD-50 / S-IFD-75; filters only when ``ifd_threshold`` is given (keep ``ifd >= threshold``)."""
    name, requires_logprobs = 'sifd', True

    def __init__(self, ifd_threshold: Optional[float] = None):
        self.ifd_threshold = ifd_threshold

    def score(self, contexts):
        out = []
        for c in contexts:
            fam = ifd_family(c.features.get('cond_lp'), c.features.get('asst_lp'), c.cond_ids, c.asst_ids, c.n_prompt)
            s = fam.get('ifd')
            out.append(ScoreResult(s, self.ifd_threshold is None or s is None or s >= self.ifd_threshold, dict(fam)))
        return out


_JUDGE_PROMPT = ('You are grading an answer against a reference. Decide whether the candidate answer is correct and complete with '
                 'respect to the reference; wording may differ. Reply with <verdict>PASS</verdict> or <verdict>FAIL</verdict>.')
_PASS_FAIL_TAG = re.compile(r'<verdict>\s*(PASS|FAIL)\s*</verdict>', re.I)


class PassNScorer:
    """The policy answers the round's prompt ``n`` times; a judge model compares each answer with the recorded one.
    Score = pass rate. Rounds the policy already solves (rate above ``max_pass_rate``) fail the filter — they teach
    nothing — as do, optionally, rounds below ``min_pass_rate`` (out of reach)."""
    name, requires_logprobs = 'pass_n', False

    def __init__(self, backend: LLMBackend, judge: Optional[LLMBackend] = None, n: int = 4, max_pass_rate: float = 0.75,
                 min_pass_rate: float = 0.0, temperature: float = 1.0, max_tokens: int = 1024, judge_max_tokens: int = 64,
                 max_chars: int = 6000):
        self.backend, self.judge = backend, judge or backend
        self.n, self.max_rate, self.min_rate = n, max_pass_rate, min_pass_rate
        self.temperature, self.max_tokens, self.judge_max_tokens, self.max_chars = temperature, max_tokens, judge_max_tokens, max_chars

    def _clip(self, text: str) -> str:
        if len(text) <= self.max_chars:
            return text
        half = self.max_chars // 2
        return text[:half] + '\n…\n' + text[-half:]

    @staticmethod
    def parse_verdict(text: str) -> Optional[bool]:
        found = _PASS_FAIL_TAG.findall(text or '')
        if found:
            return found[-1].upper() == 'PASS'
        t = (text or '').upper()
        if ('PASS' in t) != ('FAIL' in t):
            return 'PASS' in t
        return None

    def score(self, contexts):
        if not contexts:
            return []
        rollouts = self.backend.chat_batch([c.context_messages for c in contexts], temperature=self.temperature, max_tokens=self.max_tokens,
                                           n=self.n)
        jobs, owner = [], []
        for ci, (c, choices) in enumerate(zip(contexts, rollouts)):
            for ch in choices:
                jobs.append([{'role': 'system', 'content': _JUDGE_PROMPT},
                             {'role': 'user', 'content': f'[Question]\n{self._clip(c.user_prompt)}\n\n[Reference]\n{self._clip(c.asst_text)}\n\n'
                                                         f'[Candidate]\n{self._clip(ch.get("content", ""))}'}])
                owner.append(ci)
        verdicts = self.judge.chat_batch(jobs, temperature=0.0, max_tokens=self.judge_max_tokens, n=1) if jobs else []
        per: Dict[int, List[Optional[bool]]] = {}
        for ci, v in zip(owner, verdicts):
            per.setdefault(ci, []).append(self.parse_verdict(v[0]['content']) if v else None)
        out = []
        for ci, c in enumerate(contexts):
            vs = [v for v in per.get(ci, []) if v is not None]
            if not vs:
                out.append(ScoreResult(None, True, {'rollouts': 0}))
                continue
            rate = sum(vs) / len(vs)
            out.append(ScoreResult(rate, self.min_rate <= rate <= self.max_rate, {'rollouts': len(vs), 'verdicts': vs}))
        return out


_MIN_RESPONSE_TOKENS = 6


def _ids(x: Any) -> List[int]:
    if isinstance(x, dict) or hasattr(x, 'keys'):
        x = x['input_ids']
    if hasattr(x, 'tolist'):
        x = x.tolist()
    return [int(t) for t in x]


def _encode_text(template, text: str) -> List[int]:
    return _ids(template.tokenizer(text, add_special_tokens=False))


def _encode_prompt(template, ctx_msgs: List[Dict[str, Any]], budget: int) -> List[int]:
    """Templated prompt (generation prompt appended) within ``budget`` tokens: oldest non-system turns are removed
    first; a single over-long turn keeps its tail."""
    ctx = list(ctx_msgs)
    enc = lambda: _ids(template.encode({'messages': ctx}, add_generation_prompt=True))  # noqa: E731
    ids = enc()
    if budget <= 0 or len(ids) <= budget:
        return ids
    first = 1 if ctx and ctx[0].get('role') == 'system' else 0
    while len(ctx) - first > 1:
        ctx.pop(first)
        ids = enc()
        if len(ids) <= budget:
            return ids
    return ids[-budget:]


class ParaphraseScorer:
    """The recorded answer may be written in a style the policy would never use, which inflates its difficulty. So the
    policy first restates the answer in its own words (the recorded answer is shown as a reference), and ``chr_min`` is
    computed on that restatement against the *original* prompt. Filters only when ``chr_min_threshold`` is set."""
    name, requires_logprobs = 'paraphrase', False

    def __init__(self, backend: LLMBackend, template, chr_min_threshold: Optional[float] = None, prompt_budget: int = 4096,
                 sample_temperature: float = 0.7, sample_max_tokens: int = 4096, max_prompt_tokens: int = 1024):
        self.backend, self.template, self.threshold = backend, template, chr_min_threshold
        self.prompt_budget, self.temperature, self.max_tokens, self.max_prompt_tokens = prompt_budget, sample_temperature, sample_max_tokens, max_prompt_tokens

    @staticmethod
    def with_reference(context_messages: List[Dict[str, Any]], answer: str) -> List[Dict[str, Any]]:
        note = ('A reference answer to the question above follows, for your eyes only:\n<reference_answer>\n' + answer +
                '\n</reference_answer>\nUsing it, give a complete answer to the question in your own words and reasoning. Answer '
                'directly and do not copy the reference word for word.')
        msgs = [dict(m) for m in context_messages]
        if msgs and msgs[-1].get('role') == 'user' and isinstance(msgs[-1].get('content'), str):
            msgs[-1]['content'] = msgs[-1]['content'] + '\n\n' + note
        else:
            msgs.append({'role': 'user', 'content': note})
        return msgs

    def _fit_answer(self, text: str, n_prompt: int) -> Optional[str]:
        room = self.prompt_budget - n_prompt - 80  # 80 tokens for the instruction around the reference
        if room < 50:
            return None
        ids = _encode_text(self.template, text)
        return text if len(ids) <= room else self.template.tokenizer.decode(ids[:room])

    def score(self, contexts):
        out = [ScoreResult(None, True, {'reason': 'paraphrase skipped'}) for _ in contexts]
        todo, prompts = [], []
        for i, c in enumerate(contexts):
            ans = self._fit_answer(c.asst_text, c.n_prompt) if c.context_messages else None
            if ans is not None:
                todo.append(i)
                prompts.append(self.with_reference(c.context_messages, ans))
        if not todo:
            return out
        choices = self.backend.chat_batch(prompts, temperature=self.temperature, max_tokens=self.max_tokens, n=1) or []
        ready = []
        for i, ch in zip(todo, choices):
            text = ch[0].get('content') if ch and isinstance(ch[0], dict) else None
            if not isinstance(text, str) or not text.strip():
                continue
            p = _encode_prompt(self.template, contexts[i].context_messages, self.max_prompt_tokens)
            a = _encode_text(self.template, text)
            if len(a) >= _MIN_RESPONSE_TOKENS:
                ready.append((i, p + a, len(p), a, text))
        if not ready:
            return out
        cond = self.backend.prompt_logprobs_ids([r[1] for r in ready])
        alone = self.backend.prompt_logprobs_ids([r[3] for r in ready])
        for (i, cond_ids, n_prompt, a, text), c_lp, a_lp in zip(ready, cond, alone):
            s = chr_min_distinct(c_lp, a_lp, cond_ids, a, n_prompt)
            out[i] = ScoreResult(s, self.threshold is None or s is None or s < self.threshold,
                                 {'paraphrase_text': text, 'n_prompt': n_prompt, 'threshold': self.threshold})
        return out


class RoundScoreFilter(Preprocessor):
    """Scores candidate assistant turns with a set of scorers; a round survives when every scorer passes it.

    Candidates are ``user_data['key_rounds']`` (as written by :class:`IntentClassifier`) or, without them, every
    assistant turn; ``intents`` restricts scoring to rounds with those intents. Rows that had key rounds keep the
    surviving ones (and are dropped when none survive); rows without key rounds are dropped when any round fails
    (``drop_row_on_any_fail``). Log-probabilities are fetched once, in two batched calls, when a scorer needs them.
    ``trace_dir`` receives one JSON file per scored round."""

    def __init__(self, template, backend: LLMBackend, scorers: List[Scorer], intents: Optional[Iterable[str]] = None,
                 keep_if_no_key_rounds: bool = False, drop_row_on_any_fail: bool = True, max_prompt_tokens: int = 1024,
                 trace_dir: Optional[str] = None):
        if not hasattr(template, 'encode') or not hasattr(template, 'tokenizer'):
            raise TypeError(f'RoundScoreFilter needs a Template, got {type(template).__name__}')
        self.template, self.backend, self.scorers = template, backend, list(scorers)
        self.intents = None if intents is None else set(intents)
        self.keep_if_no_key_rounds, self.drop_row_on_any_fail = keep_if_no_key_rounds, drop_row_on_any_fail
        self.max_prompt_tokens, self.trace_dir = max_prompt_tokens, trace_dir
        if trace_dir:
            os.makedirs(trace_dir, exist_ok=True)

    # -- candidates
    def _context(self, row, ri: int, k: int, ai: int) -> Optional[RoundContext]:
        from ..data_format import user_data_get
        msgs = row['messages']
        if not (isinstance(ai, int) and 0 < ai < len(msgs)) or not isinstance(msgs[ai], dict) or msgs[ai].get('role') != 'assistant':
            return None
        intent = (user_data_get(row.get('user_data'), 'intents') or {}).get(str(ai))
        if self.intents is not None and intent not in self.intents:
            return None
        text = _content_text(msgs[ai])
        if not text.strip():
            return None
        a = _encode_text(self.template, text)  # raw ids: the same tokens in both the conditioned and the lone pass
        if len(a) < _MIN_RESPONSE_TOKENS:
            return None
        ctx_msgs = msgs[:ai]
        p = _encode_prompt(self.template, ctx_msgs, self.max_prompt_tokens)
        shown = '\n\n'.join(f"[{m.get('role', 'user')}] {_content_text(m).strip()}" for m in ctx_msgs if isinstance(m, dict) and _content_text(m).strip())
        return RoundContext(ri, k, ai, row, intent, msgs, ctx_msgs, p + a, len(p), a, text, shown)

    def build_contexts(self, rows: Rows) -> List[RoundContext]:
        from ..data_format import user_data_get
        out = []
        for ri, row in enumerate(rows):
            msgs = row.get('messages')
            if not isinstance(msgs, list):
                continue
            rounds = user_data_get(row.get('user_data'), 'key_rounds')
            if not isinstance(rounds, list) or not rounds:
                rounds = [i for i, m in enumerate(msgs) if isinstance(m, dict) and m.get('role') == 'assistant']
            for k, ai in enumerate(rounds):
                c = self._context(row, ri, k, ai)
                if c is not None:
                    out.append(c)
        return out

    # -- scoring
    def score_contexts(self, contexts: List[RoundContext]) -> List[Dict[str, ScoreResult]]:
        if any(getattr(s, 'requires_logprobs', False) for s in self.scorers):
            cond = self.backend.prompt_logprobs_ids([c.cond_ids for c in contexts])
            alone = self.backend.prompt_logprobs_ids([c.asst_ids for c in contexts])
            for c, cl, al in zip(contexts, cond, alone):
                c.features['cond_lp'], c.features['asst_lp'] = cl, al
        table: List[Dict[str, ScoreResult]] = [dict() for _ in contexts]
        for s in self.scorers:
            res = s.score(contexts)
            if len(res) != len(contexts):
                raise RuntimeError(f'scorer {s.name!r} returned {len(res)} results for {len(contexts)} rounds')
            for i, r in enumerate(res):
                table[i][s.name] = r
        return table

    def _trace(self, contexts, table) -> None:
        for c, scores in zip(contexts, table):
            rec = {'row': c.row_idx, 'round': c.rnd_idx, 'assistant_index': c.asst_idx, 'intent': c.intent, 'prompt': c.user_prompt,
                   'answer': c.asst_text, 'n_prompt': c.n_prompt, 'n_answer': len(c.asst_ids),
                   'scores': {k: {'score': v.score, 'passed': v.passed, 'extras': v.extras} for k, v in scores.items()}}
            with open(os.path.join(self.trace_dir, f'row{c.row_idx:06d}_round{c.rnd_idx:03d}.json'), 'w', encoding='utf-8') as f:
                json.dump(rec, f, ensure_ascii=False, indent=1, default=str)

    def __call__(self, rows: Rows) -> Step:
        from ..data_format import user_data_get, user_data_set
        rows = list(rows)
        contexts = self.build_contexts(rows)
        if not contexts and self.intents is None and self.keep_if_no_key_rounds:
            return rows, []
        table = self.score_contexts(contexts) if contexts else []
        if self.trace_dir and contexts:
            self._trace(contexts, table)
        per_row: Dict[int, Dict[str, Any]] = {}
        for c, scores in zip(contexts, table):
            slot = per_row.setdefault(c.row_idx, {'kept': [], 'failed': 0})
            if all(r.passed for r in scores.values()):
                slot['kept'].append(c.asst_idx)
            else:
                slot['failed'] += 1
        kept, dropped = [], []
        for ri, row in enumerate(rows):
            kr = user_data_get(row.get('user_data'), 'key_rounds')
            had = isinstance(kr, list) and bool(kr)
            d = per_row.get(ri)
            if d is None:  # nothing to score: no assistant text, or every round filtered out by intent
                if (had or self.intents is not None) and not self.keep_if_no_key_rounds:
                    dropped.append(dict(row, drop_reason='score_no_context'))
                else:
                    kept.append(row)
            elif had:
                if d['kept']:
                    kept.append(dict(row, user_data=user_data_set(row.get('user_data'), 'key_rounds', d['kept'])))
                else:
                    dropped.append(dict(row, drop_reason='score_all_rounds_failed'))
            elif d['failed'] and self.drop_row_on_any_fail:
                dropped.append(dict(row, drop_reason='score_round_failed'))
            else:
                kept.append(row)
        logger.info(f'[RoundScoreFilter] {len(contexts)} rounds scored, kept {len(kept)}/{len(rows)} rows')
        return kept, dropped


# --------------------------------------------------------------------------------------------------------- pipeline
class QualityPreprocessor(Preprocessor):
    """Runs quality steps in order and reports how many rows each one removed. A step is any callable on a list of
    rows that returns either ``(kept, dropped)`` or just the kept rows (plain ``Preprocessor`` / ``DataFilter``
    objects). ``dropped_log_path`` receives one JSON line per dropped row with the step's name; the file is rewritten
    per pipeline object and appended to under a file lock, so several dataset workers can share it."""

    def __init__(self, pipeline: Sequence[Callable], dropped_log_path: str = ''):
        self.pipeline, self.dropped_log_path = list(pipeline), dropped_log_path
        self.last_stats: List[Dict[str, Any]] = []
        if dropped_log_path:
            os.makedirs(os.path.dirname(os.path.abspath(dropped_log_path)), exist_ok=True)
            if os.path.exists(dropped_log_path):
                os.remove(dropped_log_path)

    def _log(self, step: str, dropped: Rows) -> None:
        if not self.dropped_log_path or not dropped:
            return
        import fcntl
        with open(self.dropped_log_path, 'a', encoding='utf-8') as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                for r in dropped:
                    f.write(json.dumps({'step': step, 'row': r}, ensure_ascii=False, default=str) + '\n')
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)

    def __call__(self, rows: Rows) -> Rows:
        rows = list(rows)
        self.last_stats = []
        for step in self.pipeline:
            if not rows:
                break
            name = getattr(step, '__name__', None) or type(step).__name__
            before, t0 = rows, time.perf_counter()
            res = step(rows)
            if isinstance(res, tuple) and len(res) == 2:
                rows, dropped = list(res[0]), list(res[1])
            else:
                rows = list(res)
                alive = {id(r) for r in rows}
                dropped = [dict(r, drop_reason=name) for r in before if id(r) not in alive] if len(rows) < len(before) else []
            self.last_stats.append({'step': name, 'before': len(before), 'after': len(rows), 'seconds': time.perf_counter() - t0})
            self._log(name, dropped)
        logger.info('[QualityPreprocessor] ' + ', '.join(f"{s['step']}: {s['before']}->{s['after']}" for s in self.last_stats))
        return rows
