"""Context management for long agent trajectories: chunking, condensing, and the rollout that uses them.

What it covers: reference ``src/twinkle_agentic/data_format/chunks.py``, ``chunker/native.py``,
``condenser/{base,keyword}.py``, ``tools/extract_condensed.py``, ``rollout/multi_turn_condense.py``.
A trajectory is cut into ``Chunk``s (role-tagged text pieces of bounded size); a ``Condenser`` replaces chunks the
policy no longer needs verbatim by a short digest and numbers them; the ``ExtractCondensed`` tool lets the policy
ask for the original text of a numbered block back.  The reference's keyword condenser relies on a spaCy
pipeline; no spaCy model can be loaded offline, so the digest here is built from sentence position and term
frequency (opening sentence + highest-scoring terms), which needs nothing but the text.
"""
from __future__ import annotations

import math
import re
from abc import ABC, abstractmethod
from collections import Counter
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence

from ..data_format.types import Message, Trajectory
from .rollout import MultiTurnRollout
from .tools import Tool, ToolManager


@dataclass
class Chunk:
    role: str
    content: str
    message_index: int
    tool_call_id: Optional[str] = None
    condensed: bool = False
    original: Optional[str] = None   # full text when ``condensed``
    block: Optional[int] = None      # number under which the original can be requested back
    extra: Dict[str, Any] = field(default_factory=dict)


class Chunks:

    def __init__(self, chunks: Sequence[Chunk], trajectory: Optional[Trajectory] = None):
        self.chunks = list(chunks)
        self.trajectory = trajectory

    def __iter__(self) -> Iterator[Chunk]:
        return iter(self.chunks)

    def __len__(self) -> int:
        return len(self.chunks)

    def to_trajectory(self) -> Trajectory:
        """Messages rebuilt from the chunks (pieces of one message are re-joined; condensed pieces carry their
        block number so the policy can refer to them)."""
        msgs: List[Message] = []
        src = (self.trajectory or {}).get('messages', [])
        cur = None
        for c in self.chunks:
            text = f'[block {c.block}, condensed] {c.content}' if c.condensed else c.content
            if cur is not None and cur[0] == c.message_index:
                cur[1]['content'] += text
                continue
            m: Message = {'role': c.role, 'content': text}
            if c.tool_call_id:
                m['tool_call_id'] = c.tool_call_id
            if c.message_index < len(src) and src[c.message_index].get('tool_calls'):
                m['tool_calls'] = src[c.message_index]['tool_calls']
            msgs.append(m)
            cur = (c.message_index, m)
        out = dict(self.trajectory or {})
        out['messages'] = msgs
        return out


class Chunker(ABC):

    @abstractmethod
    def __call__(self, trajectory: Trajectory) -> Chunks:
        ...


class NativeChunker(Chunker):
    """Recursive separator splitting (paragraph → line → sentence → word → hard cut) with a merge pass that packs the
    pieces back up to ``chunk_size`` characters."""

    SEPARATORS = ['\n\n', '\n', '. ', ' ']

    def __init__(self, chunk_size: int = 1200, min_chunk: int = 200, roles: Sequence[str] = ('tool', 'user', 'assistant')):
        self.chunk_size, self.min_chunk, self.roles = chunk_size, min_chunk, set(roles)

    def __call__(self, trajectory: Trajectory) -> Chunks:
        out: List[Chunk] = []
        for i, m in enumerate(trajectory.get('messages', [])):
            content = m.get('content', '')
            if not isinstance(content, str):
                content = ' '.join(p.get('text', '') for p in content if isinstance(p, dict))
            pieces = self._split(content, 0) if (m['role'] in self.roles and len(content) > self.chunk_size) else [content]
            for p in self._merge(pieces):
                out.append(Chunk(m['role'], p, i, m.get('tool_call_id')))
        return Chunks(out, trajectory)

    def _split(self, text: str, level: int) -> List[str]:
        if len(text) <= self.chunk_size:
            return [text]
        if level >= len(self.SEPARATORS):
            return [text[i:i + self.chunk_size] for i in range(0, len(text), self.chunk_size)]
        sep = self.SEPARATORS[level]
        parts = text.split(sep)
        parts = [p + sep for p in parts[:-1]] + [parts[-1]]
        out: List[str] = []
        for p in parts:
            if p:
                out.extend(self._split(p, level + 1))
        return out

    def _merge(self, pieces: List[str]) -> List[str]:
        out: List[str] = []
        for p in pieces:
            if out and len(out[-1]) + len(p) <= self.chunk_size:
                out[-1] += p
            else:
                out.append(p)
        if len(out) > 1 and len(out[-1]) < self.min_chunk and len(out[-2]) + len(out[-1]) <= 2 * self.chunk_size:
            last = out.pop()
            out[-1] += last
        return out


class Condenser(ABC):

    @abstractmethod
    def __call__(self, chunks: Chunks, **kwargs) -> Chunks:
        ...


_WORD = re.compile(r"[A-Za-z][A-Za-z0-9_\-']+|\d+(?:\.\d+)?")
_STOP = frozenset('the a an and or of to in on for with by is are was were be been it this that these those as at from not but if then '
                  'than so such can could will would should may might have has had do does did i you he she we they them his her its our '
                  'your their there here what which who whom when where why how all any each other some no nor only own same too very'.split())


class KeywordCondenser(Condenser):
    """Condenses chunks that are (a) long enough, (b) of a condensable role and (c) not among the most recent
    ``keep_last`` chunks: the digest is the opening sentence plus the top terms by tf·log-length weight."""

    def __init__(self, min_chars: int = 600, budget_chars: int = 240, keep_last: int = 4, roles: Sequence[str] = ('tool', ), top_k: int = 12):
        self.min_chars, self.budget, self.keep_last, self.roles, self.top_k = min_chars, budget_chars, keep_last, set(roles), top_k

    def __call__(self, chunks: Chunks, **kwargs) -> Chunks:
        out: List[Chunk] = []
        next_block = 1 + max([c.block or 0 for c in chunks] + [0])
        n = len(chunks)
        for i, c in enumerate(chunks):
            if c.condensed or c.role not in self.roles or len(c.content) < self.min_chars or i >= n - self.keep_last:
                out.append(c)
                continue
            out.append(Chunk(c.role, self._digest(c.content), c.message_index, c.tool_call_id, True, c.content, next_block, dict(c.extra)))
            next_block += 1
        return Chunks(out, chunks.trajectory)

    def _digest(self, text: str) -> str:
        first = re.split(r'(?<=[.!?])\s+|\n', text.strip(), maxsplit=1)[0][:self.budget // 2]
        words = [w.lower() for w in _WORD.findall(text)]
        tf = Counter(w for w in words if w not in _STOP and len(w) > 2)
        scored = sorted(tf.items(), key=lambda kv: (-kv[1] * math.log(2 + len(kv[0])), kv[0]))
        seen = set(w.lower() for w in _WORD.findall(first))
        terms = [w for w, _ in scored if w not in seen][:self.top_k]
        digest = first
        for t in terms:
            if len(digest) + len(t) + 2 > self.budget:
                break
            digest += ('; ' if digest else '') + t
        return digest


_CONDENSE_SYSTEM = ('You compress passages for a reader who must still answer questions from them. Keep names, numbers, dates, '
                    'identifiers and causal links; drop filler. Output the compressed passage only.')
_CONDENSE_USER = 'Question the reader cares about: {query}\n\nCompress the passage below to at most about {budget} characters.\n\n{text}'
_FENCED = re.compile(r'^```[\w-]*\n([\s\S]*?)\n?```$')


class ModelCondenser(Condenser):
    """Condenses chunks by asking a language model (through a sampler of this framework) for a shorter restatement.

    A chunk is sent when its role is condensable, it is at least ``min_chars`` long, not among the newest ``keep_last``
    chunks, not already condensed and does not match ``skip_pattern``. ``compression_ratio`` sets the character budget
    named in the prompt (never below ``min_budget_chars``) and the token limit of the request; the model's text is not
    cut to the budget, but a reply that is empty, has no letters or digits, or is not strictly shorter than the
    passage is discarded and the passage kept. ``related_query(chunk)`` marks chunks that carry the question; the most
    recent one is put in the prompts of the chunks that follow. Requests go out in batches of ``batch_size`` (the last
    batch padded with a repeat so data-parallel samplers get a full batch). By default the base model answers
    (``use_base_model=True`` is passed to the sampler so a policy adapter under training is bypassed); ``lora_path``
    selects a dedicated adapter instead.

    Parity: reference ``src/twinkle_agentic/condenser/model.py:104-455``."""

    def __init__(self, sampler, compression_ratio: float = 3.0, sampling_params=None, system_prompt: str = _CONDENSE_SYSTEM,
                 user_prompt_template: str = _CONDENSE_USER, min_chars: int = 600, min_budget_chars: int = 120, keep_last: int = 0,
                 roles: Sequence[str] = ('tool', ), skip_pattern: Optional[str] = None, related_query=None, batch_size: int = 8,
                 lora_path: Optional[str] = None, template=None, chars_per_token: float = 3.0):
        if compression_ratio <= 1:
            raise ValueError('compression_ratio must be > 1')
        if '{text}' not in user_prompt_template or '{budget}' not in user_prompt_template:
            raise ValueError('user_prompt_template needs {budget} and {text}')
        self.sampler, self.ratio, self.sampling_params = sampler, float(compression_ratio), sampling_params
        self.system_prompt, self.user_prompt_template = system_prompt, user_prompt_template
        self.min_chars, self.min_budget, self.keep_last, self.roles = min_chars, min_budget_chars, keep_last, set(roles)
        self.skip_re = re.compile(skip_pattern, re.M) if skip_pattern else None
        self.related_query, self.batch_size, self.lora_path = related_query, max(1, batch_size), lora_path
        self.template, self.chars_per_token = template if template is not None else getattr(sampler, 'template', None), chars_per_token

    def eligible(self, c: Chunk, index: int, total: int) -> bool:
        if c.condensed or c.role not in self.roles or len(c.content) < self.min_chars or index >= total - self.keep_last:
            return False
        return not (self.skip_re and self.skip_re.search(c.content))

    def budget(self, text: str) -> int:
        return max(self.min_budget, math.ceil(len(text) / self.ratio))

    def _special_tokens(self) -> Sequence[str]:
        tok = getattr(self.template, 'tokenizer', None)
        return tuple(t for t in (getattr(tok, 'all_special_tokens', None) or ()) if isinstance(t, str) and t)

    def clean(self, reply: str, original: str) -> Optional[str]:
        text = (reply or '').strip()
        m = _FENCED.match(text)
        if m:
            text = m.group(1).strip()
        for t in self._special_tokens():
            text = text.replace(t, '')
        text = text.strip()
        if not text or not any(ch.isalnum() for ch in text) or len(text) >= len(original):
            return None
        return text

    def _ask(self, jobs: List[Dict[str, Any]]) -> List[str]:
        from ..data_format import SamplingParams
        trajs = [{'messages': [{'role': 'system', 'content': self.system_prompt},
                               {'role': 'user', 'content': self.user_prompt_template.format(budget=j['budget'], text=j['text'], query=j['query'])}]}
                 for j in jobs]
        params = self.sampling_params or SamplingParams(temperature=0.0, max_tokens=max(32, int(max(j['budget'] for j in jobs) / self.chars_per_token * 1.5)))
        kw = {'adapter_path': self.lora_path} if self.lora_path else {'use_base_model': True}
        out: List[str] = []
        for i in range(0, len(trajs), self.batch_size):
            batch = trajs[i:i + self.batch_size]
            real = len(batch)
            batch = batch + [batch[-1]] * (self.batch_size - real if len(trajs) > self.batch_size else 0)
            resps = self.sampler.sample(batch, params, **kw)
            for r in list(resps)[:real]:
                seqs = getattr(r, 'sequences', None) if not isinstance(r, dict) else r.get('sequences')
                seq = seqs[0] if seqs else None
                out.append(((getattr(seq, 'decoded', None) if not isinstance(seq, dict) else seq.get('decoded')) or '') if seq is not None else '')
        return out

    def __call__(self, chunks: Chunks, **kwargs) -> Chunks:
        items = list(chunks)
        jobs, query = [], None
        for i, c in enumerate(items):
            if self.related_query is not None:
                q = self.related_query(c)
                if q:
                    query = q
            if self.eligible(c, i, len(items)):
                jobs.append({'index': i, 'text': c.content, 'budget': self.budget(c.content), 'query': query or '(not stated)'})
        if not jobs:
            return chunks
        replies = self._ask(jobs)
        next_block = 1 + max([c.block or 0 for c in items] + [0])
        for j, reply in zip(jobs, replies):
            c = items[j['index']]
            text = self.clean(reply, c.content)
            if text is None:
                continue
            items[j['index']] = Chunk(c.role, text, c.message_index, c.tool_call_id, True, c.content, next_block, dict(c.extra))
            next_block += 1
        return Chunks(items, chunks.trajectory)


class ExtractCondensed(Tool):
    """Tool through which the policy gets the original text of condensed blocks back."""

    def __init__(self, chunks: Chunks):
        self.originals = {c.block: c.original for c in chunks if c.condensed and c.block is not None}

    def tool_info(self):
        return {'tool_name': 'extract_condensed', 'description': 'Return the full original text of condensed blocks.',
                'parameters': {'type': 'object', 'properties': {'blocks': {'type': 'array', 'items': {'type': 'integer'}}}, 'required': ['blocks']}}

    def __call__(self, tool_name: str, arguments: Dict[str, Any]) -> str:
        blocks = arguments.get('blocks', [])
        if isinstance(blocks, int):
            blocks = [blocks]
        parts = []
        for b in blocks:
            try:
                b = int(b)
            except (TypeError, ValueError):
                parts.append(f'[block {b}] not a block number')
                continue
            parts.append(f'[block {b}] {self.originals[b]}' if b in self.originals else f'[block {b}] unknown; known: {sorted(self.originals)}')
        return '\n\n'.join(parts) if parts else 'no blocks requested'

    def __len__(self) -> int:
        return len(self.originals)

    def __contains__(self, n: Any) -> bool:
        return n in self.originals


class MultiTurnCondenseRollout(MultiTurnRollout):
    """``MultiTurnRollout`` that re-chunks and condenses every live trajectory before each sampling turn once it is
    longer than ``condense_above_chars``, and offers ``extract_condensed`` next to the task's own tools."""

    def __init__(self, sampler, chunker: Optional[Chunker] = None, condenser: Optional[Condenser] = None, condense_above_chars: int = 12000, **kw):
        super().__init__(sampler, **kw)
        self.chunker, self.condenser, self.condense_above_chars = chunker or NativeChunker(), condenser or KeywordCondenser(), condense_above_chars

    def __call__(self, trajectories: List[Trajectory], **kwargs) -> List[Trajectory]:
        base_sampler = self.sampler
        outer = self

        class _CondensingSampler:
            """Presents condensed views to the sampler; the stored trajectories keep their full messages."""

            def sample(self, trajs, params, **kws):
                views = []
                for t in trajs:
                    size = sum(len(m.get('content', '')) for m in t.get('messages', []) if isinstance(m.get('content', ''), str))
                    if size <= outer.condense_above_chars:
                        views.append(t)
                        continue
                    chunks = outer.condenser(outer.chunker(t))
                    view = chunks.to_trajectory()
                    tool = ExtractCondensed(chunks)
                    if len(tool):
                        view['tools'] = list(view.get('tools') or []) + [tool.tool_info()]
                        t.setdefault('user_data', {})
                        if isinstance(t['user_data'], dict):
                            t['user_data']['_extract_condensed'] = tool
                    views.append(view)
                return base_sampler.sample(views, params, **kws)

        # the rollout copies trajectories shallowly, so a user_data dict created here is shared with its working copy
        prepared = []
        for t in trajectories:
            t = dict(t)
            if not isinstance(t.get('user_data'), dict):
                t['user_data'] = {} if t.get('user_data') is None else {'value': t['user_data']}
            prepared.append(t)
        trajectories = prepared
        self.sampler = _CondensingSampler()
        try:
            managers = self._managers(trajectories)
            wrapped = []
            for t, m in zip(trajectories, managers):
                m = m or ToolManager()
                m.register(_LateBound(t))
                wrapped.append(m)
            saved, self.tool_manager = self.tool_manager, wrapped
            try:
                out = super().__call__(trajectories, **kwargs)
            finally:
                self.tool_manager = saved
        finally:
            self.sampler = base_sampler
        for t in out:
            if isinstance(t.get('user_data'), dict):
                t['user_data'].pop('_extract_condensed', None)
        return out


class _LateBound(Tool):
    """``extract_condensed`` bound to whatever condensed view the trajectory had at its latest sampling turn."""

    def __init__(self, traj: Trajectory):
        self.traj = traj

    def tool_info(self):
        return ExtractCondensed(Chunks([])).tool_info()

    def __call__(self, tool_name, arguments):
        tool = (self.traj.get('user_data') or {}).get('_extract_condensed') if isinstance(self.traj.get('user_data'), dict) else None
        return tool(tool_name, arguments) if tool is not None else 'nothing has been condensed yet'
