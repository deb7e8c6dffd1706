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
