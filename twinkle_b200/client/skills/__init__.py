"""Skills: markdown documents with a small front-matter header that are put into the auto agent's system prompt.

Parity: reference ``src/twinkle_client/skills/`` (``Skill``, ``SkillProvider`` with a cache directory and markdown
scan, local-directory provider, hub provider, ``SkillManager.format_for_prompt``).  A skill file looks like::

    ---
    name: twinkle-training
    description: how to write a training script
    ---
    # body in markdown …

The hub-backed provider resolves a repository through :class:`twinkle_b200.hub.HubOperation`, which only reads
local caches when the host is offline; a provider that cannot fetch contributes nothing and is reported, never fatal.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional


@dataclass
class Skill:
    name: str
    description: str
    content: str
    source: str = ''
    path: Optional[str] = None
    meta: Dict[str, str] = field(default_factory=dict)


_FRONT = re.compile(r'\A---\s*\n(.*?)\n---\s*\n', re.S)


def parse_skill(text: str, default_name: str, source: str = '', path: Optional[str] = None) -> Skill:
    meta: Dict[str, str] = {}
    m = _FRONT.match(text)
    body = text
    if m:
        body = text[m.end():]
        for ln in m.group(1).splitlines():
            if ':' in ln and not ln.lstrip().startswith('#'):
                k, v = ln.split(':', 1)
                meta[k.strip().lower()] = v.strip().strip('"\'')
    if 'description' not in meta:
        first = next((ln.strip('# ').strip() for ln in body.splitlines() if ln.strip()), '')
        meta['description'] = first[:200]
    return Skill(meta.get('name') or default_name, meta['description'], body.strip(), source, path, meta)


class SkillProvider:
    name = 'provider'

    def fetch(self) -> None:
        """Bring the skill files to local disk if they are not there (no-op for local providers)."""

    def root(self) -> Optional[Path]:
        raise NotImplementedError

    def load(self) -> List[Skill]:
        self.fetch()
        root = self.root()
        if root is None or not root.is_dir():
            return []
        out = []
        for f in sorted(root.rglob('*.md')):
            if f.name.lower() in ('readme.md', 'license.md'):
                continue
            try:
                out.append(parse_skill(f.read_text(encoding='utf-8'), f.stem, self.name, str(f)))
            except OSError:
                continue
        return out


class LocalSkillProvider(SkillProvider):

    def __init__(self, directory: os.PathLike, name: Optional[str] = None):
        self.directory = Path(directory).expanduser()
        self.name = name or f'local:{self.directory.name}'

    def root(self) -> Optional[Path]:
        return self.directory


class BundledSkillProvider(LocalSkillProvider):

    def __init__(self):
        super().__init__(Path(__file__).parent / 'bundled', 'bundled')


class HubSkillProvider(SkillProvider):
    """Skills kept in a model-hub repository (``ms://org/repo`` or ``hf://org/repo``)."""

    def __init__(self, repo_id: str, subdir: str = ''):
        self.repo_id, self.subdir, self.name = repo_id, subdir, f'hub:{repo_id}'
        self._dir: Optional[Path] = None

    def fetch(self) -> None:
        if self._dir is None:
            from ...hub import HubOperation
            self._dir = Path(HubOperation.download_model(self.repo_id)) / self.subdir

    def root(self) -> Optional[Path]:
        return self._dir


class SkillManager:

    def __init__(self, providers: Optional[List[SkillProvider]] = None):
        self.providers: List[SkillProvider] = list(providers or [])
        self.skills: List[Skill] = []
        self.errors: Dict[str, str] = {}

    def register(self, provider: SkillProvider) -> None:
        self.providers.append(provider)

    def load_all(self) -> List[Skill]:
        """Later providers override earlier ones on a name clash, so a user's directory can replace a bundled skill."""
        by_name: Dict[str, Skill] = {}
        self.errors = {}
        for p in self.providers:
            try:
                for s in p.load():
                    by_name[s.name] = s
            except Exception as e:
                self.errors[p.name] = f'{type(e).__name__}: {e}'
        self.skills = list(by_name.values())
        return self.skills

    def names(self) -> List[str]:
        return [s.name for s in self.skills]

    def format_for_prompt(self, max_chars: int = 60_000) -> str:
        """All skills in full while they fit; after that only name and description, so the model at least knows
        what it could ask the user to paste."""
        if not self.skills:
            return ''
        parts, used = ['# Skills\nReference material for this installation. Follow it when writing scripts.'], 0
        for s in self.skills:
            block = f'\n## Skill: {s.name}\n{s.description}\n\n{s.content}\n'
            if used + len(block) > max_chars:
                block = f'\n## Skill: {s.name} (summary only)\n{s.description}\n'
            parts.append(block)
            used += len(block)
        return ''.join(parts)


def default_manager(extra_dirs: Optional[List[str]] = None) -> SkillManager:
    m = SkillManager([BundledSkillProvider()])
    user = Path(os.environ.get('TWINKLE_SKILLS_DIR', str(Path.home() / '.config' / 'twinkle_b200' / 'skills')))
    if user.is_dir():
        m.register(LocalSkillProvider(user, 'user'))
    for d in extra_dirs or []:
        m.register(HubSkillProvider(d) if '://' in d else LocalSkillProvider(d))
    return m
