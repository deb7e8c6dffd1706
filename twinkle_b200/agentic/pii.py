"""Rewrites personal data in trajectories instead of dropping the rows: every detected span is masked, replaced with a
plausible fake value, removed, or hashed — chosen per entity type — and the same source value always gets the same
replacement, so a dialogue that mentions an address twice stays coherent.

Detection is pattern- and checksum-based and needs no model: e-mail, URL, IPv4, phone (international and mainland-China
mobile), payment card (Luhn-checked), IBAN (mod-97 checked), US SSN, mainland-China resident id (check digit verified).
Names, places and organisations need a tagger; ``ner_fn(text) -> [(start, end, 'PERSON' | 'LOCATION' | 'ORGANIZATION')]``
plugs one in.

Parity: reference ``src/twinkle_agentic/preprocessor/pii_presidio_filter.py`` (Presidio + spaCy + Faker there; none of the
three is available offline, so detection and fake values are restated on the standard library)."""
from __future__ import annotations

import hashlib
import re
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from ..preprocessor import Preprocessor


class Strategy(str, Enum):
    MASK = 'mask'        # keep the edges, star the middle (ids, cards, phones)
    REPLACE = 'replace'  # a fake value of the same kind (names, e-mail) — keeps the text fluent
    REDACT = 'redact'    # remove the span
    HASH = 'hash'        # 12 hex digits of sha256 — de-identified but still joinable

    @classmethod
    def coerce(cls, v) -> 'Strategy':
        try:
            return v if isinstance(v, cls) else cls(v)
        except ValueError:
            raise ValueError(f'unknown strategy {v!r}; allowed: {[s.value for s in cls]}') from None


def luhn_ok(s: str) -> bool:
    d = [int(c) for c in s if c.isdigit()]
    if len(d) < 13:
        return False
    total = 0
    for i, x in enumerate(reversed(d)):
        if i % 2:
            x = x * 2 - 9 if x * 2 > 9 else x * 2
        total += x
    return total % 10 == 0


def cn_id_ok(s: str) -> bool:
    if len(s) != 18 or not s[:17].isdigit():
        return False
    w = (7, 9, 10, 5, 8, 4, 2, 1, 6, 3, 7, 9, 10, 5, 8, 4, 2)
    return '10X98765432'[sum(int(c) * k for c, k in zip(s, w)) % 11] == s[17].upper()


def iban_ok(s: str) -> bool:
    s = s.replace(' ', '').upper()
    if not (15 <= len(s) <= 34) or not s[:2].isalpha() or not s[2:4].isdigit():
        return False
    moved = s[4:] + s[:4]
    return int(''.join(str(int(c, 36)) for c in moved)) % 97 == 1


def mask_keep_edges(s: str, head: int = 3, tail: int = 4, ch: str = '*') -> str:
    return ch * len(s) if len(s) <= head + tail else s[:head] + ch * (len(s) - head - tail) + s[-tail:]


def hash_short(s: str, salt: str = '') -> str:
    return hashlib.sha256((salt + s).encode()).hexdigest()[:12]


# entity → (pattern, validator or None). Order matters: earlier entities win overlaps.
_PATTERNS: List[Tuple[str, 're.Pattern', Optional[Callable[[str], bool]]]] = [
    ('EMAIL_ADDRESS', re.compile(r'\b[\w.+-]+@[\w-]+(?:\.[\w-]+)+\b'), None),
    ('URL', re.compile(r'\bhttps?://[^\s<>"\')\]]+(?<![.,;:!?])', re.I), None),
    ('CN_ID', re.compile(r'(?<![\dA-Za-z])\d{17}[\dXx](?![\dA-Za-z])'), cn_id_ok),
    ('IBAN_CODE', re.compile(r'\b[A-Z]{2}\d{2}(?: ?[A-Z0-9]{4}){2,7}(?: ?[A-Z0-9]{1,4})?\b'), iban_ok),
    ('CREDIT_CARD', re.compile(r'(?<!\d)(?:\d[ -]?){12,18}\d(?!\d)'), luhn_ok),
    ('US_SSN', re.compile(r'(?<!\d)(?!000|666|9\d\d)\d{3}-(?!00)\d{2}-(?!0000)\d{4}(?!\d)'), None),
    ('IP_ADDRESS', re.compile(r'(?<![\d.])(?:(?:25[0-5]|2[0-4]\d|1?\d?\d)\.){3}(?:25[0-5]|2[0-4]\d|1?\d?\d)(?![\d.])'), None),
    ('CN_PHONE', re.compile(r'(?<!\d)(?:\+?86[ -]?)?1[3-9]\d{9}(?!\d)'), None),
    ('PHONE_NUMBER', re.compile(r'(?<![\d+])(?<!\d[ -])(?:\+\d{1,3}[ -]?)?(?:\(\d{2,4}\)[ -]?|\d{2,4}[ -])\d{3,4}[ -]\d{3,4}(?![ -]?\d)'), None),
]

DEFAULT_STRATEGY: Dict[str, Strategy] = {
    'EMAIL_ADDRESS': Strategy.REPLACE, 'URL': Strategy.REPLACE, 'IP_ADDRESS': Strategy.REPLACE, 'PERSON': Strategy.REPLACE,
    'LOCATION': Strategy.REPLACE, 'ORGANIZATION': Strategy.REPLACE, 'PHONE_NUMBER': Strategy.MASK, 'CN_PHONE': Strategy.MASK,
    'CREDIT_CARD': Strategy.MASK, 'IBAN_CODE': Strategy.MASK, 'US_SSN': Strategy.MASK, 'CN_ID': Strategy.MASK,
}

_FIRST = ('Alex', 'Sam', 'Jordan', 'Taylor', 'Morgan', 'Casey', 'Riley', 'Jamie', 'Avery', 'Quinn', 'Robin', 'Drew')
_LAST = ('Hale', 'Marsh', 'Lund', 'Voss', 'Keane', 'Rowe', 'Pike', 'Dunn', 'Frost', 'Wren', 'Cole', 'Nash')
_PLACE = ('Elmford', 'Lakemont', 'Ashbury', 'Northvale', 'Pinehurst', 'Redwater', 'Stonefield', 'Westbrook')
_ORG = ('Northwind Ltd', 'Bluepeak Group', 'Harbor Labs', 'Cinder Systems', 'Vale & Co', 'Orchard Works')


def fake_value(entity: str, source: str, salt: str = '') -> str:
    """Deterministic stand-in of the right kind, derived from a hash of the source value (no random state)."""
    h = int(hashlib.sha256((salt + entity + source).encode()).hexdigest(), 16)
    pick = lambda seq, shift=0: seq[(h >> shift) % len(seq)]  # noqa: E731
    if entity == 'EMAIL_ADDRESS':
        return f'{pick(_FIRST).lower()}.{pick(_LAST, 8).lower()}{h % 100}@example.com'
    if entity == 'URL':
        return f'https://example.com/{hash_short(source, salt)[:8]}'
    if entity == 'IP_ADDRESS':
        return f'192.0.2.{h % 254 + 1}'  # TEST-NET-1, never routed
    if entity == 'PERSON':
        return f'{pick(_FIRST)} {pick(_LAST, 8)}'
    if entity == 'LOCATION':
        return pick(_PLACE)
    if entity == 'ORGANIZATION':
        return pick(_ORG)
    digits = ''.join(str((h >> (4 * i)) % 10) if c.isdigit() else c for i, c in enumerate(source))
    return digits


class PIIRewriter(Preprocessor):
    """Pipeline step ``rows -> (rows, [])``: rewrites string contents of the given roles in place of the originals.

    ``entity_strategy`` overrides :data:`DEFAULT_STRATEGY` per entity; ``entities`` restricts detection; ``salt`` makes
    hashes and fake values specific to a deployment; ``persistent_consistency`` keeps the source → replacement map
    across calls (default: per call). ``last_report`` counts the rewrites of the latest call per entity."""

    def __init__(self, entity_strategy: Optional[Dict[str, Any]] = None, entities: Optional[Sequence[str]] = None,
                 roles: Sequence[str] = ('system', 'user', 'assistant', 'tool'), ner_fn: Optional[Callable[[str], List[Tuple[int, int, str]]]] = None,
                 salt: str = '', persistent_consistency: bool = False):
        self.strategy = dict(DEFAULT_STRATEGY)
        for k, v in (entity_strategy or {}).items():
            self.strategy[k] = Strategy.coerce(v)
        self.entities = set(entities) if entities is not None else None
        self.roles, self.ner_fn, self.salt, self.persistent = set(roles), ner_fn, salt, persistent_consistency
        self._map: Dict[Tuple[str, str], str] = {}
        self.last_report: Dict[str, int] = {}

    def detect(self, text: str) -> List[Tuple[int, int, str]]:
        """Non-overlapping ``(start, end, entity)`` spans, left to right."""
        spans: List[Tuple[int, int, str]] = []
        taken = [False] * (len(text) + 1)
        found = []
        for ent, pat, ok in _PATTERNS:
            if self.entities is not None and ent not in self.entities:
                continue
            found.extend((m.start(), m.end(), ent) for m in pat.finditer(text) if ok is None or ok(m.group(0)))
        if self.ner_fn is not None:
            found.extend((a, b, e) for a, b, e in self.ner_fn(text) if self.entities is None or e in self.entities)
        for a, b, ent in found:  # pattern order = priority
            if a < b and not any(taken[a:b]):
                taken[a:b] = [True] * (b - a)
                spans.append((a, b, ent))
        return sorted(spans)

    def _replacement(self, ent: str, src: str) -> str:
        key = (ent, src)
        if key not in self._map:
            how = self.strategy.get(ent, Strategy.MASK)
            self._map[key] = {Strategy.MASK: lambda: mask_keep_edges(src), Strategy.REPLACE: lambda: fake_value(ent, src, self.salt),
                              Strategy.REDACT: lambda: '', Strategy.HASH: lambda: hash_short(src, self.salt)}[how]()
        return self._map[key]

    def rewrite(self, text: str) -> str:
        out, last = [], 0
        for a, b, ent in self.detect(text):
            out.append(text[last:a])
            out.append(self._replacement(ent, text[a:b]))
            self.last_report[ent] = self.last_report.get(ent, 0) + 1
            last = b
        out.append(text[last:])
        return ''.join(out)

    def __call__(self, rows: List[Dict[str, Any]]):
        if not self.persistent:
            self._map = {}
        self.last_report = {}
        rows = list(rows)
        for row in rows:
            for m in row.get('messages') or []:
                if isinstance(m, dict) and m.get('role') in self.roles and isinstance(m.get('content'), str):
                    m['content'] = self.rewrite(m['content'])
        return rows, []


PIIPresidioFilter = PIIRewriter  # the reference's class name for this pipeline step
