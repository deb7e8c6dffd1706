"""Deterministic seeds from arbitrary keys.  Parity: reference
``src/twinkle/utils/seed.py`` (sha256-based ``stable_seed``)."""
from __future__ import annotations

import hashlib
import json


def stable_seed(*parts, modulo: int = 2**31 - 1) -> int:
    blob = json.dumps([repr(p) if not isinstance(p, (str, int, float, bool, type(None))) else p for p in parts],
                      sort_keys=True, separators=(',', ':')).encode()
    return int.from_bytes(hashlib.sha256(blob).digest()[:8], 'big') % modulo
