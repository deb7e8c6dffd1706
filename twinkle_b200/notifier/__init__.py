"""Exception notifiers.

Parity: reference ``src/twinkle/notifier/base.py:10-93`` and ``ding_notifier.py:13-124``: an exception in a
remote call is forwarded to an IM webhook; among all ranks only the one that wins a file-lock claim sends;
the notifier serialises to an environment variable so worker processes can rebuild it.
"""
from __future__ import annotations

import base64
import hashlib
import hmac
import json
import os
import time
import urllib.parse
from typing import Any, Dict, Optional

from ..utils.parallel import claim_once

_ENV = 'TWINKLE_NOTIFIER'


class Notifier:
    kind = 'base'

    def __init__(self, dedup_ttl: float = 60.0, **kwargs):
        self.dedup_ttl = dedup_ttl
        self.sent = []

    def notify(self, text: str) -> bool:
        key = hashlib.sha1(text[:200].encode()).hexdigest()
        if not claim_once(f'notify:{key}', self.dedup_ttl):
            return False
        self._send(text)
        return True

    def _send(self, text: str) -> None:
        self.sent.append(text)

    def to_env(self) -> None:
        os.environ[_ENV] = json.dumps({'kind': self.kind, **self._state()})

    def _state(self) -> Dict[str, Any]:
        return {'dedup_ttl': self.dedup_ttl}

    @staticmethod
    def from_env() -> Optional['Notifier']:
        raw = os.environ.get(_ENV)
        if not raw:
            return None
        d = json.loads(raw)
        cls = {'base': Notifier, 'ding': DingNotifier}[d.pop('kind')]
        return cls(**d)


class DingNotifier(Notifier):
    kind = 'ding'

    def __init__(self, webhook: str = '', secret: str = '', title: str = 'twinkle', **kw):
        super().__init__(**kw)
        self.webhook, self.secret, self.title = webhook, secret, title

    def _state(self):
        return {'webhook': self.webhook, 'secret': self.secret, 'title': self.title, 'dedup_ttl': self.dedup_ttl}

    def _signed_url(self) -> str:
        if not self.secret:
            return self.webhook
        ts = str(round(time.time() * 1000))
        sig = base64.b64encode(hmac.new(self.secret.encode(), f'{ts}\n{self.secret}'.encode(), hashlib.sha256).digest())
        return f'{self.webhook}&timestamp={ts}&sign={urllib.parse.quote_plus(sig)}'

    def _send(self, text: str) -> None:
        super()._send(text)
        if not self.webhook:
            return
        import requests
        try:
            requests.post(self._signed_url(), json={'msgtype': 'markdown', 'markdown': {'title': self.title, 'text': f'### {self.title}\n```\n{text[:3500]}\n```'}},
                          timeout=5)
        except Exception:
            pass
