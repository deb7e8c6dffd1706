"""Chat-completion clients for the auto agent: an OpenAI-compatible HTTP client and a scripted stand-in.

Parity: reference ``src/twinkle_client/auto/agent/core.py:112-178`` (streamed chat completion with tool calls
against an OpenAI-compatible endpoint).  The reply is one dict: ``{'content': str, 'tool_calls': [{'id', 'name',
'arguments': dict}]}``; streaming delivers text pieces to ``on_text`` as they arrive.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Iterable, List, Optional

Reply = Dict[str, Any]


def _parse_args(raw: Any) -> Dict[str, Any]:
    if isinstance(raw, dict):
        return raw
    try:
        v = json.loads(raw or '{}')
        return v if isinstance(v, dict) else {'value': v}
    except ValueError:
        return {'_raw': raw}


class ChatLLM:
    """``POST {base_url}/chat/completions``.  Environment: ``TWINKLE_AUTO_LLM_URL`` / ``_KEY`` / ``_MODEL``
    (falling back to ``OPENAI_BASE_URL`` / ``OPENAI_API_KEY``)."""

    def __init__(self, base_url: Optional[str] = None, api_key: Optional[str] = None, model: Optional[str] = None, timeout: float = 300.0):
        self.base_url = (base_url or os.environ.get('TWINKLE_AUTO_LLM_URL') or os.environ.get('OPENAI_BASE_URL') or 'http://127.0.0.1:8000/v1').rstrip('/')
        self.api_key = api_key or os.environ.get('TWINKLE_AUTO_LLM_KEY') or os.environ.get('OPENAI_API_KEY') or 'EMPTY'
        self.model = model or os.environ.get('TWINKLE_AUTO_LLM_MODEL') or 'default'
        self.timeout = timeout

    def chat(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]] = None, temperature: float = 0.3,
             max_tokens: int = 4096, on_text: Optional[Callable[[str], None]] = None) -> Reply:
        import requests
        body: Dict[str, Any] = dict(model=self.model, messages=messages, temperature=temperature, max_tokens=max_tokens, stream=on_text is not None)
        if tools:
            body['tools'] = tools
        r = requests.post(self.base_url + '/chat/completions', json=body, timeout=self.timeout, stream=on_text is not None,
                          headers={'Authorization': f'Bearer {self.api_key}'})
        r.raise_for_status()
        if on_text is None:
            msg = r.json()['choices'][0]['message']
            calls = [dict(id=c.get('id', ''), name=c['function']['name'], arguments=_parse_args(c['function'].get('arguments')))
                     for c in msg.get('tool_calls') or []]
            return dict(content=msg.get('content') or '', tool_calls=calls)
        return merge_stream(iter_sse(r.iter_lines()), on_text)


def iter_sse(lines: Iterable[bytes]) -> Iterable[Dict[str, Any]]:
    for ln in lines:
        if isinstance(ln, bytes):
            ln = ln.decode('utf-8', 'replace')
        if not ln.startswith('data:'):
            continue
        data = ln[5:].strip()
        if data == '[DONE]':
            return
        try:
            yield json.loads(data)
        except ValueError:
            continue


def merge_stream(chunks: Iterable[Dict[str, Any]], on_text: Optional[Callable[[str], None]] = None) -> Reply:
    """Fold streamed deltas into one reply.  Tool-call fragments are keyed by their ``index``; the name arrives
    once and the argument string in pieces."""
    text: List[str] = []
    calls: Dict[int, Dict[str, str]] = {}
    for ch in chunks:
        for choice in ch.get('choices') or []:
            d = choice.get('delta') or {}
            if d.get('content'):
                text.append(d['content'])
                if on_text:
                    on_text(d['content'])
            for tc in d.get('tool_calls') or []:
                slot = calls.setdefault(int(tc.get('index', 0)), dict(id='', name='', arguments=''))
                slot['id'] = tc.get('id') or slot['id']
                fn = tc.get('function') or {}
                slot['name'] = fn.get('name') or slot['name']
                slot['arguments'] += fn.get('arguments') or ''
    return dict(content=''.join(text),
                tool_calls=[dict(id=c['id'] or f'call_{i}', name=c['name'], arguments=_parse_args(c['arguments'])) for i, c in sorted(calls.items()) if c['name']])


class ScriptedLLM:
    """Replays prepared replies (strings, reply dicts, or callables of the message list).  Used by tests and by
    ``twinkle-auto --dry-run``; records every request it saw in ``requests``."""

    def __init__(self, replies: Iterable[Any], default: str = 'LGTM'):
        self.replies = list(replies)
        self.default = default
        self.requests: List[Dict[str, Any]] = []

    def chat(self, messages, tools=None, temperature: float = 0.3, max_tokens: int = 4096, on_text=None) -> Reply:
        self.requests.append(dict(messages=[dict(m) for m in messages], tools=tools))
        r = self.replies.pop(0) if self.replies else self.default
        if callable(r):
            r = r(messages)
        if isinstance(r, str):
            r = dict(content=r, tool_calls=[])
        r = dict(content=r.get('content', ''), tool_calls=[dict(id=c.get('id', f'call_{i}'), name=c['name'], arguments=_parse_args(c.get('arguments', {})))
                                                          for i, c in enumerate(r.get('tool_calls') or [])])
        if on_text and r['content']:
            on_text(r['content'])
        return r
