"""Tool-call wire formats: turning assistant text into ``ToolCall`` records and back.

Covers the four formats the reference ships parsers for (``src/twinkle/template/tools/{qwen,react,cline,vcp}.py``):

* ``hermes`` — ``<tool_call>{"name": …, "arguments": {…}}</tool_call>`` (Qwen / Hermes chat templates);
* ``react``  — ``Action: name`` / ``Action Input: {…}`` lines, observations fed back as ``Observation: …``;
* ``cline``  — one XML element per call, its children are the arguments: ``<read_file><path>a.py</path></read_file>``;
* ``vcp``    — ``<<<[TOOL_REQUEST]>>>`` blocks with ``key:「始」value「末」`` pairs (``「始ESCAPE」…「末ESCAPE」`` when the value
  itself contains markers); the function name is the ``tool_name`` pair.

Every format offers ``detect``, ``parse`` (→ list of ``ToolCall``), ``strip`` (text with the call syntax removed) and
``render`` (a call back to text, used when a trajectory recorded in one format is re-templated in another).
``parse_tool_calls`` tries the formats in order and returns the first that matches.
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..data_format.types import ToolCall


def _call(name: str, arguments: Any) -> ToolCall:
    return ToolCall(id=f'call_{uuid.uuid4().hex[:8]}', type='function', tool_name=name, arguments=arguments)


def _loads_lenient(text: str) -> Any:
    text = text.strip()
    if not text:
        return {}
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        pass
    try:  # single quotes / trailing commas written by small models
        fixed = re.sub(r',\s*([}\]])', r'\1', text.replace("'", '"'))
        return json.loads(fixed)
    except json.JSONDecodeError:
        return text


class ToolCallFormat:
    name = ''

    def detect(self, text: str) -> bool:
        raise NotImplementedError

    def parse(self, text: str) -> List[ToolCall]:
        raise NotImplementedError

    def strip(self, text: str) -> str:
        raise NotImplementedError

    def render(self, call: ToolCall) -> str:
        raise NotImplementedError


class HermesFormat(ToolCallFormat):
    name = 'hermes'
    _RE = re.compile(r'<tool_call>\s*(.*?)\s*</tool_call>', re.S)

    def detect(self, text):
        return '<tool_call>' in (text or '')

    def parse(self, text):
        out = []
        for m in self._RE.finditer(text or ''):
            obj = _loads_lenient(m.group(1))
            if isinstance(obj, dict) and (obj.get('name') or obj.get('tool_name')):
                out.append(_call(obj.get('name') or obj.get('tool_name'), obj.get('arguments', obj.get('parameters', {}))))
        return out

    def strip(self, text):
        return self._RE.sub('', text or '').strip()

    def render(self, call):
        args = call.get('arguments', {})
        if isinstance(args, str):
            args = _loads_lenient(args)
        return '<tool_call>\n' + json.dumps({'name': call.get('tool_name'), 'arguments': args}, ensure_ascii=False) + '\n</tool_call>'


class ReActFormat(ToolCallFormat):
    name = 'react'
    _RE = re.compile(r'Action\s*:\s*(?P<name>[^\n]+?)\s*\n\s*Action Input\s*:\s*(?P<args>.*?)(?=\n\s*(?:Observation|Thought|Action)\s*:|\Z)', re.S)

    def detect(self, text):
        return bool(re.search(r'^\s*Action\s*:', text or '', re.M)) and 'Action Input' in (text or '')

    def parse(self, text):
        return [_call(m.group('name').strip(), _loads_lenient(m.group('args'))) for m in self._RE.finditer(text or '')]

    def strip(self, text):
        return self._RE.sub('', text or '').strip()

    def render(self, call):
        args = call.get('arguments', {})
        return f"Action: {call.get('tool_name')}\nAction Input: {args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}"


class ClineFormat(ToolCallFormat):
    """``known_tools`` limits which element names count as calls (prose may contain other tags such as ``<thinking>``)."""
    name = 'cline'
    _SKIP = {'thinking', 'think', 'answer', 'tool_call', 'tool_response', 'tools'}

    def __init__(self, known_tools: Optional[Sequence[str]] = None):
        self.known = set(known_tools) if known_tools else None
        self._outer = re.compile(r'<(?P<tag>[A-Za-z_][\w\-]*)>\s*(?P<body>(?:<[A-Za-z_][\w\-]*>.*?</[A-Za-z_][\w\-]*>\s*)+)</(?P=tag)>', re.S)
        self._inner = re.compile(r'<(?P<k>[A-Za-z_][\w\-]*)>(?P<v>.*?)</(?P=k)>', re.S)

    def _is_call(self, tag: str) -> bool:
        return tag in self.known if self.known is not None else tag not in self._SKIP

    def detect(self, text):
        return any(self._is_call(m.group('tag')) for m in self._outer.finditer(text or ''))

    def parse(self, text):
        out = []
        for m in self._outer.finditer(text or ''):
            if not self._is_call(m.group('tag')):
                continue
            args = {i.group('k'): i.group('v').strip() for i in self._inner.finditer(m.group('body'))}
            out.append(_call(m.group('tag'), args))
        return out

    def strip(self, text):
        return self._outer.sub(lambda m: '' if self._is_call(m.group('tag')) else m.group(0), text or '').strip()

    def render(self, call):
        args = call.get('arguments', {})
        if isinstance(args, str):
            args = _loads_lenient(args)
        body = '\n'.join(f'<{k}>{v}</{k}>' for k, v in (args.items() if isinstance(args, dict) else [('input', args)]))
        return f"<{call.get('tool_name')}>\n{body}\n</{call.get('tool_name')}>"


class VCPFormat(ToolCallFormat):
    name = 'vcp'
    OPEN, CLOSE = '<<<[TOOL_REQUEST]>>>', '<<<[END_TOOL_REQUEST]>>>'
    _BLOCK = re.compile(re.escape(OPEN) + r'(.*?)' + re.escape(CLOSE), re.S)
    _PAIR = re.compile(r'(?P<k>[A-Za-z_]\w*)\s*:\s*(?:「始ESCAPE」(?P<e>.*?)「末ESCAPE」|「始」(?P<v>.*?)「末」)', re.S)

    def detect(self, text):
        return self.OPEN in (text or '')

    def parse(self, text):
        out = []
        for block in self._BLOCK.findall(text or ''):
            name, args = '', {}
            for m in self._PAIR.finditer(block):
                val = m.group('e') if m.group('e') is not None else m.group('v')
                if m.group('k') == 'tool_name':
                    name = (val or '').strip()
                else:
                    args[m.group('k')] = val
            if name:
                out.append(_call(name, args))
        return out

    def strip(self, text):
        return self._BLOCK.sub('', text or '').strip()

    def render(self, call):
        args = call.get('arguments', {})
        if isinstance(args, str):
            args = _loads_lenient(args)

        def wrap(v):
            v = v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)
            return f'「始ESCAPE」{v}「末ESCAPE」' if ('「末」' in v or self.OPEN in v) else f'「始」{v}「末」'

        lines = [f"tool_name:{wrap(call.get('tool_name', ''))}"] + [f'{k}:{wrap(v)}' for k, v in (args.items() if isinstance(args, dict) else [])]
        return self.OPEN + '\n' + ',\n'.join(lines) + '\n' + self.CLOSE


FORMATS: Dict[str, type] = {'hermes': HermesFormat, 'qwen': HermesFormat, 'react': ReActFormat, 'cline': ClineFormat, 'vcp': VCPFormat}


def get_format(name: str, **kwargs) -> ToolCallFormat:
    if name not in FORMATS:
        raise KeyError(f'unknown tool-call format {name!r}; known: {sorted(FORMATS)}')
    return FORMATS[name](**kwargs) if name == 'cline' else FORMATS[name]()


def parse_tool_calls(text: str, formats: Sequence[str] = ('hermes', 'vcp', 'react', 'cline'), known_tools: Optional[Sequence[str]] = None) -> Tuple[List[ToolCall], str, Optional[str]]:
    """(calls, text without the call syntax, name of the format that matched or None)."""
    for name in formats:
        f = get_format(name, **({'known_tools': known_tools} if name == 'cline' else {}))
        if f.detect(text):
            calls = f.parse(text)
            if calls:
                return calls, f.strip(text), f.name
    return [], text or '', None


def tools_system_prompt(tools: Sequence[Dict[str, Any]], fmt: str = 'hermes') -> str:
    """A system-prompt section that describes the tools and the expected call syntax of ``fmt``."""
    f = get_format(fmt)
    specs = '\n'.join(json.dumps({'name': t.get('tool_name'), 'description': t.get('description', ''), 'parameters': t.get('parameters', {})},
                                 ensure_ascii=False) for t in tools)
    example = f.render(ToolCall(tool_name='tool_name', arguments={'argument': 'value'}))
    return f'# Tools\nYou may call these functions:\n{specs}\n\nTo call one, write:\n{example}'
