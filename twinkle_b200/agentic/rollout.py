"""Multi-turn rollouts: the policy samples an assistant turn, tool calls are executed, observations are appended,
until every trajectory stops calling tools or the turn budget is spent.

What it covers: reference ``src/twinkle_agentic/rollout/{base,multi_turn,bridge,api_multi_turn}.py``.  All live
trajectories of a batch are sampled together each turn (one ``sampler.sample`` call per turn).  For training the
token-exact history matters: the tokens the sampler produced are kept as they are and only the *bridge* — what the
chat template puts between the end of one assistant turn and the next generation prompt (tool results, role
headers) — is tokenised and appended with ``labels = -100``, so log-probs computed at training time line up with
the sampled tokens.
"""
from __future__ import annotations

import json
import os
import re
import uuid
from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

from ..data_format.sampling import SamplingParams
from ..data_format.types import Message, ToolCall, Trajectory
from .tools import ToolManager

_TOOL_CALL = re.compile(r'<tool_call>\s*(\{.*?\})\s*</tool_call>', re.S)


def parse_tool_calls(text: str) -> List[ToolCall]:
    """Hermes / Qwen style ``<tool_call>{"name": …, "arguments": {…}}</tool_call>`` blocks."""
    calls = []
    for m in _TOOL_CALL.finditer(text or ''):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        name = obj.get('name') or obj.get('tool_name')
        if not name:
            continue
        calls.append(ToolCall(id=f'call_{uuid.uuid4().hex[:8]}', type='function', tool_name=name, arguments=obj.get('arguments', {})))
    return calls


def strip_tool_calls(text: str) -> str:
    return _TOOL_CALL.sub('', text or '').strip()


class Rollout(ABC):

    @abstractmethod
    def __call__(self, trajectories: List[Trajectory], **kwargs) -> List[Trajectory]:
        ...


def extend_with_bridge(template, feature: Dict[str, Any], messages: List[Message], new_messages: List[Message], tools=None) -> Dict[str, Any]:
    """Append the tokens the chat template renders for ``new_messages`` (+ the next generation prompt) to a
    token-exact ``feature``; the appended span is excluded from the loss."""
    before = template._render(messages, tools=tools, add_generation_prompt=False)
    after = template._render(messages + new_messages, tools=tools, add_generation_prompt=True)
    # the rendered prefix may differ from the sampled tokens (e.g. whitespace normalisation): only the tail is used
    common = 0
    for a, b in zip(before, after):
        if a != b:
            break
        common += 1
    bridge = list(after[common:])
    out = dict(feature)
    out['input_ids'] = list(feature['input_ids']) + bridge
    out['labels'] = list(feature.get('labels', [-100] * len(feature['input_ids']))) + [-100] * len(bridge)
    if 'completion_mask' in feature:
        out['completion_mask'] = list(feature['completion_mask']) + [0] * len(bridge)
    out['length'] = len(out['input_ids'])
    if feature.get('mrope_position_ids') is not None:  # vision-language state: the appended text continues all three position rows
        import torch
        m = torch.as_tensor(feature['mrope_position_ids']).long()
        nxt = int(m.max()) + 1 if m.numel() else 0
        out['mrope_position_ids'] = torch.cat([m, torch.arange(nxt, nxt + len(bridge)).expand(3, -1)], 1)
    for k in ('position_ids', 'attention_mask'):
        if k in out:
            out[k] = list(range(out['length'])) if k == 'position_ids' else [1] * out['length']
    return out


class MultiTurnRollout(Rollout):
    """``sampler`` needs ``sample(trajectories, sampling_params)`` returning one ``SampleResponse`` per trajectory
    (decoded text in ``sequences[0].decoded``) — the native sampler, its HTTP twin and ``RouterSampler`` all do."""

    def __init__(self, sampler, tool_manager: Union[ToolManager, Sequence[ToolManager], Callable[[Sequence[Trajectory]], List[ToolManager]], None] = None,
                 max_turns: int = 8, sampling_params: Optional[SamplingParams] = None, stop_on_no_tool_call: bool = True,
                 trace_dir: Optional[str] = None, adapter_name: Optional[str] = None, tool_format: str = 'hermes'):
        # tool_format: 'hermes' (the <tool_call> JSON blocks Qwen models write), 'react', 'cline', 'vcp', or 'auto' (first that matches)
        self.tool_format = tool_format
        self.sampler, self.tool_manager = sampler, tool_manager
        self.max_turns, self.stop_on_no_tool_call = max_turns, stop_on_no_tool_call
        self.sampling_params = sampling_params or SamplingParams(max_tokens=512)
        self.trace_dir, self.adapter_name = trace_dir, adapter_name

    def _managers(self, trajectories: Sequence[Trajectory]) -> List[Optional[ToolManager]]:
        tm = self.tool_manager
        if tm is None:
            return [None] * len(trajectories)
        if isinstance(tm, ToolManager):
            return [tm.copy() for _ in trajectories]
        if callable(tm) and not isinstance(tm, (list, tuple)):
            return list(tm(trajectories))
        if len(tm) != len(trajectories):
            raise ValueError('one tool manager per trajectory is required')
        return list(tm)

    def __call__(self, trajectories: List[Trajectory], **kwargs) -> List[Trajectory]:
        managers = self._managers(trajectories)
        trajs: List[Trajectory] = []
        for t, m in zip(trajectories, managers):
            t = dict(t)
            t['messages'] = [dict(x) for x in t.get('messages', [])]
            if m is not None and not t.get('tools'):
                t['tools'] = m.tool_infos()
            t.setdefault('user_data', {})
            trajs.append(t)
        live = list(range(len(trajs)))
        stats = [{'turns': 0, 'tool_calls': 0, 'tokens': 0, 'logprobs': [], 'stop': 'max_turns'} for _ in trajs]
        for _turn in range(self.max_turns):
            if not live:
                break
            resps = self.sampler.sample([trajs[i] for i in live], self.sampling_params,
                                        **({'adapter_name': self.adapter_name} if self.adapter_name else {}))
            if callable(resps):  # lazy collect
                resps = resps()
            nxt = []
            for i, resp in zip(live, resps):
                seq = resp.sequences[0]
                text = seq.decoded if seq.decoded is not None else ''
                if self.tool_format == 'hermes':
                    calls = parse_tool_calls(text)
                    clean = strip_tool_calls(text) if calls else text
                else:
                    from ..template.tools import parse_tool_calls as parse_any
                    fmts = ('hermes', 'vcp', 'react', 'cline') if self.tool_format == 'auto' else (self.tool_format, )
                    known = managers[i].names() if managers[i] is not None else None
                    calls, clean, _ = parse_any(text, fmts, known_tools=known)
                msg: Message = {'role': 'assistant', 'content': clean}
                if calls:
                    msg['tool_calls'] = calls
                trajs[i]['messages'].append(msg)
                st = stats[i]
                st['turns'] += 1
                st['tokens'] += len(seq.tokens)
                if seq.logprobs:
                    st['logprobs'].append(list(seq.logprobs))
                if seq.stop_reason == 'length':
                    st['stop'] = 'length'
                    continue
                m = managers[i]
                if not calls or m is None:
                    if self.stop_on_no_tool_call or m is None:
                        st['stop'] = 'answer'
                        continue
                for c in calls:
                    obs = m(c)
                    trajs[i]['messages'].append({'role': 'tool', 'content': obs, 'tool_call_id': c['id']})
                    st['tool_calls'] += 1
                done = any(getattr(t, 'done', False) for t in getattr(m, '_tools', {}).values())
                if done:
                    st['stop'] = 'env_done'
                    continue
                nxt.append(i)
            live = nxt
        for t, st, m in zip(trajs, stats, managers):
            ud = t['user_data'] if isinstance(t['user_data'], dict) else {'value': t['user_data']}
            ud['rollout'] = {k: v for k, v in st.items() if k != 'logprobs'}
            if m is not None:
                rewards = [tool.episode_reward for tool in getattr(m, '_tools', {}).values() if hasattr(tool, 'episode_reward')]
                if rewards:
                    ud['env_reward'] = max(rewards)
            t['user_data'] = ud
        if self.trace_dir:
            self._write_traces(trajs)
        return trajs

    def _write_traces(self, trajs: Sequence[Trajectory]) -> None:
        os.makedirs(self.trace_dir, exist_ok=True)
        path = os.path.join(self.trace_dir, f'rollout_{uuid.uuid4().hex[:8]}.jsonl')
        with open(path, 'w') as f:
            for t in trajs:
                f.write(json.dumps({'messages': t['messages'], 'user_data': t.get('user_data')}, ensure_ascii=False, default=str) + '\n')


class ChatAPI(ABC):
    """``(messages, tools, **params) -> assistant message`` over some wire protocol."""

    @abstractmethod
    def __call__(self, messages: List[Message], tools: Optional[List[Dict[str, Any]]] = None, **kwargs) -> Message:
        ...


class OpenAIChatAPI(ChatAPI):
    """OpenAI-compatible ``/chat/completions`` endpoint (also what this framework's gateway serves)."""

    def __init__(self, base_url: str, model: str, api_key: Optional[str] = None, timeout: float = 120.0, **defaults):
        self.base_url, self.model, self.api_key, self.timeout, self.defaults = base_url.rstrip('/'), model, api_key, timeout, defaults

    def __call__(self, messages, tools=None, **kwargs) -> Message:
        import requests
        body = {'model': self.model, 'messages': [self._wire(m) for m in messages], **self.defaults, **kwargs}
        if tools:
            body['tools'] = [{'type': 'function', 'function': {'name': t.get('tool_name'), 'description': t.get('description', ''),
                                                                 'parameters': t.get('parameters', {})}} for t in tools]
        headers = {'Authorization': f'Bearer {self.api_key}'} if self.api_key else {}
        r = requests.post(self.base_url + '/chat/completions', json=body, headers=headers, timeout=self.timeout)
        r.raise_for_status()
        choice = r.json()['choices'][0]['message']
        msg: Message = {'role': 'assistant', 'content': choice.get('content') or ''}
        if choice.get('reasoning_content'):
            msg['reasoning_content'] = choice['reasoning_content']
        calls = []
        for c in choice.get('tool_calls') or []:
            fn = c.get('function', {})
            calls.append(ToolCall(id=c.get('id') or f'call_{uuid.uuid4().hex[:8]}', type='function', tool_name=fn.get('name'),
                                  arguments=fn.get('arguments', {})))
        if calls:
            msg['tool_calls'] = calls
        return msg

    @staticmethod
    def _wire(m: Message) -> Dict[str, Any]:
        out = {'role': m['role'], 'content': m.get('content', '')}
        if m.get('tool_call_id'):
            out['tool_call_id'] = m['tool_call_id']
        if m.get('tool_calls'):
            out['tool_calls'] = [{'id': c.get('id'), 'type': 'function',
                                  'function': {'name': c.get('tool_name'),
                                               'arguments': c['arguments'] if isinstance(c.get('arguments'), str) else json.dumps(c.get('arguments', {}))}}
                                 for c in m['tool_calls']]
        return out


class APIMultiTurnRollout(Rollout):
    """The same loop against a chat API (a teacher model, or this framework's own gateway): used to collect
    demonstrations, so no token ids are kept."""

    def __init__(self, api: ChatAPI, tool_manager: Optional[ToolManager] = None, max_turns: int = 8, max_workers: int = 8, **api_kwargs):
        self.api, self.tool_manager, self.max_turns, self.max_workers, self.api_kwargs = api, tool_manager, max_turns, max_workers, api_kwargs

    def _run_one(self, traj: Trajectory) -> Trajectory:
        t = dict(traj)
        t['messages'] = [dict(m) for m in traj.get('messages', [])]
        m = self.tool_manager.copy() if self.tool_manager is not None else None
        tools = t.get('tools') or (m.tool_infos() if m else None)
        for _ in range(self.max_turns):
            reply = self.api(t['messages'], tools, **self.api_kwargs)
            t['messages'].append(reply)
            calls = reply.get('tool_calls') or []
            if not calls or m is None:
                break
            for c in calls:
                t['messages'].append({'role': 'tool', 'content': m(c), 'tool_call_id': c.get('id', '')})
        return t

    def __call__(self, trajectories: List[Trajectory], **kwargs) -> List[Trajectory]:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=max(1, min(self.max_workers, len(trajectories)))) as ex:
            return list(ex.map(self._run_one, trajectories))
