"""TypedDict records.  All keys are optional (``total=False``) because every
stage adds its own fields: the template adds ``input_ids``/``labels``, the
processor adds ``position_ids``/``attention_mask``, RL loops add
``old_logps``/``advantages``."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, TypedDict, Union

import numpy as np

try:  # torch is always present at run time; keep the types importable without it
    import torch
    Tensor = torch.Tensor
except Exception:  # pragma: no cover
    Tensor = Any

Array = Union[List[int], 'np.ndarray', 'Tensor']


class ToolCall(TypedDict, total=False):
    id: str
    type: str
    tool_name: str
    arguments: Union[str, Dict[str, Any]]


class Tool(TypedDict, total=False):
    tool_name: str
    description: str
    parameters: Dict[str, Any]


class FunctionCall(TypedDict, total=False):
    """OpenAI wire form of a call: ``{"name": …, "arguments": "<json>"}`` (nested under ``function`` in a tool call)."""
    name: str
    arguments: Union[str, Dict[str, Any]]


class FunctionSpec(TypedDict, total=False):
    """OpenAI wire form of a tool declaration (nested under ``function`` with ``type: "function"``)."""
    name: str
    description: str
    parameters: Dict[str, Any]


def tool_to_openai(tool: Union[Tool, Dict[str, Any]]) -> Dict[str, Any]:
    """``Tool`` → ``{"type": "function", "function": FunctionSpec}``; already-wrapped declarations pass through."""
    if 'function' in tool:
        return dict(tool)
    return {'type': 'function', 'function': {'name': tool.get('tool_name') or tool.get('name'), 'description': tool.get('description', ''),
                                             'parameters': tool.get('parameters') or {'type': 'object', 'properties': {}}}}


def tool_call_to_openai(call: Union[ToolCall, Dict[str, Any]]) -> Dict[str, Any]:
    """``ToolCall`` → ``{"id", "type": "function", "function": FunctionCall}`` with JSON-string arguments."""
    import json
    fn = call.get('function') or {}
    args = call.get('arguments', fn.get('arguments', {}))
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {'id': call.get('id', ''), 'type': 'function', 'function': {'name': call.get('tool_name') or fn.get('name'), 'arguments': args}}


class Message(TypedDict, total=False):
    role: str  # system | user | assistant | tool
    content: Union[str, List[Dict[str, Any]]]
    reasoning_content: str
    tool_calls: List[ToolCall]
    tool_call_id: str
    loss: bool  # False → excluded from the training labels


class Trajectory(TypedDict, total=False):
    messages: List[Message]
    tools: List[Tool]
    user_data: Any
    images: List[Any]
    videos: List[Any]
    audios: List[Any]
    prompt: str


class InputFeature(TypedDict, total=False):
    input_ids: Array
    attention_mask: Array
    position_ids: Array
    labels: Array  # already shifted: labels[t] is the target of logits[t]; −100 = ignore
    completion_mask: Array
    length: int
    routed_experts: Any
    # RL extras carried alongside
    old_logps: Any
    ref_logps: Any
    advantages: Any


class ModelOutput(TypedDict, total=False):
    logits: Any
    loss: Any
    logps: Any
    entropies: Any
    num_tokens: Any
    embeddings: Any
    routed_experts: Any
    aux_loss: Any


class LossOutput(TypedDict, total=False):
    loss: Any
    num_tokens: Any


def to_input_feature(obj: Dict[str, Any]) -> InputFeature:
    """Keep only known keys, convert arrays to python lists lazily."""
    keep = InputFeature.__annotations__.keys()
    return {k: v for k, v in obj.items() if k in keep}  # type: ignore[return-value]


def pack_value(value: Any) -> str:
    """JSON text of one ``user_data`` value (columnar stores keep ``user_data`` as ``(key, json)`` pairs so that rows
    with different value types share one schema). Parity: reference ``data_format/trajectory.py:26-44``."""
    import json
    return json.dumps(value, ensure_ascii=False, default=str)


def user_data_get(user_data: Any, key: str, default: Any = None) -> Any:
    """Value of ``key`` in ``user_data`` given as a dict or as a list of ``(key, value-or-json)`` pairs."""
    import json
    if isinstance(user_data, dict):
        return user_data.get(key, default)
    if not isinstance(user_data, (list, tuple)):
        return default
    for entry in user_data:
        if isinstance(entry, (list, tuple)) and len(entry) == 2 and entry[0] == key:
            v = entry[1]
            if isinstance(v, str):
                try:
                    return json.loads(v)
                except ValueError:
                    return v
            return v
    return default


def user_data_set(user_data: Any, key: str, value: Any) -> Any:
    """Copy of ``user_data`` with ``key`` replaced: dicts stay dicts, pair lists get a packed ``(key, json)`` entry."""
    if isinstance(user_data, dict):
        return {**user_data, key: value}
    items = [e for e in (user_data or []) if not (isinstance(e, (list, tuple)) and len(e) == 2 and e[0] == key)]
    items.append((key, pack_value(value)))
    return items
