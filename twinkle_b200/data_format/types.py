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
