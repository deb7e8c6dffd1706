"""Loss interface.

Parity: reference ``src/twinkle/loss/base.py:5-12``.  A loss is a callable
``(inputs, outputs, **kw) -> LossOutput{loss, num_tokens}``.  Three class flags
tell the model forward what to materialise: ``require_logits`` (keep the
``[T, V]`` logits), ``require_entropy`` (per-token entropy from the fused
logprob kernel), ``require_logps`` (default).  ``num_tokens`` follows the
normalisation contract: sum-reduction losses report the number of valid tokens
(gradients are later divided by the global token count); mean-style losses
report 0.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..data_format import LossOutput

IGNORE_INDEX = -100


class Loss:
    require_logits: bool = False
    require_entropy: bool = False
    require_logps: bool = True
    ignore_index: int = IGNORE_INDEX

    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], **kwargs) -> LossOutput:  # pragma: no cover
        raise NotImplementedError


def as_2d_labels(inputs: Dict[str, Any]) -> torch.Tensor:
    labels = inputs.get('labels')
    if labels is None:
        raise AssertionError("inputs must contain 'labels'")
    if not torch.is_tensor(labels):
        labels = torch.as_tensor(labels)
    if labels.dim() == 1:
        labels = labels.unsqueeze(0)
    return labels


def token_logps(outputs: Dict[str, Any], labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """``outputs['logps']`` if present, else computed from ``outputs['logits']``
    with masked labels replaced by 0 before the gather."""
    logps = outputs.get('logps')
    if logps is not None:
        if logps.dim() == 1:
            logps = logps.unsqueeze(0)
        return logps
    from ..utils.torch_utils import selective_log_softmax
    logits = outputs['logits']
    if logits.shape[-2] != labels.shape[-1]:
        logits = logits[..., -labels.shape[-1]:, :]
    safe = labels.clamp_min(0).to(logits.device)
    return selective_log_softmax(logits, safe)
