"""Hang guards: a failing rank must still take part in the step's collectives.

Parity: reference ``src/twinkle/utils/nccl_safe.py:36-333``.  Active when
``TWINKLE_FAIL_FAST=0``:

* ``safe_loss`` wraps a loss; an exception inside it (bad payload: ragged
  ``old_logps`` of the wrong length, NaN inputs, all labels masked…) becomes a
  zero loss that is still connected to the model outputs, so backward runs and
  every gradient reduce-scatter fires on all ranks.
* ``collective_safe`` wraps a model method: if the forward ran but the backward
  did not (exception in between), a zero backward is forced before re-raising
  is suppressed, keeping ranks in lock-step.

With ``TWINKLE_FAIL_FAST=1`` (default) exceptions propagate unchanged.
"""
from __future__ import annotations

import functools
import os
from typing import Any, Callable, Dict

import torch

from ..data_format import LossOutput
from .logger import get_logger

logger = get_logger()


def fail_fast() -> bool:
    return os.environ.get('TWINKLE_FAIL_FAST', '1').lower() not in ('0', 'false', 'no')


def _connected_zero(outputs: Dict[str, Any]) -> torch.Tensor:
    for k in ('logps', 'logits', 'hidden_states', 'embeddings'):
        v = outputs.get(k) if isinstance(outputs, dict) else None
        if torch.is_tensor(v) and v.requires_grad:
            return torch.nan_to_num(v.float(), nan=0.0, posinf=0.0, neginf=0.0).sum() * 0.0
    return torch.zeros((), requires_grad=True)


class SafeLossWrapper:

    def __init__(self, loss: Callable):
        self.loss = loss
        self.last_error = None

    def __getattr__(self, item):
        return getattr(self.__dict__['loss'], item)

    def __call__(self, inputs, outputs, **kwargs):
        if fail_fast():
            return self.loss(inputs, outputs, **kwargs)
        try:
            out = self.loss(inputs, outputs, **kwargs)
            loss = out['loss'] if isinstance(out, dict) else out
            if torch.is_tensor(loss) and not bool(torch.isfinite(loss.detach()).all()):
                raise FloatingPointError('non-finite loss')
            self.last_error = None
            return out
        except Exception as e:  # noqa: BLE001 — any failure must not desynchronise ranks
            self.last_error = e
            logger.warning(f'loss raised {type(e).__name__}: {e}; substituting a graph-connected zero', ranks='all')
            return LossOutput(loss=_connected_zero(outputs), num_tokens=0)


def safe_loss(loss):
    if loss is None or isinstance(loss, SafeLossWrapper):
        return loss
    return SafeLossWrapper(loss)


def collective_safe(method):
    """For ``forward_backward``-style methods of a model that exposes
    ``_forward_ran`` / ``_backward_ran`` flags and ``_force_zero_backward()``."""

    @functools.wraps(method)
    def wrapper(self, *args, **kwargs):
        if fail_fast():
            return method(self, *args, **kwargs)
        self._forward_ran = self._backward_ran = False
        try:
            return method(self, *args, **kwargs)
        except Exception as e:  # noqa: BLE001
            logger.warning(f'{method.__name__} raised {type(e).__name__}: {e}', ranks='all')
            if getattr(self, '_forward_ran', False) and not getattr(self, '_backward_ran', False):
                try:
                    self._force_zero_backward()
                except Exception as e2:  # pragma: no cover
                    logger.error(f'zero backward failed: {e2}')
            return {'loss': 0.0, 'error': f'{type(e).__name__}: {e}'}

    return wrapper


nccl_safe = collective_safe
