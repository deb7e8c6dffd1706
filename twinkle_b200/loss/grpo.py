"""Policy-gradient losses with importance ratios.

Parity: reference ``src/twinkle/loss/grpo.py:13-437`` — GRPO plus the GSPO,
SAPO, CISPO, BNPO and DR-GRPO variants, including the alignment rules for
ragged ``old_logps`` / ``ref_logps`` / ``advantages``.  Each variant here is a
(ratio rule, surrogate rule, aggregation rule) triple on one class.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..data_format import LossOutput
from .base import Loss, as_2d_labels, token_logps


def align_to_mask(values, mask: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Bring ``values`` to the ``[B, S]`` grid of ``mask``.

    Accepted per row: a scalar (broadcast on the mask); a vector whose length
    equals the number of masked positions (scattered onto them in order); a
    vector at least as long as the row (sliced to S; values sit at their own
    positions).  Anything else is an error.  A ``[B, S]`` tensor passes through.
    """
    device = mask.device
    B, S = mask.shape
    if torch.is_tensor(values) and values.dim() == 2 and tuple(values.shape) == (B, S):
        return values.to(device=device, dtype=dtype)
    if isinstance(values, np.ndarray):
        values = torch.from_numpy(values)
    if torch.is_tensor(values) and values.dim() <= 1:
        values = values.reshape(-1).tolist()
        if len(values) == 1 and B > 1:
            values = values * B
    elif torch.is_tensor(values):
        values = [v for v in values]
    if isinstance(values, (int, float)):
        values = [float(values)] * B
    if len(values) != B:
        raise AssertionError(f'expected {B} rows, got {len(values)}')
    out = torch.zeros(B, S, dtype=dtype, device=device)
    for b, row in enumerate(values):
        m = mask[b]
        n_valid = int(m.sum())
        r = torch.as_tensor(row, dtype=dtype, device=device).reshape(-1)
        if r.numel() == 1:
            out[b] = r * m.to(dtype)
        elif r.numel() == n_valid:
            out[b, m] = r
        elif r.numel() >= S:
            out[b, m] = r[:S][m]  # indexed, not multiplied: a NaN or inf parked in a padding position must not reach the loss
        else:
            raise AssertionError(f'row {b}: cannot align {r.numel()} values to {n_valid} target tokens of a length-{S} row')
    return out


class GRPOLoss(Loss):

    def __init__(self, epsilon: float = 0.2, epsilon_high: Optional[float] = None, beta: float = 0.0,
                 entropy_coef: float = 0.0, ignore_index: int = -100, **kwargs):
        self.epsilon = epsilon
        self.epsilon_high = epsilon if epsilon_high is None else epsilon_high
        self.beta = beta
        self.entropy_coef = entropy_coef
        self.require_entropy = entropy_coef > 0.0
        self.ignore_index = ignore_index

    # rules ---------------------------------------------------------------
    def _log_ratio(self, logps, old_logps, mask):
        return torch.clamp(logps - old_logps, -20.0, 20.0)

    def _surrogate(self, ratio, adv, logps):
        clipped = torch.clamp(ratio, 1.0 - self.epsilon, 1.0 + self.epsilon_high)
        return -torch.min(ratio * adv, clipped * adv)

    def _aggregate(self, per_token, mask, **kwargs):
        m = mask.to(per_token.dtype)
        per_seq = (per_token * m).sum(-1) / m.sum(-1).clamp_min(1.0)
        return per_seq.mean()

    # call ----------------------------------------------------------------
    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], *, old_logps=None, ref_logps=None,
                 advantages=None, **kwargs) -> LossOutput:
        labels = as_2d_labels(inputs)
        logps = token_logps(outputs, labels, self.ignore_index)
        mask = (labels != self.ignore_index).to(logps.device)
        if advantages is None:
            return LossOutput(loss=logps.sum() * 0.0, num_tokens=0)
        old = logps.detach() if old_logps is None else align_to_mask(old_logps, mask, logps.dtype)
        adv = align_to_mask(advantages, mask, logps.dtype)
        ratio = torch.exp(self._log_ratio(logps, old, mask))
        per_token = self._surrogate(ratio, adv, logps)
        if self.beta > 0.0 and ref_logps is not None:
            d = align_to_mask(ref_logps, mask, logps.dtype) - logps
            per_token = per_token + self.beta * (torch.exp(d) - d - 1.0)
        if self.entropy_coef > 0.0:
            ent = outputs.get('entropies')
            if ent is None:
                raise AssertionError("entropy_coef > 0 needs outputs['entropies']")
            per_token = per_token - self.entropy_coef * ent.to(per_token.dtype)
        return LossOutput(loss=self._aggregate(per_token, mask, **kwargs), num_tokens=0)

    # metrics helpers -----------------------------------------------------
    @torch.no_grad()
    def diagnostics(self, logps, old_logps, mask) -> Dict[str, float]:
        lr = self._log_ratio(logps, old_logps, mask)
        ratio = lr.exp()
        m = mask.float()
        n = m.sum().clamp_min(1)
        kl = ((ratio - 1) - lr) * m
        low = ((ratio < 1 - self.epsilon) * m).sum() / n
        high = ((ratio > 1 + self.epsilon_high) * m).sum() / n
        return {'kl': float(kl.sum() / n), 'clip_low': float(low), 'clip_high': float(high)}


class GSPOLoss(GRPOLoss):
    """Sequence-level ratio: masked mean of the token log ratios, broadcast."""

    def _log_ratio(self, logps, old_logps, mask):
        m = mask.to(logps.dtype)
        # every token's log ratio is clamped first, then averaged (reference ``loss/grpo.py:323-324``)
        lr = torch.clamp(logps - old_logps, -20.0, 20.0)
        seq = (lr * m).sum(-1, keepdim=True) / m.sum(-1, keepdim=True).clamp_min(1.0)
        return seq.expand_as(logps)


class SAPOLoss(GRPOLoss):
    """Soft gate ``σ(τ(r−1))·4/τ`` with a temperature chosen by the sign of A."""

    def __init__(self, tau_pos: float = 1.0, tau_neg: float = 1.0, **kw):
        super().__init__(**kw)
        self.tau_pos, self.tau_neg = tau_pos, tau_neg

    def _surrogate(self, ratio, adv, logps):
        tau = torch.where(adv > 0, torch.full_like(adv, self.tau_pos), torch.full_like(adv, self.tau_neg))
        gate = torch.sigmoid(tau * (ratio - 1.0)) * 4.0 / tau
        return -gate * adv


class CISPOLoss(GRPOLoss):

    def _surrogate(self, ratio, adv, logps):
        return -torch.clamp(ratio, max=1.0 + self.epsilon).detach() * adv * logps  # reference loss/grpo.py:379

    def _aggregate(self, per_token, mask, **kwargs):
        n = kwargs.get('num_items_in_batch')
        n = mask.sum() if n is None else n
        return (per_token * mask).sum() / n


class BNPOLoss(GRPOLoss):

    def _aggregate(self, per_token, mask, **kwargs):
        return (per_token * mask).sum() / mask.sum().clamp_min(1.0)


class DRGRPOLoss(GRPOLoss):

    def __init__(self, max_completion_length: int = 1024, **kw):
        super().__init__(**kw)
        self.max_completion_length = max_completion_length

    def _aggregate(self, per_token, mask, **kwargs):
        return (per_token * mask).sum() / (mask.shape[0] * self.max_completion_length)
