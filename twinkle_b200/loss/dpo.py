"""Preference losses on interleaved (chosen, rejected) batches.

Parity: reference ``src/twinkle/loss/dpo.py:20-569`` — DPO with sigmoid /
hinge / ipo / kto_pair forms, label smoothing, ``sft_weight``,
``reference_free``; SimPO, CPO, ORPO.  Rows ``0::2`` are chosen and ``1::2``
rejected, so a contiguous data-parallel slice of even length keeps pairs whole.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F

from ..data_format import LossOutput
from .base import Loss, as_2d_labels, token_logps


class PreferenceLoss(Loss):

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index

    def _seq_logps(self, inputs, outputs):
        labels = as_2d_labels(inputs)
        logps = token_logps(outputs, labels, self.ignore_index)
        mask = (labels != self.ignore_index).to(logps.device)
        if logps.shape[0] % 2 != 0:
            raise AssertionError('preference batches interleave chosen/rejected rows; got an odd number of rows')
        seq = (logps * mask).sum(-1)
        return logps, mask, seq

    @staticmethod
    def _nll(chosen_seq_logps: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """Negative log-likelihood of the chosen rows per chosen *token* over the whole batch (total divided by the
        number of chosen tokens, reference ``loss/dpo.py:64-71``), not a mean of per-sequence means."""
        return -chosen_seq_logps.sum() / mask[0::2].sum().clamp_min(1)

    @staticmethod
    def _align_ref(ref, logps, mask):
        """Reference logps may be per-token ``[B, S']`` (S' ≥ or ≤ S), or
        already per-sequence ``[B]``."""
        if ref is None:
            return None
        if isinstance(ref, dict):
            ref = ref.get('logps')
        ref = torch.as_tensor(ref) if not torch.is_tensor(ref) else ref
        ref = ref.to(logps.device, logps.dtype)
        if ref.dim() == 1:
            return ref
        S = mask.shape[1]
        if ref.shape[1] < S:
            ref = F.pad(ref, (0, S - ref.shape[1]))
        return (ref[:, :S] * mask).sum(-1)


class DPOLoss(PreferenceLoss):

    def __init__(self, beta: float = 0.1, label_smoothing: float = 0.0, ignore_index: int = -100,
                 loss_type: str = 'sigmoid', reference_free: bool = False, sft_weight: float = 0.0, **kwargs):
        super().__init__(ignore_index)
        if loss_type not in ('sigmoid', 'hinge', 'ipo', 'kto_pair'):
            raise ValueError(f'Unknown loss_type: {loss_type}')
        if label_smoothing > 0 and loss_type != 'sigmoid':
            raise ValueError('label_smoothing is only defined for loss_type="sigmoid"')
        self.beta, self.label_smoothing, self.loss_type = beta, label_smoothing, loss_type
        self.reference_free, self.sft_weight = reference_free, sft_weight

    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], *, ref_outputs=None, ref_logps=None,
                 ref_chosen_logps=None, ref_rejected_logps=None, **kwargs) -> LossOutput:
        """The reference policy comes as ``ref_outputs`` / ``ref_logps`` (per token or per sequence, rows interleaved
        like the batch) or as the two sequence-level vectors ``ref_chosen_logps`` / ``ref_rejected_logps``
        (reference ``src/twinkle/loss/dpo.py:257-320``)."""
        logps, mask, seq = self._seq_logps(inputs, outputs)
        pc, pr = seq[0::2], seq[1::2]
        ref = None
        if ref_chosen_logps is not None and ref_rejected_logps is not None:
            rc = torch.as_tensor(ref_chosen_logps).to(pc.device, pc.dtype).reshape(-1)
            rr = torch.as_tensor(ref_rejected_logps).to(pc.device, pc.dtype).reshape(-1)
            if rc.numel() != pc.numel() or rr.numel() != pr.numel():
                raise ValueError(f'ref_chosen_logps / ref_rejected_logps must hold one value per pair ({pc.numel()}), got {rc.numel()} / {rr.numel()}')
        else:
            ref = self._align_ref(ref_outputs if ref_outputs is not None else ref_logps, logps, mask)
            if ref is None and not self.reference_free:
                return LossOutput(loss=logps.sum() * 0.0, num_tokens=0)
            if ref is None:
                rc = rr = torch.zeros_like(pc)
            else:
                rc, rr = ref[0::2], ref[1::2]
        dc, dr = pc - rc, pr - rr
        z = self.beta * (dc - dr)
        if self.loss_type == 'sigmoid':
            ls = self.label_smoothing
            per_pair = -F.logsigmoid(z) * (1 - ls) - F.logsigmoid(-z) * ls
        elif self.loss_type == 'hinge':
            per_pair = torch.relu(1 - z)
        elif self.loss_type == 'ipo':
            per_pair = (z - 1 / (2 * self.beta))**2  # on the β-scaled margin, as the reference (dpo.py:234-237)
        else:  # kto_pair
            per_pair = 1 - torch.sigmoid(self.beta * dc) + torch.sigmoid(self.beta * dr)
        loss = per_pair.mean()
        if self.sft_weight > 0:
            loss = loss + self.sft_weight * self._nll(pc, mask)
        self.last_stats = {
            'rewards/chosen': float((self.beta * dc).mean().detach()), 'rewards/rejected': float((self.beta * dr).mean().detach()),
            'rewards/margins': float((self.beta * (dc - dr)).mean().detach()), 'rewards/accuracies': float((dc > dr).float().mean()),
            'logps/chosen': float(pc.mean().detach()), 'logps/rejected': float(pr.mean().detach()),
        }
        return LossOutput(loss=loss, num_tokens=0)


class SimPOLoss(PreferenceLoss):
    """Length-normalised, reference-free: ``−logσ(β(avg_c − avg_r) − γ)``."""

    def __init__(self, beta: float = 2.5, gamma: float = 0.5, ignore_index: int = -100, **kwargs):
        super().__init__(ignore_index)
        self.beta, self.gamma = beta, gamma

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        logps, mask, seq = self._seq_logps(inputs, outputs)
        avg = seq / mask.sum(-1).clamp_min(1)
        z = self.beta * (avg[0::2] - avg[1::2]) - self.gamma
        return LossOutput(loss=(-F.logsigmoid(z)).mean(), num_tokens=0)


class CPOLoss(PreferenceLoss):
    """``−logσ(β(π_c − π_r)) + bc_coef · NLL(chosen)``."""

    def __init__(self, beta: float = 0.1, bc_coef: float = 1.0, ignore_index: int = -100, **kwargs):
        super().__init__(ignore_index)
        self.beta, self.bc_coef = beta, bc_coef

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        logps, mask, seq = self._seq_logps(inputs, outputs)
        pref = -F.logsigmoid(self.beta * (seq[0::2] - seq[1::2])).mean()
        return LossOutput(loss=pref + self.bc_coef * self._nll(seq[0::2], mask), num_tokens=0)


class ORPOLoss(PreferenceLoss):
    """NLL(chosen) − λ·logσ(log odds ratio) on length-averaged logps."""

    def __init__(self, lambda_orpo: float = 0.1, ignore_index: int = -100, **kwargs):
        super().__init__(ignore_index)
        self.lambda_orpo = lambda_orpo

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        logps, mask, seq = self._seq_logps(inputs, outputs)
        avg = seq / mask.sum(-1).clamp_min(1)
        c, r = avg[0::2], avg[1::2]
        log_odds = (c - r) - (torch.log1p(-torch.exp(c).clamp(max=1 - 1e-6)) - torch.log1p(-torch.exp(r).clamp(max=1 - 1e-6)))
        loss = self._nll(seq[0::2], mask) - self.lambda_orpo * F.logsigmoid(log_odds).mean()
        return LossOutput(loss=loss, num_tokens=0)
