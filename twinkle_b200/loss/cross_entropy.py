"""Cross-entropy family.

Parity: reference ``src/twinkle/loss/cross_entropy.py:6-31`` (from logps;
``sum`` / ``mean``; DFT variant ``−logp·exp(logp)``), ``chunked_cross_entropy.py:
20-159`` and ``liger_fused_linear_cross_entropy.py:88-208``.  The chunked and
fused variants of the reference exist to bound memory; here both map onto the
fused lm_head+CE kernel (``ops.fused_linear_logprob``) on B200 and onto a
chunked PyTorch formula elsewhere.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..data_format import LossOutput
from .base import Loss, as_2d_labels, token_logps


class CrossEntropyLoss(Loss):

    def __init__(self, reduction: str = 'sum', ignore_index: int = -100, dft: bool = False, **kwargs):
        if reduction not in ('sum', 'mean'):
            raise ValueError(f'reduction must be sum|mean, got {reduction}')
        self.reduction = reduction
        self.ignore_index = ignore_index
        self.dft = dft

    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], **kwargs) -> LossOutput:
        labels = as_2d_labels(inputs)
        logps = token_logps(outputs, labels, self.ignore_index)
        mask = (labels != self.ignore_index).to(logps.device)
        per_token = -logps
        if self.dft:
            per_token = per_token * logps.detach().exp()
        total = (per_token * mask).sum()
        count = mask.sum().clamp_min(1)
        if self.reduction == 'mean':
            return LossOutput(loss=total / count, num_tokens=0)
        return LossOutput(loss=total, num_tokens=count)


class DFTLoss(CrossEntropyLoss):

    def __init__(self, **kw):
        kw['dft'] = True
        super().__init__(**kw)


class ChunkedCrossEntropyLoss(Loss):
    """Consumes ``outputs['logits']`` chunk by chunk; gradient of each chunk is
    formed in place so that at most ``chunk_size × V`` fp32 values are live."""
    require_logits = True
    require_logps = False

    def __init__(self, chunk_size: int = 1024, reduction: str = 'sum', ignore_index: int = -100, **kwargs):
        self.chunk_size = chunk_size
        self.reduction = reduction
        self.ignore_index = ignore_index

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        labels = as_2d_labels(inputs).reshape(-1)
        logits = outputs['logits'].reshape(-1, outputs['logits'].shape[-1])
        labels = labels.to(logits.device)
        total = _ChunkedCE.apply(logits, labels, self.chunk_size, self.ignore_index)
        count = (labels != self.ignore_index).sum().clamp_min(1)
        if self.reduction == 'mean':
            return LossOutput(loss=total / count, num_tokens=0)
        return LossOutput(loss=total, num_tokens=count)


class _ChunkedCE(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, labels, chunk, ignore_index):
        total = logits.new_zeros((), dtype=torch.float32)
        grad = torch.empty_like(logits) if logits.requires_grad else None
        for s in range(0, logits.shape[0], chunk):
            x = logits[s:s + chunk].float()
            y = labels[s:s + chunk]
            valid = y != ignore_index
            lse = torch.logsumexp(x, -1)
            tgt = x.gather(-1, y.clamp_min(0)[:, None]).squeeze(-1)
            total = total + ((lse - tgt) * valid).sum()
            if grad is not None:
                p = torch.softmax(x, -1)
                p.scatter_add_(-1, y.clamp_min(0)[:, None], -torch.ones_like(tgt)[:, None])
                p.mul_(valid[:, None])
                grad[s:s + chunk] = p.to(grad.dtype)
        ctx.save_for_backward(grad)
        return total

    @staticmethod
    def backward(ctx, g):
        (grad, ) = ctx.saved_tensors
        return grad * g.to(grad.dtype), None, None, None


class FusedLinearCrossEntropyLoss(Loss):
    """Hidden states × lm_head fused with CE: the model forward (task
    ``fused_lm_ce``) skips the logits and hands ``hidden_states`` plus the head
    weight to this loss."""
    require_logits = False
    require_logps = False
    require_hidden = True

    def __init__(self, reduction: str = 'sum', ignore_index: int = -100, **kwargs):
        self.reduction = reduction
        self.ignore_index = ignore_index

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        labels = as_2d_labels(inputs).reshape(-1)
        if 'logps' in outputs and outputs['logps'] is not None:
            logps = outputs['logps'].reshape(-1)
        else:
            from ..ops import fused_linear_logprob
            hidden = outputs['hidden_states'].reshape(-1, outputs['hidden_states'].shape[-1])
            logps, _ = fused_linear_logprob(hidden, outputs['lm_head_weight'], labels.clamp_min(0).to(hidden.device))
        mask = (labels != self.ignore_index).to(logps.device)
        total = -(logps * mask).sum()
        count = mask.sum().clamp_min(1)
        if self.reduction == 'mean':
            return LossOutput(loss=total / count, num_tokens=0)
        return LossOutput(loss=total, num_tokens=count)


LigerFusedLinearCrossEntropyLoss = FusedLinearCrossEntropyLoss


class MSELoss(Loss):
    require_logits = True
    require_logps = False

    def __init__(self, **kwargs):
        pass

    def __call__(self, inputs, outputs, **kwargs) -> LossOutput:
        pred = outputs['logits'].float().squeeze(-1)
        target = torch.as_tensor(inputs['labels']).to(pred.device, torch.float32).reshape(pred.shape)
        return LossOutput(loss=torch.mean((pred - target)**2), num_tokens=0)
