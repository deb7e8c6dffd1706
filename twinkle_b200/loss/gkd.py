"""Generalised knowledge distillation (generalised Jensen–Shannon).

Parity: reference ``src/twinkle/loss/gkd.py:11-242`` — β=0 → KL(T‖S), β=1 →
KL(S‖T), else ``β·KL(T‖M) + (1−β)·KL(S‖M)`` with
``M = logsumexp(S + log(1−β), T + log β)``; teacher given as full logits,
local top-k, or remote top-k logprobs + indices; valid tokens processed in
chunks; vocab mismatch padded from the other side; mean over valid tokens.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F

from ..data_format import LossOutput
from .base import Loss, as_2d_labels


def generalized_jsd(student_logp: torch.Tensor, teacher_logp: torch.Tensor, beta: float) -> torch.Tensor:
    """Per-row divergence between two log-distributions over the last dim."""
    if beta <= 0.0:
        return (teacher_logp.exp() * (teacher_logp - student_logp)).sum(-1)
    if beta >= 1.0:
        return (student_logp.exp() * (student_logp - teacher_logp)).sum(-1)
    mix = torch.logsumexp(torch.stack([student_logp + math.log1p(-beta), teacher_logp + math.log(beta)]), dim=0)
    kl_t = (teacher_logp.exp() * (teacher_logp - mix)).sum(-1)
    kl_s = (student_logp.exp() * (student_logp - mix)).sum(-1)
    return beta * kl_t + (1.0 - beta) * kl_s


class GKDLoss(Loss):
    require_logits = True
    require_logps = False

    def __init__(self, beta: float = 0.5, temperature: float = 1.0, chunk_size: int = 512, topk: Optional[int] = None,
                 ignore_index: int = -100, **kwargs):
        self.beta, self.temperature, self.chunk_size, self.topk = beta, temperature, chunk_size, topk
        self.ignore_index = ignore_index

    @staticmethod
    def _match_vocab(a: torch.Tensor, b: torch.Tensor):
        va, vb = a.shape[-1], b.shape[-1]
        if va < vb:
            a = torch.cat([a, b[..., va:].to(a.dtype)], -1)
        elif vb < va:
            b = torch.cat([b, a[..., vb:].detach().to(b.dtype)], -1)
        return a, b

    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], *, teacher_logits=None,
                 teacher_topk_logprobs=None, teacher_topk_indices=None, **kwargs) -> LossOutput:
        labels = as_2d_labels(inputs)
        s_logits = outputs['logits']
        if s_logits.dim() == 2:
            s_logits = s_logits.unsqueeze(0)
        mask = (labels != self.ignore_index).to(s_logits.device).reshape(-1)
        s_flat = s_logits.reshape(-1, s_logits.shape[-1])
        idx = mask.nonzero(as_tuple=True)[0]
        if idx.numel() == 0:
            return LossOutput(loss=s_flat.sum() * 0.0, num_tokens=0)
        total = s_flat.new_zeros((), dtype=torch.float32)
        t_flat = ti_flat = tl_flat = None
        if teacher_logits is not None:
            t = torch.as_tensor(teacher_logits).to(s_flat.device)
            t_flat = t.reshape(-1, t.shape[-1])
        elif teacher_topk_logprobs is not None:
            tl = torch.as_tensor(teacher_topk_logprobs).to(s_flat.device)
            ti = torch.as_tensor(teacher_topk_indices).to(s_flat.device).long()
            tl_flat, ti_flat = tl.reshape(-1, tl.shape[-1]), ti.reshape(-1, ti.shape[-1])
        else:
            raise AssertionError('GKDLoss needs teacher_logits or teacher_topk_logprobs + teacher_topk_indices')
        for s in range(0, idx.numel(), self.chunk_size):
            rows = idx[s:s + self.chunk_size]
            sl = s_flat[rows].float() / self.temperature
            if t_flat is not None:
                tl_ = t_flat[rows].float() / self.temperature
                if self.topk:
                    top_v, top_i = tl_.topk(self.topk, -1)
                    sp = F.log_softmax(sl.gather(-1, top_i), -1)
                    tp = F.log_softmax(top_v, -1)
                else:
                    sl, tl_ = self._match_vocab(sl, tl_)
                    sp, tp = F.log_softmax(sl, -1), F.log_softmax(tl_, -1)
            else:
                sp = F.log_softmax(sl.gather(-1, ti_flat[rows]), -1)
                tp = F.log_softmax(tl_flat[rows].float(), -1)
            total = total + generalized_jsd(sp, tp, self.beta).sum()
        return LossOutput(loss=total / idx.numel(), num_tokens=0)
