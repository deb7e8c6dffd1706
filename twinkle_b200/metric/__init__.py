"""Training metrics.

Parity: reference ``src/twinkle/metric/*.py`` — ``accumulate / calculate /
reset``; results are strings (``'loss': '0.1234'``) as in the reference, and
cross-rank reduction happens through an object gather on the data-parallel
group.
"""
from __future__ import annotations

import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..utils.framework import Torch


def _f(x) -> float:
    if torch.is_tensor(x):
        return float(x.detach().float().mean().item()) if x.numel() else 0.0
    return float(x)


class Metric:

    def __init__(self, device_mesh=None, process_group=None, **kwargs):
        self.device_mesh = device_mesh
        self.process_group = process_group
        self.reset()

    def accumulate(self, inputs: Any, outputs: Any, **kwargs) -> None:  # pragma: no cover
        raise NotImplementedError

    def calculate(self) -> Dict[str, Any]:  # pragma: no cover
        raise NotImplementedError

    def reset(self) -> None:
        pass

    def _gather(self, obj):
        return Torch.gather_object(obj, self.process_group)


class LossMetric(Metric):
    """Σloss / Σtokens across ranks (mean-style losses count 1 per call) and the
    max grad-norm seen."""

    def reset(self):
        self.loss_sum, self.tokens, self.calls, self.grad_norm = 0.0, 0.0, 0, None

    def accumulate(self, inputs, outputs, **kwargs):
        loss = outputs.get('loss') if isinstance(outputs, dict) else outputs
        if loss is None:
            return
        self.loss_sum += _f(loss)
        nt = outputs.get('num_tokens', 0) if isinstance(outputs, dict) else 0
        self.tokens += _f(nt) if nt is not None else 0.0
        self.calls += 1
        gn = kwargs.get('grad_norm')
        if gn is not None:
            self.grad_norm = max(self.grad_norm or 0.0, _f(gn))

    def calculate(self):
        parts = self._gather((self.loss_sum, self.tokens, self.calls, self.grad_norm))
        ls = sum(p[0] for p in parts)
        tk = sum(p[1] for p in parts)
        calls = sum(p[2] for p in parts)
        out = {'loss': f'{(ls / tk) if tk > 0 else (ls / max(calls, 1)):.4f}'}
        gns = [p[3] for p in parts if p[3] is not None]
        if gns:
            out['grad_norm'] = f'{max(gns):.4f}'
        self.reset()
        return out


class Accuracy(Metric):

    def reset(self):
        self.correct, self.total = 0, 0

    def accumulate(self, inputs, outputs, **kwargs):
        logits = outputs.get('logits') if isinstance(outputs, dict) else None
        labels = inputs.get('labels') if isinstance(inputs, dict) else None
        if labels is None:
            return
        labels = torch.as_tensor(labels)
        if logits is not None:
            pred = logits.argmax(-1).reshape(labels.shape).cpu()
        elif isinstance(outputs, dict) and outputs.get('predictions') is not None:
            pred = torch.as_tensor(outputs['predictions']).reshape(labels.shape).cpu()
        else:
            return
        m = labels.cpu() != -100
        self.correct += int(((pred == labels.cpu()) & m).sum())
        self.total += int(m.sum())

    def calculate(self):
        parts = self._gather((self.correct, self.total))
        c, t = sum(p[0] for p in parts), sum(p[1] for p in parts)
        self.reset()
        return {'accuracy': f'{c / max(t, 1):.4f}'}


class TrainMetric(Metric):
    """lr, iteration count, elapsed time, iters/s — plus device-timed tokens/s
    when the engine reports ``step_ms`` and ``step_tokens``."""

    def reset(self):
        if not hasattr(self, 'start'):
            self.start, self.iters = time.time(), 0
        self.lr, self.step_ms, self.step_tokens = None, [], 0

    def accumulate(self, inputs, outputs, **kwargs):
        self.iters += 1 if kwargs.get('step_done', True) else 0
        if 'lr' in kwargs:
            self.lr = kwargs['lr']
        if 'step_ms' in kwargs:
            self.step_ms.append(float(kwargs['step_ms']))
            self.step_tokens += int(kwargs.get('step_tokens', 0))

    def calculate(self):
        el = max(time.time() - self.start, 1e-9)
        out = {'iters': str(self.iters), 'elapsed': f'{el:.1f}s', 'speed': f'{self.iters / el:.2f} iters/s'}
        if self.lr is not None:
            out['lr'] = f'{self.lr:.3e}' if not isinstance(self.lr, (list, tuple)) else ','.join(f'{x:.3e}' for x in self.lr)
        if self.step_ms:
            out['tokens_per_s'] = f'{self.step_tokens / (sum(self.step_ms) / 1e3):.1f}'
        self.lr, self.step_ms, self.step_tokens = None, [], 0
        return out


class CompletionRewardMetric(Metric):

    def reset(self):
        self.rewards, self.lengths, self.gen_time, self.sync_time = [], [], [], []

    def accumulate(self, inputs=None, outputs=None, *, rewards=None, completion_lengths=None, generate_time=None,
                   weight_sync_time=None, **kwargs):
        if rewards is not None:
            self.rewards += [float(r) for r in np.asarray(rewards).reshape(-1)]
        if completion_lengths is not None:
            self.lengths += [int(x) for x in np.asarray(completion_lengths).reshape(-1)]
        if generate_time is not None:
            self.gen_time.append(float(generate_time))
        if weight_sync_time is not None:
            self.sync_time.append(float(weight_sync_time))

    def calculate(self):
        out = {}
        if self.rewards:
            out['reward_mean'] = f'{np.mean(self.rewards):.4f}'
            out['reward_std'] = f'{np.std(self.rewards):.4f}'
        if self.lengths:
            out['completion_length'] = f'{np.mean(self.lengths):.1f}'
        if self.gen_time:
            out['generate_time'] = f'{np.mean(self.gen_time):.2f}s'
        if self.sync_time:
            out['weight_sync_time'] = f'{np.mean(self.sync_time):.2f}s'
        self.reset()
        return out


class GRPOMetric(Metric):
    """KL(old‖new) estimate and clip fractions from logps / old_logps."""
    epsilon, epsilon_high = 0.2, 0.2

    def reset(self):
        self.acc: Dict[str, List[float]] = {}

    def _push(self, k, v):
        self.acc.setdefault(k, []).append(float(v))

    def accumulate(self, inputs, outputs, *, old_logps=None, advantages=None, **kwargs):
        logps = outputs.get('logps') if isinstance(outputs, dict) else None
        labels = inputs.get('labels') if isinstance(inputs, dict) else None
        if logps is None or labels is None:
            return
        from ..loss.grpo import align_to_mask
        labels = torch.as_tensor(labels)
        if labels.dim() == 1:
            labels = labels[None]
        logps = logps.detach().float().cpu().reshape(labels.shape)
        mask = labels != -100
        old = logps if old_logps is None else align_to_mask(old_logps, mask, torch.float32).cpu()
        lr = torch.clamp(logps - old, -20, 20)
        ratio = self._ratio(lr, mask)
        n = mask.sum().clamp_min(1)
        self._push('kl', (((ratio - 1) - torch.log(ratio)) * mask).sum() / n)
        self._push('clip_ratio_low', ((ratio < 1 - self.epsilon) & mask).sum() / n)
        self._push('clip_ratio_high', ((ratio > 1 + self.epsilon_high) & mask).sum() / n)
        self._push('ratio_mean', (ratio * mask).sum() / n)
        if advantages is not None:
            self._push('advantage_abs', align_to_mask(advantages, mask, torch.float32).abs().sum() / n)

    def _ratio(self, log_ratio, mask):
        return log_ratio.exp()

    def calculate(self):
        parts = self._gather({k: (sum(v), len(v)) for k, v in self.acc.items()})
        out = {}
        for k in self.acc:
            s = sum(p[k][0] for p in parts if k in p)
            c = sum(p[k][1] for p in parts if k in p)
            out[k] = f'{s / max(c, 1):.6f}'
        self.reset()
        return out


class GSPOMetric(GRPOMetric):

    def _ratio(self, log_ratio, mask):
        m = mask.float()
        return ((log_ratio * m).sum(-1, keepdim=True) / m.sum(-1, keepdim=True).clamp_min(1)).exp().expand_as(log_ratio)


class CISPOMetric(GRPOMetric):
    pass


class DPOMetric(Metric):

    def reset(self):
        self.acc: Dict[str, List[float]] = {}

    def accumulate(self, inputs, outputs, *, loss_instance=None, **kwargs):
        stats = getattr(loss_instance, 'last_stats', None) or kwargs.get('stats')
        for k, v in (stats or {}).items():
            self.acc.setdefault(k, []).append(float(v))

    def calculate(self):
        out = {k: f'{np.mean(v):.4f}' for k, v in self.acc.items()}
        self.reset()
        return out


class EmbeddingMetric(Metric):
    """In-batch retrieval accuracy and mean positive / negative cosine."""

    def reset(self):
        self.hits, self.n, self.pos, self.neg = 0, 0, [], []

    def accumulate(self, inputs, outputs, group_size: int = 2, **kwargs):
        emb = outputs.get('embeddings')
        if emb is None:
            return
        e = torch.nn.functional.normalize(emb.detach().float().cpu(), dim=-1)
        q, d = e[0::group_size], e[1::group_size]
        sim = q @ d.t()
        self.hits += int((sim.argmax(-1) == torch.arange(len(q))).sum())
        self.n += len(q)
        self.pos.append(float(sim.diag().mean()))
        if len(q) > 1:
            off = sim[~torch.eye(len(q), dtype=torch.bool)]
            self.neg.append(float(off.mean()))

    def calculate(self):
        parts = self._gather((self.hits, self.n))
        out = {'retrieval_acc': f'{sum(p[0] for p in parts) / max(sum(p[1] for p in parts), 1):.4f}'}
        if self.pos:
            out['pos_sim'] = f'{np.mean(self.pos):.4f}'
        if self.neg:
            out['neg_sim'] = f'{np.mean(self.neg):.4f}'
        self.reset()
        return out


metric_mapping = {c.__name__: c for c in (LossMetric, Accuracy, TrainMetric, CompletionRewardMetric, GRPOMetric, GSPOMetric,
                                          CISPOMetric, DPOMetric, EmbeddingMetric)}
__all__ = ['Metric', 'metric_mapping'] + list(metric_mapping)
