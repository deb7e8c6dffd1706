"""Advantage estimators.

Parity: reference ``src/twinkle/advantage/grpo.py:10-68`` and ``rloo.py:10-63``.
Rewards arrive flat, ``num_generations`` consecutive entries per prompt.
"""
from __future__ import annotations

from typing import List, Sequence, Union

import torch


class Advantage:

    def __call__(self, rewards, num_generations: int = 1, scale: str = 'group', **kwargs) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


def _as_groups(rewards, num_generations: int) -> torch.Tensor:
    r = torch.as_tensor(rewards, dtype=torch.float32).reshape(-1)
    if num_generations < 1 or r.numel() % num_generations != 0:
        raise ValueError(f'{r.numel()} rewards cannot be grouped by {num_generations}')
    return r.view(-1, num_generations)


class GRPOAdvantage(Advantage):
    """``A = r − mean(group)``; divided by the group's (unbiased) std for
    ``scale='group'``, by the whole batch's std for ``'batch'``, left alone for
    ``'none'``.  ε = 1e−8."""

    def __call__(self, rewards, num_generations: int = 1, scale: str = 'group', **kwargs) -> torch.Tensor:
        g = _as_groups(rewards, num_generations)
        adv = g - g.mean(dim=1, keepdim=True)
        if scale == 'group':
            std = g.std(dim=1, keepdim=True) if num_generations > 1 else torch.zeros_like(adv[:, :1])
            adv = adv / (std + 1e-8)
        elif scale == 'batch':
            std = g.reshape(-1).std() if g.numel() > 1 else torch.tensor(0.0)
            adv = adv / (std + 1e-8)
        elif scale not in ('none', None):
            raise ValueError(f'scale must be group|batch|none, got {scale}')
        return adv.reshape(-1)


class RLOOAdvantage(Advantage):
    """Leave-one-out baseline: ``A_i = r_i − mean_{j≠i} r_j``."""

    def __call__(self, rewards, num_generations: int = 1, scale: str = 'none', **kwargs) -> torch.Tensor:
        g = _as_groups(rewards, num_generations)
        if num_generations == 1:
            return g.reshape(-1)
        baseline = (g.sum(dim=1, keepdim=True) - g) / (num_generations - 1)
        adv = g - baseline
        if scale == 'group':
            adv = adv / (g.std(dim=1, keepdim=True) + 1e-8)
        elif scale == 'batch':
            adv = adv / (g.reshape(-1).std() + 1e-8)
        return adv.reshape(-1)


advantage_mapping = {'grpo': GRPOAdvantage, 'rloo': RLOOAdvantage, 'GRPOAdvantage': GRPOAdvantage, 'RLOOAdvantage': RLOOAdvantage}
__all__ = ['Advantage', 'GRPOAdvantage', 'RLOOAdvantage', 'advantage_mapping']
