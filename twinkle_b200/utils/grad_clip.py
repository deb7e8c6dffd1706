"""Gradient normalisation + clipping for plain (non-bucketed) parameter lists.

Parity: reference ``src/twinkle/utils/grad_clip.py:31-377``: divide gradients
by the global token count in place, compute the L2 / inf norm with a reduction
over the sharding group (experts: first over ``ep_fsdp`` then ``ep``), clip.
The bucketed engine folds the same arithmetic into its fused AdamW scale
(``model/native.py``); this helper serves replicated parameters (LoRA pools)
and user code.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


def _reduce(t: torch.Tensor, group, op) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and group is not False:
        if group is None or dist.get_world_size(group) > 1:
            dist.all_reduce(t, op=op, group=group)
    return t


def normalize_and_clip_grad_norm(params: Iterable[torch.nn.Parameter], num_tokens: float = 1.0, max_grad_norm: float = 1.0,
                                 norm_type: float = 2.0, group=False, ep_params: Optional[List[torch.nn.Parameter]] = None,
                                 ep_group=None, ep_fsdp_group=None, sharded: bool = False) -> float:
    """``sharded=True`` means each rank holds a disjoint slice of every
    gradient (norm partials are summed over ``group``); otherwise gradients are
    replicated and no reduction is needed.  Returns the pre-clip norm."""
    params = [p for p in params if p.grad is not None]
    ep_ids = {id(p) for p in (ep_params or [])}
    dense = [p for p in params if id(p) not in ep_ids]
    experts = [p for p in params if id(p) in ep_ids]
    if num_tokens and num_tokens != 1.0:
        for p in params:
            p.grad.div_(num_tokens)
    dev = params[0].grad.device if params else torch.device('cpu')
    inf = math.isinf(norm_type)

    def partial(ps):
        if not ps:
            return torch.zeros((), device=dev)
        if inf:
            return torch.stack([p.grad.detach().abs().max().float() for p in ps]).max()
        return torch.stack([p.grad.detach().float().norm(norm_type)**norm_type for p in ps]).sum()

    op = dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM
    d = partial(dense)
    if sharded:
        d = _reduce(d, group, op)
    e = partial(experts)
    if experts:
        if ep_fsdp_group is not None:
            e = _reduce(e, ep_fsdp_group, op)
        if ep_group is not None:
            e = _reduce(e, ep_group, op)
    total = torch.maximum(d, e) if inf else (d + e)**(1.0 / norm_type)
    total_f = float(total)
    if max_grad_norm is not None and max_grad_norm > 0:
        coef = min(1.0, max_grad_norm / (total_f + 1e-6))
        if coef < 1.0:
            for p in params:
                p.grad.mul_(coef)
    return total_f
