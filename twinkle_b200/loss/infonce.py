"""In-batch contrastive loss for the embedding task.

Parity: reference ``src/twinkle/loss/infonce.py:73-292`` — rows come as
(query, positive[, negatives…]) groups, similarities are cosine / temperature,
negatives are every other document in the (optionally cross-rank gathered)
batch.  The gather keeps gradients for the local shard only.
"""
from __future__ import annotations

from typing import Any, Dict

import torch
import torch.nn.functional as F

from ..data_format import LossOutput
from .base import Loss


def gather_with_local_grad(x: torch.Tensor, group=None) -> torch.Tensor:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return x
    n = torch.tensor([x.shape[0]], device=x.device)
    sizes = [torch.zeros_like(n) for _ in range(dist.get_world_size(group))]
    dist.all_gather(sizes, n, group=group)
    m = int(max(s.item() for s in sizes))
    padded = F.pad(x.detach(), (0, 0, 0, m - x.shape[0]))
    bufs = [torch.zeros_like(padded) for _ in sizes]
    dist.all_gather(bufs, padded, group=group)
    r = dist.get_rank(group)
    parts = [x if i == r else b[:int(s.item())] for i, (b, s) in enumerate(zip(bufs, sizes))]
    return torch.cat(parts, 0)


class InfonceLoss(Loss):
    require_logits = False
    require_logps = False

    def __init__(self, temperature: float = 0.05, group_size: int = 2, cross_rank: bool = True, **kwargs):
        self.temperature, self.group_size, self.cross_rank = temperature, group_size, cross_rank

    def __call__(self, inputs: Dict[str, Any], outputs: Dict[str, Any], **kwargs) -> LossOutput:
        emb = F.normalize(outputs['embeddings'].float(), dim=-1)
        g = self.group_size
        q, docs = emb[0::g], torch.cat([emb[i::g] for i in range(1, g)], 0)
        n_local = q.shape[0]
        if self.cross_rank:
            all_docs = gather_with_local_grad(docs, kwargs.get('group'))
            import torch.distributed as dist
            offset = 0
            if dist.is_available() and dist.is_initialized() and all_docs.shape[0] != docs.shape[0]:
                offset = dist.get_rank(kwargs.get('group')) * docs.shape[0]
        else:
            all_docs, offset = docs, 0
        sim = q @ all_docs.t() / self.temperature
        target = torch.arange(n_local, device=sim.device) + offset
        return LossOutput(loss=F.cross_entropy(sim, target), num_tokens=0)
