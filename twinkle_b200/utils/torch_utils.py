"""Token log-prob helpers.

Parity: reference ``src/twinkle/utils/torch_utils.py:61-147`` —
``selective_log_softmax(logits, index)`` returns ``log softmax(logits)[index]``
without keeping a ``[T, V]`` fp32 copy, optionally with per-token entropy.
On B200 the row-loop of the reference is replaced by one fused kernel
(``ops.fused_logprob``); the chunked PyTorch formula below is the oracle and
the CPU path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def selective_log_softmax_reference(logits: torch.Tensor, index: torch.Tensor, chunk: int = 4096,
                                    with_entropy: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    flat = logits.reshape(-1, logits.shape[-1])
    idx = index.reshape(-1)
    logps = torch.empty(flat.shape[0], dtype=torch.float32, device=flat.device)
    ent = torch.empty_like(logps) if with_entropy else None
    for s in range(0, flat.shape[0], chunk):
        x = flat[s:s + chunk].float()
        lse = torch.logsumexp(x, dim=-1)
        logps[s:s + chunk] = x.gather(-1, idx[s:s + chunk, None]).squeeze(-1) - lse
        if with_entropy:
            p = torch.softmax(x, dim=-1)
            ent[s:s + chunk] = lse - (p * x).sum(-1)
    shape = index.shape
    return logps.view(shape), (ent.view(shape) if with_entropy else None)


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor, with_entropy: bool = False):
    """Differentiable w.r.t. ``logits``.  Returns logps, or (logps, entropy)."""
    if logits.is_cuda:
        from ..ops import logprob_from_logits
        out = logprob_from_logits(logits, index, with_entropy=with_entropy)
        return out if with_entropy else out[0]
    x = logits.float()
    lse = torch.logsumexp(x, dim=-1)
    lp = x.gather(-1, index.unsqueeze(-1)).squeeze(-1) - lse
    if not with_entropy:
        return lp
    p = torch.softmax(x, dim=-1)
    return lp, lse - (p * x).sum(-1)


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    x = logits.float()
    lse = torch.logsumexp(x, dim=-1)
    return lse - (torch.softmax(x, -1) * x).sum(-1)


def pad_and_stack(tensors, pad_value=0, side: str = 'right') -> torch.Tensor:
    """Stack 1-D/ N-D tensors whose first dim differs, padding with ``pad_value``."""
    n = max(t.shape[0] for t in tensors)
    out = []
    for t in tensors:
        pad = n - t.shape[0]
        if pad:
            filler = t.new_full((pad, ) + tuple(t.shape[1:]), pad_value)
            t = torch.cat([t, filler] if side == 'right' else [filler, t], 0)
        out.append(t)
    return torch.stack(out, 0)


# ---------------------------------------------------------------- small helpers (reference ``utils/torch_utils.py:11-60, 235-260``)
def to_device(data, device, non_blocking: bool = False):
    """Tensors inside (nested) mappings, lists and tuples moved to ``device``; everything else returned as it is."""
    if isinstance(data, dict):
        return type(data)((k, to_device(v, device, non_blocking)) for k, v in data.items())
    if isinstance(data, (list, tuple)):
        return type(data)(to_device(v, device, non_blocking) for v in data)
    return data.to(device, non_blocking=non_blocking) if isinstance(data, torch.Tensor) else data


def clone_state_dict_to_cpu(state_dict) -> dict:
    """Detached host copies of every tensor of a state dict (other values pass through)."""
    return {k: (v.detach().to('cpu', copy=True) if isinstance(v, torch.Tensor) else v) for k, v in state_dict.items()}


def pad_sequence_to_length(tensor: torch.Tensor, max_seq_len: int, pad_value: float = 0.0, left_pad: bool = False) -> torch.Tensor:
    """The last dimension padded with ``pad_value`` up to ``max_seq_len`` (unchanged when it is already that long)."""
    n = max_seq_len - tensor.shape[-1]
    if n <= 0:
        return tensor
    return torch.nn.functional.pad(tensor, (n, 0) if left_pad else (0, n), value=pad_value)


def pad_and_stack_tensors(tensors, pad_value: float = -200, concat: bool = True) -> torch.Tensor:
    """Tensors of equal rank and differing sizes padded (at the end of every dimension) to their common largest shape, then
    concatenated along the first dimension (``concat=True``: rows of all tensors in one batch) or stacked on a new one."""
    if not tensors:
        raise ValueError('no tensors to pad')
    rank = tensors[0].dim()
    if any(t.dim() != rank for t in tensors):
        raise ValueError('tensors must have the same number of dimensions')
    dims = range(1, rank) if concat else range(rank)
    target = {d: max(t.shape[d] for t in tensors) for d in dims}
    out = []
    for t in tensors:
        pad = []
        for d in reversed(range(rank)):
            pad += [0, (target[d] - t.shape[d]) if d in target else 0]
        out.append(torch.nn.functional.pad(t, pad, value=pad_value))
    return torch.cat(out, 0) if concat else torch.stack(out, 0)
