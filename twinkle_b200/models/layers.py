"""Building blocks of the owned decoder: LoRA-capable linears, norms, embedding.

The LoRA slot pool follows the contract of the reference's
``src/twinkle/model/multi_lora.py:209-330``: ``max_loras`` physical adapters
of rank ``max_r`` exist on every target linear from start-up; a tenant bound to
a slot uses only the first ``r`` rows of ``A`` / columns of ``B`` and its own
``alpha/r`` (or ``alpha/√r``) scale; modules not matched by the tenant's
``target_modules`` skip the delta.  Unlike the reference (one tenant per
forward) a batch may carry several tenants: ``LoraBatch`` names, per token
segment, which slot applies, and the segmented kernel (``ops.sgmv``) serves
them in one launch.
"""
from __future__ import annotations

import math
import re
from contextlib import contextmanager
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class LoraBatch:
    """Per-forward LoRA routing: segment ``i`` covers token rows ``lo:hi`` and uses adapter slot ``slot``
    (−1 = base only) at rank ``rank`` with scale ``scale``.  Segments are kept on the host (they are built
    from Python integers) so that no kernel launch needs a device→host read; device copies are cached."""

    def __init__(self, segments, device, targets=None):
        self.host = [(int(lo), int(hi), int(slot), int(rank), float(scale)) for lo, hi, slot, rank, scale in segments]
        self.device = device
        self.targets: List[Optional[object]] = list(targets) if targets is not None else [None] * len(self.host)
        self._cache: Dict[tuple, tuple] = {}

    def tensors(self, keep: Optional[tuple] = None):
        """(seg_starts int32 [n+1], seg_slots int32 [n], seg_ranks int32 [n], seg_scales fp32 [n], host list) with
        the slots of segments where ``keep[i]`` is False forced to −1."""
        key = keep if keep is not None else ()
        hit = self._cache.get(key)
        if hit is None:
            host = [(lo, hi, (s if (keep is None or keep[i]) else -1), r, c) for i, (lo, hi, s, r, c) in enumerate(self.host)]
            dev = self.device
            hit = (torch.tensor([h[0] for h in host] + [host[-1][1] if host else 0], dtype=torch.int32, device=dev),
                   torch.tensor([h[2] for h in host], dtype=torch.int32, device=dev),
                   torch.tensor([h[3] for h in host], dtype=torch.int32, device=dev),
                   torch.tensor([h[4] for h in host], dtype=torch.float32, device=dev), host)
            self._cache[key] = hit
        return hit

    # tensor views of the unfiltered routing (used by code that inspects the batch)
    seg_starts = property(lambda self: self.tensors()[0])
    seg_slots = property(lambda self: self.tensors()[1])
    seg_ranks = property(lambda self: self.tensors()[2])
    seg_scales = property(lambda self: self.tensors()[3])

    @staticmethod
    def single(num_tokens: int, slot: int, rank: int, scale: float, device, target=None) -> 'LoraBatch':
        return LoraBatch([(0, num_tokens, slot, rank, scale)], device, [target])


class _LoraContext:
    batch: Optional[LoraBatch] = None


_CTX = _LoraContext()


@contextmanager
def lora_batch(batch: Optional[LoraBatch]):
    prev = _CTX.batch
    _CTX.batch = batch
    try:
        yield
    finally:
        _CTX.batch = prev


def current_lora_batch() -> Optional[LoraBatch]:
    return _CTX.batch


class TargetFilter:
    """``'all-linear'``, a list of module-name suffixes, or a full-match regex; ``exclude`` (same forms, PEFT's
    ``exclude_modules``) takes modules back out."""

    def __init__(self, spec, exclude=None):
        self.spec = spec
        self._re = None
        if isinstance(spec, str) and spec not in ('all-linear', 'all'):
            self._re = re.compile(spec)
        self.exclude = [exclude] if isinstance(exclude, str) and not any(c in exclude for c in '.*+?[(|') else exclude
        self._ex_re = re.compile(exclude) if isinstance(self.exclude, str) else None

    def matches(self, full_name: str, short_name: str) -> bool:
        if short_name == 'q_gate':      # the output gate is the second half of HF's q_proj: one adapter covers both
            short_name, full_name = 'q_proj', full_name[:-len('q_gate')] + 'q_proj'
        if self._ex_re is not None:
            if self._ex_re.fullmatch(full_name):
                return False
        elif self.exclude and any(full_name == t or full_name.endswith('.' + t) or short_name == t for t in self.exclude):
            return False
        s = self.spec
        if s is None or s in ('all-linear', 'all'):
            return short_name not in ('lm_head', 'gate')  # PEFT's all-linear excludes the output head; router kept off
        if self._re is not None:
            return self._re.fullmatch(full_name) is not None
        return any(full_name == t or full_name.endswith('.' + t) or short_name == t for t in s)


class Linear(nn.Module):
    """``y = x Wᵀ (+ b)`` with an optional LoRA slot pool.

    ``parts`` names the logical HF projections fused along the output dim, e.g.
    ``[('q_proj', 4096), ('k_proj', 1024), ('v_proj', 1024)]``; each part owns its
    own ``A``/``B`` so adapters stay PEFT-compatible per projection.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = False,
                 parts: Optional[Sequence[Tuple[str, int]]] = None, name: str = ''):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        # every use of this weight goes through a backward that can add dW into a buffer it is handed (`_wgrad_out`),
        # which lets a sharding engine skip the per-parameter gradient tensor altogether
        self.weight._direct_wgrad = True
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.parts = list(parts) if parts else [(name or 'linear', out_features)]
        assert sum(n for _, n in self.parts) == out_features
        self.full_name = ''  # set by the model after construction
        self.lora_A = nn.ParameterDict()
        self.lora_B = nn.ParameterDict()
        self.max_loras = 0
        self.max_r = 0
        self.wgrad_out: Optional[torch.Tensor] = None  # flat-bucket view to accumulate dW into
        self.gate_head_dim: Optional[int] = None  # set on a q|k|v|gate projection: head width used to interleave q and gate rows for export
        self.tp = None  # tensor-parallel context (parallel.tensor.TPContext)
        self.tp_mode: Optional[str] = None  # 'col' | 'row'

    # ------------------------------------------------------------- LoRA pool
    def add_lora_pool(self, max_loras: int, max_r: int, dtype=None, device=None) -> None:
        dtype = dtype or self.weight.dtype
        device = device or self.weight.device
        self.max_loras, self.max_r = max_loras, max_r
        for pname, n in self.parts:
            if pname == 'q_gate' and 'q_proj' in self.lora_A:
                # query and output gate are one projection in the checkpoint format (and for PEFT): they share the
                # adapter's A and each keeps its rows of B
                self.lora_A[pname] = self.lora_A['q_proj']
            else:
                a = torch.empty(max_loras, max_r, self.in_features, dtype=dtype, device=device)
                for s in range(max_loras):
                    nn.init.kaiming_uniform_(a[s], a=math.sqrt(5))
                self.lora_A[pname] = nn.Parameter(a)
            self.lora_B[pname] = nn.Parameter(torch.zeros(max_loras, n, max_r, dtype=dtype, device=device))

    def has_lora(self) -> bool:
        return self.max_loras > 0

    def _lora_delta(self, x2: torch.Tensor, lb: LoraBatch) -> Optional[torch.Tensor]:
        prefix = self.full_name.rsplit('.', 1)[0] if '.' in self.full_name else ''
        outs: List[Optional[torch.Tensor]] = []
        for pname, n in self.parts:
            keep = None
            if any(t is not None for t in lb.targets):
                keep = tuple(t is None or t.matches(f'{prefix}.{pname}' if prefix else pname, pname) for t in lb.targets)
                if not any(keep):
                    outs.append(None)
                    continue
                if all(keep):
                    keep = None
            st, sl, rk, sc, host = lb.tensors(keep)
            outs.append(ops.sgmv(x2, self.lora_A[pname], self.lora_B[pname], st, sl, rk, sc, host))
        if all(o is None for o in outs):
            return None
        outs = [o if o is not None else x2.new_zeros(x2.shape[0], n) for o, (_, n) in zip(outs, self.parts)]
        return outs[0] if len(outs) == 1 else torch.cat(outs, -1)

    def forward(self, x: torch.Tensor, value_unused: bool = False) -> torch.Tensor:
        """``value_unused``: this is the last linear of a layer; when the layer is only re-run to rebuild its graph the
        base product is skipped (the LoRA branch still runs: its intermediate is needed by its own backward)."""
        if self.tp_mode is not None:
            from ..parallel.tensor import tp_linear_forward
            return tp_linear_forward(self, x)
        wgrad_out = None
        if self.weight.requires_grad:  # set by the sharding engine while the flat gradient buffer is bound
            wgrad_out = self.wgrad_out if self.wgrad_out is not None else getattr(self.weight, '_wgrad_out', None)
        y = ops.linear(x, self.weight, self.bias, wgrad_out, value_unused)
        lb = _CTX.batch
        if lb is not None and self.max_loras > 0:
            x2 = x.reshape(-1, x.shape[-1])
            fused = self._lora_into(x2, y, lb)
            if fused is not None:
                return fused
            d = self._lora_delta(x2, lb)
            if d is not None:
                y = y + d.view(y.shape)
        return y

    def _lora_into(self, x2: torch.Tensor, y: torch.Tensor, lb: LoraBatch) -> Optional[torch.Tensor]:
        """GPU path: one shrink over the pools of all fused projections (stacked along the rank axis) and one expand
        whose epilogue adds the delta into ``y`` in place — no per-projection launches, no concatenation, no separate
        add.  Returns None when it does not apply (CPU / fp32, or tenants whose ``target_modules`` differ between the
        fused projections)."""
        if not ops.sgmv_fused_supported(x2) or y.dtype != torch.bfloat16 or y.dim() != 2 or not y.is_contiguous():
            return None
        prefix = self.full_name.rsplit('.', 1)[0] if '.' in self.full_name else ''
        keep = None
        if any(t is not None for t in lb.targets):
            keeps = [tuple(t is None or t.matches(f'{prefix}.{pname}' if prefix else pname, pname) for t in lb.targets) for pname, _ in self.parts]
            if any(k != keeps[0] for k in keeps[1:]):
                return None
            keep = keeps[0]
            if not any(keep):
                return y
            if all(keep):
                keep = None
        st, sl, rk, sc, host = lb.tensors(keep)
        names = [p for p, _ in self.parts]
        if len(names) == 1:
            a, b = self.lora_A[names[0]], self.lora_B[names[0]]
        else:
            P, R = len(names), self.max_r
            a = torch.cat([self.lora_A[p] for p in names], 1)                                              # [S, P·R, K]
            b = torch.cat([F.pad(self.lora_B[p], (i * R, (P - 1 - i) * R)) for i, p in enumerate(names)], 1)   # block-diagonal [S, N, P·R]
        return ops.sgmv(x2, a, b, st, sl, rk, sc, host, out=y, repeat=len(names))


class RMSNorm(nn.Module):

    def __init__(self, dim: int, eps: float = 1e-6, offset: float = 0.0):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim) if offset == 0.0 else torch.zeros(dim))
        self.eps, self.offset = eps, offset

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.offset)

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor):
        """``(norm(x + residual), x + residual)`` — the residual add rides in the norm kernel."""
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, self.offset)


class Embedding(nn.Module):

    def __init__(self, num: int, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num, dim))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.embedding(ids, self.weight)
