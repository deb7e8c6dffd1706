"""Context parallelism for causal attention over zig-zag sharded sequences.

What it replaces: the reference's zig-zag ring flash attention (``model/transformers/strategy/sequence_parallel/
zigzag_ring_attn.py``: ring ``isend``/``irecv`` of K and V, three mask cases per step, online-softmax merge of the
partial outputs).  Every sequence is cut into ``2·cp`` chunks and rank ``r`` holds chunks ``r`` and ``2cp−1−r``
(``processor.zigzag_indices``), so every rank has the same amount of causal work.

Design here: keys and values are small next to queries under GQA, so they are all-gathered once per layer (one
collective instead of ``cp−1`` ring steps) and the attention kernel is called ONCE with ``2·n`` entries — the two
local chunks of every sequence — each attending to its own key prefix through the kernel's separate key boundaries
and bottom-right causal alignment.  No partial outputs exist, so nothing has to be merged, and the backward is the
ordinary flash backward followed by the reduce-scatter that is the all-gather's adjoint.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from .comm import Communicator


class _AllGatherRows(torch.autograd.Function):
    """fwd: all-gather along dim 0 → [cp·T, …]; bwd: reduce-scatter (sum over ranks of the slice that is ours)."""

    @staticmethod
    def forward(ctx, x, comm: Communicator):
        ctx.comm, ctx.n = comm, x.shape[0]
        return comm.all_gather_tensor(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        comm = ctx.comm
        g = g.contiguous()
        out = g.new_empty((ctx.n, ) + tuple(g.shape[1:]))
        import torch.distributed as dist
        dist.reduce_scatter_tensor(out, g, group=comm.group)
        return out, None


def cp_key_index(seq_lens: Sequence[int], cp: int, rank: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int, int]:
    """For the local layout ``[chunk r ; chunk 2cp−1−r]`` per sequence: (rows of the rank-major gathered K/V to pack as
    keys, cu_q [2n+1], cu_k [2n+1], max q length, max k length).  ``seq_lens`` are the full lengths (multiples of 2·cp)."""
    t_loc = sum(n // cp for n in seq_lens)
    rows: List[torch.Tensor] = []
    cu_q, cu_k = [0], [0]
    a = 0
    max_q = max_k = 0
    for n in seq_lens:
        c = n // (2 * cp)

        def chunk_rows(j: int) -> torch.Tensor:  # global chunk j of this sequence inside the gathered tensor
            owner, second = (j, 0) if j < cp else (2 * cp - 1 - j, 1)
            start = owner * t_loc + a + second * c
            return torch.arange(start, start + c)

        for last in (rank, 2 * cp - 1 - rank):           # first local chunk sees chunks 0…r, second 0…2cp−1−r
            rows.extend(chunk_rows(j) for j in range(last + 1))
            cu_q.append(cu_q[-1] + c)
            cu_k.append(cu_k[-1] + (last + 1) * c)
            max_q, max_k = max(max_q, c), max(max_k, (last + 1) * c)
        a += 2 * c
    idx = torch.cat(rows) if rows else torch.zeros(0, dtype=torch.long)
    return (idx.to(device), torch.tensor(cu_q, dtype=torch.int32, device=device), torch.tensor(cu_k, dtype=torch.int32, device=device),
            max_q, max_k)


class ContextParallelAttention:
    """Strategy plugged into ``Attention.attn_parallel`` (``attention`` replaces the local flash-attention call)."""

    def __init__(self, comm: Communicator):
        self.comm, self.cp, self.rank = comm, comm.world_size, comm.rank
        self._cache_key, self._cache = None, None

    def _index(self, seq_lens: Sequence[int], device):
        key = (tuple(seq_lens), str(device))
        if key != self._cache_key:
            self._cache_key, self._cache = key, cp_key_index(seq_lens, self.cp, self.rank, device)
        return self._cache

    def attention(self, q, k, v, seq_lens: Sequence[int], scale: float) -> torch.Tensor:
        idx, cu_q, cu_k, max_q, max_k = self._index(seq_lens, q.device)
        kg = _AllGatherRows.apply(k, self.comm).index_select(0, idx)
        vg = _AllGatherRows.apply(v, self.comm).index_select(0, idx)
        return ops.flash_attn_varlen(q, kg, vg, cu_q, max_q, True, scale, cu_seqlens_k=cu_k, max_seqlen_k=max_k)


def gather_zigzag_rows(x: torch.Tensor, comm: Communicator, seq_lens: Sequence[int], fill, differentiable: bool) -> torch.Tensor:
    """Per-token values of the context-parallel peers put back at their positions in the full packed row: every rank
    ends up with whole sequences (the loss needs them), and — when ``differentiable`` — back-propagates only into its
    own zig-zag pieces, so the loss is counted once."""
    from ..processor import zigzag_indices
    from .ulysses import gather_tokens
    cp = comm.world_size
    pieces = []
    for r in range(cp):
        off = 0
        for n in seq_lens:
            pieces.append(zigzag_indices(n, cp, r) + off)
            off += n
    perm = torch.cat(pieces).to(x.device)
    g = gather_tokens(x, comm) if differentiable else comm.all_gather_tensor(x)
    return g.new_full((perm.numel(), ) + tuple(g.shape[1:]), fill).index_copy(0, perm, g)


_CP_GROUPS = {}


def cp_group_for(mesh):
    """Process group of the ranks that share this rank's sequences (the mesh's ``cp`` dimension)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or not mesh.has_dim('cp') or mesh.get_dim_size('cp') <= 1:
        return None
    key = mesh.signature()
    if key not in _CP_GROUPS:
        _CP_GROUPS[key] = mesh.get_dim_group('cp')
    return _CP_GROUPS[key]


def apply_context_parallel(model, mesh) -> Optional[ContextParallelAttention]:
    group = cp_group_for(mesh)
    if group is None:
        return None
    dev = next(model.parameters()).device
    strat = ContextParallelAttention(Communicator(group, dev))
    for layer in model.layers:
        layer.self_attn.attn_parallel = strat
    return strat
