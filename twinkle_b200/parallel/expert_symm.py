"""Expert parallelism over peer memory: dispatch and combine as gathers from the peers' symmetric buffers.

What it replaces: the reference's expert-parallel data plane — ``all_gather`` of token counts,
``all_to_all_single`` dispatch with host-side split sizes, a local permute, the per-expert loop, the inverse permute
and the combine ``all_to_all_single`` (``src/twinkle/model/transformers/moe/ep_utils.py:183-288``,
``moe/expert_parallel.py:333-378``).  Here every rank *publishes* its tokens (and its sort order) in symmetric
memory, passes one flag barrier, and the expert side *pulls* exactly the rows it needs straight into the
128-aligned expert-grouped layout the grouped GEMM consumes; the way back is the mirror image, fused with the
weighted sum over a token's k experts.  No host read of split sizes, no staging buffer, no NCCL call.

Index bookkeeping (all on the device, derived from the ``[ep, E]`` matrix of per-rank expert counts that every
rank can compute identically after reading the peers' count vectors):

* token side — sorted pair ``p`` (expert ``e``) of rank ``s`` lands on rank ``e // El`` in row
  ``off[e] + before[s, e] + (p - start[s, e])``;
* expert side — row ``r`` of local expert ``e`` is fed by rank ``s`` at sorted position
  ``start[s, e] + (r - off[e] - before[s, e])``, or is padding.

``off`` are the 128-aligned segment starts (per destination rank), ``before`` the exclusive prefix over source
ranks, ``start`` the exclusive prefix over experts inside one source rank's sorted list.

The functions below take the "peer buffers" as lists of per-rank tensors when run on CPU (so the index math is
testable with all ranks emulated in one process) and as lists of device pointers on GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops


@dataclass
class EPMeta:
    """Everything one rank needs for one MoE layer pass."""
    order: torch.Tensor        # [n] flat (token, slot) index of the p-th sorted pair
    tok_sorted: torch.Tensor   # [n] int32 token of the p-th sorted pair
    dst_rank: torch.Tensor     # [T, k] int32 destination rank of every (token, slot); −1 = dropped (over capacity)
    dst_row: torch.Tensor      # [T, k] int32 row on that rank
    src_rank: torch.Tensor     # [cap] int32 source rank feeding each local row; −1 = padding
    src_pos: torch.Tensor      # [cap] int32 sorted position on that source rank
    offsets: torch.Tensor      # [El + 1] int32 aligned segment starts of the local experts
    total_rows: torch.Tensor   # [1] int32 rows the local experts need (may exceed cap → reported by the kernel)


def ep_metadata(flat_idx: torch.Tensor, counts_all: torch.Tensor, me: int, k: int, cap: int, align: int) -> EPMeta:
    """``flat_idx [n]`` = expert of every (token, slot) pair of this rank; ``counts_all [ep, E]`` = pairs per expert of
    every rank (row ``me`` must equal this rank's own histogram)."""
    dev = flat_idx.device
    ep, E = counts_all.shape
    El = E // ep
    n = flat_idx.numel()
    ca = counts_all.to(torch.int64)
    start = ca.cumsum(1) - ca                                   # [ep, E] exclusive prefix over experts per source rank
    before = ca.cumsum(0) - ca                                  # [ep, E] exclusive prefix over source ranks per expert
    tot = ca.sum(0)                                             # [E]
    padded = (tot + align - 1) // align * align
    pv = padded.view(ep, El)
    off = (pv.cumsum(1) - pv).reshape(-1)                       # [E] aligned start of every expert on its owner rank

    # ---- token side
    order = torch.argsort(_sort_keys(flat_idx, ca.shape[1]), stable=True)
    e_sorted = flat_idx[order]
    p = torch.arange(n, device=dev)
    row_sorted = off[e_sorted] + before[me][e_sorted] + (p - start[me][e_sorted])
    rank_sorted = e_sorted // El
    rank_sorted = torch.where(row_sorted < cap, rank_sorted, torch.full_like(rank_sorted, -1))
    dst_rank = torch.empty(n, dtype=torch.int32, device=dev)
    dst_row = torch.empty(n, dtype=torch.int32, device=dev)
    dst_rank[order] = rank_sorted.to(torch.int32)
    dst_row[order] = row_sorted.clamp_max(max(cap - 1, 0)).to(torch.int32)

    # ---- expert side: segments in (local expert, source rank) order, each expert followed by its padding
    lo = me * El
    seg = torch.empty(El, ep + 1, dtype=torch.int64, device=dev)
    seg[:, :ep] = ca[:, lo:lo + El].t()
    seg[:, ep] = (padded - tot)[lo:lo + El]
    seg_end = seg.reshape(-1).cumsum(0)                         # [El·(ep+1)]
    seg_begin = seg_end - seg.reshape(-1)
    r = torch.arange(cap, device=dev)
    sid = torch.searchsorted(seg_end, r, right=True)            # rows past the last segment get sid = El·(ep+1)
    valid = sid < seg_end.numel()
    sid_c = sid.clamp_max(seg_end.numel() - 1)
    e_l, s = sid_c // (ep + 1), sid_c % (ep + 1)
    is_pad = (~valid) | (s == ep)
    s_c = s.clamp_max(ep - 1)
    pos = start[s_c, lo + e_l] + (r - seg_begin[sid_c])
    src_rank = torch.where(is_pad, torch.full_like(s, -1), s).to(torch.int32)
    src_pos = torch.where(is_pad, torch.zeros_like(pos), pos).to(torch.int32)
    offsets = torch.zeros(El + 1, dtype=torch.int64, device=dev)
    offsets[1:] = padded[lo:lo + El].cumsum(0)
    total_rows = offsets[-1:].to(torch.int32)
    offsets = offsets.clamp_max(cap // align * align).to(torch.int32)
    return EPMeta(order, (order // k).to(torch.int32), dst_rank.view(-1, k), dst_row.view(-1, k), src_rank, src_pos, offsets, total_rows)


# --------------------------------------------------------------------- peer pulls (CUDA kernels / CPU emulation)
def pull_rows(x_bufs, tok_bufs, w_bufs, meta: EPMeta, H: int, tok_cap: int = 0, x_rows: int = 0) -> torch.Tensor:
    """``out[r] = (w_s[pos]) · x_s[tok_s[pos]]``; buffers are per-rank tensors (CPU) or device pointers (CUDA).
    ``tok_cap`` / ``x_rows``: capacities of every peer's token list and activation buffer — the kernel checks each
    position and token it reads from a peer against them before using it as an address."""
    if isinstance(x_bufs[0], int):
        return ops.ext().ep_rows_gather(list(x_bufs), list(tok_bufs), list(w_bufs) if w_bufs else [], meta.src_rank, meta.src_pos, H, meta.total_rows,
                                        tok_cap, x_rows)
    out = x_bufs[0].new_zeros(meta.src_rank.numel(), H)
    for s in range(len(x_bufs)):
        m = meta.src_rank == s
        pos = meta.src_pos[m].long()
        rows = x_bufs[s][tok_bufs[s][pos].long()]
        if w_bufs:
            rows = rows * w_bufs[s][pos].to(rows.dtype).unsqueeze(-1)
        out[m] = rows
    return out


def pull_combine(y_bufs, meta: EPMeta, w: Optional[torch.Tensor], H: int, y_rows: int = 0) -> torch.Tensor:
    """``out[t] = Σ_j w[t, j] · y_d[row]`` (``y_rows``: row capacity of every peer's buffer, checked in the kernel)."""
    if isinstance(y_bufs[0], int):
        return ops.ext().ep_rows_combine(list(y_bufs), meta.dst_rank, meta.dst_row, None if w is None else w.float().contiguous(), H, y_rows)
    T, k = meta.dst_rank.shape
    out = y_bufs[0].new_zeros(T, H)
    for d in range(len(y_bufs)):
        m = (meta.dst_rank == d)
        g = y_bufs[d][meta.dst_row.clamp_min(0).long().reshape(-1)].view(T, k, H)
        c = m.to(g.dtype) if w is None else m.to(g.dtype) * w.to(g.dtype)
        out += (g * c.unsqueeze(-1)).sum(1)
    return out


def pull_wgrad(g: torch.Tensor, y_bufs, meta: EPMeta, y_rows: int = 0) -> torch.Tensor:
    """``dw[t, j] = <g[t], y_d[row]>``."""
    if isinstance(y_bufs[0], int):
        return ops.ext().ep_combine_wgrad(g.contiguous(), list(y_bufs), meta.dst_rank, meta.dst_row, y_rows)
    T, k = meta.dst_rank.shape
    dw = torch.zeros(T, k, dtype=torch.float32, device=g.device)
    for d in range(len(y_bufs)):
        m = (meta.dst_rank == d)
        yy = y_bufs[d][meta.dst_row.clamp_min(0).long().reshape(-1)].view(T, k, -1)
        dw += (yy.float() * g.float().unsqueeze(1)).sum(-1) * m
    return dw


# ------------------------------------------------------------------------------------------- the strategy object
class _Slots:
    """One set of symmetric buffers (token-side rows, expert-side rows, sort order, sorted weights, counts)."""

    def __init__(self, comm, T: int, cap: int, H: int, n: int, E: int, dtype):
        self.x = comm.alloc(T * H, dtype).view(T, H)
        self.y = comm.alloc(cap * H, dtype).view(cap, H)
        self.tok = comm.alloc(n, torch.int32)
        self.w = comm.alloc(n, torch.float32)
        self.counts = comm.alloc(E, torch.int32)
        self.x_ptrs, self.y_ptrs = comm.peer_ptrs(self.x), comm.peer_ptrs(self.y)
        self.tok_ptrs, self.w_ptrs, self.counts_ptrs = comm.peer_ptrs(self.tok), comm.peer_ptrs(self.w), comm.peer_ptrs(self.counts)


class SymmExpertParallel:
    """``MoEBlock.moe_parallel`` strategy on a ``SymmCommunicator``.

    Buffer sets alternate between publish events.  A set is overwritten two events after it was published; by then
    this rank has passed the barrier of the event in between, which every peer reaches only after its pulls from the
    older set have been issued on its stream — so no extra "buffer free" barrier is needed.
    """

    def __init__(self, comm, num_experts: int, capacity_factor: float = 1.5):
        self.comm, self.ep, self.rank = comm, comm.world_size, comm.rank
        assert num_experts % self.ep == 0
        self.num_experts, self.local = num_experts, num_experts // self.ep
        self.capacity_factor = capacity_factor
        self._sets: List[_Slots] = []
        self._event = 0
        self._shape = None

    def _ensure(self, T: int, H: int, k: int, dtype) -> int:
        """Symmetric buffers must have one size on every rank: the first call agrees on the largest token count of
        the group (one host-side reduction) and allocates for it; later calls only check that they fit."""
        if self._shape is None:
            t = torch.tensor([T], device=self.comm.device, dtype=torch.int64)
            self.comm.all_reduce(t, 'max')
            T_alloc = (int(t.item()) + 1023) // 1024 * 1024
            n = T_alloc * k
            cap = (int(n * self.capacity_factor) + self.local * 127 + 127) // 128 * 128
            self._sets = [_Slots(self.comm, T_alloc, cap, H, n, self.num_experts, dtype) for _ in range(2)]
            self._shape = (T_alloc, H, k, dtype)
        T_alloc, H0, k0, dt0 = self._shape
        if T > T_alloc or (H, k, dtype) != (H0, k0, dt0):
            raise RuntimeError(f'expert-parallel buffers were sized for {T_alloc} tokens per rank (hidden {H0}, top-{k0}); '
                               f'got {T} tokens (hidden {H}, top-{k}). Start with the largest micro-batch first.')
        return self._sets[0].y.shape[0]

    def _next(self) -> _Slots:
        s = self._sets[self._event % 2]
        self._event += 1
        return s

    def forward(self, block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        k = idx.shape[1]
        cap = self._ensure(T, H, k, x.dtype)
        hist = getattr(block, '_hist', None)
        flat = idx.reshape(-1)
        if hist is None:
            hist = torch.zeros(self.num_experts, dtype=torch.int32, device=x.device).scatter_add_(
                0, flat, torch.ones_like(flat, dtype=torch.int32))
        xs, meta = _EPDispatch.apply(x, self, flat, hist.to(torch.int32), k, cap)
        ys = block.experts(xs, meta.offsets)
        return _EPCombine.apply(ys, w, self, meta)

    # one publish event: copy into the set, barrier, return the set
    def publish(self, x=None, y=None, tok=None, w=None, counts=None) -> _Slots:
        s = self._next()
        if x is not None:
            s.x[:x.shape[0]].copy_(x)
        if y is not None:
            s.y[:y.shape[0]].copy_(y)
        if tok is not None:
            s.tok[:tok.numel()].copy_(tok)
        if w is not None:
            s.w[:w.numel()].copy_(w)
        if counts is not None:
            s.counts.copy_(counts)
        self.comm.barrier_kernel()
        return s


def _sort_keys(expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Expert ids as one-byte keys when they fit: the device radix sort then makes one pass instead of eight."""
    return expert_ids.to(torch.uint8) if (expert_ids.is_cuda and num_experts <= 256) else expert_ids


class _EPDispatch(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, strat: SymmExpertParallel, flat, hist, k, cap):
        order = torch.argsort(_sort_keys(flat, strat.num_experts), stable=True)
        s = strat.publish(x=x, tok=(order // k).to(torch.int32), counts=hist)
        counts_all = torch.empty(strat.ep, strat.num_experts, dtype=torch.int32, device=x.device)
        strat.comm.ext.peer_all_gather(counts_all, s.counts_ptrs, strat.num_experts * 4, strat.rank, 1)
        meta = ep_metadata(flat, counts_all, strat.rank, k, cap, 128)
        xs = pull_rows(s.x_ptrs, s.tok_ptrs, None, meta, x.shape[1], s.tok.numel(), s.x.shape[0])
        ctx.strat, ctx.meta, ctx.H = strat, meta, x.shape[1]
        ctx.set_materialize_grads(False)
        return xs, meta

    @staticmethod
    def backward(ctx, gxs, _gmeta):
        if gxs is None:
            return None, None, None, None, None, None
        s = ctx.strat.publish(y=gxs.contiguous())
        gx = pull_combine(s.y_ptrs, ctx.meta, None, ctx.H, s.y.shape[0])
        return gx, None, None, None, None, None


class _EPCombine(torch.autograd.Function):

    @staticmethod
    def forward(ctx, ys, w, strat: SymmExpertParallel, meta: EPMeta):
        s = strat.publish(y=ys)
        out = pull_combine(s.y_ptrs, meta, w, ys.shape[1], s.y.shape[0])
        ctx.save_for_backward(ys, w)
        ctx.strat, ctx.meta = strat, meta
        return out

    @staticmethod
    def backward(ctx, g):
        ys, w = ctx.saved_tensors
        meta, strat = ctx.meta, ctx.strat
        g = g.contiguous()
        w_sorted = w.reshape(-1).float()[meta.order]
        s = strat.publish(x=g, y=ys, tok=meta.tok_sorted, w=w_sorted)
        gys = pull_rows(s.x_ptrs, s.tok_ptrs, s.w_ptrs, meta, g.shape[1], s.tok.numel(), s.x.shape[0])
        gw = pull_wgrad(g, s.y_ptrs, meta, s.y.shape[0])
        return gys, gw.to(w.dtype), None, None
