"""Expert parallelism: experts are split over the ``ep`` group, tokens travel to their experts and back.

Parity: reference ``src/twinkle/model/transformers/moe/expert_parallel.py:16-606`` and ``moe/ep_utils.py:
13-288`` (slice experts ``[start:end]`` per rank, router → counts exchange → permute by expert → uneven
all-to-all → per-expert FFN → all-to-all back → weight and scatter-add).  Differences by design:

* the per-expert ``F.linear`` loop with one host sync per expert becomes one grouped GEMM over an
  expert-sorted, 128-row-aligned layout built entirely on the device (``expert_layout``);
* the baseline data plane is ``all_to_all_single`` (NCCL / gloo — needs the split sizes on the host, one sync
  per layer as in the reference); the peer-memory plane (``SymmCommunicator``) pushes rows straight into
  the destination rank's buffer with device-side offsets and needs no host sync.

EP groups are consecutive blocks of ``ep_size`` ranks in the flattened (dp, fsdp) order; expert gradients
are therefore already summed over the tokens of the whole EP group by the backward all-to-all and only need
reducing across EP *replicas* (the ``ep_fsdp`` dimension).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .comm import Communicator

_EP_GROUPS = {}


def ep_group_for(mesh):
    ep = mesh.ep_size or 1
    if ep <= 1 or not (dist.is_available() and dist.is_initialized()):
        return None
    key = (mesh.signature(), ep)
    if key in _EP_GROUPS:
        return _EP_GROUPS[key][0]
    ranks = sorted(mesh._coord_of, key=lambda r: (mesh._flat_data_index(r), r))
    me, mine, mine_rep = dist.get_rank(), None, None
    for i in range(0, len(ranks), ep):
        grp = ranks[i:i + ep]
        g = dist.new_group(ranks=grp)
        if me in grp:
            mine = g
    # replica groups: same position inside every EP block
    for j in range(ep):
        grp = ranks[j::ep]
        g = dist.new_group(ranks=grp)
        if me in grp:
            mine_rep = g
    _EP_GROUPS[key] = (mine, mine_rep)
    return mine


def ep_replica_group_for(mesh):
    ep_group_for(mesh)
    return _EP_GROUPS.get((mesh.signature(), mesh.ep_size or 1), (None, None))[1]


def expert_layout(expert_ids: torch.Tensor, num_experts: int, align: int,
                  counts: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """Rows for an expert-grouped GEMM.  ``expert_ids [n]`` → (``order`` = argsort by expert, ``rows [n]`` =
    destination row of ``order[i]``, ``offsets [E+1]`` int32 with every expert's segment starting on a
    multiple of ``align``, upper bound of total rows known without a device sync)."""
    n = expert_ids.numel()
    # expert ids fit one byte for up to 256 experts: the radix sort then takes one pass over the keys instead of eight
    keys = expert_ids.to(torch.uint8) if (expert_ids.is_cuda and num_experts <= 256) else expert_ids
    order = torch.argsort(keys, stable=True)
    if counts is None:  # scatter-add instead of bincount: no device→host read
        counts = torch.zeros(num_experts, dtype=torch.int64, device=expert_ids.device).scatter_add_(
            0, expert_ids, torch.ones_like(expert_ids, dtype=torch.int64))
    counts = counts.to(torch.int64)
    padded = (counts + align - 1) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=expert_ids.device)
    offsets[1:] = padded.cumsum(0)
    starts = torch.zeros(num_experts, dtype=torch.int64, device=expert_ids.device)
    starts[1:] = counts.cumsum(0)[:-1]
    e_sorted = expert_ids[order]
    rows = offsets[:-1][e_sorted] + (torch.arange(n, device=expert_ids.device) - starts[e_sorted])
    bound = (n + num_experts * (align - 1) + align - 1) // align * align if align > 1 else n
    return order, rows, offsets.to(torch.int32), bound


class _AllToAll(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, comm: Communicator, in_splits: List[int], out_splits: List[int]):
        ctx.comm, ctx.in_splits, ctx.out_splits = comm, in_splits, out_splits
        out = x.new_empty((sum(out_splits), ) + tuple(x.shape[1:]))
        comm.all_to_all_single(out, x.contiguous(), out_splits, in_splits)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits), ) + tuple(g.shape[1:]))
        ctx.comm.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits)
        return out, None, None, None


class ExpertParallel:
    """Strategy object plugged into ``MoEBlock.moe_parallel``."""

    def __init__(self, comm: Communicator, num_experts: int):
        self.comm, self.ep = comm, comm.world_size
        assert num_experts % self.ep == 0, f'{num_experts} experts do not divide over ep={self.ep}'
        self.num_experts, self.local = num_experts, num_experts // self.ep

    def forward(self, block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        k, E, El, ep = idx.shape[1], self.num_experts, self.local, self.ep
        flat = idx.reshape(-1)
        # 1. sort (token, slot) pairs by global expert: contiguous per destination rank
        order = torch.argsort(flat, stable=True)
        tok = order // k
        send = x.index_select(0, tok)
        counts = torch.bincount(flat, minlength=E)                       # [E] pairs per expert on this rank
        # 2. exchange counts: recv_counts[s, e_local] = pairs rank s sends for my expert e_local
        recv_counts = torch.empty(ep, El, dtype=counts.dtype, device=x.device)
        self.comm.all_to_all_single(recv_counts.view(-1), counts.contiguous())
        in_splits = counts.view(ep, El).sum(1).tolist()                  # host sync (baseline data plane)
        out_splits = recv_counts.sum(1).tolist()
        # 3. dispatch
        recv = _AllToAll.apply(send, self.comm, in_splits, out_splits)  # grouped by source rank, then expert
        # 4. regroup by local expert into the aligned layout
        src_expert = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(ep), recv_counts.reshape(-1))
        align = 128 if x.is_cuda else 1
        o2, rows, offsets, bound = expert_layout(src_expert, El, align)
        xs = x.new_zeros(bound, H)
        xs = xs.index_copy(0, rows, recv.index_select(0, o2))
        ys = block.experts(xs, offsets)
        # 5. back to arrival order, combine
        back = torch.empty_like(recv).index_copy(0, o2, ys.index_select(0, rows))
        ret = _AllToAll.apply(back, self.comm, out_splits, in_splits)
        ret = ret * w.reshape(-1)[order].to(ret.dtype).unsqueeze(-1)
        out = torch.zeros(T, H, dtype=ret.dtype, device=x.device)
        return out.index_add(0, tok, ret)


def shard_experts(model, strat, ep_rank: int, rep_comm: Optional[Communicator]) -> None:
    """Keep the experts ``[ep_rank·E_local, (ep_rank+1)·E_local)`` of every MoE block (cut from the identically
    initialised full tensors), route the blocks through ``strat``, and mark the expert tensors as EP-local: their
    gradients are summed over ``rep_comm`` (the ranks that hold the same experts), never over the whole data group."""
    El = strat.local
    lo = ep_rank * El
    for layer in model.layers:
        if not getattr(layer, 'is_moe', False):
            continue
        ex = layer.mlp.experts
        with torch.no_grad():
            ex.gate_up_proj = torch.nn.Parameter(ex.gate_up_proj.data[lo:lo + El].clone(), requires_grad=ex.gate_up_proj.requires_grad)
            ex.down_proj = torch.nn.Parameter(ex.down_proj.data[lo:lo + El].clone(), requires_grad=ex.down_proj.requires_grad)
            for key in list(ex.lora.keys()):
                ex.lora[key] = torch.nn.Parameter(ex.lora[key].data[:, lo:lo + El].clone())
            if getattr(ex, 'gate_up_bias', None) is not None:
                ex.gate_up_bias = torch.nn.Parameter(ex.gate_up_bias.data[lo:lo + El].clone(), requires_grad=ex.gate_up_bias.requires_grad)
                ex.down_bias = torch.nn.Parameter(ex.down_bias.data[lo:lo + El].clone(), requires_grad=ex.down_bias.requires_grad)
        # expert tensors differ per EP rank: their gradients are summed only over the ranks that hold the same
        # experts, and their squared norms are summed over the EP group when the global norm is taken
        for p in [ex.gate_up_proj, ex.down_proj] + list(ex.lora.values()) + [b for b in (getattr(ex, 'gate_up_bias', None), getattr(ex, 'down_bias', None)) if b is not None]:
            p._ep_local = True
            p._ep_replica_comm = rep_comm
        ex.num_local, ex.first_expert = El, lo
        layer.mlp.moe_parallel = strat


def apply_expert_parallel(model, mesh, cfg, backend: str = 'auto'):
    """Keep only this rank's experts (a view of the freshly initialised full tensors, so every layout starts
    from identical values) and route MoE blocks through ``ExpertParallel``."""
    dev = next(model.parameters()).device
    comm = Communicator(ep_group_for(mesh), dev)
    if comm.world_size <= 1:
        return
    strat = None
    if dev.type == 'cuda' and backend in ('auto', 'symm'):
        try:
            from .expert_symm import SymmExpertParallel
            from .symm import SymmCommunicator
            strat = SymmExpertParallel(SymmCommunicator(comm.group, dev), cfg.num_experts)
        except Exception as e:  # the NCCL data plane stays correct
            if backend == 'symm':
                raise
            import logging
            logging.getLogger('twinkle_b200').warning(f'peer-memory expert parallel unavailable ({e}); using NCCL all-to-all')
    if strat is None:
        strat = ExpertParallel(comm, cfg.num_experts)
    rep_group = ep_replica_group_for(mesh)
    rep_comm = Communicator(rep_group, dev) if rep_group is not None else None
    if rep_comm is not None and rep_comm.world_size <= 1:
        rep_comm = None
    shard_experts(model, strat, comm.rank, rep_comm)
    model._ep_comm = comm
    return strat
