"""Ulysses sequence parallelism: head ↔ sequence exchange around attention.

Parity: reference ``src/twinkle/model/transformers/strategy/sequence_parallel/
utils.py:269-401`` (``_SeqAllToAll`` / ``DistributedAttention``) and
``__init__.py:597-671`` (``GatherLoss``).  Each rank holds a contiguous chunk of
the packed row; before attention q/k/v go from ``[T/sp, H, D]`` to
``[T, H/sp, D]`` (all-to-all), after attention the output goes back.  Ranks of
one SP group are consecutive in the flattened (dp, fsdp) order, as in the
reference (``data_rank = flat_index // ulysses_size``).

Two data planes implement the exchange: ``torch.distributed.all_to_all_single``
(baseline; gloo on CPU) and the peer-memory kernel of ``parallel.symm`` that
writes each head slice straight into the destination rank's buffer.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .comm import Communicator

_SP_GROUPS = {}


def sp_group_for(mesh):
    """Process group of this rank's Ulysses peers (created collectively once)."""
    sp = mesh.ulysses_size or 1
    if sp <= 1 or not (dist.is_available() and dist.is_initialized()):
        return None
    key = (mesh.signature(), sp)
    if key in _SP_GROUPS:
        return _SP_GROUPS[key]
    # order ranks by their flat data index so that consecutive ``sp`` of them share a data rank
    ranks = sorted(mesh._coord_of, key=lambda r: (mesh._flat_data_index(r), r))
    by_other = {}
    for r in ranks:
        c = mesh.coord_of(r)
        other = tuple(v for i, v in enumerate(c) if mesh.mesh_dim_names[i] not in ('dp', 'fsdp'))
        by_other.setdefault(other, []).append(r)
    mine = None
    me = dist.get_rank()
    for other, rs in sorted(by_other.items()):
        for i in range(0, len(rs), sp):
            grp_ranks = rs[i:i + sp]
            g = dist.new_group(ranks=grp_ranks)
            if me in grp_ranks:
                mine = g
    _SP_GROUPS[key] = mine
    return mine


class _HeadScatter(torch.autograd.Function):
    """``[T_local, H, D]`` → ``[T_local·sp, H/sp, D]`` (forward) and the inverse (backward)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Communicator):
        ctx.comm = comm
        return _seq_to_head(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g.contiguous(), ctx.comm), None


class _HeadGather(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Communicator):
        ctx.comm = comm
        return _head_to_seq(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g.contiguous(), ctx.comm), None


def _pulls(comm, x: torch.Tensor) -> bool:
    return (hasattr(comm, 'exchange_heads') and not comm.legacy_kernels and x.is_cuda and x.dim() == 3
            and (x.shape[-1] * x.element_size()) % 16 == 0)


class _ExchangeMany(torch.autograd.Function):
    """Several tensors through ONE exchange (one barrier, one kernel): q, k and v on the way in, their gradients on the
    way back.  ``seq_to_head`` picks the forward direction; backward runs the inverse."""

    @staticmethod
    def forward(ctx, comm, seq_to_head: bool, *xs):
        ctx.comm, ctx.s2h = comm, seq_to_head
        return tuple(comm.exchange_heads(list(xs), seq_to_head))

    @staticmethod
    def backward(ctx, *gs):
        return (None, None) + tuple(ctx.comm.exchange_heads([g.contiguous() for g in gs], not ctx.s2h))


class _ExchangeReuse(torch.autograd.Function):
    """The recompute pass of a layer: the forward values are the tensors the first forward already received (kept by
    the engine beside the attention output), so nothing crosses NVLink; backward still returns the gradients with the
    inverse exchange."""

    @staticmethod
    def forward(ctx, comm, seq_to_head: bool, kept, *xs):
        ctx.comm, ctx.s2h = comm, seq_to_head
        return tuple(t.view(t.shape) for t in kept)

    @staticmethod
    def backward(ctx, *gs):
        return (None, None, None) + tuple(ctx.comm.exchange_heads([g.contiguous() for g in gs], not ctx.s2h))


def _exchange(comm, seq_to_head: bool, xs):
    """One exchange of ``xs``; inside the sharding engine's per-layer forward the results are kept, and its recompute
    pass takes them back instead of exchanging again (two of the six cross-GPU meeting points per layer go away)."""
    from .. import ops
    st = ops.AttentionStash.current
    if st is not None and st.exchanges is not None and st.mode == 'save' and not torch.is_grad_enabled():
        outs = tuple(comm.exchange_heads(list(xs), seq_to_head))
        st.exchanges.append(outs)
        return outs
    if st is not None and st.exchanges is not None and st.mode == 'reuse' and st._j < len(st.exchanges):
        kept = st.exchanges[st._j]
        st._j += 1
        return _ExchangeReuse.apply(comm, seq_to_head, kept, *xs)
    return _ExchangeMany.apply(comm, seq_to_head, *xs)


def _symm_out(comm, shape, dtype, tag):
    """Destination buffers in symmetric memory, two per (shape, direction) used alternately so a
    consumer of the previous exchange never races with the next push.  The cache lives on the
    communicator, so it goes away with the symmetric arena it points into."""
    cache = comm.__dict__.setdefault('_exchange_buffers', {})
    key = (tuple(shape), dtype, tag)
    ent = cache.get(key)
    if ent is None:
        n = 1
        for v in shape:
            n *= v
        ent = {'bufs': [comm.alloc(n, dtype).view(shape) for _ in range(2)], 'next': 0}
        cache[key] = ent
    t = ent['bufs'][ent['next']]
    ent['next'] ^= 1
    return t


def _seq_to_head(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    sp = comm.world_size
    t, h, d = x.shape
    if hasattr(comm, 'ulysses_exchange') and x.is_cuda and (d * x.element_size()) % 16 == 0 and x.dtype == torch.bfloat16:
        out = _symm_out(comm, (sp * t, h // sp, d), x.dtype, 's2h')
        comm.ulysses_exchange(x.contiguous(), out, True, h)
        return out.clone()
    assert h % sp == 0, f'{h} heads do not divide over sp={sp}'
    send = x.view(t, sp, h // sp, d).transpose(0, 1).contiguous()  # [sp, t, h/sp, d] : block j goes to rank j
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send)
    return recv.view(sp * t, h // sp, d)  # blocks arrive in rank order = sequence order


def _head_to_seq(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    sp = comm.world_size
    tt, hl, d = x.shape
    t = tt // sp
    if hasattr(comm, 'ulysses_exchange') and x.is_cuda and (d * x.element_size()) % 16 == 0 and x.dtype == torch.bfloat16:
        out = _symm_out(comm, (t, sp * hl, d), x.dtype, 'h2s')
        comm.ulysses_exchange(x.contiguous(), out, False, sp * hl)
        return out.clone()
    send = x.view(sp, t, hl, d).contiguous()  # block j (token chunk j) returns to rank j
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send)
    return recv.transpose(0, 1).reshape(t, sp * hl, d)  # [t, sp, hl, d] → heads back in order


def fused_projection_enabled() -> bool:
    """``TWINKLE_ULYSSES_FUSED=1``: the q|k|v projection scatters heads to the peers from its own epilogue."""
    import os
    return os.environ.get('TWINKLE_ULYSSES_FUSED', '0') == '1'


class _ProjectScatter(torch.autograd.Function):
    """``x [T_local, H] · Wqkvᵀ`` delivered as ``[T_local·sp, (Hq + 2 Hkv)/sp · D]`` on every peer: the GEMM epilogue
    stores each 128-column block into the buffer of the rank that owns those heads (reference
    ``sequence_parallel/utils.py:345-401`` does projection, then three all-to-alls).  Backward returns the three
    gradient sections with the head → sequence exchange and runs the usual dX / dW GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, strat, hq, hkv, d, wgrad_out):
        comm, sp = strat.comm, strat.sp
        t = x.shape[0]
        out = _symm_out(comm, (sp * t, weight.shape[0] // sp), x.dtype, 'qkv')
        comm.head_scatter_gemm(x, weight, out, t, hq * d // 128, hkv * d // 128)
        ctx.save_for_backward(x, weight)
        ctx.strat, ctx.dims, ctx.wgrad_out = strat, (hq, hkv, d), wgrad_out
        # saved by the consumer for its backward, while the symmetric buffer is reused two exchanges later
        return out.clone() if any(ctx.needs_input_grad[:2]) else out

    @staticmethod
    def backward(ctx, g):
        from .. import ops
        x, weight = ctx.saved_tensors
        comm, sp = ctx.strat.comm, ctx.strat.sp
        hq, hkv, d = ctx.dims
        tt = g.shape[0]
        ql, kl = hq // sp * d, hkv // sp * d
        parts = [_head_to_seq(g[:, a:b].reshape(tt, (b - a) // d, d).contiguous(), comm).reshape(tt // sp, -1)
                 for a, b in ((0, ql), (ql, ql + kl), (ql + kl, ql + 2 * kl))]
        g2 = torch.cat(parts, dim=-1)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = ops.gemm(g2, weight, 'nn')
        if ctx.needs_input_grad[1]:
            if ctx.wgrad_out is not None:
                ops.gemm(g2, x, 'tn', out=ctx.wgrad_out, accumulate=True)
            else:
                gw = ops.gemm(g2, x, 'tn')
        return gx, gw, None, None, None, None, None


def kv_replication(num_kv_heads: int, sp: int) -> int:
    """How often every K/V head is repeated before the head exchange so that the K/V heads divide over ``sp`` ranks:
    ``sp / gcd(num_kv_heads, sp)``. With query heads divisible by ``sp`` (required anyway) and a whole number of query
    heads per K/V head, the repeated heads always split so that each rank's query heads find their K/V head locally
    (``sp/gcd`` divides the group size), for every ``sp`` — 8 K/V heads over 16 ranks, or 2 over 3. This takes the
    place of a ring among the ranks that share a K/V head (reference ``sequence_parallel/utils.py:90-99`` derives
    ``rp = ulysses / gcd`` ring ranks there); the price is ``kv_rep`` × the K/V volume in the exchange."""
    return sp // math.gcd(num_kv_heads, sp)


class UlyssesAttention:
    """Strategy object plugged into ``Attention.attn_parallel``."""

    def __init__(self, comm: Communicator, num_kv_heads: int):
        self.comm = comm
        self.sp = comm.world_size
        self.kv_rep = kv_replication(num_kv_heads, self.sp)

    def scatter_heads(self, q, k, v):
        if self.kv_rep > 1:
            k = k.repeat_interleave(self.kv_rep, dim=1)
            v = v.repeat_interleave(self.kv_rep, dim=1)
        if _pulls(self.comm, q) and q.dtype == k.dtype == v.dtype:
            return _exchange(self.comm, True, (q, k, v))
        return (_HeadScatter.apply(q.contiguous(), self.comm), _HeadScatter.apply(k.contiguous(), self.comm),
                _HeadScatter.apply(v.contiguous(), self.comm))

    def gather_heads(self, o):
        if _pulls(self.comm, o):
            return _exchange(self.comm, False, (o, ))[0]
        return _HeadGather.apply(o.contiguous(), self.comm)

    # ---- exchange inside the projection
    def _fusable(self, hq: int, hkv: int, d: int) -> bool:
        return (fused_projection_enabled() and hasattr(self.comm, 'head_scatter_gemm') and self.kv_rep == 1
                and (hq * d) % (128 * self.sp) == 0 and (hkv * d) % (128 * self.sp) == 0 and hq % self.sp == 0)

    def full_rope(self, cos, sin):
        """(cos, sin) of all tokens of the row (ranks hold consecutive chunks), or None when the fused path is off."""
        if not (fused_projection_enabled() and hasattr(self.comm, 'head_scatter_gemm') and cos.is_cuda):
            return None
        with torch.no_grad():
            return self.comm.all_gather_tensor(cos), self.comm.all_gather_tensor(sin)

    def project_scatter(self, x, proj, hq: int, hkv: int, d: int):
        """q|k|v projection + sequence → head exchange in one kernel; None when this call cannot use it (bias, LoRA
        on the projection, tensor parallelism, dtype, head counts that do not split into 128-column blocks)."""
        from ..models.layers import current_lora_batch
        if not (self._fusable(hq, hkv, d) and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and proj.bias is None
                and getattr(proj, 'tp_mode', None) is None and x.shape[-1] % 8 == 0):
            return None
        if getattr(proj, 'max_loras', 0) > 0 and current_lora_batch() is not None:
            return None
        w = proj.weight
        if w.dtype != torch.bfloat16 or not w.is_contiguous():
            return None
        return _ProjectScatter.apply(x.contiguous(), w, self, hq, hkv, d, proj.wgrad_out if w.requires_grad else None)

    # ---- linear attention (Gated DeltaNet): per-head scalars and the depth-wise convolution follow the heads
    def scatter_scalar_heads(self, x):
        """``[T_local, H]`` → ``[T_full, H/sp]``."""
        return _HeadScatter.apply(x.unsqueeze(-1).contiguous(), self.comm).squeeze(-1)

    def conv_after_scatter(self, q, k, v, conv_weight, cu_seqlens, hk, hv, dk, dv):
        """Causal conv1d on whole sequences with this rank's slice of the depth-wise filters (channels are laid out
        ``[q heads | k heads | v heads]``; the rank owns heads ``[r·H/sp, (r+1)·H/sp)`` of each block)."""
        from ..models.linear_attention import causal_conv1d_varlen
        sp, r = self.sp, self.comm.rank
        hkl, hvl = hk // sp, hv // sp
        kd = hk * dk
        wq = conv_weight[r * hkl * dk:(r + 1) * hkl * dk]
        wk = conv_weight[kd + r * hkl * dk:kd + (r + 1) * hkl * dk]
        wv = conv_weight[2 * kd + r * hvl * dv:2 * kd + (r + 1) * hvl * dv]
        T = q.shape[0]
        x = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1)
        y = causal_conv1d_varlen(x, torch.cat([wq, wk, wv], 0), cu_seqlens)
        a, b = hkl * dk, 2 * hkl * dk
        return y[:, :a].reshape(T, hkl, dk), y[:, a:b].reshape(T, hkl, dk), y[:, b:].reshape(T, hvl, dv)


class _GatherTokens(torch.autograd.Function):
    """All-gather along dim 0; backward keeps this rank's slice of the gradient.
    Every SP peer computes the same loss from the gathered values, and each
    back-propagates only into its own chunk, so the loss is counted once."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Communicator):
        ctx.comm, ctx.n = comm, x.shape[0]
        return comm.all_gather_tensor(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        r = ctx.comm.rank
        return g[r * ctx.n:(r + 1) * ctx.n].contiguous(), None


def gather_tokens(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    if comm.world_size == 1:
        return x
    return _GatherTokens.apply(x, comm)


def apply_ulysses(model, mesh, cfg, backend: str = 'auto') -> None:
    dev = next(model.parameters()).device
    comm = Communicator(sp_group_for(mesh), dev)
    if comm.world_size <= 1:
        return
    if backend in ('auto', 'symm') and dev.type == 'cuda':
        try:
            from .symm import SymmCommunicator
            comm = SymmCommunicator(comm.group, dev)
        except Exception:
            if backend == 'symm':
                raise
    if cfg.num_attention_heads % comm.world_size != 0:
        raise ValueError(f'{cfg.num_attention_heads} query heads do not divide over ulysses_size={comm.world_size}; '
                         f"shard the sequence with the mesh's cp dimension (zig-zag context parallelism) instead")
    strat = UlyssesAttention(comm, cfg.num_key_value_heads)
    linear = None
    for layer in model.layers:
        if getattr(layer, 'is_linear', False):
            if linear is None:
                assert cfg.linear_num_key_heads % comm.world_size == 0, 'linear-attention key heads must divide over the Ulysses group'
                linear = UlyssesAttention(comm, cfg.linear_num_key_heads)
            layer.self_attn.attn_parallel = linear
        else:
            layer.self_attn.attn_parallel = strat
