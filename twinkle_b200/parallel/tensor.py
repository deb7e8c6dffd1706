"""Tensor parallelism with sequence-parallel activations (the Megatron-style layout).

What it replaces: megatron-core / TransformerEngine column- and row-parallel linears reached by the
reference through ``src/twinkle/model/megatron/strategy/megatron.py:37-118`` (``tensor_model_parallel_size``,
``sequence_parallel``), and the fused vocab-parallel cross entropy (``utils/torch_utils.py:139-147``).

Layout: ``qkv_proj`` / ``gate_up_proj`` are column-parallel (output rows split per logical part so each rank
owns whole heads), ``o_proj`` / ``down_proj`` row-parallel (input columns split), embedding and head
vocab-parallel.  With ``sequence_parallel`` the residual stream is sharded over tokens inside the TP group:
an all-gather precedes every column-parallel GEMM and a reduce-scatter follows every row-parallel GEMM
(without it: identity / all-reduce).  Collectives go through ``Communicator`` (NCCL / gloo); the fused
all-gather→GEMM and GEMM→reduce-scatter kernels plug in at the same two call sites.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..models.bridge import tp_shard
from .comm import Communicator


def _rs(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    n = x.shape[0] // comm.world_size
    out = x.new_empty((n, ) + tuple(x.shape[1:]))
    dist.reduce_scatter_tensor(out, x.contiguous(), group=comm.group)
    return out


class GatherTokens(torch.autograd.Function):
    """fwd: all-gather along tokens; bwd: reduce-scatter."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return comm.all_gather_tensor(x)

    @staticmethod
    def backward(ctx, g):
        return _rs(g, ctx.comm), None


class ScatterTokens(torch.autograd.Function):
    """fwd: reduce-scatter along tokens; bwd: all-gather."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _rs(x, comm)

    @staticmethod
    def backward(ctx, g):
        return ctx.comm.all_gather_tensor(g.contiguous()), None


class ReduceFromTP(torch.autograd.Function):
    """fwd: all-reduce; bwd: identity."""

    @staticmethod
    def forward(ctx, x, comm):
        x = x.contiguous().clone()
        comm.all_reduce(x)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class CopyToTP(torch.autograd.Function):
    """fwd: identity; bwd: all-reduce."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        ctx.comm.all_reduce(g)
        return g, None


class SliceTokens(torch.autograd.Function):
    """fwd: keep this rank's token chunk; bwd: all-gather (used to enter the sequence-parallel region)."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        n = x.shape[0] // comm.world_size
        return x[comm.rank * n:(comm.rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return ctx.comm.all_gather_tensor(g.contiguous()), None


class TPContext:

    def __init__(self, comm: Communicator, sequence_parallel: bool):
        self.comm, self.sp = comm, sequence_parallel
        self.size, self.rank = comm.world_size, comm.rank
        self.fused = None  # parallel.tensor_fused.FusedTP when the group has a peer-memory communicator

    def before_column(self, x):
        return GatherTokens.apply(x, self.comm) if self.sp else CopyToTP.apply(x, self.comm)

    def after_row(self, y):
        return ScatterTokens.apply(y, self.comm) if self.sp else ReduceFromTP.apply(y, self.comm)


def tp_linear_forward(lin, x: torch.Tensor) -> torch.Tensor:
    """Forward of a ``models.layers.Linear`` whose weight is a TP shard (``lin.tp_mode`` in {'col', 'row'})."""
    tp: TPContext = lin.tp
    f = tp.fused
    from ..models.layers import current_lora_batch
    lb = current_lora_batch() if lin.max_loras > 0 else None
    if lb is not None:
        # Adapters on a sharded linear (reference ``model/multi_lora.py:289-475``).  Column-parallel: ``A`` is replicated
        # and ``B`` holds this rank's output rows, so the delta lands on the local output shard.  Row-parallel: ``A``
        # holds this rank's input columns and ``B`` is replicated; ``B·(A_r x_r)`` is added to the partial product
        # BEFORE the reduction, which sums the ranks' parts of ``A x`` for free.
        if lin.tp_mode == 'col':
            xg = tp.before_column(x)
            y = ops.linear(xg, lin.weight, lin.bias)
            d = lin._lora_delta(xg.reshape(-1, xg.shape[-1]), lb)
            return y if d is None else y + d.view(y.shape)
        y = ops.linear(x, lin.weight, None)
        d = lin._lora_delta(x.reshape(-1, x.shape[-1]), lb)
        if d is not None:
            y = y + d.view(y.shape)
        y = tp.after_row(y)
        return y if lin.bias is None else y + lin.bias
    if f is not None and tp.sp and x.is_cuda and x.dim() == 2:
        from .tensor_fused import ColumnLinearFused, FusedTP, RowLinearFused
        if lin.tp_mode == 'col' and FusedTP.eligible(x.shape[0], x.shape[1], lin.weight.shape[0], x.dtype):
            y = ColumnLinearFused.apply(x, lin.weight, f)
            return y if lin.bias is None else y + lin.bias
        if lin.tp_mode == 'row' and x.shape[0] % tp.size == 0 and FusedTP.eligible(x.shape[0] // tp.size, x.shape[1], lin.weight.shape[0], x.dtype):
            y = RowLinearFused.apply(x, lin.weight, f)
            return y if lin.bias is None else y + lin.bias
    if lin.tp_mode == 'col':
        return ops.linear(tp.before_column(x), lin.weight, lin.bias)
    y = ops.linear(x, lin.weight, None)
    y = tp.after_row(y)
    return y if lin.bias is None else y + lin.bias


def vocab_parallel_embedding(ids: torch.Tensor, weight: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """``weight`` holds vocabulary rows ``[rank·Vl, (rank+1)·Vl)``; out-of-range ids contribute zeros and the
    partial results are summed (reduce-scattered over tokens under sequence parallelism)."""
    vl = weight.shape[0]
    lo = tp.rank * vl
    local = ids - lo
    ok = (local >= 0) & (local < vl)
    e = F.embedding(local.clamp(0, vl - 1), weight) * ok.unsqueeze(-1).to(weight.dtype)
    return tp.after_row(e)


class _VocabParallelLogprob(torch.autograd.Function):
    """log softmax(hidden·Wᵀ)[labels] with the vocabulary split over the TP group: local max / sum-exp /
    target-logit partials are combined with two tiny all-reduces; logits never leave the rank."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, comm: Communicator, temperature: float):
        vl = weight.shape[0]
        lo = comm.rank * vl
        logits = ops.gemm(hidden, weight, 'nt', out_dtype=torch.float32).float() / temperature if hidden.is_cuda else (
            hidden.float() @ weight.float().t()) / temperature
        m = logits.max(-1).values
        comm.all_reduce(m, 'max')
        ex = torch.exp(logits - m[:, None])
        s = ex.sum(-1)
        comm.all_reduce(s)
        local = labels - lo
        ok = (local >= 0) & (local < vl)
        tgt = logits.gather(-1, local.clamp(0, vl - 1)[:, None]).squeeze(-1) * ok
        comm.all_reduce(tgt)
        lse = m + torch.log(s)
        ctx.save_for_backward(hidden, weight, ex / s[:, None], local, ok)
        ctx.comm, ctx.temperature = comm, temperature
        return tgt - lse

    @staticmethod
    def backward(ctx, g):
        hidden, weight, p, local, ok = ctx.saved_tensors
        d = -p * g[:, None]
        idx = local.clamp(0, weight.shape[0] - 1)
        d.scatter_add_(-1, idx[:, None], (g * ok)[:, None])
        d = (d / ctx.temperature).to(hidden.dtype)
        gh = ops.gemm(d, weight, 'nn') if hidden.is_cuda and hidden.dtype == torch.bfloat16 else (d.float() @ weight.float()).to(hidden.dtype)
        gh = gh.contiguous()  # partial over this rank's vocabulary shard; the caller's gather / copy op sums the shards
        gw = ops.gemm(d, hidden, 'tn') if hidden.is_cuda and hidden.dtype == torch.bfloat16 else (d.float().t() @ hidden.float()).to(weight.dtype)
        return gh, gw, None, None, None


class _VocabParallelLogprobChunked(torch.autograd.Function):
    """GPU form of the op above on the log-prob kernels: the head GEMM runs chunk by chunk over the tokens and each
    chunk's logits (bf16, this rank's vocabulary shard) are reduced to ``(target logit, log-sum-exp)`` by one kernel, so
    neither fp32 logits nor probabilities are kept; the shards' statistics are merged with two small all-reduces.
    Backward re-forms each chunk's logits, turns them in place into dlogits with the *global* log-sum-exp, and feeds the
    two gradient GEMMs (the same scheme as the single-GPU ``ops.fused_linear_logprob``)."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, comm: Communicator, temperature: float, chunk: int):
        E = ops.ext()
        T, vl = hidden.shape[0], weight.shape[0]
        local = labels.to(torch.int64) - comm.rank * vl
        local = torch.where((local >= 0) & (local < vl), local, torch.full_like(local, -1))   # −1: not in this shard
        stats = torch.empty(2, T, dtype=torch.float32, device=hidden.device)                 # [shard lse, shard target logit]
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = ops.gemm(hidden[s:e], weight, 'nt')
            lp, lse_l, _ = E.logprob_fwd(logits, local[s:e], temperature, False)
            stats[0, s:e] = lse_l
            stats[1, s:e] = lp + lse_l                     # the kernel reports (target − lse) with target = 0 outside the shard
        m = stats[0].clone()
        comm.all_reduce(m, 'max')
        packed = torch.stack([torch.exp(stats[0] - m), stats[1]])
        comm.all_reduce(packed)                            # Σ exp(lse_shard − m) and the target logit (one shard holds it)
        lse = m + torch.log(packed[0])
        ctx.save_for_backward(hidden, weight, local, lse)
        ctx.comm, ctx.temperature, ctx.chunk = comm, temperature, chunk
        return packed[1] - lse

    @staticmethod
    def backward(ctx, g):
        E = ops.ext()
        hidden, weight, local, lse = ctx.saved_tensors
        T = hidden.shape[0]
        g = g.contiguous().float()
        gh = torch.empty_like(hidden)
        gw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        for s in range(0, T, ctx.chunk):
            e = min(s + ctx.chunk, T)
            logits = ops.gemm(hidden[s:e], weight, 'nt')
            d = E.logprob_bwd(logits, local[s:e], lse[s:e], None, g[s:e], None, ctx.temperature)
            ops.gemm(d, weight, 'nn', out=gh[s:e])         # partial over this rank's shard; the caller's gather / copy op sums
            ops.gemm(d, hidden[s:e], 'tn', out=gw, accumulate=True)
        return gh, gw.to(weight.dtype), None, None, None, None


def vocab_parallel_logprob(hidden, weight, labels, tp: TPContext, temperature: float = 1.0, chunk: int = 4096):
    if hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        return _VocabParallelLogprobChunked.apply(hidden.contiguous(), weight, labels.clamp_min(0), tp.comm, temperature, chunk)
    return _VocabParallelLogprob.apply(hidden, weight, labels.clamp_min(0), tp.comm, temperature)


def make_fused_tp(comm: Communicator, device, sequence_parallel: bool, backend: str = 'auto'):
    """A ``FusedTP`` (peer-memory GEMM+collective kernels) for this TP group, or None when NCCL collectives are to be used."""
    if not (sequence_parallel and device.type == 'cuda' and backend in ('auto', 'symm') and 1 < comm.world_size <= 8):
        return None
    try:
        from .symm import SymmCommunicator
        from .tensor_fused import FusedTP
        return FusedTP(SymmCommunicator(comm.group, device))
    except Exception as e:  # NCCL collectives around the GEMM stay correct
        if backend == 'symm':
            raise
        import logging
        logging.getLogger('twinkle_b200').warning(f'fused tensor-parallel kernels unavailable ({e}); using NCCL collectives')
        return None


def apply_tensor_parallel(model, cfg, comm: Communicator, sequence_parallel: bool, fused=None) -> Optional[TPContext]:
    """Replace every parallelisable weight by this rank's shard (cut from the identically initialised full
    tensor) and switch the modules to their TP forward."""
    if comm.world_size <= 1:
        return None
    if getattr(cfg, 'attn_sinks', False) or getattr(cfg, 'expert_bias', False):
        raise NotImplementedError('attention sinks and biased experts / output projections (GPT-OSS) have no tensor-parallel split here; '
                                  'use tp_size=1 (data, sharded-data, expert and pipeline parallelism apply)')
    if getattr(cfg, 'qk_norm_full', False):
        raise NotImplementedError('q / k norms over the whole projection (OLMo-2) need statistics of all heads: no tensor-parallel split here; use tp_size=1')
    if getattr(cfg, 'is_mla', False):
        raise NotImplementedError('multi-head latent attention has no tensor-parallel split here; use tp_size=1 '
                                  '(data, sharded-data, expert and pipeline parallelism apply)')
    tp = TPContext(comm, sequence_parallel)
    tp.fused = fused
    assert cfg.num_key_value_heads % tp.size == 0 and cfg.num_attention_heads % tp.size == 0, 'heads must divide over tp'
    names = dict(model.named_parameters())
    with torch.no_grad():
        for name, p in list(names.items()):
            # internal names are relative to the chunk; layer indices are global already
            shard = tp_shard(name, p.data, cfg, tp.rank, tp.size)
            if shard.shape != p.shape:
                p.data = shard.contiguous().clone()
    for layer in model.layers:
        if getattr(layer, 'is_linear', False):
            raise NotImplementedError('linear-attention (Gated DeltaNet) layers are not split over a tensor-parallel group; '
                                      'use tp_size=1 for hybrid stacks (pipeline, data, sequence and context parallelism apply)')
        at = layer.self_attn
        at.hq, at.hkv = cfg.num_attention_heads // tp.size, cfg.num_key_value_heads // tp.size
        pairs = [(at.qkv_proj, 'col'), (at.o_proj, 'row')]
        if not layer.is_moe:
            pairs += [(layer.mlp.gate_up_proj, 'col'), (layer.mlp.down_proj, 'row')]
        elif getattr(cfg, 'expert_tensor_parallel', False):
            layer.mlp.etp = tp      # the expert tensors were cut above (bridge.tp_rule: 'ecol' / 'erow')
        for lin, mode in pairs:
            lin.tp, lin.tp_mode = tp, mode
            # the module's declared sizes follow its shard, so that an adapter pool created afterwards has the local
            # shapes (B rows of a column-parallel part, A columns of a row-parallel input)
            if mode == 'col':
                lin.parts = [(n, k // tp.size) for n, k in lin.parts]
                lin.out_features //= tp.size
            else:
                lin.in_features //= tp.size
    model.tp = tp
    return tp


def lora_param_is_replicated(name: str, tp_mode: Optional[str], expert_tp: bool = False) -> bool:
    """Whether an adapter-pool tensor is the same on every rank of the tensor-parallel group (its gradient is then a
    partial sum that must be all-reduced): ``A`` of a column-parallel linear and ``B`` of a row-parallel one; the other
    two are shards.  Expert pools (``…experts.lora.gate_up_A`` …) are whole on every rank unless the experts themselves
    are split over the group (``expert_tp``): then ``gate_up`` behaves like a column-parallel linear (``B`` holds this
    rank's rows) and ``down`` like a row-parallel one (``A`` holds this rank's columns)."""
    if '.lora.' in name:
        return not expert_tp or name.endswith('gate_up_A') or name.endswith('down_B')
    is_a = 'lora_A' in name
    return (tp_mode == 'col' and is_a) or (tp_mode == 'row' and not is_a) or tp_mode is None
