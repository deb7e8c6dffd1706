"""Operator layer: autograd-aware entry points for every hot op.

On CUDA tensors each op launches a hand-written sm_100a kernel from the
in-tree extension ``twinkle_b200/ops/_C*.so`` (sources in ``ops/csrc``); if the
extension cannot be loaded on a machine that has a GPU the import fails loudly
instead of falling back.  On CPU tensors the fp32 formulas of
``ops.reference`` run (used by gloo tests and as oracles).

Kernel ↔ reference-site map (what each op replaces in the reference project):
``linear`` → ``F.linear`` everywhere; ``flash_attn_varlen`` → flash-attn varlen
(``model/transformers/strategy/sequence_parallel/__init__.py:230-337``);
``rmsnorm``/``swiglu``/``qk_norm_rope`` → Liger kernels (``kernel/liger.py``);
``fused_linear_logprob`` → ``utils/torch_utils.py:61-137`` +
``loss/liger_fused_linear_cross_entropy.py``; ``adamw_step`` → ``torch.optim.AdamW``;
``sgmv`` → ``model/multi_lora.py:320-326``; ``moe_*`` →
``model/transformers/moe/expert_parallel.py``.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import reference as ref

_EXT = None


def ext():
    """The compiled extension; loaded on first use."""
    global _EXT
    if _EXT is None:
        from .build import load_extension
        _EXT = load_extension()
    return _EXT


def has_ext() -> bool:
    try:
        return ext() is not None
    except Exception:
        return False


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# ------------------------------------------------------------------ linear
class _DeadValues:
    """While a layer is re-run only to rebuild its autograd graph (activation recompute in backward), the values of
    its last operations are never read: their backward needs the operands, not the result.  Inside this context
    the operations that opt in return uninitialised tensors of the right shape instead of computing."""
    on = False


class dead_values:

    def __enter__(self):
        self.prev, _DeadValues.on = _DeadValues.on, True

    def __exit__(self, *exc):
        _DeadValues.on = self.prev
        return False


def dead_values_enabled() -> bool:
    return _DeadValues.on


class _AddDead(torch.autograd.Function):
    """``a + b`` whose value nobody reads: returns an uninitialised tensor, passes the gradient to both."""

    @staticmethod
    def forward(ctx, a, b):
        return torch.empty_like(a)

    @staticmethod
    def backward(ctx, g):
        return g, g


def add(a: torch.Tensor, b: torch.Tensor, value_unused: bool = False) -> torch.Tensor:
    if value_unused and _DeadValues.on and a.is_cuda:
        return _AddDead.apply(a, b)
    return a + b


class _Linear(torch.autograd.Function):
    """y = x @ Wᵀ with three tcgen05 GEMM layouts: NT forward, NN for dX, TN for dW."""

    @staticmethod
    def forward(ctx, x, weight, bias, wgrad_out, dead=False):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.wgrad_out = wgrad_out
        if dead:  # graph only: dX needs W and dW needs x, nobody needs x·Wᵀ
            return torch.empty(*x.shape[:-1], weight.shape[0], dtype=x.dtype, device=x.device)
        x2 = x.reshape(-1, x.shape[-1])
        # the result is allocated in its final shape (not returned as a view of a 2-D product): a later op may then
        # accumulate into it in place, which autograd refuses for views created inside a custom Function
        y = torch.empty(*x.shape[:-1], weight.shape[0], dtype=x.dtype, device=x.device)
        gemm(x2, weight, 'nt', out=y.view(-1, weight.shape[0]))
        if bias is not None:
            y += bias
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = gemm(g2, weight, 'nn').view(x.shape)
        if ctx.needs_input_grad[1]:
            if ctx.wgrad_out is not None:
                # accumulate straight into the flat gradient bucket (fp32 or bf16)
                gemm(g2, x2, 'tn', out=ctx.wgrad_out, accumulate=True)
                gw = None
            else:
                gw = gemm(g2, x2, 'tn')
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g2.float().sum(0).to(gy.dtype)
        return gx, gw, gb, None, None


def gemm(a: torch.Tensor, b: torch.Tensor, layout: str = 'nt', out: Optional[torch.Tensor] = None,
         accumulate: bool = False, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``nt``: a[M,K]·b[N,K]ᵀ; ``nn``: a[M,K]·b[K,N]; ``tn``: a[K,M]ᵀ·b[K,N].  bf16
    operands, fp32 accumulation in tensor memory, bf16 or fp32 output."""
    if _cuda(a) and a.dtype == torch.bfloat16:
        return ext().gemm(a, b, layout, out, accumulate, out_dtype)
    af, bf = a.float(), b.float()
    r = af @ bf.t() if layout == 'nt' else (af @ bf if layout == 'nn' else af.t() @ bf)
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r)
        return out
    return r.to(out_dtype or a.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, wgrad_out: Optional[torch.Tensor] = None,
           value_unused: bool = False):
    """``value_unused``: the caller never reads the result when the graph is being rebuilt (see ``dead_values``)."""
    if _cuda(x) and x.dtype == torch.bfloat16:
        return _Linear.apply(x, weight, bias, wgrad_out, value_unused and _DeadValues.on)
    return torch.nn.functional.linear(x, weight, bias)


# ------------------------------------------------------------------- norms
class _RMSNorm(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, eps, offset):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()       # a column slice of a wider tensor arrives strided
        y, rstd = ext().rmsnorm_fwd(x2, weight, eps, offset)
        ctx.save_for_backward(x2, weight, rstd)
        ctx.offset = offset
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, weight, rstd = ctx.saved_tensors
        gx, gw = ext().rmsnorm_bwd(gy.reshape(x2.shape).contiguous(), x2, weight, rstd, ctx.offset)
        return gx.view(ctx.shape), gw.to(weight.dtype), None, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    if _cuda(x) and x.dtype == torch.bfloat16:
        return _RMSNorm.apply(x, weight, eps, offset)
    return ref.rmsnorm(x, weight, eps, offset)


class _AddRMSNorm(torch.autograd.Function):
    """``h = x + residual``; ``y = rmsnorm(h)`` in one kernel.  Backward: the gradient that reaches ``h`` directly (the
    residual stream) is added inside the RMSNorm backward kernel, and the sum is the gradient of both inputs."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps, offset):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, x.shape[-1])
        y, rstd, h = ext().rmsnorm_fwd(x2.contiguous(), weight, eps, offset, r2.contiguous())
        ctx.save_for_backward(h, weight, rstd)
        ctx.offset = offset
        ctx.shape = x.shape
        return y.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, gy, gh):
        h, weight, rstd = ctx.saved_tensors
        if gy is None:
            return gh, gh, None, None, None
        gadd = gh.reshape(h.shape).contiguous() if gh is not None else None
        gx, gw = ext().rmsnorm_bwd(gy.reshape(h.shape).contiguous(), h, weight, rstd, ctx.offset, gadd)
        gx = gx.view(ctx.shape)
        return gx, gx, gw.to(weight.dtype), None, None


def add_rmsnorm(x, residual, weight, eps: float = 1e-6, offset: float = 0.0):
    """Returns ``(rmsnorm(x + residual), x + residual)``; one kernel on CUDA (the add costs no pass of its own, forward
    or backward)."""
    if _cuda(x) and x.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16:
        return _AddRMSNorm.apply(x, residual, weight, eps, offset)
    return ref.add_rmsnorm(x, residual, weight, eps, offset)


# -------------------------------------------------------------------- rope
class _QKNormRope(torch.autograd.Function):
    """In: fused qkv ``[T, (Hq+2Hkv)·D]``; out: q ``[T,Hq,D]``, k ``[T,Hkv,D]``,
    v ``[T,Hkv,D]`` — per-head RMSNorm on q,k then rotate-half RoPE, one pass."""

    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, cos, sin, hq, hkv, d, eps):
        q, k, v, rstd = ext().qk_norm_rope_fwd(qkv, q_weight, k_weight, cos, sin, hq, hkv, d, eps)
        ctx.save_for_backward(qkv, q_weight, k_weight, cos, sin, rstd)
        ctx.dims = (hq, hkv, d, eps)
        return q, k, v

    @staticmethod
    def backward(ctx, gq, gk, gv):
        qkv, qw, kw, cos, sin, rstd = ctx.saved_tensors
        hq, hkv, d, eps = ctx.dims
        gqkv, gqw, gkw = ext().qk_norm_rope_bwd(gq.contiguous(), gk.contiguous(), gv.contiguous(), qkv, qw, kw, cos, sin,
                                                rstd, hq, hkv, d)
        return gqkv, gqw.to(qw.dtype), gkw.to(kw.dtype), None, None, None, None, None, None


_WARNED_HEAD_DIM = set()


def _head_dim_ok(d: int) -> bool:
    """The attention-side kernels are written for 128-wide heads (every Qwen3 / Llama-3 size). Other widths — the tiny
    presets used in tests, vision towers — run on the PyTorch restatement; said once per width."""
    if d == 128:
        return True
    if d not in _WARNED_HEAD_DIM:
        _WARNED_HEAD_DIM.add(d)
        import logging
        logging.getLogger('twinkle_b200').warning(f'head_dim {d}: attention, q/k-norm + RoPE and paged decode run on PyTorch ops (the sm_100a kernels are for head_dim 128)')
    return False


def qkv_norm_rope(qkv: torch.Tensor, q_weight, k_weight, cos, sin, hq: int, hkv: int, d: int, eps: float = 1e-6, offset: float = 0.0):
    """Split fused qkv, apply q/k RMSNorm (if weights given; ``offset`` 1.0 = "1 + w") and RoPE on the leading
    ``2·cos.shape[-1]`` dims of every head.  The fused kernel serves full rotary with plain norm weights."""
    if (_cuda(qkv) and qkv.dtype == torch.bfloat16 and q_weight is not None and _head_dim_ok(d) and offset == 0.0
            and 2 * cos.shape[-1] == d):
        return _QKNormRope.apply(qkv.contiguous(), q_weight, k_weight, cos, sin, hq, hkv, d, eps)
    T = qkv.shape[0]
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.reshape(T, hq, d), k.reshape(T, hkv, d), v.reshape(T, hkv, d)
    q, k = ref.qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps, offset)
    return q, k, v


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float = 1e6, scaling: Optional[dict] = None):
    return ref.rope_tables(positions, head_dim, theta, scaling)


# ------------------------------------------------------------------ swiglu
class _SwiGLU(torch.autograd.Function):

    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return ext().swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, gy):
        (gate_up, ) = ctx.saved_tensors
        return ext().swiglu_bwd(gy.contiguous(), gate_up)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    if _cuda(gate_up) and gate_up.dtype == torch.bfloat16:
        return _SwiGLU.apply(gate_up)
    return ref.swiglu(gate_up)


class _GeGLU(torch.autograd.Function):

    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return ext().geglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, gy):
        (gate_up, ) = ctx.saved_tensors
        return ext().geglu_bwd(gy.contiguous(), gate_up)


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``[T, 2I]`` laid out as ``[gate | up]`` → ``gelu_tanh(gate) * up`` (Gemma-family MLPs); same kernel family as
    :func:`swiglu` (reference ``kernel/liger_impls/swiglu.py:26-32``)."""
    if _cuda(gate_up) and gate_up.dtype == torch.bfloat16:
        lead = gate_up.shape[:-1]
        return _GeGLU.apply(gate_up.reshape(-1, gate_up.shape[-1])).reshape(*lead, -1)
    return ref.geglu(gate_up)


# --------------------------------------------------------------- attention
class _FlashAttnVarlen(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale, cu_k=None, max_seqlen_k=0):
        out, lse = ext().flash_attn_fwd(q, k, v, cu_seqlens, max_seqlen, causal, scale, cu_k)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens, cu_k if cu_k is not None else cu_seqlens)
        ctx.args = (max_seqlen, causal, scale, cu_k is not None, max_seqlen_k)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, gout, _glse):
        q, k, v, out, lse, cu, cu_k = ctx.saved_tensors
        max_seqlen, causal, scale, has_k, max_k = ctx.args
        dq, dk, dv = ext().flash_attn_bwd(gout.contiguous(), q, k, v, out, lse, cu, max_seqlen, causal, scale, cu_k if has_k else None, max_k)
        return dq, dk, dv, None, None, None, None, None, None


class _FlashAttnReuse(torch.autograd.Function):
    """Forward returns an attention output computed earlier (with its log-sum-exp); backward is the normal
    flash backward.  Lets an activation-recompute pass skip the attention forward."""

    @staticmethod
    def forward(ctx, q, k, v, out, lse, cu_seqlens, max_seqlen, causal, scale):
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens)
        ctx.args = (max_seqlen, causal, scale)
        return out.view_as(out)

    @staticmethod
    def backward(ctx, gout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        max_seqlen, causal, scale = ctx.args
        dq, dk, dv = ext().flash_attn_bwd(gout.contiguous(), q, k, v, out, lse, cu, max_seqlen, causal, scale)
        return dq, dk, dv, None, None, None, None, None, None


class AttentionStash:
    """``mode='save'``: every attention call in scope appends its (out, lse); ``mode='reuse'``: calls consume
    them in the same order instead of recomputing."""
    current = None

    def __init__(self, mode: str, items=None, exchanges=None):
        """``items``: attention outputs; ``exchanges``: tensors received by sequence-parallel exchanges of the same
        layer (``None`` = do not keep them: the recompute pass exchanges again)."""
        self.mode, self.items, self._i = mode, ([] if items is None else items), 0
        self.exchanges, self._j = exchanges, 0

    def __enter__(self):
        self._prev = AttentionStash.current
        AttentionStash.current = self
        return self

    def __exit__(self, *exc):
        AttentionStash.current = self._prev


def flash_attn_varlen(q, k, v, cu_seqlens, max_seqlen: int, causal: bool = True, scale: Optional[float] = None,
                      cu_seqlens_k=None, max_seqlen_k: int = 0, return_lse: bool = False, window: Optional[int] = None,
                      softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None):
    """Packed causal attention with GQA.  ``q [T,Hq,D]``, ``k,v [Tk,Hkv,D]``.  ``cu_seqlens_k``: the keys of every
    sequence are a (longer) range of their own; the causal diagonal is aligned bottom-right.  A sliding ``window`` shorter
    than the longest row, a score ``softcap`` or per-head ``sinks`` select the PyTorch form (the kernels compute plain causal attention)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if window is not None and window >= max(int(max_seqlen), int(max_seqlen_k)):
        window = None           # no row reaches past the window: plain causal attention
    if window is not None or softcap or sinks is not None:
        return ref.attention_varlen(q, k, v, cu_seqlens, causal, scale, return_lse, cu_seqlens_k, window, softcap, sinks)
    if cu_seqlens_k is not None or return_lse:
        if _cuda(q) and q.dtype == torch.bfloat16 and _head_dim_ok(q.shape[-1]):
            out, lse = _FlashAttnVarlen.apply(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens.to(torch.int32), int(max_seqlen), causal,
                                              scale, None if cu_seqlens_k is None else cu_seqlens_k.to(torch.int32), int(max_seqlen_k))
        else:
            out, lse = ref.attention_varlen(q, k, v, cu_seqlens, causal, scale, True, cu_seqlens_k)
        return (out, lse) if return_lse else out
    if _cuda(q) and q.dtype == torch.bfloat16 and _head_dim_ok(q.shape[-1]):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        cu = cu_seqlens.to(torch.int32)
        st = AttentionStash.current
        if st is not None and st.mode == 'save' and not torch.is_grad_enabled():
            out, lse = ext().flash_attn_fwd(q, k, v, cu, int(max_seqlen), causal, scale)
            st.items.append((out, lse))
            return out
        if st is not None and st.mode == 'reuse' and st._i < len(st.items):
            out, lse = st.items[st._i]
            st._i += 1
            return _FlashAttnReuse.apply(q, k, v, out, lse, cu, int(max_seqlen), causal, scale)
        return _FlashAttnVarlen.apply(q, k, v, cu, int(max_seqlen), causal, scale)[0]
    return ref.attention_varlen(q, k, v, cu_seqlens, causal, scale)


def paged_attention_decode(q, k_cache, v_cache, block_tables, seq_lens, scale: Optional[float] = None, window: Optional[int] = None,
                           softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None):
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if window is not None or softcap or sinks is not None:
        return ref.paged_attention_decode(q, k_cache, v_cache, block_tables, seq_lens, scale, window, softcap, sinks)
    if _cuda(q) and q.dtype == torch.bfloat16 and _head_dim_ok(q.shape[-1]):
        return ext().paged_attn_decode(q.contiguous(), k_cache, v_cache, block_tables.to(torch.int32),
                                       seq_lens.to(torch.int32), scale)
    return ref.paged_attention_decode(q, k_cache, v_cache, block_tables, seq_lens, scale)


# ------------------------------------------------------ gated delta net (linear attention)
def _segment_starts(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """``[T]`` int32: for every packed token the index of the first token of its sequence."""
    cu = cu_seqlens.to(torch.int64)
    lens = cu[1:] - cu[:-1]
    return torch.repeat_interleave(cu[:-1], lens, output_size=total).to(torch.int32)


class _CausalConv1d(torch.autograd.Function):
    """Forward: one kernel (depth-wise taps + SiLU, no leakage across packed sequences).  Backward: the gradient of the
    same op formed by autograd on the PyTorch expression (the convolution is a small share of a layer's backward)."""

    @staticmethod
    def forward(ctx, x, weight, cu_seqlens, activation):
        ctx.save_for_backward(x, weight, cu_seqlens)
        ctx.activation = activation
        return ext().causal_conv1d_fwd(x, weight.to(x.dtype).contiguous(), _segment_starts(cu_seqlens, x.shape[0]), activation)

    @staticmethod
    def backward(ctx, gy):
        from ..models.linear_attention import causal_conv1d_varlen_torch
        x, weight, cu = ctx.saved_tensors
        with torch.enable_grad():
            xd, wd = x.detach().requires_grad_(True), weight.detach().requires_grad_(True)
            y = causal_conv1d_varlen_torch(xd, wd, cu, ctx.activation)
            gx, gw = torch.autograd.grad(y, (xd, wd), gy)
        return gx, gw, None, None


def causal_conv1d_varlen(x: torch.Tensor, weight: torch.Tensor, cu_seqlens: torch.Tensor, activation: bool = True) -> torch.Tensor:
    """Depth-wise causal convolution (+ SiLU) over packed tokens: ``x [T, C]``, ``weight [C, W]``."""
    from ..models.linear_attention import causal_conv1d_varlen_torch
    if (_cuda(x) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and 2 <= weight.shape[1] <= 4 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
        return _CausalConv1d.apply(x, weight, cu_seqlens, activation)
    return causal_conv1d_varlen_torch(x, weight, cu_seqlens, activation)


def gdn_kernel_supported(q: torch.Tensor, v: torch.Tensor) -> bool:
    return (_cuda(q) and q.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)
            and q.stride(2) == 1 and q.stride(1) == q.shape[2] and v.stride(2) == 1 and v.stride(1) == v.shape[2])


class _GatedDeltaRule(torch.autograd.Function):
    """Forward: the recurrent kernel (q / k L2 normalisation and the grouped-head repeat inside).  Backward: autograd
    through the chunk-parallel PyTorch evaluator of the same function, re-run from the saved inputs."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, cu_seqlens, scale, chunk):
        o, _ = ext().gdn_recurrent_fwd(q, k, v, g.float().contiguous(), beta.float().contiguous(), cu_seqlens.to(torch.int32).contiguous(),
                                       None, scale, False)
        ctx.save_for_backward(q, k, v, g, beta, cu_seqlens)
        ctx.scale, ctx.chunk = scale, chunk
        return o

    @staticmethod
    def backward(ctx, go):
        from ..models.linear_attention import gated_delta_rule_varlen_torch
        q, k, v, g, beta, cu = ctx.saved_tensors
        with torch.enable_grad():
            ins = [t.detach().requires_grad_(True) for t in (q, k, v, g, beta)]
            o = gated_delta_rule_varlen_torch(*ins, cu, ctx.scale, chunk=ctx.chunk, normalize=True)
            grads = torch.autograd.grad(o, ins, go)
        return (*grads, None, None, None)


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None, chunk: int = 64, init_state=None,
                            return_states: bool = False):
    """Gated delta rule over packed sequences with **unnormalised** ``q, k [T, Hk, dk]`` (they are L2-normalised per head
    inside), ``v [T, Hv, dv]`` (``Hv`` a multiple of ``Hk``), ``g`` (log decay) and ``beta [T, Hv]``.  Returns
    ``o [T, Hv, dv]`` and, with ``return_states``, the final state per sequence ``[n, Hv, dk, dv]`` (fp32).
    ``init_state`` continues from earlier tokens (decoding); it and ``return_states`` are inference-only."""
    from ..models.linear_attention import gated_delta_rule_varlen_torch
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if gdn_kernel_supported(q, v) and gdn_kernel_supported(k, v):
        if init_state is None and not return_states:
            return _GatedDeltaRule.apply(q, k, v, g, beta, cu_seqlens, scale, chunk)
        if not torch.is_grad_enabled() or not any(t.requires_grad for t in (q, k, v, g, beta)):
            o, fin = ext().gdn_recurrent_fwd(q, k, v, g.float().contiguous(), beta.float().contiguous(),
                                             cu_seqlens.to(torch.int32).contiguous(),
                                             init_state.float().contiguous() if init_state is not None else None, scale, return_states)
            return (o, fin) if return_states else o
    return gated_delta_rule_varlen_torch(q, k, v, g, beta, cu_seqlens, scale, chunk=chunk, normalize=True, init_state=init_state,
                                         return_states=return_states)


# ------------------------------------------------------------- logprob / CE
class _LogprobFromLogits(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, labels, temperature, with_entropy):
        x = logits.reshape(-1, logits.shape[-1])
        lp, lse, ent = ext().logprob_fwd(x, labels.reshape(-1).to(torch.int64), temperature, with_entropy)
        ctx.save_for_backward(x, labels.reshape(-1).to(torch.int64), lse, ent if with_entropy else lse)
        ctx.temperature, ctx.with_entropy, ctx.shape = temperature, with_entropy, logits.shape
        out_shape = labels.shape
        return lp.view(out_shape), (ent.view(out_shape) if with_entropy else lp.new_zeros(()))

    @staticmethod
    def backward(ctx, glp, gent):
        x, labels, lse, ent = ctx.saved_tensors
        gent_flat = gent.reshape(-1).contiguous().float() if ctx.with_entropy else None
        gx = ext().logprob_bwd(x.clone(), labels, lse, ent if ctx.with_entropy else None, glp.reshape(-1).contiguous().float(), gent_flat,
                               ctx.temperature)
        return gx.view(ctx.shape), None, None, None


def logprob_from_logits(logits, labels, temperature: float = 1.0, with_entropy: bool = False):
    """(logps, entropy|None); differentiable w.r.t. logits."""
    if _cuda(logits) and logits.dtype in (torch.bfloat16, torch.float32):
        lp, ent = _LogprobFromLogits.apply(logits.contiguous(), labels, temperature, with_entropy)
        return lp, (ent if with_entropy else None)
    return ref.logprob_from_logits(logits, labels, temperature, with_entropy)


class _FusedLinearLogprob(torch.autograd.Function):
    """lm_head GEMM + online-softmax statistics, chunked over tokens so the
    ``[T, V]`` logits never exist; backward re-forms each chunk's logits,
    converts them in place to dlogits and feeds the two gradient GEMMs."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature, with_entropy, chunk, wgrad_out):
        T = hidden.shape[0]
        lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        lse = torch.empty_like(lp)
        ent = torch.empty_like(lp) if with_entropy else None
        labels = labels.to(torch.int64)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = gemm(hidden[s:e], weight, 'nt')
            a, b, c = ext().logprob_fwd(logits, labels[s:e], temperature, with_entropy)
            lp[s:e], lse[s:e] = a, b
            if with_entropy:
                ent[s:e] = c
        ctx.save_for_backward(hidden, weight, labels, lse, ent if with_entropy else lse)
        ctx.cfg = (temperature, with_entropy, chunk)
        ctx.wgrad_out = wgrad_out
        return lp, (ent if with_entropy else lp.new_zeros(()))

    @staticmethod
    def backward(ctx, glp, gent):
        hidden, weight, labels, lse, ent = ctx.saved_tensors
        temperature, with_entropy, chunk = ctx.cfg
        T = hidden.shape[0]
        glp = glp.contiguous().float()
        gent = gent.contiguous().float() if with_entropy else None
        gh = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        need_w = ctx.needs_input_grad[1]
        gw = ctx.wgrad_out
        if need_w and gw is None:
            gw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = gemm(hidden[s:e], weight, 'nt')
            dlogits = ext().logprob_bwd(logits, labels[s:e], lse[s:e], ent[s:e] if with_entropy else None, glp[s:e],
                                        gent[s:e] if with_entropy else None, temperature)
            if gh is not None:
                gemm(dlogits, weight, 'nn', out=gh[s:e])
            if need_w:
                gemm(dlogits, hidden[s:e], 'tn', out=gw, accumulate=True)
        gw_ret = None
        if need_w and ctx.wgrad_out is None:
            gw_ret = gw.to(weight.dtype)
        return gh, gw_ret, None, None, None, None, None


def fused_linear_logprob(hidden, weight, labels, temperature: float = 1.0, with_entropy: bool = False, chunk: int = 4096,
                         wgrad_out: Optional[torch.Tensor] = None):
    """(logps [T] fp32, entropy|None) of ``labels`` under ``softmax(hidden·Wᵀ/T)``."""
    if _cuda(hidden) and hidden.dtype == torch.bfloat16:
        lp, ent = _FusedLinearLogprob.apply(hidden, weight, labels, temperature, with_entropy, chunk, wgrad_out)
        return lp, (ent if with_entropy else None)
    return ref.fused_linear_logprob(hidden, weight, labels, temperature, with_entropy)


# ------------------------------------------------------------------- adamw
def adamw_step(master, exp_avg, exp_avg_sq, grad, param_out, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    if _cuda(master):
        ext().adamw_step(master, exp_avg, exp_avg_sq, grad, param_out, float(lr), float(beta1), float(beta2), float(eps),
                         float(weight_decay), int(step), float(grad_scale))
    else:
        ref.adamw_step(master, exp_avg, exp_avg_sq, grad, param_out, lr, beta1, beta2, eps, weight_decay, step, grad_scale)


def sumsq(t: torch.Tensor) -> torch.Tensor:
    """Σ t² in fp32 as a 0-d tensor (partial of an L2 grad norm)."""
    if _cuda(t) and t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous():
        return ext().sumsq(t)
    return t.float().pow(2).sum()


# -------------------------------------------------------------------- lora
class _SGMV(torch.autograd.Function):
    """Segmented multi-LoRA on the tensor cores: shrink and expand are two expert-grouped tcgen05 GEMMs in
    which a *segment of tokens* plays the role of an expert and ``seg_slots`` maps it to its adapter block
    (−1 = no adapter → rows stay zero).  The rank mask (``r`` ≤ pool rank) and the ``alpha/r`` scale are one
    small element-wise pass over the ``[T, R]`` intermediate.  Weight gradients are per-segment ``tn`` GEMMs
    over 64-row-aligned token windows whose rows outside the segment are zeroed."""

    @staticmethod
    def forward(ctx, x, lora_a, lora_b, seg_starts, seg_slots, seg_ranks, seg_scales, host_segments, y_in=None, repeat=1):
        """``y_in`` (optional): the base projection's output; the delta is accumulated into it by the expand GEMM's
        epilogue instead of being produced as a tensor of its own and added.  ``repeat``: the pools of ``repeat``
        fused projections stacked along the rank axis (``A [S, repeat·R, K]``, ``B`` block-diagonal) — the rank mask
        then repeats per block."""
        E = ext()
        R = lora_a.shape[1]
        rowmask = _sgmv_rowmask(host_segments, R // repeat, x.device, x.dtype, repeat)   # [T, R] = scale where col < rank else 0
        h = E.grouped_gemm(x, lora_a, seg_starts, 'nt', seg_slots)             # [T, R]
        hm = h * rowmask
        if y_in is not None:
            E.grouped_gemm(hm, lora_b, seg_starts, 'nt', seg_slots, y_in, True)
            ctx.mark_dirty(y_in)
            y = y_in
        else:
            y = E.grouped_gemm(hm, lora_b, seg_starts, 'nt', seg_slots)        # [T, N]
        ctx.save_for_backward(x, lora_a, lora_b, hm, rowmask, seg_starts, seg_slots)
        ctx.host_segments = host_segments
        ctx.has_y = y_in is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        E = ext()
        x, a, b, hm, rowmask, st, sl = ctx.saved_tensors
        gy = gy.contiguous()
        ghm = E.grouped_gemm(gy, b, st, 'nn', sl)                               # [T, R]   (b[s] is [N, R] = [K, N_out])
        gh = ghm * rowmask
        gx = E.grouped_gemm(gh, a, st, 'nn', sl) if ctx.needs_input_grad[0] else None
        ga = torch.zeros_like(a, dtype=torch.float32)
        gb = torch.zeros_like(b, dtype=torch.float32)
        T = x.shape[0]
        for (lo, hi, slot, rank, scale) in ctx.host_segments:
            if slot < 0 or rank == 0 or hi <= lo:
                continue
            a0, b0 = lo // 64 * 64, min((hi + 63) // 64 * 64, T)
            if a0 == lo and (b0 == hi or hi == T):       # the segment fills its 64-row windows: no rows to blank out
                ghs, hms = gh[a0:b0], hm[a0:b0]
            else:
                ghs, hms = gh[a0:b0].clone(), hm[a0:b0].clone()
                ghs[:lo - a0].zero_(), ghs[hi - a0:].zero_()
                hms[:lo - a0].zero_(), hms[hi - a0:].zero_()
            n = b0 - a0
            if n >= 8192:
                # split-K: the outputs are a handful of tiles ([R, K] and [N, R]) over a reduction of n rows — as one
                # GEMM that is a few CTAs walking the whole batch.  The K-grouped kernel gives every 1/32 of the rows
                # its own CTAs; the partial sums are added afterwards (32 small fp32 tensors)
                off = _split_k_offsets(n, x.device)
                ga[slot] += E.grouped_gemm_wgrad(ghs, x[a0:b0], off, off.numel() - 1).sum(0)
                gb[slot] += E.grouped_gemm_wgrad(gy[a0:b0], hms, off, off.numel() - 1).sum(0)
            else:
                E.gemm(ghs, x[a0:b0], 'tn', ga[slot], True, None)               # dA[slot] += ghᵀ x
                E.gemm(gy[a0:b0], hms, 'tn', gb[slot], True, None)              # dB[slot] += gyᵀ h
        return gx, ga.to(a.dtype), gb.to(b.dtype), None, None, None, None, None, (gy if ctx.has_y else None), None


_ROWMASKS: 'dict' = {}
_SPLITK: 'dict' = {}


def _split_k_offsets(n: int, device) -> torch.Tensor:
    """int32 boundaries that cut ``n`` reduction rows into at most 32 chunks whose sizes are multiples of 64."""
    key = (n, str(device))
    hit = _SPLITK.get(key)
    if hit is None:
        chunk = max(1024, ((n + 31) // 32 + 63) // 64 * 64)
        cuts = list(range(0, n, chunk)) + [n]
        hit = torch.tensor(cuts, dtype=torch.int32, device=device)
        if len(_SPLITK) >= 64:
            _SPLITK.pop(next(iter(_SPLITK)))
        _SPLITK[key] = hit
    return hit


def _sgmv_rowmask(host_segments, R: int, device, dtype, repeat: int = 1) -> torch.Tensor:
    """``[T, R]``: the segment's scale in the first ``rank`` columns of its rows, zero elsewhere.  Every LoRA linear of
    every layer asks for the same mask during one forward/backward (and its recompute), so the last few are kept: the
    mask is built on the host and copied once instead of by a dozen small kernels per call."""
    key = (tuple(host_segments), R, str(device), dtype, repeat)
    hit = _ROWMASKS.get(key)
    if hit is not None:
        return hit
    if repeat > 1:
        mask = _sgmv_rowmask(host_segments, R, device, dtype).repeat(1, repeat)
        if len(_ROWMASKS) >= 16:
            _ROWMASKS.pop(next(iter(_ROWMASKS)))
        _ROWMASKS[key] = mask
        return mask
    per_seg = torch.zeros(max(len(host_segments), 1), R, dtype=torch.float32)
    lens = []
    for i, (lo, hi, slot, rank, scale) in enumerate(host_segments):
        if slot >= 0:
            per_seg[i, :rank] = scale
        lens.append(hi - lo)
    if host_segments:
        rep = torch.tensor(lens, dtype=torch.int64, device=device)
        mask = per_seg[:len(host_segments)].to(device=device, dtype=dtype).repeat_interleave(rep, dim=0, output_size=sum(lens))
    else:
        mask = torch.zeros(0, R, device=device, dtype=dtype)
    if len(_ROWMASKS) >= 16:
        _ROWMASKS.pop(next(iter(_ROWMASKS)))
    _ROWMASKS[key] = mask
    return mask


def sgmv_fused_supported(x: torch.Tensor) -> bool:
    """Whether :func:`sgmv` can accumulate into the base output (``out=``) and take rank-stacked pools (``repeat=``)."""
    return _cuda(x) and x.dtype == torch.bfloat16


def sgmv(x, lora_a, lora_b, seg_starts, seg_slots, seg_ranks, seg_scales, host_segments=None, out=None, repeat: int = 1):
    """Multi-tenant LoRA delta for a token-segmented batch (see ``reference.sgmv``).  ``host_segments`` =
    ``[(lo, hi, slot, rank, scale)]`` mirrors the device tensors so the CUDA path needs no device read.  On a GPU
    ``out`` (the base projection's output ``[T, N]``) receives the delta in place and is returned; ``repeat`` says that
    ``lora_a`` / ``lora_b`` stack that many projections' pools along the rank axis."""
    if _cuda(x) and x.dtype == torch.bfloat16:
        if host_segments is None:
            starts = seg_starts.tolist()
            host_segments = [(starts[i], starts[i + 1], int(s), int(r), float(c)) for i, (s, r, c) in enumerate(
                zip(seg_slots.tolist(), seg_ranks.tolist(), seg_scales.tolist()))]
        T = x.shape[0]
        if any(hi > T for (_, hi, _, _, _) in host_segments):  # an open-ended segment ("all remaining tokens")
            host_segments = [(lo, min(hi, T), s, r, c) for (lo, hi, s, r, c) in host_segments if lo < T]
            seg_starts = torch.tensor([h[0] for h in host_segments] + [host_segments[-1][1]], dtype=torch.int32, device=x.device)
            seg_slots = torch.tensor([h[2] for h in host_segments], dtype=torch.int32, device=x.device)
        return _SGMV.apply(x.contiguous(), lora_a, lora_b, seg_starts, seg_slots, seg_ranks, seg_scales, host_segments, out, repeat)
    assert out is None and repeat == 1, 'in-place / stacked form is for the CUDA path'
    return _sgmv_autograd_cpu(x, lora_a, lora_b, seg_starts, seg_slots, seg_ranks, seg_scales)


def _sgmv_autograd_cpu(x, lora_a, lora_b, seg_starts, seg_slots, seg_ranks, seg_scales):
    outs = []
    starts = seg_starts.tolist()
    for i in range(len(starts) - 1):
        xs = x[starts[i]:starts[i + 1]]
        slot, r = int(seg_slots[i]), int(seg_ranks[i])
        if slot < 0 or r == 0:
            outs.append(xs.new_zeros(xs.shape[0], lora_b.shape[1]))
        else:
            outs.append((xs @ lora_a[slot, :r].t().to(xs.dtype)) @ lora_b[slot, :, :r].t().to(xs.dtype) * float(seg_scales[i]))
    return torch.cat(outs, 0) if outs else x.new_zeros(0, lora_b.shape[1])


# --------------------------------------------------------------------- moe
class _Router(torch.autograd.Function):
    """Fused fp32 softmax + top-k + renormalisation + expert histogram.  Backward is the closed form on the
    ``[T, E]`` probabilities (a few element-wise passes over a small tensor)."""

    @staticmethod
    def forward(ctx, logits, top_k, renorm, forced):
        w, idx, probs, hist = ext().moe_router(logits.contiguous(), top_k, renorm)
        if forced is not None:  # router replay: keep the probabilities, take the given experts (rows of -1: no replay)
            forced = forced.to(idx.device).long()
            idx = torch.where(forced[:, :1] < 0, idx, forced)
            w = probs.gather(-1, idx)
            if renorm:
                w = w / w.sum(-1, keepdim=True)
            hist = torch.zeros_like(hist).scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=hist.dtype, device=hist.device))
        ctx.save_for_backward(probs, idx, w)
        ctx.renorm = renorm
        ctx.mark_non_differentiable(idx, hist)
        return w, idx, probs, hist

    @staticmethod
    def backward(ctx, gw, _gidx, gprobs, _ghist):
        probs, idx, w = ctx.saved_tensors
        dp = gprobs.clone() if gprobs is not None else torch.zeros_like(probs)
        if gw is not None:
            if ctx.renorm:
                S = probs.gather(-1, idx).sum(-1, keepdim=True)
                g_sel = (gw - (gw * w).sum(-1, keepdim=True)) / S
            else:
                g_sel = gw
            dp.scatter_add_(-1, idx, g_sel)
        dlogits = probs * (dp - (probs * dp).sum(-1, keepdim=True))
        return dlogits, None, None, None


def moe_router(logits, top_k: int, renormalize: bool = True, forced=None):
    """(weights [T,k] fp32, indices [T,k] int64, probs [T,E] fp32, histogram [E] | None)."""
    if _cuda(logits):
        return _Router.apply(logits, top_k, renormalize, forced)
    probs = torch.softmax(logits.float(), -1)
    w, idx = probs.topk(top_k, -1)
    if forced is not None:  # rows of -1 keep the router's own choice (tokens the sampler did not record)
        forced = forced.long()
        idx = torch.where(forced[:, :1] < 0, idx, forced)
        w = probs.gather(-1, idx)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs, None


class _GroupedGemm(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, offsets):
        ctx.save_for_backward(x, weight, offsets)
        return ext().grouped_gemm(x, weight, offsets, 'nt', None)

    @staticmethod
    def backward(ctx, gy):
        x, weight, offsets = ctx.saved_tensors
        gy = gy.contiguous()
        gx = ext().grouped_gemm(gy, weight, offsets, 'nn', None) if ctx.needs_input_grad[0] else None
        gw = ext().grouped_gemm_wgrad(gy, x, offsets, weight.shape[0]).to(weight.dtype) if ctx.needs_input_grad[1] else None
        return gx, gw, None


def grouped_gemm(x, weight, offsets):
    """Per-expert GEMM over expert-sorted rows (``offsets [E+1]`` int32 on device)."""
    if _cuda(x) and x.dtype == torch.bfloat16:
        return _GroupedGemm.apply(x, weight, offsets.to(torch.int32))
    outs = []
    off = offsets.tolist()
    for e in range(weight.shape[0]):
        outs.append(x[off[e]:off[e + 1]] @ weight[e].t().to(x.dtype))
    return torch.cat(outs, 0)


# ------------------------------------------------------- moe token permutation
def moe_index_maps(order: torch.Tensor, rows: torch.Tensor, bound: int, k: int):
    """From the expert sort (``order[i]`` = flat (token, slot) index of the i-th sorted pair, ``rows[i]`` = its row in
    the expert-grouped layout) build the two gather maps: ``row_of [T, k]`` (row of every (token, slot)),
    ``src_tok [bound]`` (token feeding each row, −1 = padding) and ``slot_of_row [bound]`` (flat index, −1 = padding)."""
    n = order.numel()
    dev = order.device
    row_of = torch.empty(n, dtype=torch.int32, device=dev)
    row_of[order] = rows.to(torch.int32)
    slot_of_row = torch.full((bound, ), -1, dtype=torch.int32, device=dev)
    slot_of_row[rows] = order.to(torch.int32)
    src_tok = torch.where(slot_of_row >= 0, slot_of_row // k, slot_of_row)
    return row_of.view(-1, k), src_tok, slot_of_row


def _rows_gather(x, src, scale=None):
    if _cuda(x) and x.dtype == torch.bfloat16:
        return ext().moe_rows_gather(x.contiguous(), src, scale)
    out = x.index_select(0, src.clamp_min(0).long()) * (src >= 0).to(x.dtype).unsqueeze(-1)
    return out if scale is None else out * scale.to(x.dtype).unsqueeze(-1)


def _rows_combine(y, row_of, w=None):
    if _cuda(y) and y.dtype == torch.bfloat16:
        return ext().moe_rows_combine(y.contiguous(), row_of, None if w is None else w.float().contiguous())
    g = y.index_select(0, row_of.reshape(-1).clamp_min(0).long()).view(row_of.shape[0], row_of.shape[1], -1)
    m = (row_of >= 0).to(y.dtype)
    if w is not None:
        m = m * w.to(y.dtype)
    return (g * m.unsqueeze(-1)).sum(1)


class _MoEDispatch(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, src_tok, row_of):
        ctx.save_for_backward(row_of)
        return _rows_gather(x, src_tok)

    @staticmethod
    def backward(ctx, g):
        row_of, = ctx.saved_tensors
        return _rows_combine(g.contiguous(), row_of), None, None


class _MoECombine(torch.autograd.Function):

    @staticmethod
    def forward(ctx, y, w, row_of, src_tok, slot_of_row):
        ctx.save_for_backward(y, w, row_of, src_tok, slot_of_row)
        return _rows_combine(y, row_of, w)

    @staticmethod
    def backward(ctx, g):
        y, w, row_of, src_tok, slot_of_row = ctx.saved_tensors
        g = g.contiguous()
        w_row = w.reshape(-1).float().index_select(0, slot_of_row.clamp_min(0).long())
        gy = _rows_gather(g, src_tok, w_row)
        if _cuda(y) and y.dtype == torch.bfloat16:
            gw = ext().moe_combine_wgrad(g, y, row_of)
        else:
            yy = y.index_select(0, row_of.reshape(-1).clamp_min(0).long()).view(row_of.shape[0], row_of.shape[1], -1)
            gw = (yy.float() * g.float().unsqueeze(1)).sum(-1) * (row_of >= 0)
        return gy, gw.to(w.dtype), None, None, None


def moe_dispatch(x, src_tok, row_of):
    """Token rows → expert-grouped rows (zero padding rows); backward sums every token's k rows."""
    return _MoEDispatch.apply(x, src_tok, row_of)


def moe_combine(y, w, row_of, src_tok, slot_of_row):
    """``out[t] = Σ_j w[t, j] · y[row_of[t, j]]`` with gradients for ``y`` and the routing weights ``w``."""
    return _MoECombine.apply(y, w, row_of, src_tok, slot_of_row)


class _ExpertLinearLora(torch.autograd.Function):
    """``y = x Wᵀ + s · (x Aᵀ) Bᵀ`` per expert over expert-grouped rows.  The low-rank term rides in the base GEMM as a
    second operand pair (``[x | h] · [W | s·B]ᵀ`` summed in tensor memory), forward and input-gradient alike, so the
    ``[rows, out]`` / ``[rows, in]`` tensors are written once and never re-read by an accumulate pass.
    ``TWINKLE_EXPERT_LORA_SPLIT=1`` keeps the earlier form (a separate rank-r GEMM accumulating into the output)."""

    @staticmethod
    def forward(ctx, x, weight, a, b, offsets, scale):
        E = ext()
        h = E.grouped_gemm(x, a, offsets, 'nt', None)                     # [rows, r]
        bs = (b.float() * scale).to(b.dtype)                               # [E, out, r] — scale folded into the small operand
        if _EXPERT_LORA_SPLIT:
            y = E.grouped_gemm(x, weight, offsets, 'nt', None)
            E.grouped_gemm(h, bs, offsets, 'nt', None, y, True)
        else:
            y = E.grouped_gemm(x, weight, offsets, 'nt', None, None, False, h, bs)
        ctx.save_for_backward(x, weight, a, bs, h, offsets)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, gy):
        E = ext()
        x, weight, a, bs, h, offsets = ctx.saved_tensors
        gy = gy.contiguous()
        n_e = weight.shape[0]
        gh = E.grouped_gemm(gy, bs, offsets, 'nn', None)                   # [rows, r] = gy · (s·B)
        gx = None
        if ctx.needs_input_grad[0]:
            if _EXPERT_LORA_SPLIT:
                gx = E.grouped_gemm(gy, weight, offsets, 'nn', None)
                E.grouped_gemm(gh, a, offsets, 'nn', None, gx, True)
            else:
                gx = E.grouped_gemm(gy, weight, offsets, 'nn', None, None, False, gh, a)
        gw = E.grouped_gemm_wgrad(gy, x, offsets, n_e).to(weight.dtype) if ctx.needs_input_grad[1] else None
        ga = E.grouped_gemm_wgrad(gh, x, offsets, n_e).to(a.dtype) if ctx.needs_input_grad[2] else None
        gb = (E.grouped_gemm_wgrad(gy, h, offsets, n_e) * ctx.scale).to(bs.dtype) if ctx.needs_input_grad[3] else None
        return gx, gw, ga, gb, None, None


_EXPERT_LORA_SPLIT = os.environ.get('TWINKLE_EXPERT_LORA_SPLIT', '0') == '1'


def expert_linear(x, weight, offsets, lora_a=None, lora_b=None, scale: float = 1.0):
    """Per-expert linear over expert-grouped rows with an optional per-expert LoRA pair (``lora_a [E, r, in]``,
    ``lora_b [E, out, r]``)."""
    if lora_a is None:
        return grouped_gemm(x, weight, offsets)
    if _cuda(x) and x.dtype == torch.bfloat16:
        r = lora_a.shape[1]
        if r % 8:  # TMA rows must be 16-byte multiples: pad the rank with zero rows / columns
            pad = 8 - r % 8
            lora_a = torch.nn.functional.pad(lora_a, (0, 0, 0, pad))
            lora_b = torch.nn.functional.pad(lora_b, (0, pad))
        return _ExpertLinearLora.apply(x, weight, lora_a.contiguous(), lora_b.contiguous(), offsets.to(torch.int32), float(scale))
    return grouped_gemm(x, weight, offsets) + grouped_gemm(grouped_gemm(x, lora_a, offsets), lora_b, offsets) * scale


def sample_tokens(logits, temperature=1.0, top_k=-1, top_p=1.0, generator=None, seeds=None):
    """(tokens [B], logprob of each under the processed distribution [B]).  On CUDA every row draws from its
    own counter-based stream keyed by ``seeds[row]`` (fresh seeds when none are given)."""
    if _cuda(logits):
        if seeds is None:
            seeds = torch.randint(0, 2**62, (logits.shape[0], ), device=logits.device, dtype=torch.int64, generator=generator)
        tok, lp = ext().sample_tokens(logits.float().contiguous(), float(temperature), int(top_k), float(top_p), seeds)
        return tok, lp
    return ref.sample_tokens(logits, temperature, top_k, top_p, generator)


__all__ = [n for n in dir() if not n.startswith('_')]
