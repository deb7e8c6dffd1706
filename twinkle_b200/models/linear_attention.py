"""Gated DeltaNet linear attention (the "linear_attention" layers of Qwen3.5 / Qwen3-Next style hybrids).

What it covers: the reference's sequence-parallel wrapper around FLA's Triton kernels
(``model/transformers/strategy/sequence_parallel/linear_attention_sp.py:266-308``: in-projection → short causal
conv1d → ``chunk_gated_delta_rule`` → gated RMSNorm → out-projection, with Ulysses head scatter).  The state update
per head is

    S_t = α_t · S_{t-1} · (I − β_t k_t k_tᵀ) + β_t k_t v_tᵀ ,      o_t = S_tᵀ q_t            (S ∈ R^{dk×dv})

with decay α_t = exp(g_t) ∈ (0, 1] and write strength β_t ∈ (0, 1).  Two evaluators are provided: the plain recurrence
(exact, O(T) sequential steps) and a chunk-parallel form (WY / UT transform inside chunks of ``chunk`` tokens, one
sequential step per chunk) that is what training uses.  Both take packed sequences through ``cu_seqlens``: state and
convolution history are reset at every boundary.  On a GPU in bf16 the convolution (+SiLU) and the forward recurrence
(with the q / k normalisation and the grouped-head repeat inside) are CUDA kernels (``ops/csrc/gdn.cu``: one warp per
sequence × value head × 32 state columns, state in registers); their backward is autograd on the chunk-parallel
evaluator below, which is also the CPU / fp32 path.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Linear


def gated_delta_rule_recurrent(q, k, v, g, beta, scale: Optional[float] = None, state=None):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g, beta [T, H]`` → (``o [T, H, dv]``, final state ``[H, dk, dv]``)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    S = q.new_zeros(H, dk, dv, dtype=torch.float32) if state is None else state.float().clone()
    out = []
    qf, kf, vf, gf, bf = q.float() * scale, k.float(), v.float(), g.float(), beta.float()
    for t in range(T):
        S = S * gf[t].exp()[:, None, None]
        kv = torch.einsum('hk,hkv->hv', kf[t], S)                       # what the memory currently returns for k_t
        S = S + torch.einsum('hk,hv->hkv', kf[t], (vf[t] - kv) * bf[t][:, None])
        out.append(torch.einsum('hk,hkv->hv', qf[t], S))
    return torch.stack(out).to(q.dtype), S


def gated_delta_rule_chunked(q, k, v, g, beta, scale: Optional[float] = None, chunk: int = 64, state=None):
    """Same contract as the recurrence, evaluated chunk-parallel."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    N = (T + pad) // chunk
    # [H, N, C, ·]
    qc = (q.float() * scale).view(N, chunk, H, dk).permute(2, 0, 1, 3)
    kc = k.float().view(N, chunk, H, dk).permute(2, 0, 1, 3)
    vc = v.float().view(N, chunk, H, dv).permute(2, 0, 1, 3)
    bc = beta.float().view(N, chunk, H).permute(2, 0, 1)
    gc = g.float().view(N, chunk, H).permute(2, 0, 1).cumsum(-1)       # log decay from the chunk start (inclusive)
    kb, vb = kc * bc[..., None], vc * bc[..., None]
    tri = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device)
    strict_lower, lower = tri.tril(-1), tri.tril()
    rel = (gc[..., :, None] - gc[..., None, :]).masked_fill(~lower, float('-inf')).exp()    # decay from token j to token i ≥ j
    # (I + A)^{-1} with A = strictly-lower(β_i k_i·k_j · decay): forward substitution, row by row
    A = -(kb @ kc.transpose(-1, -2) * rel).masked_fill(~strict_lower, 0.0)
    rows = [A[..., 0, :]]
    for i in range(1, chunk):                                            # out of place: the loop stays differentiable
        a = A[..., i, :]
        rows.append(a + (a[..., :i, None] * torch.stack(rows, -2)).sum(-2))
    A = torch.stack(rows, -2) + torch.eye(chunk, device=q.device)
    u = A @ vb                                                          # values corrected for intra-chunk interactions
    w = A @ (kb * gc.exp()[..., None])                                   # what must be subtracted per unit of incoming state
    S = q.new_zeros(H, dk, dv, dtype=torch.float32) if state is None else state.float().clone()
    outs = []
    for n in range(N):
        qn, kn, gn = qc[:, n], kc[:, n], gc[:, n]
        v_new = u[:, n] - w[:, n] @ S
        attn = (qn @ kn.transpose(-1, -2) * rel[:, n]).masked_fill(~lower, 0.0)
        outs.append((qn * gn.exp()[..., None]) @ S + attn @ v_new)
        last = gn[:, -1]
        S = S * last.exp()[:, None, None] + (kn * (last[:, None] - gn).exp()[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, 1).permute(1, 2, 0, 3).reshape(N * chunk, H, dv)[:T]
    return o.to(q.dtype), S


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None, chunk: int = 64, recurrent: bool = False,
                            return_states: bool = False):
    """Packed sequences: every segment starts from an empty state. With ``return_states`` also the final state of every
    (non-empty) segment, stacked ``[n, H, dk, dv]`` — what a decoder carries on from after the prompt."""
    fn = gated_delta_rule_recurrent if recurrent else (lambda *a, **kw: gated_delta_rule_chunked(*a, chunk=chunk, **kw))
    bounds = cu_seqlens.tolist()
    res = [fn(q[a:b], k[a:b], v[a:b], g[a:b], beta[a:b], scale) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
    out = torch.cat([r[0] for r in res], 0) if res else q.new_zeros(0, q.shape[1], v.shape[-1])
    if return_states:
        return out, (torch.stack([r[1] for r in res]) if res else q.new_zeros(0, q.shape[1], q.shape[2], v.shape[-1], dtype=torch.float32))
    return out


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x / sqrt(Σx² + eps)`` over the last dim in fp32 — the q / k normalisation of the FLA kernels the Hugging Face
    implementation follows (not ``F.normalize``, whose epsilon clamps the norm instead)."""
    xf = x.float()
    return xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) + eps)


def gated_delta_rule_varlen_torch(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None, chunk: int = 64, normalize: bool = True,
                                  init_state=None, return_states: bool = False):
    """The whole op on PyTorch: ``q, k [T, Hk, dk]`` are L2-normalised per head (``normalize``) and repeated to the ``Hv``
    value heads, then every packed segment is evaluated chunk-parallel from ``init_state[i]`` (or an empty state)."""
    rep = v.shape[1] // q.shape[1]
    if normalize:
        q, k = l2norm(q).to(q.dtype), l2norm(k).to(k.dtype)
    if rep > 1:
        q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    bounds = cu_seqlens.tolist()
    segs = [(a, b) for a, b in zip(bounds[:-1], bounds[1:])]
    res = []
    for i, (a, b) in enumerate(segs):
        st = init_state[i] if init_state is not None else None
        if b > a:
            res.append(gated_delta_rule_chunked(q[a:b], k[a:b], v[a:b], g[a:b], beta[a:b], scale, chunk=chunk, state=st))
        else:   # an empty segment keeps its state
            res.append((q.new_zeros(0, v.shape[1], v.shape[-1]),
                        st.float() if st is not None else q.new_zeros(v.shape[1], q.shape[2], v.shape[-1], dtype=torch.float32)))
    out = torch.cat([r[0] for r in res], 0) if res else q.new_zeros(0, v.shape[1], v.shape[-1])
    if return_states:
        return out, (torch.stack([r[1] for r in res]) if res else q.new_zeros(0, v.shape[1], q.shape[2], v.shape[-1], dtype=torch.float32))
    return out


def causal_conv1d_varlen(x: torch.Tensor, weight: torch.Tensor, cu_seqlens: torch.Tensor, activation: bool = True) -> torch.Tensor:
    """Depth-wise causal convolution over packed tokens (kernel on a GPU in bf16, PyTorch otherwise)."""
    from .. import ops
    return ops.causal_conv1d_varlen(x, weight, cu_seqlens, activation)


def causal_conv1d_varlen_torch(x: torch.Tensor, weight: torch.Tensor, cu_seqlens: torch.Tensor, activation: bool = True) -> torch.Tensor:
    """Depth-wise causal convolution over packed tokens: ``x [T, C]``, ``weight [C, W]``; no leakage across segments."""
    T, C = x.shape
    W = weight.shape[1]
    bounds = cu_seqlens.tolist()
    outs = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b <= a:
            continue
        seg = F.pad(x[a:b].t().unsqueeze(0), (W - 1, 0))                # [1, C, L + W − 1]
        outs.append(F.conv1d(seg, weight.unsqueeze(1).to(x.dtype), groups=C)[0].t())
    y = torch.cat(outs, 0) if outs else x.new_zeros(0, C)
    return F.silu(y) if activation else y


class GatedDeltaNet(nn.Module):
    """Drop-in replacement of the softmax-attention block for ``linear_attention`` layers."""

    def __init__(self, hidden_size: int, num_k_heads: int, num_v_heads: int, head_k_dim: int, head_v_dim: int, conv_kernel: int = 4,
                 eps: float = 1e-6, chunk: int = 64):
        super().__init__()
        assert num_v_heads % num_k_heads == 0
        self.hk, self.hv, self.dk, self.dv, self.chunk, self.eps = num_k_heads, num_v_heads, head_k_dim, head_v_dim, chunk, eps
        kd, vd = num_k_heads * head_k_dim, num_v_heads * head_v_dim
        self.in_proj_qkvz = Linear(hidden_size, 2 * kd + 2 * vd, name='in_proj_qkvz')
        self.in_proj_ba = Linear(hidden_size, 2 * num_v_heads, name='in_proj_ba')
        self.conv_weight = nn.Parameter(torch.empty(2 * kd + vd, conv_kernel))
        self.dt_bias = nn.Parameter(torch.ones(num_v_heads))
        self.A_log = nn.Parameter(torch.zeros(num_v_heads))
        self.norm_weight = nn.Parameter(torch.ones(head_v_dim))
        self.out_proj = Linear(vd, hidden_size, name='out_proj')
        self.attn_parallel = None  # Ulysses strategy: heads are scattered exactly like softmax attention heads
        nn.init.kaiming_uniform_(self.conv_weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor, cu_seqlens: torch.Tensor, state_sink=None) -> torch.Tensor:
        """``state_sink(conv_tail [n, W−1, C], state [n, Hv, dk, dv])``, when given, receives what :meth:`step` needs to
        continue every segment token by token: the last ``W−1`` pre-convolution rows (zero-padded on the left for short
        segments) and the final recurrent state."""
        T = x.shape[0]
        kd, vd = self.hk * self.dk, self.hv * self.dv
        qkvz = self.in_proj_qkvz(x)
        qkv, z = qkvz[:, :2 * kd + vd], qkvz[:, 2 * kd + vd:]
        if state_sink is not None:
            assert self.attn_parallel is None, 'decoding state is collected on unsharded sequences'
            w1 = self.conv_weight.shape[1] - 1
            bounds = cu_seqlens.tolist()
            tails = [F.pad(qkv[max(a, b - w1):b], (0, 0, w1 - min(w1, b - a), 0)) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
        b, a = self.in_proj_ba(x).chunk(2, -1)
        beta = torch.sigmoid(b.float())
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias.float())      # log decay ≤ 0
        ap = self.attn_parallel
        if ap is None:
            qkv = causal_conv1d_varlen(qkv, self.conv_weight, cu_seqlens)
        q, k, v = qkv[:, :kd].view(T, self.hk, self.dk), qkv[:, kd:2 * kd].view(T, self.hk, self.dk), qkv[:, 2 * kd:].view(T, self.hv, self.dv)
        if ap is not None:
            # sequence → head exchange first (every rank then owns whole sequences for a slice of the heads), then the
            # convolution with this rank's slice of the depth-wise filters; the exchange is the same one attention uses
            q, k, v = ap.scatter_heads(q.contiguous(), k.contiguous(), v.contiguous())
            beta, g = ap.scatter_scalar_heads(beta), ap.scatter_scalar_heads(g)
            q, k, v = ap.conv_after_scatter(q, k, v, self.conv_weight, cu_seqlens, self.hk, self.hv, self.dk, self.dv)
        from .. import ops
        if state_sink is not None:
            o, states = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk=self.chunk, return_states=True)
            keep = (cu_seqlens[1:] > cu_seqlens[:-1]).tolist()
            if not all(keep):   # the sink takes the non-empty segments only
                states = states[torch.tensor(keep, device=states.device)]
            state_sink(torch.stack(tails) if tails else qkv.new_zeros(0, w1, qkv.shape[1]), states)
        else:
            o = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk=self.chunk)
        if ap is not None:
            o = ap.gather_heads(o.contiguous())
        # gated RMSNorm per head, gate z
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.eps) * self.norm_weight.float()
        of = of * F.silu(z.float().view(T, self.hv, self.dv))
        return self.out_proj(of.to(x.dtype).reshape(T, vd))

    @torch.no_grad()
    def step(self, x: torch.Tensor, conv_state: torch.Tensor, state: torch.Tensor):
        """One token per row: ``x [B, hidden]``, ``conv_state [B, W−1, C]`` (previous pre-convolution rows),
        ``state [B, Hv, dk, dv]`` (fp32) → (``y [B, hidden]``, new ``conv_state``, new ``state``). Same arithmetic as
        :meth:`forward` on a sequence extended by this token."""
        B = x.shape[0]
        kd, vd = self.hk * self.dk, self.hv * self.dv
        qkvz = self.in_proj_qkvz(x)
        qkv, z = qkvz[:, :2 * kd + vd], qkvz[:, 2 * kd + vd:]
        b, a = self.in_proj_ba(x).chunk(2, -1)
        beta = torch.sigmoid(b.float())
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias.float())
        window = torch.cat([conv_state.to(qkv.dtype), qkv.unsqueeze(1)], 1)                    # [B, W, C]
        conv = F.silu((window * self.conv_weight.t().to(qkv.dtype).unsqueeze(0)).sum(1))       # depth-wise causal conv, last position
        q, k, v = conv[:, :kd].view(B, self.hk, self.dk), conv[:, kd:2 * kd].view(B, self.hk, self.dk), conv[:, 2 * kd:].view(B, self.hv, self.dv)
        from .. import ops
        if ops.gdn_kernel_supported(q, v):
            # every row is a one-token sequence that continues from its own state
            cu = torch.arange(B + 1, dtype=torch.int32, device=x.device)
            o, S = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu, init_state=state, return_states=True)
            o = o.float()
        else:
            q, k = l2norm(q), l2norm(k)
            rep = self.hv // self.hk
            if rep > 1:
                q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            S = state.float() * g.exp()[:, :, None, None]
            kv = torch.einsum('bhk,bhkv->bhv', k, S)
            S = S + torch.einsum('bhk,bhv->bhkv', k, (v.float() - kv) * beta[:, :, None])
            o = torch.einsum('bhk,bhkv->bhv', q * self.dk ** -0.5, S)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.norm_weight.float()
        o = o * F.silu(z.float().view(B, self.hv, self.dv))
        return self.out_proj(o.to(x.dtype).reshape(B, vd)), window[:, 1:].contiguous(), S
