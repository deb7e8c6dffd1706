"""Plain-PyTorch fp32 restatement of every hand-written kernel.

These functions are (a) the oracle the CUDA kernels are tested against and
(b) the path taken on CPU tensors (gloo tests).  They favour clarity over
speed and never call a fused library kernel.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * (weight.float() + offset)).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``res' = x + residual`` (rounded to the storage dtype), ``y = rmsnorm(res')``."""
    new_res = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(new_res, weight, eps, offset), new_res


# ---------------------------------------------------------------------- rope
def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None, device=None,
                  seq_len: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, float]:
    """Inverse frequencies ``[head_dim/2]`` and the factor applied to cos/sin, for plain RoPE or a long-context variant
    given as a Hugging Face ``rope_scaling`` mapping (``rope_type`` / ``type``):

    * ``linear``: all frequencies ÷ ``factor``;
    * ``llama3``: wavelengths above ``original_max / low_freq_factor`` ÷ ``factor``, those below
      ``original_max / high_freq_factor`` unchanged, a linear blend between;
    * ``yarn``: per-dimension blend of interpolated (÷ ``factor``) and original frequencies along a ramp between the
      dimensions that complete ``beta_fast`` and ``beta_slow`` rotations over the original window; cos/sin scaled by
      ``attention_factor`` (default ``0.1·ln(factor) + 1``);
    * ``dynamic`` (NTK): the base grows with the sequence once it exceeds ``max_position_embeddings``:
      ``θ · (factor · L / max − (factor − 1)) ^ (d / (d − 2))``;
    * ``longrope`` (Phi-3 long-context): per-dimension divisors ``short_factor`` up to ``original_max_position_embeddings``
      tokens and ``long_factor`` beyond, cos/sin scaled by ``√(1 + ln(factor) / ln(original_max))``.

    The last two depend on the sequence length ``seq_len`` (a 0-dim tensor: largest position + 1, as Hugging Face takes
    it; chosen on the device, no host read); without it they give their short-sequence form.
    ``default`` / ``None`` give plain RoPE. Other types raise."""
    import math
    inv = 1.0 / (theta**(torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    kind = (scaling or {}).get('rope_type', (scaling or {}).get('type', 'default'))
    if not scaling or kind in ('default', None):
        return inv, 1.0
    factor = float(scaling.get('factor', 1.0))
    if kind == 'linear':
        return inv / factor, 1.0
    if kind == 'llama3':
        lo, hi = float(scaling.get('low_freq_factor', 1.0)), float(scaling.get('high_freq_factor', 4.0))
        orig = float(scaling['original_max_position_embeddings'])
        wavelen = 2 * math.pi / inv
        smooth = ((orig / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)
        blended = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, blended))
        return out, 1.0
    if kind == 'yarn':
        orig = float(scaling.get('original_max_position_embeddings') or scaling.get('max_position_embeddings', 4096))
        fast, slow = float(scaling.get('beta_fast') or 32), float(scaling.get('beta_slow') or 1)
        att = scaling.get('attention_factor')
        if att is None:
            ms, ms_all = scaling.get('mscale'), scaling.get('mscale_all_dim')
            get = lambda sc, m=1.0: 1.0 if sc <= 1 else 0.1 * m * math.log(sc) + 1.0  # noqa: E731
            att = get(factor, ms) / get(factor, ms_all) if ms and ms_all else get(factor)

        def corr_dim(rot: float) -> float:
            return head_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))

        low, high = corr_dim(fast), corr_dim(slow)
        if scaling.get('truncate', True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        keep = 1 - ramp                                  # 1 → original frequency, 0 → interpolated
        return inv / factor * (1 - keep) + inv * keep, float(att)
    if kind == 'dynamic':
        mx = float(scaling.get('max_position_embeddings', 0) or 0)
        if seq_len is None or mx <= 0 or head_dim <= 2:
            return inv, 1.0
        grow = (factor * seq_len.float().clamp_min(mx) / mx - (factor - 1.0))**(head_dim / (head_dim - 2))
        expo = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
        return 1.0 / ((theta * grow)**expo), 1.0
    if kind == 'longrope':
        orig = float(scaling.get('original_max_position_embeddings') or scaling.get('max_position_embeddings', 4096))
        short = torch.tensor(scaling['short_factor'], dtype=torch.float32, device=device)
        ext = short
        if seq_len is not None:
            ext = torch.where(seq_len > orig, torch.tensor(scaling['long_factor'], dtype=torch.float32, device=device), short)
        f = scaling.get('factor') or float(scaling.get('max_position_embeddings', orig)) / orig
        att = scaling.get('attention_factor')
        if att is None:
            att = 1.0 if f <= 1.0 else math.sqrt(1 + math.log(f) / math.log(orig))
        return inv / ext, float(att)
    raise NotImplementedError(f'rope scaling type {kind!r} is not supported (default, linear, llama3, yarn, dynamic, longrope are)')


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float = 1e6, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[T, head_dim/2]`` in fp32 for integer ``positions [T]`` (see :func:`rope_inv_freq` for ``scaling``)."""
    seq_len = None
    if scaling and scaling.get('rope_type', scaling.get('type')) in ('dynamic', 'longrope') and positions.numel():
        seq_len = positions.max() + 1
    inv_freq, att = rope_inv_freq(head_dim, theta, scaling, positions.device, seq_len)
    ang = positions.float()[:, None] * inv_freq[None, :]
    if att != 1.0:
        return ang.cos() * att, ang.sin() * att
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention (HF Llama/Qwen): pairs are (i, i + R/2) inside the leading ``R = 2·cos.shape[-1]`` dims;
    dims past ``R`` pass through (partial rotary).  ``x [T, H, D]``."""
    rot = 2 * cos.shape[-1]
    xf = x.float()
    x1, x2 = xf[..., :rot // 2], xf[..., rot // 2:rot]
    c, s = cos[:, None, :], sin[:, None, :]
    parts = [x1 * c - x2 * s, x2 * c + x1 * s]
    if rot < x.shape[-1]:
        parts.append(xf[..., rot:])
    return torch.cat(parts, -1).to(x.dtype)


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                 cos: torch.Tensor, sin: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-head RMSNorm on q and k (Qwen3; ``offset`` 1.0 for the "1 + w" form of Qwen3.5) followed by RoPE.
    ``q [T,Hq,D]``, ``k [T,Hkv,D]``."""
    if q_weight is not None:
        q = rmsnorm(q, q_weight, eps, offset)
        k = rmsnorm(k, k_weight, eps, offset)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin)


# -------------------------------------------------------------------- swiglu
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``[T, 2I]`` laid out as ``[gate | up]`` → ``silu(gate) * up`` ``[T, I]``."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.gelu(g, approximate='tanh') * u).to(gate_up.dtype)


def clamped_glu(gate_up: torch.Tensor, limit: float = 7.0, alpha: float = 1.702) -> torch.Tensor:
    """GPT-OSS expert activation on ``[gate | up]``: ``(up + 1) · gate · σ(α · gate)`` with ``gate ≤ limit`` and
    ``|up| ≤ limit``."""
    g, u = gate_up.float().chunk(2, dim=-1)
    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return ((u + 1.0) * g * torch.sigmoid(alpha * g)).to(gate_up.dtype)


# ----------------------------------------------------------------- attention
def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, causal: bool = True,
                     scale: Optional[float] = None, return_lse: bool = False, cu_seqlens_k: Optional[torch.Tensor] = None,
                     window: Optional[int] = None, softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None):
    """Packed attention.  ``q [T,Hq,D]``, ``k,v [Tk,Hkv,D]``, ``cu_seqlens`` int
    ``[n+1]``; tokens of different segments never attend to each other; GQA by
    repeating each kv head ``Hq/Hkv`` times.  With ``cu_seqlens_k`` the keys of a segment may be longer than its
    queries; the causal diagonal is then aligned bottom-right (query row r sees keys 0 … r + Lk − Lq).
    ``window``: a query sees only the last ``window`` keys up to and including its own position (sliding-window
    checkpoints); ``softcap``: scores pass through ``cap · tanh(s / cap)`` before the softmax (Gemma-2); ``sinks [Hq]``: a
    learned logit per head that takes part in the softmax and carries no value (GPT-OSS), i.e. it only enlarges the
    denominator."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = q.new_empty(T, Hq, v.shape[-1])          # values may be narrower than the score width (latent attention)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    bounds = cu_seqlens.tolist()
    kb = bounds if cu_seqlens_k is None else cu_seqlens_k.tolist()
    for a, b, ka, kbnd in zip(bounds[:-1], bounds[1:], kb[:-1], kb[1:]):
        if b <= a:
            continue
        qs = q[a:b].float().transpose(0, 1)  # [Hq, L, D]
        ks = k[ka:kbnd].float().transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[ka:kbnd].float().transpose(0, 1).repeat_interleave(rep, 0)
        s = qs @ ks.transpose(1, 2) * scale
        if softcap:
            s = torch.tanh(s / softcap) * softcap
        if causal:
            L, Lk = b - a, kbnd - ka
            s = s.masked_fill(torch.ones(L, Lk, dtype=torch.bool, device=q.device).triu(1 + Lk - L), float('-inf'))
            if window and Lk > window:
                s = s.masked_fill(torch.ones(L, Lk, dtype=torch.bool, device=q.device).tril(Lk - L - window), float('-inf'))
        l = torch.logsumexp(s, -1)
        if sinks is not None:
            l = torch.logaddexp(l, sinks.float()[:, None])
        p = torch.exp(s - l[..., None])
        out[a:b] = (p @ vs).transpose(0, 1).to(q.dtype)
        lse[:, a:b] = l
    return (out, lse) if return_lse else out


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                           seq_lens: torch.Tensor, scale: Optional[float] = None, window: Optional[int] = None,
                           softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence against a paged KV cache.
    ``q [B,Hq,D]``; caches ``[num_blocks, block_size, Hkv, D]``; ``block_tables
    [B, max_blocks]`` int; ``seq_lens [B]`` (including the current token)."""
    B, Hq, D = q.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.empty_like(q)
    for b in range(B):
        n = int(seq_lens[b])
        nb = (n + bs - 1) // bs
        blocks = block_tables[b, :nb].long()
        kk = k_cache[blocks].reshape(-1, Hkv, D)[:n].float().repeat_interleave(rep, 1)
        vv = v_cache[blocks].reshape(-1, Hkv, D)[:n].float().repeat_interleave(rep, 1)
        s = torch.einsum('hd,nhd->hn', q[b].float(), kk) * scale
        if softcap:
            s = torch.tanh(s / softcap) * softcap
        if window and n > window:
            s[:, :n - window] = float('-inf')
        if sinks is not None:
            l = torch.logaddexp(torch.logsumexp(s, -1), sinks.float())
            out[b] = torch.einsum('hn,nhd->hd', torch.exp(s - l[:, None]), vv).to(q.dtype)
            continue
        out[b] = torch.einsum('hn,nhd->hd', torch.softmax(s, -1), vv).to(q.dtype)
    return out


# ------------------------------------------------------------ logprob / loss
def logprob_from_logits(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                        with_entropy: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    x = logits.float() / temperature
    lse = torch.logsumexp(x, -1)
    lp = x.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1) - lse
    ent = None
    if with_entropy:
        ent = lse - (torch.softmax(x, -1) * x).sum(-1)
    return lp, ent


def fused_linear_logprob(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                         with_entropy: bool = False, chunk: int = 2048) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``log softmax(hidden @ weightᵀ / temperature)[labels]`` without keeping
    the ``[T, V]`` matrix (chunks over T).  Differentiable via autograd."""
    lps, ents = [], []
    for s in range(0, hidden.shape[0], chunk):
        logits = hidden[s:s + chunk].float() @ weight.float().t()
        lp, ent = logprob_from_logits(logits, labels[s:s + chunk], temperature, with_entropy)
        lps.append(lp)
        if with_entropy:
            ents.append(ent)
    return torch.cat(lps), (torch.cat(ents) if with_entropy else None)


# -------------------------------------------------------------------- adamw
def adamw_step(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, grad: torch.Tensor,
               param_out: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
               step: int, grad_scale: float = 1.0) -> None:
    """Decoupled weight decay Adam on fp32 master weights; ``grad_scale``
    multiplies the gradient first (1/num_tokens × clip coefficient);
    ``param_out`` (bf16 working copy) receives the rounded result."""
    g = grad.float() * grad_scale
    master.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    master.addcdiv_(exp_avg / bc1, denom, value=-lr)
    if param_out is not None:
        param_out.copy_(master)


# --------------------------------------------------------------------- lora
def sgmv(x: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor, seg_starts: torch.Tensor, seg_slots: torch.Tensor,
         seg_ranks: torch.Tensor, seg_scales: torch.Tensor) -> torch.Tensor:
    """Segmented multi-LoRA: rows ``seg_starts[i]:seg_starts[i+1]`` of ``x [T,K]``
    use slot ``seg_slots[i]`` (−1 = no adapter) with rank ``seg_ranks[i]`` and
    scale ``seg_scales[i]``.  ``lora_a [S, R, K]``, ``lora_b [S, N, R]``.
    Returns the delta ``[T, N]`` in x's dtype."""
    T = x.shape[0]
    out = torch.zeros(T, lora_b.shape[1], dtype=x.dtype, device=x.device)
    starts = seg_starts.tolist()
    for i in range(len(starts) - 1):
        slot, r = int(seg_slots[i]), int(seg_ranks[i])
        if slot < 0 or r == 0 or starts[i + 1] <= starts[i]:
            continue
        a = lora_a[slot, :r].float()
        b = lora_b[slot, :, :r].float()
        xs = x[starts[i]:starts[i + 1]].float()
        out[starts[i]:starts[i + 1]] = ((xs @ a.t()) @ b.t() * float(seg_scales[i])).to(x.dtype)
    return out


# ---------------------------------------------------------------------- moe
def moe_router(logits: torch.Tensor, top_k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 softmax → top-k → optional renormalisation.  Returns (weights [T,k]
    fp32, indices [T,k] int64, full probabilities [T,E] fp32)."""
    probs = torch.softmax(logits.float(), -1)
    w, idx = probs.topk(top_k, -1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs


def moe_aux_loss(probs: torch.Tensor, indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Switch-style load-balance loss: ``E · Σ_e f_e · P_e`` with ``f_e`` the
    fraction of routed slots and ``P_e`` the mean router probability."""
    T, k = indices.shape
    f = torch.zeros(num_experts, dtype=torch.float32, device=probs.device)
    f.scatter_add_(0, indices.reshape(-1), torch.ones(T * k, device=probs.device))
    f = f / (T * k)
    return num_experts * (f * probs.mean(0)).sum()


def grouped_gemm(x: torch.Tensor, weight: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """Rows ``offsets[e]:offsets[e+1]`` of ``x [R, K]`` times ``weight[e]ᵀ`` with
    ``weight [E, N, K]`` → ``[R, N]``."""
    out = torch.zeros(x.shape[0], weight.shape[1], dtype=x.dtype, device=x.device)
    off = offsets.tolist()
    for e in range(weight.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            out[a:b] = (x[a:b].float() @ weight[e].float().t()).to(x.dtype)
    return out


def moe_experts(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor) -> torch.Tensor:
    """Dense-math MoE FFN: ``Σ_k weights[t,k] · down_e(swiglu(gate_up_e(x_t)))``."""
    T, k = indices.shape
    out = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    for e in range(w_gate_up.shape[0]):
        tok, slot = (indices == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = swiglu((x[tok].float() @ w_gate_up[e].float().t()).to(x.dtype))
        y = h.float() @ w_down[e].float().t()
        out.index_add_(0, tok, y * weights[tok, slot, None].float())
    return out.to(x.dtype)


# ----------------------------------------------------------------- sampling
def sample_tokens(logits: torch.Tensor, temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0,
                  generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (token ids [B], logprob of the chosen token under the *processed*
    distribution [B])."""
    x = logits.float()
    if temperature <= 0:
        tok = x.argmax(-1)
        return tok, torch.zeros(x.shape[0], device=x.device)
    x = x / temperature
    if top_k and top_k > 0:
        kth = x.topk(min(top_k, x.shape[-1]), -1).values[..., -1:]
        x = x.masked_fill(x < kth, float('-inf'))
    if top_p < 1.0:
        sorted_x, order = x.sort(-1, descending=True)
        cum = torch.softmax(sorted_x, -1).cumsum(-1)
        drop = cum - torch.softmax(sorted_x, -1) >= top_p
        sorted_x = sorted_x.masked_fill(drop, float('-inf'))
        x = torch.full_like(x, float('-inf')).scatter(-1, order, sorted_x)
    logp = torch.log_softmax(x, -1)
    tok = torch.multinomial(logp.exp(), 1, generator=generator).squeeze(-1)
    return tok, logp.gather(-1, tok[:, None]).squeeze(-1)
