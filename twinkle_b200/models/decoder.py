"""The owned decoder-only transformer (Qwen3 dense / Qwen3-MoE / Llama-style).

The reference wraps Hugging Face modules (``src/twinkle/model/transformers/
transformers.py:203-233``); here the network is written once against the
``ops`` layer so that every hot op is our own kernel on B200 and the same code
runs in fp32 on CPU for the gloo tests.  Tensors are always *packed*:
``[T, hidden]`` rows of all sequences back to back, with ``cu_seqlens``
delimiting them (padding-free; reference ``processor/base.py:501-524``).

Parallel behaviour is injected, not hard-coded: ``attn_parallel`` (Ulysses
head↔sequence exchange), ``moe_parallel`` (expert-parallel dispatch/combine) and
``tp`` (tensor-parallel linears) are small strategy objects set by the engine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .config import DecoderConfig
from .layers import Embedding, Linear, RMSNorm


@dataclass
class PackedBatch:
    """What one forward consumes (already on the right device)."""
    input_ids: torch.Tensor  # [T] int64
    position_ids: torch.Tensor  # [T] int64
    cu_seqlens: torch.Tensor  # [n+1] int32 — boundaries of the *full* (un-split) sequences
    max_seqlen: int
    labels: Optional[torch.Tensor] = None  # [T] int64, pre-shifted, −100 = ignore
    # router replay: per layer [T, k] expert ids to force (reference moe/router_replay.py)
    routed_experts: Optional[List[torch.Tensor]] = None
    inputs_embeds: Optional[torch.Tensor] = None
    seq_lens: Optional[List[int]] = None  # full (un-split) sequence lengths on the host; needed by context parallelism
    # (cos, sin) of the whole row; set by the model forward when the Ulysses strategy scatters heads inside the q|k|v
    # projection, because q/k-norm and RoPE then run after the exchange on all tokens of this rank's heads
    rope_full: Optional[tuple] = None
    # (cos, sin) from the rotary base of sliding-window layers, for families that give those layers their own (Gemma-3)
    rope_local: Optional[tuple] = None
    # vision-language: flat patches of every image in the batch (in token order) and their (t, h, w) patch grids; the
    # tower's output replaces the embeddings of the image placeholder tokens. position_ids is then [3, T].
    pixel_values: Optional[torch.Tensor] = None
    image_grid_thw: Optional[torch.Tensor] = None
    # (row indices of the placeholder tokens, features per early layer) — set by ``embed`` for towers with deep-stack outputs
    deepstack: Optional[tuple] = None
    # under sequence / context parallelism: rows of the tower's output that belong to this rank's placeholder tokens
    vision_rows: Optional[torch.Tensor] = None


class Attention(nn.Module):

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        h, d = cfg.hidden_size, cfg.head_dim
        self.hq, self.hkv, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, d
        # output gate (Qwen3.5, reference HF ``Qwen3_5Attention``): a second q-sized projection whose sigmoid scales the
        # attention output per head and dim; kept as a fourth part of the fused projection, after q | k | v
        self.gated = bool(cfg.attn_output_gate)
        parts = [('q_proj', cfg.q_size), ('k_proj', cfg.kv_size), ('v_proj', cfg.kv_size)] + ([('q_gate', cfg.q_size)] if self.gated else [])
        self.qkv_proj = Linear(h, sum(n for _, n in parts), bias=cfg.attention_bias, parts=parts)
        if self.gated:
            self.qkv_proj.gate_head_dim = d
        self.o_proj = Linear(cfg.q_size, h, bias=cfg.o_proj_bias, name='o_proj')
        # GPT-OSS: one learned logit per head that joins the softmax without a value (an always-available place for attention mass)
        self.sinks = nn.Parameter(torch.zeros(cfg.num_attention_heads)) if cfg.attn_sinks else None
        # the per-head norms follow the model's norm convention ("1 + w" for Qwen3.5; plain weights have offset 0)
        self.norm_offset = float(cfg.rms_norm_offset) if cfg.qk_norm else 0.0
        self.qk_norm_full = bool(cfg.qk_norm and cfg.qk_norm_full)       # OLMo-2: one norm over all heads of the projection
        if self.qk_norm_full:
            self.q_norm = RMSNorm(cfg.q_size, cfg.rms_norm_eps, self.norm_offset)
            self.k_norm = RMSNorm(cfg.kv_size, cfg.rms_norm_eps, self.norm_offset)
        elif cfg.qk_norm:
            self.q_norm = RMSNorm(d, cfg.rms_norm_eps, self.norm_offset)
            self.k_norm = RMSNorm(d, cfg.rms_norm_eps, self.norm_offset)
        else:
            self.q_norm = self.k_norm = None
        self.attn_parallel = None  # Ulysses strategy or None
        self.scale = cfg.attn_scale
        self.window = cfg.layer_window(layer_idx)          # sliding-window layers see the last ``window`` keys only
        self.softcap = cfg.attn_logit_softcapping
        self.local_rope = bool(cfg.rope_local_theta) and self.window is not None     # Gemma-3: these layers rotate with their own base
        self.use_rope = not (cfg.no_rope_layers and not cfg.no_rope_layers[layer_idx])   # SmolLM3 leaves position out of some layers

    def heads(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """Fused projection output → ``(q [T,Hq,D], k [T,Hkv,D], v [T,Hkv,D], gate [T,Hq·D] | None)`` after the per-head
        norms and the rotary embedding (head counts are this rank's under tensor parallelism)."""
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        if not self.use_rope:          # the identity rotation
            cos, sin = torch.ones_like(cos), torch.zeros_like(sin)
        gate = None
        if self.gated:
            w = (self.hq + 2 * self.hkv) * self.d
            qkv, gate = qkv[:, :w], qkv[:, w:]
        if self.qk_norm_full:
            q, k, v = qkv.split([self.hq * self.d, self.hkv * self.d, self.hkv * self.d], dim=-1)
            qkv, qw, kw = torch.cat([self.q_norm(q.contiguous()), self.k_norm(k.contiguous()), v], -1), None, None
        q, k, v = ops.qkv_norm_rope(qkv, qw, kw, cos, sin, self.hq, self.hkv, self.d, self.cfg.rms_norm_eps, self.norm_offset)
        return q, k, v, gate

    def heads_from(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        return self.heads(self.qkv_proj(x), cos, sin)

    def _plain(self, max_seqlen: int) -> bool:
        """Whether this layer is ordinary causal attention for rows up to ``max_seqlen`` (what the sequence-parallel
        strategies and the fused paths compute)."""
        return not self.softcap and self.sinks is None and (self.window is None or self.window >= int(max_seqlen))

    @staticmethod
    def cache_entry(k: torch.Tensor, v: torch.Tensor):
        return k, v

    def project_out(self, o: torch.Tensor, gate: Optional[torch.Tensor]) -> torch.Tensor:
        o = o.reshape(o.shape[0], -1)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.o_proj(o)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, batch: PackedBatch,
                kv_sink=None) -> torch.Tensor:
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        ap = self.attn_parallel
        if (ap is not None and getattr(batch, 'rope_full', None) is not None and kv_sink is None and hasattr(ap, 'project_scatter')
                and not self.gated and self.norm_offset == 0.0 and self._plain(batch.max_seqlen) and not self.local_rope and not self.qk_norm_full and self.use_rope):
            # projection whose epilogue already delivers [T_full, (Hq + 2 Hkv)/sp · D] to every peer
            qkv_full = ap.project_scatter(x, self.qkv_proj, self.hq, self.hkv, self.d)
            if qkv_full is not None:
                q, k, v = ops.qkv_norm_rope(qkv_full, qw, kw, batch.rope_full[0], batch.rope_full[1], self.hq // ap.sp, self.hkv // ap.sp,
                                            self.d, self.cfg.rms_norm_eps)
                o = ops.flash_attn_varlen(q, k, v, batch.cu_seqlens, batch.max_seqlen, True, self.scale)
                o = ap.gather_heads(o)
                return self.o_proj(o.reshape(o.shape[0], -1))
        if self.local_rope:
            cos, sin = batch.rope_local
        q, k, v, gate = self.heads(self.qkv_proj(x), cos, sin)
        if kv_sink is not None:  # sampler prefill: keep K/V for the paged cache
            kv_sink(self.layer_idx, k, v)
        if ap is not None and not self._plain(batch.max_seqlen):
            raise NotImplementedError('sliding-window / soft-capped / sink attention layers are not wired to the sequence-parallel attention '
                                      'strategies; use data, sharded-data or pipeline parallelism, or rows no longer than the window')
        if ap is not None and hasattr(ap, 'attention'):  # context parallel: zig-zag local chunks against gathered keys
            o = ap.attention(q, k, v, batch.seq_lens, self.scale)
            return self.project_out(o, gate)
        if ap is not None:
            q, k, v = ap.scatter_heads(q, k, v)  # [T_local,H,D] → [T_full,H/sp,D]
        o = ops.flash_attn_varlen(q, k, v, batch.cu_seqlens, batch.max_seqlen, True, self.scale, window=self.window, softcap=self.softcap,
                                  sinks=self.sinks)
        if ap is not None:
            o = ap.gather_heads(o)  # back to [T_local, Hq, D]
        return self.project_out(o, gate)   # the gate is per token of this rank: applied after the heads are back


class MLAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V2 / V3; Hugging Face ``DeepseekV3Attention``).  Queries come through a
    low-rank bottleneck with a norm in the middle (or a plain projection), keys and values are expanded from one normalised
    latent per token, and the rotary part of the key is a single head shared by all query heads.  Scores use the
    ``qk_nope + qk_rope`` wide heads, values are ``v_head_dim`` wide, so this block runs the generic packed attention
    (``ops.flash_attn_varlen`` routes widths other than 128 to its PyTorch form)."""

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        h, nh = cfg.hidden_size, cfg.num_attention_heads
        self.nh, self.nope, self.rope, self.vd = nh, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        qk = self.nope + self.rope
        if cfg.q_lora_rank:
            self.q_a_proj = Linear(h, cfg.q_lora_rank, bias=cfg.attention_bias, name='q_a_proj')
            self.q_a_layernorm = RMSNorm(cfg.q_lora_rank, cfg.rms_norm_eps)
            self.q_b_proj = Linear(cfg.q_lora_rank, nh * qk, name='q_b_proj')
            self.q_proj = None
        else:
            self.q_proj = Linear(h, nh * qk, name='q_proj')
            self.q_a_proj = self.q_a_layernorm = self.q_b_proj = None
        self.kv_a_proj_with_mqa = Linear(h, cfg.kv_lora_rank + self.rope, bias=cfg.attention_bias, name='kv_a_proj_with_mqa')
        self.kv_a_layernorm = RMSNorm(cfg.kv_lora_rank, cfg.rms_norm_eps)
        self.kv_b_proj = Linear(cfg.kv_lora_rank, nh * (self.nope + self.vd), name='kv_b_proj')
        self.o_proj = Linear(nh * self.vd, h, bias=cfg.attention_bias, name='o_proj')
        self.attn_parallel = None
        self.scale = cfg.attn_scale

    def _rotate(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        if self.cfg.mla_rope_interleave:     # checkpoint pairs are (2i, 2i+1): bring them to (i, i + R/2) first
            x = x.reshape(*x.shape[:-1], self.rope // 2, 2).transpose(-1, -2).reshape(x.shape)
        return ops.ref.apply_rope(x, cos, sin)

    def heads_from(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """Layer input → ``(q [T,H,Dqk], k [T,H,Dqk], v [T,H,Dv], None)`` with the rotary part applied."""
        T = x.shape[0]
        q = self.q_proj(x) if self.q_proj is not None else self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        q = q.view(T, self.nh, self.nope + self.rope)
        ckv = self.kv_a_proj_with_mqa(x)
        latent, k_rot = ckv[:, :self.cfg.kv_lora_rank], ckv[:, self.cfg.kv_lora_rank:]
        kv = self.kv_b_proj(self.kv_a_layernorm(latent.contiguous())).view(T, self.nh, self.nope + self.vd)
        q_rot = self._rotate(q[..., self.nope:], cos, sin)
        k_rot = self._rotate(k_rot.reshape(T, 1, self.rope), cos, sin).expand(T, self.nh, self.rope)
        return torch.cat([q[..., :self.nope], q_rot], -1), torch.cat([kv[..., :self.nope], k_rot], -1), kv[..., self.nope:], None

    def cache_entry(self, k: torch.Tensor, v: torch.Tensor):
        """Keys and values as the paged cache keeps them: one width for both, values zero-padded to the score width."""
        return k, F.pad(v, (0, k.shape[-1] - v.shape[-1]))

    def project_out(self, o: torch.Tensor, gate=None) -> torch.Tensor:
        return self.o_proj(o[..., :self.vd].reshape(o.shape[0], self.nh * self.vd))

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, batch: PackedBatch, kv_sink=None) -> torch.Tensor:
        if self.attn_parallel is not None:
            raise NotImplementedError('multi-head latent attention is not wired to the sequence-parallel attention strategies '
                                      '(unequal key / value widths); use data, sharded-data, expert or pipeline parallelism')
        q, k, v, _ = self.heads_from(x, cos, sin)
        if kv_sink is not None:
            kv_sink(self.layer_idx, *self.cache_entry(k, v))
        o = ops.flash_attn_varlen(q, k, v, batch.cu_seqlens, batch.max_seqlen, True, self.scale)
        return self.project_out(o)


class MLP(nn.Module):

    def __init__(self, cfg: DecoderConfig, intermediate: Optional[int] = None):
        super().__init__()
        i = intermediate or cfg.intermediate_size
        self.gate_up_proj = Linear(cfg.hidden_size, 2 * i, parts=[('gate_proj', i), ('up_proj', i)])
        self.down_proj = Linear(i, cfg.hidden_size, name='down_proj')
        self.act = ops.geglu if cfg.hidden_act.startswith('gelu') else ops.swiglu

    def forward(self, x: torch.Tensor, value_unused: bool = True) -> torch.Tensor:
        """``value_unused=True`` (the block's output only feeds the residual add) lets a recompute pass skip the last GEMM;
        callers that multiply or otherwise read the output pass ``False``."""
        return self.down_proj(self.act(self.gate_up_proj(x)), value_unused=value_unused)


class Experts(nn.Module):
    """Fused expert weights ``gate_up_proj [E, 2I, H]`` and ``down_proj [E, H, I]``
    (local experts only under expert parallelism), with an optional per-expert
    LoRA pool ``A [S, E, R, in]`` / ``B [S, E, out, R]`` (reference
    ``model/multi_lora_target_parameters.py:38-118``)."""

    def __init__(self, cfg: DecoderConfig, num_local: Optional[int] = None):
        super().__init__()
        e = num_local if num_local is not None else cfg.num_experts
        self.num_local, self.first_expert = e, 0
        self.gate_up_proj = nn.Parameter(torch.empty(e, 2 * cfg.moe_intermediate_size, cfg.hidden_size))
        self.down_proj = nn.Parameter(torch.empty(e, cfg.hidden_size, cfg.moe_intermediate_size))
        if cfg.expert_bias:
            self.gate_up_bias = nn.Parameter(torch.zeros(e, 2 * cfg.moe_intermediate_size))
            self.down_bias = nn.Parameter(torch.zeros(e, cfg.hidden_size))
        else:
            self.gate_up_bias = self.down_bias = None
        self.act = ops.ref.clamped_glu if cfg.expert_act == 'clamped_glu' else ops.swiglu
        self.lora = nn.ParameterDict()
        self.max_loras = 0

    def add_lora_pool(self, max_loras: int, max_r: int) -> None:
        e, two_i, h = self.gate_up_proj.shape
        i = two_i // 2
        dev, dt = self.gate_up_proj.device, self.gate_up_proj.dtype
        self.max_loras, self.max_r = max_loras, max_r

        def mk_a(inp):
            a = torch.empty(max_loras, e, max_r, inp, device=dev, dtype=dt)
            nn.init.kaiming_uniform_(a.view(-1, inp), a=math.sqrt(5))
            return nn.Parameter(a)

        self.lora['gate_up_A'] = mk_a(h)
        self.lora['gate_up_B'] = nn.Parameter(torch.zeros(max_loras, e, two_i, max_r, device=dev, dtype=dt))
        self.lora['down_A'] = mk_a(i)
        self.lora['down_B'] = nn.Parameter(torch.zeros(max_loras, e, h, max_r, device=dev, dtype=dt))

    def _expert_lora(self, which: str):
        """(A [E, r, in], B [E, out, r], scale) of the tenant active in this forward, or None."""
        from .layers import current_lora_batch
        lb = current_lora_batch()
        if lb is None or self.max_loras == 0:
            return None
        active = [i for i, h in enumerate(lb.host) if h[2] >= 0]
        if not active:
            return None
        if len({lb.host[i][2] for i in active}) > 1:
            raise NotImplementedError('expert LoRA serves one tenant per forward; token-level tenants mix only in dense linears')
        i = active[0]
        _, _, slot, r, scale = lb.host[i]
        t = lb.targets[i] if lb.targets else None
        if t is not None and not t.matches('mlp.experts.' + which, which):
            return None
        if r == 0:
            return None
        return self.lora[which + '_A'][slot, :, :r], self.lora[which + '_B'][slot, :, :, :r], scale

    def forward(self, x_sorted: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        """``x_sorted`` rows grouped by local expert; ``offsets [E_local+1]``."""
        lo = self._expert_lora('gate_up')
        gu = ops.expert_linear(x_sorted, self.gate_up_proj, offsets, *(lo or ()))
        row_expert = None
        if self.gate_up_bias is not None:
            # expert of every row of the grouped layout (rows that pad a segment get their segment's bias and are never read)
            row_expert = torch.bucketize(torch.arange(x_sorted.shape[0], device=x_sorted.device), offsets[1:].to(torch.long), right=True)
            row_expert = row_expert.clamp_(max=self.gate_up_proj.shape[0] - 1)
            gu = gu + self.gate_up_bias[row_expert].to(gu.dtype)
        act = self.act(gu)
        lo = self._expert_lora('down')
        y = ops.expert_linear(act, self.down_proj, offsets, *(lo or ()))
        return y if row_expert is None else y + self.down_bias[row_expert].to(y.dtype)


class MoEBlock(nn.Module):
    """Router → top-k → (dispatch) → grouped experts → (combine) → weighted sum."""

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.gate = Linear(cfg.hidden_size, cfg.num_experts, bias=cfg.router_linear_bias, name='gate')
        self.experts = Experts(cfg)
        # an always-on expert beside the routed ones, scaled per token by a sigmoid gate (Qwen2-MoE / Qwen3-Next style);
        # replicated under expert parallelism (reference ``moe/expert_parallel.py:329-382``)
        if cfg.shared_expert_intermediate_size > 0:
            self.shared_expert = MLP(cfg, cfg.shared_expert_intermediate_size)
            self.shared_expert_gate = Linear(cfg.hidden_size, 1, name='shared_expert_gate') if cfg.shared_expert_gate else None
        else:
            self.shared_expert = self.shared_expert_gate = None
        # DeepSeek-V3: a per-expert bias that steers the selection only (balanced by a rule outside the loss, never by a gradient)
        self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.num_experts), requires_grad=False) if cfg.router_bias else None
        self.moe_parallel = None  # expert-parallel strategy or None
        self.etp = None           # tensor-parallel context when every expert is split over the tensor-parallel group
        self.last_routed: Optional[torch.Tensor] = None
        self.last_aux: Optional[torch.Tensor] = None
        self.record_routing = False

    def route(self, x: torch.Tensor, forced: Optional[torch.Tensor]):
        if self.cfg.router_scoring == 'topk_softmax':      # GPT-OSS: the k largest logits, then a softmax over just those
            logits = self.gate(x).float()
            top, idx = logits.topk(self.cfg.num_experts_per_tok, dim=-1)
            if forced is not None:
                idx = torch.where(forced[:, :1] < 0, idx, forced.long())
                top = logits.gather(1, idx)
            self._hist = None
            return torch.softmax(top, -1), idx, torch.softmax(logits, -1)
        if self.cfg.router_scoring != 'softmax':
            return self._route_sigmoid(x, forced)
        w, idx, probs, self._hist = ops.moe_router(self.gate(x), self.cfg.num_experts_per_tok, self.cfg.norm_topk_prob, forced)
        return w, idx, probs

    def _route_sigmoid(self, x: torch.Tensor, forced: Optional[torch.Tensor]):
        """DeepSeek-V3 routing (Hugging Face ``DeepseekV3MoE.route_tokens_to_experts``): sigmoid scores; the choice is made
        on scores plus the selection bias, restricted to the ``topk_group`` expert groups whose two best biased scores sum
        highest; the weights are the unbiased scores of the chosen experts, normalised and scaled."""
        cfg = self.cfg
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        logits = F.linear(x.float(), self.gate.weight.float())
        v2 = cfg.router_scoring == 'softmax_grouped'        # DeepSeek-V2: softmax scores, a group is as good as its best expert
        scores = torch.softmax(logits, -1) if v2 else torch.sigmoid(logits)
        choice = scores + self.e_score_correction_bias.float() if self.e_score_correction_bias is not None else scores
        if cfg.n_group > 1:
            grouped = choice.view(-1, cfg.n_group, E // cfg.n_group)
            rank = grouped.max(-1)[0] if v2 else grouped.topk(2, dim=-1)[0].sum(-1)
            best = rank.topk(cfg.topk_group, dim=-1, sorted=False)[1]
            keep = torch.zeros_like(grouped[..., 0]).scatter_(1, best, 1.0).bool()
            choice = grouped.masked_fill(~keep[..., None], 0.0).reshape(-1, E)
        idx = choice.topk(k, dim=-1, sorted=False)[1]
        if forced is not None:
            idx = torch.where(forced[:, :1] < 0, idx, forced.long())
        w = scores.gather(1, idx)
        if cfg.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        self._hist = None
        return w * cfg.routed_scaling_factor, idx, scores

    def forward(self, x: torch.Tensor, forced: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, H = x.shape
        k, E = self.cfg.num_experts_per_tok, self.cfg.num_experts
        w, idx, probs = self.route(x, forced)
        if self.record_routing:
            self.last_routed = idx.detach()
        if self.cfg.router_aux_loss_coef > 0 and torch.is_grad_enabled():
            self.last_aux = ops.ref.moe_aux_loss(probs, idx, E)
        if self.etp is not None:
            return self._with_shared(x, self._forward_expert_tp(x, w, idx))
        mp = self.moe_parallel
        if mp is not None:
            return self._with_shared(x, mp.forward(self, x, w, idx))
        return self._with_shared(x, self._routed_local(x, w, idx))

    def _forward_expert_tp(self, x, w, idx):
        """Expert tensor parallelism (reference ``megatron/strategy/megatron.py:90-107``: ``expert_tensor_parallel_size``):
        every rank of the group holds ``1/tp`` of each expert's intermediate dimension, so it needs every token of the
        group and produces a partial sum of every token's output.  Routing stays where the tokens are (the router's
        gradient is then summed like that of any other replicated tensor); the routing *results* travel with the tokens."""
        tp = self.etp
        xf, wf = tp.before_column(x), tp.before_column(w)
        idxf = tp.comm.all_gather_tensor(idx.contiguous()) if tp.sp else idx
        mp = self.moe_parallel
        if mp is not None:
            self._hist = None       # the histogram was taken over this rank's tokens only
            part = mp.forward(self, xf, wf, idxf)
        else:
            self._hist = None
            part = self._routed_local(xf, wf, idxf)
        return tp.after_row(part)

    def _routed_local(self, x, w, idx):
        T, H = x.shape
        k, E = self.cfg.num_experts_per_tok, self.cfg.num_experts
        # local: expert-sorted layout whose segments start on 128-row boundaries (grouped GEMM tiles and the
        # per-expert wgrad reduction ranges then never straddle two experts); padding rows are zero.  Dispatch and
        # combine are gathers through index maps built on the device — no host read anywhere in the block.
        from ..parallel.expert import expert_layout
        order, rows, offsets, bound = expert_layout(idx.reshape(-1), E, 128 if x.is_cuda else 1, self._hist)
        row_of, src_tok, slot_of_row = ops.moe_index_maps(order, rows, bound, k)
        xs = ops.moe_dispatch(x, src_tok, row_of)
        y = self.experts(xs, offsets)
        return ops.moe_combine(y, w, row_of, src_tok, slot_of_row)

    def _with_shared(self, x: torch.Tensor, routed: torch.Tensor) -> torch.Tensor:
        if self.shared_expert is None:
            return routed
        if self.shared_expert_gate is None:
            return routed + self.shared_expert(x, value_unused=False)
        gate = torch.sigmoid(self.shared_expert_gate(x).float()).to(x.dtype)
        return routed + gate * self.shared_expert(x, value_unused=False)


class DecoderLayer(nn.Module):

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.rms_norm_offset) if cfg.pre_norm else None
        self.is_linear = bool(cfg.layer_types) and cfg.layer_types[layer_idx] == 'linear_attention'
        if self.is_linear:
            from .linear_attention import GatedDeltaNet
            self.self_attn = GatedDeltaNet(cfg.hidden_size, cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim,
                                           cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim, cfg.rms_norm_eps)
        else:
            self.self_attn = MLAttention(cfg, layer_idx) if cfg.is_mla else Attention(cfg, layer_idx)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.rms_norm_offset) if cfg.pre_norm else None
        self.is_moe = cfg.layer_is_moe(layer_idx)          # DeepSeek keeps a dense block in its first layers
        self.residual_multiplier = float(cfg.residual_multiplier)
        self.first_moe_layer = cfg.first_k_dense_replace      # recorded routing lists have one entry per mixture-of-experts layer
        self.mlp = MoEBlock(cfg, layer_idx) if self.is_moe else MLP(cfg)
        # GLM-4: each sub-layer's output is normalised before it joins the residual stream
        if cfg.sandwich_norm:
            self.post_self_attn_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.rms_norm_offset)
            self.post_mlp_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.rms_norm_offset)
        else:
            self.post_self_attn_layernorm = self.post_mlp_layernorm = None

    def forward(self, x: torch.Tensor, cos, sin, batch: PackedBatch, kv_sink=None) -> torch.Tensor:
        if self.is_linear:
            lin = getattr(kv_sink, 'linear_state', None) if kv_sink is not None else None  # sampler prefill: keep conv tail + state
            if kv_sink is not None and lin is None:
                raise NotImplementedError('this kv_sink does not take linear-attention state (give it a linear_state attribute)')
            sink = (lambda conv, st: lin(self.layer_idx, conv, st)) if lin is not None else None
            a = self.self_attn(self.pre(x), batch.cu_seqlens, state_sink=sink)
        else:
            a = self.self_attn(self.pre(x), cos, sin, batch, kv_sink)
        n, h = self.after_attention(x, a)
        forced = batch.routed_experts[self.layer_idx - self.first_moe_layer] if (self.is_moe and batch.routed_experts is not None) else None
        return ops.add(h, self.feed_forward(n, forced), value_unused=True)

    def pre(self, x: torch.Tensor) -> torch.Tensor:
        """Input of the token mixer: the normalised stream, or the stream itself in stacks that only norm sub-layer outputs."""
        return self.input_layernorm(x) if self.input_layernorm is not None else x

    def after_attention(self, x: torch.Tensor, a: torch.Tensor):
        """Token-mixer output ``a`` joins the residual stream ``x``: ``(input of the feed-forward block, new residual)``."""
        if self.post_self_attn_layernorm is not None:
            a = self.post_self_attn_layernorm(a)
        if self.residual_multiplier != 1.0:
            a = a * self.residual_multiplier
        if self.post_attention_layernorm is None:       # no norm in front of the feed-forward block either
            h = ops.add(x, a)
            return h, h
        return self.post_attention_layernorm.forward_add(a, x)

    def feed_forward(self, n: torch.Tensor, forced=None) -> torch.Tensor:
        """What the feed-forward block adds to the residual stream."""
        if self.is_moe:
            m = self.mlp(n, forced)
        else:
            m = self.mlp(n, value_unused=self.post_mlp_layernorm is None and self.residual_multiplier == 1.0)   # a following norm or factor reads the value
        m = self.post_mlp_layernorm(m) if self.post_mlp_layernorm is not None else m
        return m * self.residual_multiplier if self.residual_multiplier != 1.0 else m


class DecoderModel(nn.Module):
    """Embedding → N layers → final norm → (lm_head).  ``forward`` returns the
    final hidden states; log-probs are formed by ``token_logprobs`` through the
    fused lm_head + log-softmax kernel so logits are only built on request."""

    def __init__(self, cfg: DecoderConfig, layer_range: Optional[Tuple[int, int]] = None, has_embed: bool = True,
                 has_head: bool = True):
        super().__init__()
        self.cfg = cfg
        lo, hi = layer_range or (0, cfg.num_hidden_layers)
        self.layer_range = (lo, hi)
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size) if has_embed else None
        self.layers = nn.ModuleList([DecoderLayer(cfg, i) for i in range(lo, hi)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.rms_norm_offset) if has_head else None
        if has_head and not cfg.tie_word_embeddings:
            self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, name='lm_head')
        else:
            self.lm_head = None
        self.has_head = has_head
        if cfg.vision and has_embed:
            from .vision import VisionConfig, VisionTower
            self.visual = VisionTower(VisionConfig.from_hf(cfg.vision))
        else:
            self.visual = None
        for name, m in self.named_modules():
            if isinstance(m, Linear):
                m.full_name = name
        self.layer_runner = None  # engine hook: runs one layer (checkpoint / FSDP unshard)
        self.tp = None  # tensor-parallel context, set by parallel.tensor.apply_tensor_parallel

    # --------------------------------------------------------------- init
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: Optional[float] = None) -> None:
        """N(0, initializer_range) for matrices, ones for norms; the generator is
        per-parameter-name so any sharding of the same model yields identical values."""
        std = std or self.cfg.initializer_range
        from ..utils.seed import stable_seed
        for name, p in self.named_parameters():
            if 'lora_' in name or name.startswith('lora'):
                continue
            if name.endswith(('bias', 'sinks')):       # also the per-expert bias matrices
                p.zero_()
                continue
            if p.dim() == 1:
                if name.endswith('bias'):
                    p.zero_()
                else:
                    p.fill_(1.0 if self.cfg.rms_norm_offset == 0.0 else 0.0)
                continue
            g = torch.Generator(device='cpu').manual_seed(stable_seed(seed, name))
            if p.numel() <= 2**24 or p.device.type == 'cpu':
                p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std))
            else:  # large matrices: draw on the device, still deterministic per name
                gd = torch.Generator(device=p.device).manual_seed(stable_seed(seed, name))
                p.normal_(0.0, std, generator=gd)

    def head_weight(self) -> torch.Tensor:
        return self.lm_head.weight if self.lm_head is not None else self.embed_tokens.weight

    # ------------------------------------------------------------ forward
    def embed_ids(self, ids: torch.Tensor) -> torch.Tensor:
        """Token embeddings, times the family's factor (Gemma: √hidden, rounded to the embeddings' dtype first)."""
        if self.tp is not None:
            from ..parallel.tensor import vocab_parallel_embedding
            x = vocab_parallel_embedding(ids, self.embed_tokens.weight, self.tp)
        else:
            x = self.embed_tokens(ids)
        if self.cfg.embed_scale != 1.0:
            x = x * torch.tensor(self.cfg.embed_scale, dtype=x.dtype, device=x.device)
        return x

    def embed(self, batch: PackedBatch) -> torch.Tensor:
        if batch.inputs_embeds is not None:
            return batch.inputs_embeds
        x = self.embed_ids(batch.input_ids)
        if batch.pixel_values is not None and self.visual is not None:
            feats, deep = self.visual(batch.pixel_values, batch.image_grid_thw, return_deepstack=True)
            if batch.vision_rows is not None:
                feats, deep = feats[batch.vision_rows], [d[batch.vision_rows] for d in deep]
            where = batch.input_ids == self.cfg.image_token_id
            if self.cfg.video_token_id is not None:
                where = where | (batch.input_ids == self.cfg.video_token_id)
            if int(where.sum()) != feats.shape[0]:
                raise ValueError(f'{int(where.sum())} image placeholder tokens in the batch but the tower produced {feats.shape[0]} embeddings')
            x = x.masked_scatter(where[:, None], feats.to(x.dtype))
            batch.deepstack = (where.nonzero(as_tuple=True)[0], deep) if deep else None
        return x

    def forward(self, batch: PackedBatch, hidden: Optional[torch.Tensor] = None, kv_sink=None) -> torch.Tensor:
        x = self.embed(batch) if hidden is None else hidden
        if batch.position_ids.dim() == 2:  # [3, T] (time, height, width) positions of a vision-language batch
            from .vision import mrope_tables
            cos, sin = mrope_tables(batch.position_ids, self.cfg.rotary_dim, self.cfg.rope_theta, self.cfg.mrope_section, self.cfg.mrope_interleaved)
        else:
            cos, sin = ops.rope_tables(batch.position_ids, self.cfg.rotary_dim, self.cfg.rope_theta, self.cfg.rope_scaling)
        if self.cfg.rope_local_theta:
            batch.rope_local = ops.rope_tables(batch.position_ids, self.cfg.rotary_dim, self.cfg.rope_local_theta, None)
        full = None
        for layer in self.layers:
            ap = getattr(getattr(layer, 'self_attn', None), 'attn_parallel', None)
            if ap is not None and hasattr(ap, 'full_rope') and not getattr(layer, 'is_linear', False):
                full = ap.full_rope(cos, sin)  # None unless the fused projection + exchange is in use
                break
        if full is not None or getattr(batch, 'rope_full', None) is not None:
            batch.rope_full = full
        run = self.layer_runner
        for layer in self.layers:
            if run is not None:
                x = run(layer, x, cos, sin, batch)
            else:
                x = layer(x, cos, sin, batch, kv_sink)
            ds = batch.deepstack
            if ds is not None and layer.layer_idx < len(ds[1]):  # deep stack: the tower's early features join the first layers' outputs
                x = x.index_add(0, ds[0], ds[1][layer.layer_idx].to(x.dtype))
        if self.norm is not None:
            x = self.norm(x)
        return x

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        z = ops.linear(hidden, self.head_weight())
        if self.cfg.logits_scaling != 1.0:
            z = z / self.cfg.logits_scaling
        cap = self.cfg.final_logit_softcapping
        return torch.tanh(z / cap) * cap if cap else z

    def token_logprobs(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                       with_entropy: bool = False):
        """(logps [T] fp32, entropies|None) with ignored labels (−100) read as id 0."""
        safe = labels.clamp_min(0)
        if self.cfg.final_logit_softcapping:
            # capped logits (Gemma-2) are outside the fused head kernel: rows in chunks through the PyTorch form
            lps, ents = [], []
            for lo in range(0, hidden.shape[0], 4096):
                lp, en = ops.ref.logprob_from_logits(self.logits(hidden[lo:lo + 4096]), safe[lo:lo + 4096], temperature, with_entropy)
                lps.append(lp)
                ents.append(en)
            return torch.cat(lps), (torch.cat(ents) if with_entropy else None)
        temperature = temperature * self.cfg.logits_scaling      # Granite divides its logits by a constant: the same thing as a temperature
        if self.tp is not None:
            from ..parallel.tensor import CopyToTP, GatherTokens, vocab_parallel_logprob
            # backward of either op sums the per-vocabulary-shard partial gradients of the hidden states
            hidden = GatherTokens.apply(hidden, self.tp.comm) if self.tp.sp else CopyToTP.apply(hidden, self.tp.comm)
            return vocab_parallel_logprob(hidden, self.head_weight(), safe, self.tp, temperature), None
        hw = self.head_weight()
        # an untied head is a Linear weight: its dW chunks can go straight into the engine's fp32 gradient buffer (a bf16
        # buffer is not used this way: the chunks are summed in fp32 first)
        wgrad_out = getattr(hw, '_wgrad_out', None) if (hw.requires_grad and getattr(hw, '_direct_wgrad', False)) else None
        if wgrad_out is not None and wgrad_out.dtype != torch.float32:
            wgrad_out = None
        return ops.fused_linear_logprob(hidden, hw, safe, temperature, with_entropy, wgrad_out=wgrad_out)

    def aux_loss(self) -> Optional[torch.Tensor]:
        terms = [l.mlp.last_aux for l in self.layers if getattr(l, 'is_moe', False) and l.mlp.last_aux is not None]
        if not terms:
            return None
        for l in self.layers:
            if getattr(l, 'is_moe', False):
                l.mlp.last_aux = None
        return torch.stack(terms).mean() * self.cfg.router_aux_loss_coef

    def collect_routed_experts(self) -> Optional[List[torch.Tensor]]:
        out = [l.mlp.last_routed for l in self.layers if getattr(l, 'is_moe', False)]
        return out if out and all(o is not None for o in out) else None

    def set_record_routing(self, on: bool) -> None:
        for l in self.layers:
            if getattr(l, 'is_moe', False):
                l.mlp.record_routing = on

    def lora_modules(self) -> List[Tuple[str, nn.Module]]:
        return [(n, m) for n, m in self.named_modules() if isinstance(m, (Linear, Experts))]


def build_model(cfg: DecoderConfig, device='cpu', dtype=torch.float32, seed: int = 0, init: bool = True,
                **kw) -> DecoderModel:
    with torch.device(device):
        model = DecoderModel(cfg, **kw)
    model.to(dtype)
    if init:
        model.init_weights(seed)
    return model
