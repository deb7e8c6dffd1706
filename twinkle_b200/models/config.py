"""Architecture description of the owned decoder family.

One config class covers Qwen3 dense, Qwen3-MoE and Llama/Qwen2-style decoders
(q/k-norm optional, attention bias optional).  ``from_hf`` reads a Hugging Face
``config.json`` dict; ``to_hf`` writes one back, so checkpoints stay loadable by
``transformers``.  Presets are the benchmark architectures with random init.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import List, Any, Dict, Optional


# config.json ``model_type`` values whose layer maths is what ``models/decoder.py`` computes (each checked against transformers)
SUPPORTED_MODEL_TYPES = frozenset({'llama', 'mistral', 'mixtral', 'qwen2', 'qwen2_moe', 'qwen3', 'qwen3_moe', 'seed_oss', 'qwen2_vl', 'qwen2_vl_text',
                                   'qwen2_5_vl', 'qwen2_5_vl_text', 'qwen3_vl', 'qwen3_vl_text', 'qwen3_vl_moe', 'qwen3_vl_moe_text',
                                   'qwen3_5', 'qwen3_5_text', 'qwen3_5_moe', 'qwen3_5_moe_text', 'qwen3_next', 'glm', 'glm4',
                                   'phi3', 'internlm2', 'internlm3', 'gemma', 'deepseek_v2', 'deepseek_v3', 'kimi_k2', 'glm4_moe', 'gemma2', 'gemma3_text', 'gemma3', 'gpt_oss', 'granite', 'olmo2', 'olmo3', 'ernie4_5', 'smollm3'})


def _rope_scaling_of(cfg: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    """``rope_scaling`` (or the newer ``rope_parameters``) of a HF config when it describes a long-context variant."""
    rs = cfg.get('rope_scaling') or cfg.get('rope_parameters')
    if not isinstance(rs, dict):
        return None
    kind = rs.get('rope_type', rs.get('type', 'default'))
    if kind in (None, 'default', 'mrope'):  # mrope is a position layout (see DecoderConfig.mrope_section), not a frequency change
        return None
    out = {k: v for k, v in rs.items() if k != 'rope_theta'}
    out.setdefault('rope_type', kind)
    if kind in ('llama3', 'yarn', 'longrope') and not out.get('original_max_position_embeddings'):
        out['original_max_position_embeddings'] = cfg.get('original_max_position_embeddings') or cfg.get('max_position_embeddings', 4096)
    if kind in ('dynamic', 'longrope'):      # these two compare the sequence length with the model's window
        out.setdefault('max_position_embeddings', cfg.get('max_position_embeddings', 4096))
    out.pop('partial_rotary_factor', None)
    return out


@dataclass
class DecoderConfig:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: Optional[Dict[str, Any]] = None  # HF mapping: {'rope_type': 'llama3' | 'yarn' | 'linear', 'factor': …}
    tie_word_embeddings: bool = False
    qk_norm: bool = True
    attention_bias: bool = False
    rms_norm_offset: float = 0.0  # 1.0 for gemma-style "1 + w"
    # Qwen3.5 full-attention layers: rotary embedding on the leading ``head_dim * partial_rotary_factor`` dims only, and a
    # per-head sigmoid gate (a second half of the q projection) on the attention output; their q/k norms are "1 + w" too
    partial_rotary_factor: float = 1.0
    attn_output_gate: bool = False
    # GLM-4 family: the checkpoint's rotary pairs are (2i, 2i+1); the bridge permutes the q / k projection rows into the
    # (i, i + R/2) convention computed here (scores are unchanged by a common permutation of q and k dims), gate and up are
    # one fused tensor in the checkpoint, and ``glm4`` norms each sub-layer's output before the residual add
    rope_interleaved: bool = False
    sandwich_norm: bool = False
    # Gemma: gate activation of the feed-forward block ('silu' | 'gelu_pytorch_tanh') and the factor √hidden on the
    # token embeddings (rounded to the compute dtype, as the Hugging Face model forms it)
    hidden_act: str = 'silu'
    embed_scale: float = 1.0
    # attention window of checkpoints trained with one (Mistral-7B-v0.1, Phi-3-mini): rows longer than the window are
    # refused — every key inside the window is what the kernels here compute
    sliding_window: Optional[int] = None
    # Gemma-2 / Gemma-3: scores through ``cap · tanh(s / cap)``, output logits likewise; softmax scale ``query_pre_attn_scalar^-½``
    # instead of ``head_dim^-½``; sliding-window layers (``layer_types`` entries ``'sliding_attention'``) of Gemma-3 use a rotary
    # base of their own, without the long-context scaling of the global layers
    # GPT-OSS: a learned per-head sink logit in the attention softmax, biases on the output projection, the router and the expert
    # tensors, routing = softmax over the top-k router logits, experts with the clamped ``(up + 1) · gate · σ(1.702 · gate)`` unit
    # Granite: what each sub-layer adds to the residual stream is multiplied by ``residual_multiplier``, output logits are divided by
    # ``logits_scaling``, the softmax scale is ``attention_multiplier`` (kept in ``query_pre_attn_scalar`` as its inverse square)
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0
    # OLMo-2 / OLMo-3: no norm in front of a sub-layer, only the one on its output (``sandwich_norm`` without ``pre_norm``), and
    # q / k norms over the whole projection instead of per head
    pre_norm: bool = True
    qk_norm_full: bool = False
    # SmolLM3: per layer, 1 = rotary embedding as usual, 0 = no position information in that layer's attention
    no_rope_layers: Optional[List[int]] = None
    attn_sinks: bool = False
    o_proj_bias: bool = False
    router_linear_bias: bool = False
    expert_bias: bool = False
    expert_act: str = 'swiglu'
    attn_logit_softcapping: Optional[float] = None
    final_logit_softcapping: Optional[float] = None
    query_pre_attn_scalar: Optional[float] = None
    rope_local_theta: Optional[float] = None
    # MoE (num_experts == 0 → dense)
    num_experts: int = 0
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    shared_expert_intermediate_size: int = 0
    # DeepSeek-V3 style routing: sigmoid scores, a per-expert selection bias that is not trained by the loss, experts in
    # ``n_group`` groups of which the ``topk_group`` best (by their two best biased scores) stay eligible, weights scaled by
    # ``routed_scaling_factor``; the first ``first_k_dense_replace`` layers keep a dense feed-forward block; the shared
    # expert has no gate of its own
    router_scoring: str = 'softmax'
    router_bias: bool = False
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0
    shared_expert_gate: bool = True
    # multi-head latent attention (DeepSeek-V2/V3): queries through a rank-``q_lora_rank`` bottleneck (None = a plain
    # projection), keys / values expanded from one rank-``kv_lora_rank`` latent per token (0 = ordinary attention); a head's
    # query / key is ``qk_nope_head_dim`` position-free dims plus ``qk_rope_head_dim`` rotary dims whose key part is shared
    # by all heads; values are ``v_head_dim`` wide
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    mla_rope_interleave: bool = True
    initializer_range: float = 0.02
    model_type: str = 'qwen3'
    torch_dtype: str = 'bfloat16'
    max_position_embeddings: int = 40960
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    # hybrid stacks: per-layer 'full_attention' | 'linear_attention' (Gated DeltaNet); None = all full attention
    layer_types: Optional[List[str]] = None
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    # vision-language (Qwen2-VL family): the vision tower's config.json section, placeholder token ids, and the split of
    # the rotary half-dimension over (time, height, width) positions
    vision: Optional[Dict[str, Any]] = None
    image_token_id: Optional[int] = None
    video_token_id: Optional[int] = None
    vision_start_token_id: Optional[int] = None
    vision_end_token_id: Optional[int] = None
    mrope_section: Optional[List[int]] = None
    mrope_interleaved: bool = False  # Qwen3-VL lays the three position components out t h w t h w … instead of in blocks

    def __post_init__(self):
        if self.vision is not None:
            from .vision import VisionConfig
            self.vision = VisionConfig.from_hf(self.vision).to_hf()  # only the fields the tower uses, in the family's spelling

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    def layer_is_moe(self, layer_idx: int) -> bool:
        return self.num_experts > 0 and layer_idx >= self.first_k_dense_replace

    def layer_window(self, layer_idx: int) -> Optional[int]:
        """Attention window of a layer: the model's ``sliding_window`` on every layer, or only on those that ``layer_types``
        marks ``'sliding_attention'``."""
        if not self.sliding_window:
            return None
        if self.layer_types and 'sliding_attention' in self.layer_types:
            return self.sliding_window if self.layer_types[layer_idx] == 'sliding_attention' else None
        return self.sliding_window

    @property
    def attn_scale(self) -> float:
        """Softmax scale of the attention scores: ``1/√d`` of the query / key width; DeepSeek's YaRN variant multiplies
        it by the square of ``0.1·mscale_all_dim·ln(factor) + 1``."""
        if not self.is_mla:
            return float(self.query_pre_attn_scalar or self.head_dim)**-0.5
        sc = (self.qk_nope_head_dim + self.qk_rope_head_dim)**-0.5
        rs = self.rope_scaling or {}
        if rs.get('mscale_all_dim') and float(rs.get('factor', 1.0)) > 1.0 and self.model_type != 'deepseek_v2':
            m = 0.1 * float(rs['mscale_all_dim']) * math.log(float(rs['factor'])) + 1.0
            sc = sc * m * m
        return sc

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def _attn_weights(self) -> int:
        h, nh = self.hidden_size, self.num_attention_heads
        if self.is_mla:
            qk = self.qk_nope_head_dim + self.qk_rope_head_dim
            q = h * self.q_lora_rank + self.q_lora_rank * nh * qk if self.q_lora_rank else h * nh * qk
            return q + h * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank * nh * (self.qk_nope_head_dim + self.v_head_dim) + nh * self.v_head_dim * h
        return h * (self.q_size + 2 * self.kv_size) + self.q_size * h + (self.q_size * h if self.attn_output_gate else 0)

    def num_params(self) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        attn = self._attn_weights() + (2 * self.head_dim if self.qk_norm else 0)
        moe = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts + 3 * h * self.shared_expert_intermediate_size
        dense = 3 * h * self.intermediate_size
        n_moe = sum(self.layer_is_moe(i) for i in range(L))
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return L * (attn + 2 * h) + n_moe * moe + (L - n_moe) * dense + emb + h

    @property
    def rotary_dim(self) -> int:
        """Leading dims of a head that carry the rotary embedding (even; the whole head unless ``partial_rotary_factor`` < 1)."""
        if self.is_mla:
            return self.qk_rope_head_dim
        return self.head_dim if self.partial_rotary_factor >= 1.0 else int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    def flops_per_token(self, avg_context: float = 0.0) -> float:
        """Forward+backward matmul FLOPs per token (6·N_active + attention)."""
        h, L = self.hidden_size, self.num_hidden_layers
        attn_w = self._attn_weights()
        moe_w = self.num_experts_per_tok * 3 * h * self.moe_intermediate_size + h * self.num_experts + 3 * h * self.shared_expert_intermediate_size
        n_moe = sum(self.layer_is_moe(i) for i in range(L))
        dense = L * attn_w + n_moe * moe_w + (L - n_moe) * 3 * h * self.intermediate_size + self.vocab_size * h
        qk_v = (self.qk_nope_head_dim + self.qk_rope_head_dim + self.v_head_dim) * self.num_attention_heads if self.is_mla else 2 * self.q_size
        attn = L * qk_v * avg_context  # QKᵀ and PV, causal average context
        return 6.0 * dense + 6.0 * attn

    # ---------------------------------------------------------------- HF I/O
    @classmethod
    def from_hf(cls, cfg: Dict[str, Any]) -> 'DecoderConfig':
        cfg = dict(cfg)
        top = cfg
        if 'text_config' in cfg:
            cfg = dict(cfg['text_config'])
        mt = cfg.get('model_type', 'qwen3')
        if mt not in SUPPORTED_MODEL_TYPES and not os.environ.get('TWINKLE_ALLOW_UNKNOWN_ARCH'):
            # an unknown type may differ in ways a shared field list does not show (scaled embeddings or residuals, other
            # norms, partial rotary …): better refused than silently computed wrongly
            raise NotImplementedError(f'model_type {mt!r} is not among the decoder families implemented here {sorted(SUPPORTED_MODEL_TYPES)}; '
                                      'set TWINKLE_ALLOW_UNKNOWN_ARCH=1 to load it as a Llama-style decoder anyway')
        vision = top.get('vision_config')
        if vision is not None:
            vision = dict(vision)
            if vision.get('model_type', top.get('model_type', 'qwen2_vl')) not in ('qwen2_vl', 'qwen2_5_vl', 'qwen3_vl', 'qwen3_vl_moe', 'qwen3_5', 'qwen3_5_moe'):
                raise NotImplementedError(f"vision tower of type {vision.get('model_type')!r} is not supported (qwen2_vl, qwen2_5_vl, qwen3_vl and qwen3_5 are)")
        rs_any = cfg.get('rope_scaling') or cfg.get('rope_parameters') or top.get('rope_scaling') or {}
        q35 = mt.startswith('qwen3_5') or mt == 'qwen3_next'      # the hybrid family: gated attention, partial rotary, "1 + w" norms
        heads = cfg.get('num_attention_heads', 32)
        mla = mt in ('deepseek_v2', 'deepseek_v3', 'kimi_k2')
        v2 = mt == 'deepseek_v2'      # softmax scores, groups ranked by their best expert, no selection bias, weights not renormalised
        dsv3 = mla or mt == 'glm4_moe'        # GLM-4.5 routes like DeepSeek-V3 over ordinary grouped-query attention
        window = cfg.get('sliding_window')
        if mt.startswith('qwen') and not cfg.get('use_sliding_window'):
            window = None                    # the Qwen configs carry a window size that is switched off by default
        gemma23 = mt in ('gemma2', 'gemma3_text', 'gemma3')
        oss = mt == 'gpt_oss'
        granite = mt == 'granite'
        olmo = mt in ('olmo2', 'olmo3')
        rope_local = cfg.get('rope_local_base_freq')
        rp = cfg.get('rope_parameters')
        if isinstance(rp, dict) and isinstance(rp.get('full_attention'), dict):      # per-layer-type rotary settings (Gemma-3)
            rope_local = (rp.get('sliding_attention') or {}).get('rope_theta', rope_local)
            cfg['rope_parameters'] = dict(rp['full_attention'])
        act = cfg.get('hidden_activation') or cfg.get('hidden_act') or 'silu'
        if mt == 'gemma':
            act = 'gelu_pytorch_tanh'        # what the Hugging Face model runs whatever the (legacy) field says
        if act not in ('silu', 'gelu_pytorch_tanh'):
            raise NotImplementedError(f'feed-forward activation {act!r} is not supported (silu and gelu_pytorch_tanh are)')
        out = cls(
            vocab_size=cfg.get('vocab_size', 151936), hidden_size=cfg.get('hidden_size', 4096),
            intermediate_size=cfg.get('intermediate_size', 12288), num_hidden_layers=cfg.get('num_hidden_layers', 36),
            num_attention_heads=heads, num_key_value_heads=cfg.get('num_key_value_heads', heads),
            head_dim=(cfg.get('head_dim') or cfg.get('hidden_size', 4096) // heads) if not mla
            else int(cfg.get('qk_nope_head_dim', 128)) + int(cfg.get('qk_rope_head_dim', 64)), rms_norm_eps=cfg.get('rms_norm_eps', 1e-6),
            rope_theta=float(cfg.get('rope_theta', (cfg.get('rope_parameters') or {}).get('rope_theta', 1e6))),
            rope_scaling=_rope_scaling_of(cfg), tie_word_embeddings=bool(cfg.get('tie_word_embeddings', False)),
            pre_norm=not olmo, qk_norm_full=olmo,
            qk_norm=olmo or mt.startswith('qwen3') or mt.startswith('gemma3') or (mt == 'glm4_moe' and bool(cfg.get('use_qk_norm'))),
            attention_bias=bool(cfg.get('attention_bias', cfg.get('qkv_bias', cfg.get('bias', False)) if mt.startswith('internlm') else mt.startswith('qwen2'))),
            router_scoring=('softmax_grouped' if v2 else 'sigmoid') if dsv3 else ('topk_softmax' if oss else 'softmax'), router_bias=dsv3 and not v2,
            n_group=int(cfg.get('n_group') or 1) if (dsv3 and not (v2 and cfg.get('topk_method', 'greedy') == 'greedy')) else 1,
            topk_group=int(cfg.get('topk_group') or 1) if dsv3 else 1, routed_scaling_factor=float(cfg.get('routed_scaling_factor', 1.0)) if dsv3 else 1.0,
            first_k_dense_replace=int(cfg.get('first_k_dense_replace', 0)) if dsv3 else 0, shared_expert_gate=not dsv3,
            q_lora_rank=cfg.get('q_lora_rank') if mla else None, kv_lora_rank=int(cfg.get('kv_lora_rank', 0)) if mla else 0,
            qk_nope_head_dim=int(cfg.get('qk_nope_head_dim', 128)), qk_rope_head_dim=int(cfg.get('qk_rope_head_dim', 64)),
            v_head_dim=int(cfg.get('v_head_dim', 128)), mla_rope_interleave=bool(cfg.get('rope_interleave', True)),
            hidden_act=act, embed_scale=float(cfg.get('embed_scale', cfg.get('hidden_size', 4096)**0.5 if mt.startswith('gemma') else (cfg.get('embedding_multiplier', 1.0) if granite else 1.0))),
            attn_sinks=oss, o_proj_bias=oss and bool(cfg.get('attention_bias', True)), router_linear_bias=oss, expert_bias=oss,
            expert_act='clamped_glu' if oss else 'swiglu',
            attn_logit_softcapping=cfg.get('attn_logit_softcapping') if gemma23 else None,
            final_logit_softcapping=cfg.get('final_logit_softcapping') if gemma23 else None,
            query_pre_attn_scalar=cfg.get('query_pre_attn_scalar') if gemma23 else (float(cfg['attention_multiplier'])**-2 if (granite and cfg.get('attention_multiplier')) else None),
            residual_multiplier=float(cfg.get('residual_multiplier', 1.0)) if granite else 1.0,
            logits_scaling=float(cfg.get('logits_scaling', 1.0)) if granite else 1.0,
            rope_local_theta=float(rope_local) if (rope_local and mt.startswith('gemma3')) else None,
            sliding_window=int(window) if window else None,
            num_experts=cfg.get('num_experts', cfg.get('num_local_experts', cfg.get('n_routed_experts', 0))) or 0,
            num_experts_per_tok=cfg.get('num_experts_per_tok', 8),
            moe_intermediate_size=cfg.get('moe_intermediate_size', cfg.get('intermediate_size', 768) if mt in ('mixtral', 'gpt_oss') else 768),
            norm_topk_prob=(True if cfg.get('norm_topk_prob') is None else bool(cfg['norm_topk_prob'])) and not v2, router_aux_loss_coef=float(cfg.get('router_aux_loss_coef', 0.0)),
            shared_expert_intermediate_size=int(cfg.get('shared_expert_intermediate_size', 0) or 0) if not dsv3
            else int(cfg.get('moe_intermediate_size', 0)) * int(cfg.get('n_shared_experts') or 0),
            rms_norm_offset=float(cfg.get('rms_norm_offset', 1.0 if (mt.startswith('gemma') or q35) else 0.0)),
            partial_rotary_factor=float(cfg.get('partial_rotary_factor', (cfg.get('rope_parameters') or {}).get('partial_rotary_factor', 1.0)) or 1.0),
            attn_output_gate=bool(cfg.get('attn_output_gate', q35)),
            rope_interleaved=bool(cfg.get('rope_interleaved', mt in ('glm', 'glm4', 'ernie4_5'))),
            no_rope_layers=[int(v) for v in cfg['no_rope_layers']] if (mt == 'smollm3' and cfg.get('no_rope_layers')) else None, sandwich_norm=bool(cfg.get('sandwich_norm', mt == 'glm4' or gemma23 or olmo)),
            layer_types=list(cfg['layer_types']) if cfg.get('layer_types') and ('linear_attention' in cfg['layer_types'] or ('sliding_attention' in cfg['layer_types'] and window)) else None,
            linear_num_key_heads=cfg.get('linear_num_key_heads', 16), linear_num_value_heads=cfg.get('linear_num_value_heads', 32),
            linear_key_head_dim=cfg.get('linear_key_head_dim', 128), linear_value_head_dim=cfg.get('linear_value_head_dim', 128),
            linear_conv_kernel_dim=cfg.get('linear_conv_kernel_dim', 4),
            vision=vision, image_token_id=top.get('image_token_id'), video_token_id=top.get('video_token_id'),
            vision_start_token_id=top.get('vision_start_token_id'), vision_end_token_id=top.get('vision_end_token_id'),
            mrope_section=list(rs_any['mrope_section']) if isinstance(rs_any, dict) and rs_any.get('mrope_section') and (vision is not None or not q35) else None,
            mrope_interleaved=bool(isinstance(rs_any, dict) and rs_any.get('mrope_interleaved')),
            initializer_range=cfg.get('initializer_range', 0.02), model_type=mt,
            torch_dtype=str(cfg.get('torch_dtype', cfg.get('dtype', 'bfloat16'))),
            max_position_embeddings=cfg.get('max_position_embeddings', 40960), pad_token_id=cfg.get('pad_token_id'),
            eos_token_id=cfg.get('eos_token_id') if not isinstance(cfg.get('eos_token_id'), list) else cfg['eos_token_id'][0])
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> 'DecoderConfig':
        with open(os.path.join(path, 'config.json')) as f:
            return cls.from_hf(json.load(f))

    def to_hf(self) -> Dict[str, Any]:
        arch = 'Qwen3MoeForCausalLM' if self.is_moe else ('Qwen3ForCausalLM' if self.qk_norm else 'LlamaForCausalLM')
        arch = {'mixtral': 'MixtralForCausalLM', 'qwen2_moe': 'Qwen2MoeForCausalLM', 'qwen2': 'Qwen2ForCausalLM', 'mistral': 'MistralForCausalLM',
                'seed_oss': 'SeedOssForCausalLM'}.get(self.model_type, arch)
        d = {
            'architectures': [arch], 'model_type': self.model_type if self.model_type in ('mixtral', 'qwen2_moe') else ('qwen3_moe' if self.is_moe else self.model_type),
            'vocab_size': self.vocab_size, 'hidden_size': self.hidden_size, 'intermediate_size': self.intermediate_size,
            'num_hidden_layers': self.num_hidden_layers, 'num_attention_heads': self.num_attention_heads,
            'num_key_value_heads': self.num_key_value_heads, 'head_dim': self.head_dim, 'rms_norm_eps': self.rms_norm_eps,
            'rope_theta': self.rope_theta, 'tie_word_embeddings': self.tie_word_embeddings, 'attention_bias': self.attention_bias,
            'hidden_act': self.hidden_act, 'initializer_range': self.initializer_range, 'torch_dtype': self.torch_dtype,
            'max_position_embeddings': self.max_position_embeddings,
        }
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                     router_aux_loss_coef=self.router_aux_loss_coef, decoder_sparse_step=1, mlp_only_layers=[])
            if self.shared_expert_intermediate_size:
                d['shared_expert_intermediate_size'] = self.shared_expert_intermediate_size
            if self.model_type == 'mixtral':
                d.update(num_local_experts=self.num_experts, intermediate_size=self.moe_intermediate_size, sliding_window=None)
        if self.rms_norm_offset:
            d['rms_norm_offset'] = self.rms_norm_offset
        if self.sliding_window:
            d['sliding_window'] = self.sliding_window
        if self.is_mla:
            d.update(architectures=['DeepseekV2ForCausalLM' if self.model_type == 'deepseek_v2' else 'DeepseekV3ForCausalLM'], model_type=self.model_type,
                     topk_method='group_limited_greedy' if self.n_group > 1 else 'greedy', q_lora_rank=self.q_lora_rank, kv_lora_rank=self.kv_lora_rank,
                     qk_nope_head_dim=self.qk_nope_head_dim, qk_rope_head_dim=self.qk_rope_head_dim, v_head_dim=self.v_head_dim,
                     rope_interleave=self.mla_rope_interleave, head_dim=self.qk_rope_head_dim, n_routed_experts=self.num_experts,
                     n_shared_experts=(self.shared_expert_intermediate_size // self.moe_intermediate_size) if self.num_experts else 0,
                     n_group=self.n_group, topk_group=self.topk_group, routed_scaling_factor=self.routed_scaling_factor,
                     first_k_dense_replace=self.first_k_dense_replace, norm_topk_prob=self.norm_topk_prob,
                     num_experts_per_tok=self.num_experts_per_tok, moe_intermediate_size=self.moe_intermediate_size)
            for k in ('num_experts', 'shared_expert_intermediate_size', 'decoder_sparse_step', 'mlp_only_layers'):
                d.pop(k, None)
        elif self.model_type == 'ernie4_5':
            d.update(architectures=['Ernie4_5ForCausalLM'], use_bias=self.attention_bias)
        elif self.model_type == 'smollm3':
            d.update(architectures=['SmolLM3ForCausalLM'], no_rope_layers=list(self.no_rope_layers or [1] * self.num_hidden_layers), use_sliding_window=False,
                     pad_token_id=self.pad_token_id if self.pad_token_id is not None else 0)
        elif self.model_type in ('olmo2', 'olmo3'):
            d.update(architectures=['Olmo3ForCausalLM' if self.model_type == 'olmo3' else 'Olmo2ForCausalLM'], model_type=self.model_type)
            if self.model_type == 'olmo3':
                d.update(sliding_window=self.sliding_window, layer_types=list(self.layer_types or ['full_attention'] * self.num_hidden_layers))
        elif self.model_type == 'granite':
            d.update(architectures=['GraniteForCausalLM'], embedding_multiplier=self.embed_scale, residual_multiplier=self.residual_multiplier,
                     logits_scaling=self.logits_scaling, attention_multiplier=self.attn_scale, mlp_bias=False)
        elif self.model_type == 'gpt_oss':
            d.update(architectures=['GptOssForCausalLM'], model_type='gpt_oss', num_local_experts=self.num_experts, intermediate_size=self.moe_intermediate_size,
                     sliding_window=self.sliding_window, layer_types=list(self.layer_types or ['full_attention'] * self.num_hidden_layers),
                     attention_bias=self.attention_bias, swiglu_limit=7.0, num_experts_per_tok=self.num_experts_per_tok,
                     router_aux_loss_coef=self.router_aux_loss_coef)
            for k in ('num_experts', 'moe_intermediate_size', 'norm_topk_prob', 'decoder_sparse_step', 'mlp_only_layers', 'shared_expert_intermediate_size'):
                d.pop(k, None)
        elif self.model_type == 'glm4_moe':
            d.update(architectures=['Glm4MoeForCausalLM'], model_type='glm4_moe', use_qk_norm=self.qk_norm, n_routed_experts=self.num_experts,
                     n_shared_experts=self.shared_expert_intermediate_size // self.moe_intermediate_size, n_group=self.n_group,
                     topk_group=self.topk_group, routed_scaling_factor=self.routed_scaling_factor, first_k_dense_replace=self.first_k_dense_replace,
                     partial_rotary_factor=self.partial_rotary_factor,
                     rope_parameters={'rope_type': 'default', 'rope_theta': self.rope_theta, 'partial_rotary_factor': self.partial_rotary_factor})
            for k in ('num_experts', 'shared_expert_intermediate_size', 'decoder_sparse_step', 'mlp_only_layers'):
                d.pop(k, None)
        elif self.model_type == 'phi3':
            d.update(architectures=['Phi3ForCausalLM'], partial_rotary_factor=self.partial_rotary_factor,
                     pad_token_id=self.pad_token_id, sliding_window=self.sliding_window,
                     original_max_position_embeddings=(self.rope_scaling or {}).get('original_max_position_embeddings', self.max_position_embeddings))
        elif self.model_type == 'gemma':
            d.update(architectures=['GemmaForCausalLM'], hidden_activation=self.hidden_act)
            d.pop('rms_norm_offset', None)
        elif self.model_type in ('gemma2', 'gemma3_text', 'gemma3'):
            g3 = self.model_type != 'gemma2'
            d.update(architectures=['Gemma3ForCausalLM' if g3 else 'Gemma2ForCausalLM'], model_type='gemma3_text' if g3 else 'gemma2',
                     hidden_activation=self.hidden_act, query_pre_attn_scalar=self.query_pre_attn_scalar, sliding_window=self.sliding_window,
                     attn_logit_softcapping=self.attn_logit_softcapping, final_logit_softcapping=self.final_logit_softcapping,
                     layer_types=list(self.layer_types or ['full_attention'] * self.num_hidden_layers))
            if g3:
                glob = dict(self.rope_scaling or {'rope_type': 'default'}, rope_theta=self.rope_theta)
                d['rope_parameters'] = {'full_attention': glob, 'sliding_attention': {'rope_type': 'default', 'rope_theta': self.rope_local_theta or self.rope_theta}}
                d.pop('rope_scaling', None)
                d.pop('rope_theta', None)
            d.pop('rms_norm_offset', None)
        elif self.model_type == 'internlm2':
            d.update(architectures=['InternLM2ForCausalLM'], bias=self.attention_bias)
        elif self.model_type == 'internlm3':
            d.update(architectures=['InternLM3ForCausalLM'], qkv_bias=self.attention_bias, bias=False)
        if self.rope_scaling:
            d['rope_scaling'] = dict(self.rope_scaling)
        if self.vision and not self.model_type.startswith('qwen3_5'):
            fam = self.vision.get('model_type', 'qwen2_vl')
            if fam == 'qwen3_vl' and self.is_moe:
                fam = 'qwen3_vl_moe'
            rope = {'type': 'mrope', 'mrope_section': list(self.mrope_section or [])}
            if fam.startswith('qwen3_vl'):
                rope = {'rope_type': 'default', 'mrope_section': list(self.mrope_section or []), 'mrope_interleaved': self.mrope_interleaved}
            text = dict(d, model_type=fam + '_text', rope_scaling=rope)
            text.pop('architectures', None)
            arch = {'qwen2_vl': 'Qwen2VLForConditionalGeneration', 'qwen2_5_vl': 'Qwen2_5_VLForConditionalGeneration',
                    'qwen3_vl': 'Qwen3VLForConditionalGeneration', 'qwen3_vl_moe': 'Qwen3VLMoeForConditionalGeneration'}[fam]
            vis = dict(self.vision, model_type=fam) if fam == 'qwen3_vl_moe' else dict(self.vision)
            return {'architectures': [arch], 'model_type': fam, 'text_config': text,
                    'vision_config': vis, 'image_token_id': self.image_token_id, 'video_token_id': self.video_token_id,
                    'vision_start_token_id': self.vision_start_token_id, 'vision_end_token_id': self.vision_end_token_id,
                    'tie_word_embeddings': self.tie_word_embeddings, 'torch_dtype': self.torch_dtype}
        if self.layer_types and 'linear_attention' not in self.layer_types:
            d['layer_types'] = list(self.layer_types)
        elif self.layer_types:
            d.update(layer_types=list(self.layer_types), linear_num_key_heads=self.linear_num_key_heads,
                     linear_num_value_heads=self.linear_num_value_heads, linear_key_head_dim=self.linear_key_head_dim,
                     linear_value_head_dim=self.linear_value_head_dim, linear_conv_kernel_dim=self.linear_conv_kernel_dim)
        if self.model_type in ('glm', 'glm4'):
            d.update(architectures=['Glm4ForCausalLM' if self.model_type == 'glm4' else 'GlmForCausalLM'], model_type=self.model_type,
                     partial_rotary_factor=self.partial_rotary_factor, pad_token_id=self.pad_token_id if self.pad_token_id is not None else 0,
                     rope_parameters={'rope_type': 'default', 'rope_theta': self.rope_theta, 'partial_rotary_factor': self.partial_rotary_factor})
        elif self.model_type == 'qwen3_next':
            d.update(architectures=['Qwen3NextForCausalLM'], model_type='qwen3_next', partial_rotary_factor=self.partial_rotary_factor,
                     rope_parameters={'rope_type': 'default', 'rope_theta': self.rope_theta, 'partial_rotary_factor': self.partial_rotary_factor},
                     layer_types=list(self.layer_types or ['full_attention'] * self.num_hidden_layers))
            d.pop('rms_norm_offset', None)
        elif self.model_type.startswith('qwen3_5'):
            # written as the text model of the family (what ``Qwen3_5ForCausalLM`` loads)
            d.update(architectures=['Qwen3_5MoeForCausalLM' if self.is_moe else 'Qwen3_5ForCausalLM'],
                     model_type='qwen3_5_moe_text' if self.is_moe else 'qwen3_5_text', partial_rotary_factor=self.partial_rotary_factor,
                     rope_parameters={'rope_type': 'default', 'rope_theta': self.rope_theta, 'partial_rotary_factor': self.partial_rotary_factor},
                     layer_types=list(self.layer_types or ['full_attention'] * self.num_hidden_layers))
            d.pop('rms_norm_offset', None)
            if self.vision:      # the full model: the Qwen3-VL tower without its deep-stack taps in front of the hybrid decoder
                fam = 'qwen3_5_moe' if self.is_moe else 'qwen3_5'
                d['rope_parameters'].update(mrope_section=list(self.mrope_section or []), mrope_interleaved=self.mrope_interleaved)
                text = {k: v for k, v in d.items() if k != 'architectures'}
                return {'architectures': ['Qwen3_5MoeForConditionalGeneration' if self.is_moe else 'Qwen3_5ForConditionalGeneration'], 'model_type': fam,
                        'text_config': text, 'vision_config': dict(self.vision, model_type=fam), 'image_token_id': self.image_token_id,
                        'video_token_id': self.video_token_id, 'vision_start_token_id': self.vision_start_token_id,
                        'vision_end_token_id': self.vision_end_token_id, 'tie_word_embeddings': self.tie_word_embeddings, 'torch_dtype': self.torch_dtype}
        elif self.partial_rotary_factor != 1.0 or self.attn_output_gate:
            d.update(partial_rotary_factor=self.partial_rotary_factor, attn_output_gate=self.attn_output_gate)
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, 'config.json'), 'w') as f:
            json.dump(self.to_hf(), f, indent=2)


PRESETS: Dict[str, Dict[str, Any]] = {
    # the smallest end-to-end configuration (LoRA SFT on CPU)
    'tiny-dense': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=True,
                       torch_dtype='float32'),
    'tiny-hybrid': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=True, torch_dtype='float32',
                        layer_types=['linear_attention', 'full_attention', 'linear_attention', 'full_attention'], linear_num_key_heads=2,
                        linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32),
    # the Qwen3.5 text stack in small: three Gated DeltaNet layers per full-attention layer, output gate, rotary on a quarter
    # of the head, "1 + w" norms
    'tiny-qwen3.5': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=True, torch_dtype='float32',
                         model_type='qwen3_5_text', rms_norm_offset=1.0, partial_rotary_factor=0.25, attn_output_gate=True,
                         layer_types=['linear_attention', 'linear_attention', 'linear_attention', 'full_attention'], linear_num_key_heads=2,
                         linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32),
    # DeepSeek-V3 in small: latent attention with a query bottleneck, one dense layer then mixture-of-experts layers with sigmoid
    # routing over expert groups, selection bias and an ungated shared expert
    'tiny-deepseek': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                          head_dim=48, rope_theta=1e4, tie_word_embeddings=False, qk_norm=False, torch_dtype='float32', model_type='deepseek_v3',
                          q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, num_experts=8,
                          num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128, shared_expert_gate=False,
                          router_scoring='sigmoid', router_bias=True, n_group=4, topk_group=2, routed_scaling_factor=2.5, first_k_dense_replace=1),
    # GPT-OSS in small: sink logits, alternating sliding-window layers, biased projections / router / experts, top-k-then-softmax routing
    'tiny-gpt-oss': dict(vocab_size=1024, hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                         rope_theta=1.5e5, tie_word_embeddings=False, qk_norm=False, torch_dtype='float32', model_type='gpt_oss', attention_bias=True,
                         o_proj_bias=True, attn_sinks=True, router_linear_bias=True, expert_bias=True, expert_act='clamped_glu',
                         router_scoring='topk_softmax', num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, sliding_window=16,
                         layer_types=['sliding_attention', 'full_attention', 'sliding_attention', 'full_attention']),
    'tiny-moe': dict(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=64, rope_theta=1e4, tie_word_embeddings=True, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=128, router_aux_loss_coef=1e-3, torch_dtype='float32'),
    'tiny-vl': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=False, attention_bias=True, torch_dtype='float32',
                    model_type='qwen2_vl_text', mrope_section=[8, 12, 12], image_token_id=265, video_token_id=267, vision_start_token_id=264,
                    vision_end_token_id=266,  # ids of these tokens in the byte-level test tokenizer
                    vision=dict(depth=2, embed_dim=64, hidden_size=256, num_heads=4, mlp_ratio=2, patch_size=14,
                                                          spatial_merge_size=2, temporal_patch_size=2, in_channels=3)),
    'tiny-vl3': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=True, torch_dtype='float32', model_type='qwen3_vl_text',
                     mrope_section=[8, 12, 12], mrope_interleaved=True, image_token_id=265, video_token_id=267, vision_start_token_id=264,
                     vision_end_token_id=266,
                     vision=dict(depth=3, hidden_size=64, out_hidden_size=256, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2,
                                 temporal_patch_size=2, in_channels=3, num_position_embeddings=64, deepstack_visual_indexes=[0, 2])),
    # Qwen3.5 vision-language in small: the Qwen3-VL tower (no deep-stack taps) in front of the hybrid decoder
    'tiny-qwen3.5-vl': dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=64, rope_theta=1e4, tie_word_embeddings=True, qk_norm=True, torch_dtype='float32', model_type='qwen3_5',
                            rms_norm_offset=1.0, partial_rotary_factor=0.25, attn_output_gate=True,
                            layer_types=['linear_attention', 'linear_attention', 'linear_attention', 'full_attention'], linear_num_key_heads=2,
                            linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32, mrope_section=[2, 3, 3], mrope_interleaved=True,
                            image_token_id=265, video_token_id=267, vision_start_token_id=264, vision_end_token_id=266,
                            vision=dict(depth=2, hidden_size=64, out_hidden_size=256, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2,
                                        temporal_patch_size=2, in_channels=3, num_position_embeddings=64)),
    'tiny-moe-shared': dict(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=64, rope_theta=1e4, tie_word_embeddings=True, num_experts=8, num_experts_per_tok=2,
                            moe_intermediate_size=128, shared_expert_intermediate_size=192, torch_dtype='float32'),
    'qwen3-0.6b': dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                       num_key_value_heads=8, head_dim=128, tie_word_embeddings=True),
    'qwen3-8b': dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128),
    'qwen3-32b': dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                      num_key_value_heads=8, head_dim=128),
    'qwen3-30b-a3b': dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32,
                          num_key_value_heads=4, head_dim=128, num_experts=128, num_experts_per_tok=8,
                          moe_intermediate_size=768, router_aux_loss_coef=1e-3),
}


def preset(name: str, **overrides) -> DecoderConfig:
    kw = dict(PRESETS[name.lower()])
    kw.update(overrides)
    return DecoderConfig(**kw)
