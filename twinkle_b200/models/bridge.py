"""HF ↔ internal-layout weight bridge.

The reference reaches Hugging Face checkpoints through ``save_pretrained``
(transformers backend) or the external ``mcore_bridge`` package (Megatron
backend, ``src/twinkle/model/megatron/megatron.py:874-945``).  This bridge is
the single converter for every parallel layout of the owned decoder:

* fused ``qkv_proj`` / ``gate_up_proj`` ⇄ separate HF ``q/k/v_proj`` and
  ``gate/up_proj`` (row concatenation, so splitting is bit-exact);
* fused expert tensors ``[E, …]`` ⇄ per-expert HF tensors;
* tensor-parallel shards ⇄ full tensors (column-parallel: rows; row-parallel:
  columns; fused projections are sharded per logical part so every rank holds
  whole heads);
* pipeline stages own disjoint layer ranges;
* PEFT adapter key names ``base_model.model.<module>.lora_A.weight``.

All conversions are pure slicing / concatenation — no arithmetic — hence a
save → load round trip is bitwise.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from .config import DecoderConfig

_LAYER = re.compile(r'^layers\.(\d+)\.(.+)$')


def _hf_layer(i: int, rest: str) -> str:
    return f'model.layers.{i}.{rest}'


_MIXTRAL = ((re.compile(r'\.mlp\.experts\.(\d+)\.gate_proj\.'), r'.block_sparse_moe.experts.\1.w1.'),
            (re.compile(r'\.mlp\.experts\.(\d+)\.up_proj\.'), r'.block_sparse_moe.experts.\1.w3.'),
            (re.compile(r'\.mlp\.experts\.(\d+)\.down_proj\.'), r'.block_sparse_moe.experts.\1.w2.'),
            (re.compile(r'\.mlp\.gate\.'), '.block_sparse_moe.gate.'))


_INTERNLM2 = (('model.embed_tokens.', 'model.tok_embeddings.'), ('lm_head.', 'output.'), ('.self_attn.qkv_proj.', '.attention.wqkv.'),
              ('.self_attn.o_proj.', '.attention.wo.'), ('.mlp.gate_proj.', '.feed_forward.w1.'), ('.mlp.up_proj.', '.feed_forward.w3.'),
              ('.mlp.down_proj.', '.feed_forward.w2.'), ('.input_layernorm.', '.attention_norm.'), ('.post_attention_layernorm.', '.ffn_norm.'))


def _family(name: str, cfg: DecoderConfig) -> str:
    """Checkpoint spelling of a tensor name for families that differ from the Qwen / Llama one (Mixtral: ``block_sparse_moe``
    with ``w1`` = gate, ``w3`` = up, ``w2`` = down; DeepSeek-V3: ``shared_experts`` and the router's selection bias under
    ``mlp.gate``; InternLM2: ``tok_embeddings`` / ``attention.wqkv`` / ``attention.wo`` /
    ``feed_forward.w1|w3|w2`` / ``attention_norm`` / ``ffn_norm`` / ``output``)."""
    if cfg.model_type == 'mixtral':
        for pat, rep in _MIXTRAL:
            name = pat.sub(rep, name)
    elif cfg.model_type in ('deepseek_v2', 'deepseek_v3', 'kimi_k2', 'glm4_moe'):
        name = name.replace('.mlp.shared_expert.', '.mlp.shared_experts.').replace('.mlp.e_score_correction_bias', '.mlp.gate.e_score_correction_bias')
    elif cfg.model_type in ('olmo2', 'olmo3'):       # only the norms on the sub-layer outputs exist there
        name = name.replace('.post_self_attn_layernorm.', '.post_attention_layernorm.').replace('.post_mlp_layernorm.', '.post_feedforward_layernorm.')
    elif cfg.model_type == 'gpt_oss':
        name = (name.replace('.mlp.gate.', '.mlp.router.').replace('.mlp.experts.gate_up_bias', '.mlp.experts.gate_up_proj_bias')
                .replace('.mlp.experts.down_bias', '.mlp.experts.down_proj_bias'))
    elif cfg.model_type in ('gemma2', 'gemma3_text', 'gemma3'):
        # four norms per layer there: input, after attention, before and after the feed-forward block
        for a, b in (('.post_attention_layernorm.', '.pre_feedforward_layernorm.'), ('.post_self_attn_layernorm.', '.post_attention_layernorm.'),
                     ('.post_mlp_layernorm.', '.post_feedforward_layernorm.')):
            if a in name:
                name = name.replace(a, b, 1)
                break
    elif cfg.model_type == 'internlm2':
        for a, b in _INTERNLM2:
            if name.startswith(a) or (a[0] == '.' and a in name):
                name = name.replace(a, b, 1)
    return name


def _fused_qkv(cfg: DecoderConfig) -> bool:
    """Families whose checkpoints keep q, k and v in one tensor: Phi-3 in this package's own ``[q | k | v]`` row order,
    InternLM2 grouped per key / value head (``[the group's query heads | its key head | its value head]``)."""
    return cfg.model_type in ('phi3', 'internlm2')


def _fused_gate_up(cfg: DecoderConfig) -> bool:
    """Families whose checkpoints keep ``[gate | up]`` as one tensor."""
    return cfg.model_type in ('glm', 'glm4', 'phi3')


def _wqkv_regroup(t: torch.Tensor, cfg: DecoderConfig, to_hf: bool) -> torch.Tensor:
    """Row permutation between ``[q | k | v]`` and InternLM2's per-group order."""
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g, tail = hq // hkv, tuple(t.shape[1:])
    if to_hf:
        q, k, v = t.split([hq * d, hkv * d, hkv * d], dim=0)
        return torch.cat([q.reshape(hkv, g, d, *tail), k.reshape(hkv, 1, d, *tail), v.reshape(hkv, 1, d, *tail)], 1).reshape(t.shape[0], *tail)
    x = t.reshape(hkv, g + 2, d, *tail)
    return torch.cat([x[:, :g].reshape(hq * d, *tail), x[:, g].reshape(hkv * d, *tail), x[:, g + 1].reshape(hkv * d, *tail)], 0)


def _split_gdn(cfg: DecoderConfig) -> bool:
    """Whether the linear-attention input projections are written the Qwen3.5 way (``in_proj_qkv`` / ``in_proj_z`` /
    ``in_proj_b`` / ``in_proj_a``) rather than as this package's two fused tensors."""
    return cfg.model_type.startswith('qwen3_5')


def rope_row_perm(cfg: DecoderConfig, heads: int, to_hf: bool) -> Optional[torch.Tensor]:
    """Row order of a q / k projection between this package's rotary convention (pairs ``(i, i + R/2)``) and a checkpoint
    that pairs ``(2i, 2i+1)`` (GLM-4 family), for ``heads`` heads; ``None`` when the conventions agree.  ``out = w[perm]``."""
    if not cfg.rope_interleaved:
        return None
    d, r = cfg.head_dim, cfg.rotary_dim
    from_hf = torch.cat([torch.arange(0, r, 2), torch.arange(1, r, 2), torch.arange(r, d)])    # ours[j] = hf[from_hf[j]]
    one = torch.argsort(from_hf) if to_hf else from_hf
    return (torch.arange(heads)[:, None] * d + one[None, :]).reshape(-1)


def _grouped_gdn(cfg: DecoderConfig) -> bool:
    """Qwen3-Next keeps the two fused linear-attention input projections, with their rows grouped per key head:
    ``[q_g | k_g | v of the group's value heads | z of the same]`` and ``[b_g | a_g]``."""
    return cfg.model_type == 'qwen3_next'


def _gdn_regroup(t: torch.Tensor, cfg: DecoderConfig, which: str, to_hf: bool) -> torch.Tensor:
    """Row permutation between this package's ``[q | k | v | z]`` / ``[b | a]`` order and the per-key-head grouping."""
    hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    rep, tail = hv // hk, tuple(t.shape[1:])
    sizes = [dk, dk, rep * dv, rep * dv] if which == 'qkvz' else [rep, rep]
    if to_hf:
        parts = t.split([hk * n for n in sizes], dim=0)
        return torch.cat([p.reshape(hk, n, *tail) for p, n in zip(parts, sizes)], 1).reshape(t.shape[0], *tail)
    parts = t.reshape(hk, sum(sizes), *tail).split(sizes, dim=1)
    return torch.cat([p.reshape(hk * n, *tail) for p, n in zip(parts, sizes)], 0)


def _gpt_oss_expert(t: torch.Tensor, rest: str, to_hf: bool) -> torch.Tensor:
    """GPT-OSS expert tensors: the checkpoint keeps ``[E, in, out]`` matrices with gate and up columns alternating
    (``gate = [..., ::2]``, ``up = [..., 1::2]``) and biases alternating the same way; here matrices are ``[E, out, in]`` with
    ``[gate | up]`` row blocks."""
    if rest.endswith('gate_up_proj') or rest.endswith('gate_up_bias'):
        if to_hf:
            if t.dim() == 3:
                t = t.transpose(1, 2)                       # [E, H, 2I] with [gate | up] columns
            g, u = t.chunk(2, dim=-1)
            return torch.stack([g, u], -1).flatten(-2).contiguous()
        t = torch.cat([t[..., ::2], t[..., 1::2]], -1)
        return t.transpose(1, 2).contiguous() if t.dim() == 3 else t.contiguous()
    if rest.endswith('down_proj'):
        return t.transpose(1, 2).contiguous()
    return t


def _vl(name: str, cfg: DecoderConfig) -> str:
    """Vision-language checkpoints nest the language model: ``model.X`` → ``model.language_model.X``."""
    return 'model.language_model.' + name[len('model.'):] if _nested(cfg) and name.startswith('model.') else name


def _nested(cfg: DecoderConfig) -> bool:
    """Checkpoints whose decoder sits under ``model.language_model``: the vision-language families and Qwen3.5 (its text-only
    class writes the same names as the full model)."""
    return bool(cfg.vision) or cfg.model_type.startswith('qwen3_5')


def internal_to_hf(name: str, tensor: torch.Tensor, cfg: DecoderConfig) -> List[Tuple[str, torch.Tensor]]:
    """One internal (full, un-sharded) tensor → one or more HF tensors."""
    if name.startswith('visual.'):
        return [('model.' + name, tensor)]
    return [(_family(_vl(n, cfg), cfg), t) for n, t in _internal_to_hf_text(name, tensor, cfg)]


def _internal_to_hf_text(name: str, tensor: torch.Tensor, cfg: DecoderConfig) -> List[Tuple[str, torch.Tensor]]:
    if name == 'embed_tokens.weight':
        return [('model.embed_tokens.weight', tensor)]
    if name == 'norm.weight':
        return [('model.norm.weight', tensor)]
    if name == 'lm_head.weight':
        return [('lm_head.weight', tensor)]
    m = _LAYER.match(name)
    if not m:
        raise KeyError(f'no HF mapping for {name}')
    i, rest = int(m.group(1)), m.group(2)
    if rest in ('self_attn.qkv_proj.weight', 'self_attn.qkv_proj.bias') and _fused_qkv(cfg):
        return [(_hf_layer(i, rest), _wqkv_regroup(tensor, cfg, True) if cfg.model_type == 'internlm2' else tensor)]
    if rest in ('self_attn.qkv_proj.weight', 'self_attn.qkv_proj.bias'):
        kind = rest.rsplit('.', 1)[1]
        if cfg.attn_output_gate:
            # HF keeps query and output gate in one projection, interleaved per head: [head 0: q (D) | gate (D), head 1: …]
            q, k, v, g = tensor.split([cfg.q_size, cfg.kv_size, cfg.kv_size, cfg.q_size], dim=0)
            hq, d = cfg.num_attention_heads, cfg.head_dim
            q = torch.cat([q.reshape(hq, d, *q.shape[1:]), g.reshape(hq, d, *g.shape[1:])], 1).reshape(2 * cfg.q_size, *q.shape[1:])
        else:
            q, k, v = tensor.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
        if cfg.rope_interleaved:
            q, k = q[rope_row_perm(cfg, cfg.num_attention_heads, True)], k[rope_row_perm(cfg, cfg.num_key_value_heads, True)]
        return [(_hf_layer(i, f'self_attn.q_proj.{kind}'), q), (_hf_layer(i, f'self_attn.k_proj.{kind}'), k),
                (_hf_layer(i, f'self_attn.v_proj.{kind}'), v)]
    if rest in ('self_attn.in_proj_qkvz.weight', 'self_attn.in_proj_ba.weight') and _grouped_gdn(cfg):
        which = 'qkvz' if 'qkvz' in rest else 'ba'
        return [(_hf_layer(i, 'linear_attn.' + rest[len('self_attn.'):]), _gdn_regroup(tensor, cfg, which, True))]
    if rest == 'self_attn.in_proj_qkvz.weight' and _split_gdn(cfg):     # Qwen3.5 keeps q|k|v and z, and b and a, as separate linears
        kd, vd = cfg.linear_num_key_heads * cfg.linear_key_head_dim, cfg.linear_num_value_heads * cfg.linear_value_head_dim
        qkv, z = tensor.split([2 * kd + vd, vd], dim=0)
        return [(_hf_layer(i, 'linear_attn.in_proj_qkv.weight'), qkv), (_hf_layer(i, 'linear_attn.in_proj_z.weight'), z)]
    if rest == 'self_attn.in_proj_ba.weight' and _split_gdn(cfg):
        b, a = tensor.chunk(2, dim=0)
        return [(_hf_layer(i, 'linear_attn.in_proj_b.weight'), b), (_hf_layer(i, 'linear_attn.in_proj_a.weight'), a)]
    if rest == 'mlp.gate_up_proj.weight' and _fused_gate_up(cfg):
        return [(_hf_layer(i, rest), tensor)]           # fused [gate | up] in the checkpoint too
    if rest in ('mlp.gate_up_proj.weight', 'mlp.shared_expert.gate_up_proj.weight'):
        g, u = tensor.chunk(2, dim=0)
        pre = rest[:-len('gate_up_proj.weight')]
        return [(_hf_layer(i, pre + 'gate_proj.weight'), g), (_hf_layer(i, pre + 'up_proj.weight'), u)]
    if rest == 'self_attn.conv_weight':          # depth-wise filters: HF keeps Conv1d's [C, 1, W], attention block named linear_attn
        return [(_hf_layer(i, 'linear_attn.conv1d.weight'), tensor.unsqueeze(1))]
    if rest == 'self_attn.norm_weight':
        return [(_hf_layer(i, 'linear_attn.norm.weight'), tensor)]
    if rest.startswith('self_attn.') and cfg.layer_types and cfg.layer_types[i] == 'linear_attention':
        return [(_hf_layer(i, 'linear_attn.' + rest[len('self_attn.'):]), tensor)]
    if rest in ('mlp.experts.gate_up_proj', 'mlp.experts.down_proj') and cfg.model_type.startswith('qwen3_5'):
        return [(_hf_layer(i, rest), tensor)]       # this family's checkpoints keep the experts fused, in the layout used here
    if cfg.model_type == 'gpt_oss' and rest.startswith('mlp.experts.'):
        return [(_hf_layer(i, rest), _gpt_oss_expert(tensor, rest, True))]
    if rest == 'mlp.experts.gate_up_proj':
        out = []
        for e in range(tensor.shape[0]):
            g, u = tensor[e].chunk(2, dim=0)
            out += [(_hf_layer(i, f'mlp.experts.{e}.gate_proj.weight'), g), (_hf_layer(i, f'mlp.experts.{e}.up_proj.weight'), u)]
        return out
    if rest == 'mlp.experts.down_proj':
        return [(_hf_layer(i, f'mlp.experts.{e}.down_proj.weight'), tensor[e]) for e in range(tensor.shape[0])]
    return [(_hf_layer(i, rest), tensor)]


def hf_names_for(name: str, cfg: DecoderConfig) -> List[str]:
    """HF tensor names that make up one internal tensor (in concat order)."""
    if name.startswith('visual.'):
        return ['model.' + name]
    return [_family(_vl(n, cfg), cfg) for n in _hf_names_for_text(name, cfg)]


def _hf_names_for_text(name: str, cfg: DecoderConfig) -> List[str]:
    meta = torch.empty(0)
    if name == 'embed_tokens.weight':
        return ['model.embed_tokens.weight']
    if name == 'norm.weight':
        return ['model.norm.weight']
    if name == 'lm_head.weight':
        return ['lm_head.weight']
    m = _LAYER.match(name)
    i, rest = int(m.group(1)), m.group(2)
    if rest.startswith('self_attn.qkv_proj.') and _fused_qkv(cfg):
        return [_hf_layer(i, rest)]
    if rest.startswith('self_attn.qkv_proj.'):
        kind = rest.rsplit('.', 1)[1]
        return [_hf_layer(i, f'self_attn.{p}_proj.{kind}') for p in 'qkv']
    if rest == 'self_attn.in_proj_qkvz.weight' and _split_gdn(cfg):
        return [_hf_layer(i, 'linear_attn.in_proj_qkv.weight'), _hf_layer(i, 'linear_attn.in_proj_z.weight')]
    if rest == 'self_attn.in_proj_ba.weight' and _split_gdn(cfg):
        return [_hf_layer(i, 'linear_attn.in_proj_b.weight'), _hf_layer(i, 'linear_attn.in_proj_a.weight')]
    if rest == 'mlp.gate_up_proj.weight' and _fused_gate_up(cfg):
        return [_hf_layer(i, rest)]
    if rest in ('mlp.gate_up_proj.weight', 'mlp.shared_expert.gate_up_proj.weight'):
        pre = rest[:-len('gate_up_proj.weight')]
        return [_hf_layer(i, pre + 'gate_proj.weight'), _hf_layer(i, pre + 'up_proj.weight')]
    if rest == 'self_attn.conv_weight':
        return [_hf_layer(i, 'linear_attn.conv1d.weight')]
    if rest == 'self_attn.norm_weight':
        return [_hf_layer(i, 'linear_attn.norm.weight')]
    if rest.startswith('self_attn.') and cfg.layer_types and cfg.layer_types[i] == 'linear_attention':
        return [_hf_layer(i, 'linear_attn.' + rest[len('self_attn.'):])]
    if rest in ('mlp.experts.gate_up_proj', 'mlp.experts.down_proj') and cfg.model_type.startswith('qwen3_5'):
        return [_hf_layer(i, rest)]
    if cfg.model_type == 'gpt_oss' and rest.startswith('mlp.experts.'):
        return [_hf_layer(i, rest)]
    if rest == 'mlp.experts.gate_up_proj':
        return [_hf_layer(i, f'mlp.experts.{e}.{p}_proj.weight') for e in range(cfg.num_experts) for p in ('gate', 'up')]
    if rest == 'mlp.experts.down_proj':
        return [_hf_layer(i, f'mlp.experts.{e}.down_proj.weight') for e in range(cfg.num_experts)]
    return [_hf_layer(i, rest)]


def hf_to_internal(name: str, cfg: DecoderConfig, get: Callable[[str], torch.Tensor],
                   expert_range: Optional[Tuple[int, int]] = None) -> torch.Tensor:
    """Assemble one internal tensor from HF tensors fetched by ``get``.  An output head that the checkpoint does not carry
    (tied embeddings saved once) is read from the embedding."""
    m = _LAYER.match(name)
    rest = m.group(2) if m else ''
    i = int(m.group(1)) if m else -1
    if cfg.model_type in ('mixtral', 'internlm2', 'deepseek_v2', 'deepseek_v3', 'kimi_k2', 'glm4_moe', 'gpt_oss'):      # names that are built without hf_names_for
        plain = get

        def get(n: str) -> torch.Tensor:  # noqa: F811
            return plain(_family(n, cfg))
    if _nested(cfg):
        raw = get

        def get(n: str) -> torch.Tensor:  # noqa: F811 — older checkpoints keep ``visual.*`` / ``model.layers.*`` at the top level
            for cand in (n, n.replace('model.language_model.', 'model.', 1), n.replace('model.visual.', 'visual.', 1), _vl(n, cfg)):
                try:
                    return raw(cand)
                except KeyError:
                    continue
            raise KeyError(n)
    if name == 'lm_head.weight':
        try:
            return get(hf_names_for(name, cfg)[0])
        except KeyError:
            return get(hf_names_for('embed_tokens.weight', cfg)[0])
    if cfg.model_type == 'gpt_oss' and rest.startswith('mlp.experts.'):
        lo, hi = expert_range or (0, cfg.num_experts)
        hf_name = hf_names_for(name, cfg)[0]
        try:
            t = get(hf_name)
        except KeyError:            # the released checkpoints keep the expert matrices as MXFP4 blocks + scales
            from ..utils.dequantizer import dequant_mxfp4
            t = dequant_mxfp4(get(hf_name + '_blocks'), get(hf_name + '_scales')).transpose(1, 2)      # [E, out, in] → the [E, in, out] of the bf16 form
        return _gpt_oss_expert(t, rest, False)[lo:hi].contiguous()
    if rest in ('mlp.experts.gate_up_proj', 'mlp.experts.down_proj'):
        # checkpoints written by newer transformers keep the experts fused, in this package's own layout
        # ([E, 2I, H] gate|up and [E, H, I]); older ones have one tensor per expert and projection
        try:
            fused = get(_hf_layer(i, rest))
        except KeyError:
            fused = None
        if fused is not None:
            lo, hi = expert_range or (0, cfg.num_experts)
            want = (2 * cfg.moe_intermediate_size, cfg.hidden_size) if rest.endswith('gate_up_proj') else (cfg.hidden_size, cfg.moe_intermediate_size)
            if tuple(fused.shape[1:]) != want:
                if tuple(fused.shape[1:]) == want[::-1]:
                    fused = fused.transpose(1, 2)       # [E, in, out] variant
                else:
                    raise ValueError(f'{name}: fused expert tensor of shape {tuple(fused.shape)}; expected [E, {want[0]}, {want[1]}]')
            return fused[lo:hi].contiguous()
    if rest == 'mlp.experts.gate_up_proj':
        lo, hi = expert_range or (0, cfg.num_experts)
        return torch.stack([torch.cat([get(_hf_layer(i, f'mlp.experts.{e}.gate_proj.weight')),
                                       get(_hf_layer(i, f'mlp.experts.{e}.up_proj.weight'))], 0) for e in range(lo, hi)])
    if rest == 'mlp.experts.down_proj':
        lo, hi = expert_range or (0, cfg.num_experts)
        return torch.stack([get(_hf_layer(i, f'mlp.experts.{e}.down_proj.weight')) for e in range(lo, hi)])
    parts = [get(n) for n in hf_names_for(name, cfg)]
    if rest.startswith('self_attn.qkv_proj.') and cfg.model_type == 'internlm2':
        return _wqkv_regroup(parts[0], cfg, False)
    if rest.startswith('self_attn.qkv_proj.') and cfg.rope_interleaved:
        parts = [parts[0][rope_row_perm(cfg, cfg.num_attention_heads, False)], parts[1][rope_row_perm(cfg, cfg.num_key_value_heads, False)], parts[2]]
    if rest.startswith('self_attn.qkv_proj.') and cfg.attn_output_gate:
        hq, d = cfg.num_attention_heads, cfg.head_dim
        qg = parts[0].reshape(hq, 2 * d, *parts[0].shape[1:])
        q, g = qg[:, :d].reshape(cfg.q_size, *parts[0].shape[1:]), qg[:, d:].reshape(cfg.q_size, *parts[0].shape[1:])
        return torch.cat([q, parts[1], parts[2], g], 0)
    if rest == 'self_attn.conv_weight' and parts[0].dim() == 3:
        return parts[0].squeeze(1)
    if rest in ('self_attn.in_proj_qkvz.weight', 'self_attn.in_proj_ba.weight') and _grouped_gdn(cfg):
        return _gdn_regroup(parts[0], cfg, 'qkvz' if 'qkvz' in rest else 'ba', False)
    return parts[0] if len(parts) == 1 else torch.cat(parts, 0)


# ------------------------------------------------------ tensor-parallel layout
def tp_rule(name: str, cfg: DecoderConfig):
    """How an internal tensor is split over a tensor-parallel group:
    ``('col', parts)`` rows sharded per logical part, ``('row', None)`` columns
    sharded, ``('vocab', None)`` rows sharded (embedding / head), or ``None`` = replicated."""
    if name in ('embed_tokens.weight', 'lm_head.weight'):
        return ('vocab', None)
    m = _LAYER.match(name)
    if not m:
        return None
    rest = m.group(2)
    if rest.startswith('self_attn.qkv_proj.'):
        return ('col', [cfg.q_size, cfg.kv_size, cfg.kv_size] + ([cfg.q_size] if cfg.attn_output_gate else []))
    if rest == 'mlp.gate_up_proj.weight':
        half = cfg.intermediate_size
        return ('col', [half, half])
    if rest in ('self_attn.o_proj.weight', 'mlp.down_proj.weight'):
        return ('row', None)
    if getattr(cfg, 'expert_tensor_parallel', False):
        # expert tensor parallelism: every expert's intermediate dimension is split over the group
        if rest == 'mlp.experts.gate_up_proj':       # [E, 2I, H]: gate rows and up rows sharded separately
            return ('ecol', [cfg.moe_intermediate_size, cfg.moe_intermediate_size])
        if rest == 'mlp.experts.down_proj':          # [E, H, I]
            return ('erow', None)
    return None


def tp_shard(name: str, full: torch.Tensor, cfg: DecoderConfig, tp_rank: int, tp_size: int) -> torch.Tensor:
    rule = tp_rule(name, cfg)
    if rule is None or tp_size == 1:
        return full
    kind, parts = rule
    if kind == 'col':
        pieces = full.split(parts, dim=0)
        return torch.cat([p.chunk(tp_size, dim=0)[tp_rank] for p in pieces], 0)
    if kind == 'row':
        return full.chunk(tp_size, dim=1)[tp_rank]
    if kind == 'ecol':
        return torch.cat([p.chunk(tp_size, dim=1)[tp_rank] for p in full.split(parts, dim=1)], 1)
    if kind == 'erow':
        return full.chunk(tp_size, dim=2)[tp_rank]
    return full.chunk(tp_size, dim=0)[tp_rank]  # vocab


def tp_unshard(name: str, shards: List[torch.Tensor], cfg: DecoderConfig) -> torch.Tensor:
    rule = tp_rule(name, cfg)
    if rule is None or len(shards) == 1:
        return shards[0]
    kind, parts = rule
    tp = len(shards)
    if kind == 'col':
        per = [p // tp for p in parts]
        split = [s.split(per, dim=0) for s in shards]
        return torch.cat([torch.cat([split[r][j] for r in range(tp)], 0) for j in range(len(parts))], 0)
    if kind == 'row':
        return torch.cat(shards, 1)
    if kind == 'ecol':
        per = [p // tp for p in parts]
        split = [s.split(per, dim=1) for s in shards]
        return torch.cat([torch.cat([split[r][j] for r in range(tp)], 1) for j in range(len(parts))], 1)
    if kind == 'erow':
        return torch.cat(shards, 2)
    return torch.cat(shards, 0)


# --------------------------------------------------------------------- PEFT
def lora_internal_to_peft(module_name: str, part: str, which: str) -> str:
    """``layers.3.self_attn.qkv_proj`` + ``q_proj`` + ``A`` →
    ``base_model.model.model.layers.3.self_attn.q_proj.lora_A.weight``."""
    prefix = module_name.rsplit('.', 1)[0] if '.' in module_name else ''
    hf_mod = f'{prefix}.{part}' if prefix else part
    if not hf_mod.startswith('lm_head'):
        hf_mod = 'model.' + hf_mod
    return f'base_model.model.{hf_mod}.lora_{which}.weight'


def lora_expert_to_peft(module_name: str, which_proj: str, which: str) -> str:
    """Expert (target-parameter) LoRA keys: ``…mlp.experts.lora_A.gate_up_proj``-style
    names collapse to ``base_model.model.model.layers.N.mlp.experts.<proj>.lora_A.weight``."""
    return f'base_model.model.model.{module_name}.{which_proj}_proj.lora_{which}.weight'
