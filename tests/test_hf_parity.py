"""The owned decoder against the Hugging Face implementations of the families it claims: random tiny models saved by
``transformers`` must give the same logits after loading here (fp32, CPU), and a checkpoint saved here must load in
``transformers`` with the same logits."""
import pytest
import torch

transformers = pytest.importorskip('transformers')

COMMON = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=512, rope_theta=10000.0)


def _cases():
    T = transformers
    return {
        'qwen3': (lambda: T.Qwen3Config(head_dim=32, tie_word_embeddings=False, **COMMON), 'Qwen3ForCausalLM'),
        'llama_tied': (lambda: T.LlamaConfig(tie_word_embeddings=True, **COMMON), 'LlamaForCausalLM'),
        'llama3_rope': (lambda: T.LlamaConfig(tie_word_embeddings=False, **{**COMMON, 'max_position_embeddings': 4096},
                                              rope_scaling={'rope_type': 'llama3', 'factor': 8.0, 'low_freq_factor': 1.0, 'high_freq_factor': 4.0,
                                                            'original_max_position_embeddings': 64}), 'LlamaForCausalLM'),
        'qwen2_bias': (lambda: T.Qwen2Config(tie_word_embeddings=False, **COMMON), 'Qwen2ForCausalLM'),
        'mistral': (lambda: T.MistralConfig(sliding_window=None, **COMMON), 'MistralForCausalLM'),
        'mixtral': (lambda: T.MixtralConfig(num_local_experts=4, num_experts_per_tok=2, sliding_window=None, **{**COMMON, 'intermediate_size': 96}),
                    'MixtralForCausalLM'),
        'seed_oss': (lambda: T.SeedOssConfig(head_dim=32, **COMMON), 'SeedOssForCausalLM'),
        'qwen3_moe': (lambda: T.Qwen3MoeConfig(head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
                                               decoder_sparse_step=1, mlp_only_layers=[], **COMMON), 'Qwen3MoeForCausalLM'),
        # hybrid stack: Gated DeltaNet layers + full attention with an output gate, partial rotary and "1 + w" norms
        'qwen3_5': (lambda: T.Qwen3_5TextConfig(head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                                                linear_value_head_dim=16, linear_conv_kernel_dim=4, tie_word_embeddings=False,
                                                layer_types=['linear_attention', 'full_attention', 'linear_attention', 'full_attention'],
                                                **{**{k: v for k, v in COMMON.items() if k != 'rope_theta'}, 'num_hidden_layers': 4},
                                                rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.25}),
                    'Qwen3_5ForCausalLM'),
        'qwen3_5_moe': (lambda: T.Qwen3_5MoeTextConfig(head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                                                       linear_value_head_dim=16, linear_conv_kernel_dim=4, tie_word_embeddings=False,
                                                       layer_types=['linear_attention', 'full_attention'], num_experts=4, num_experts_per_tok=2,
                                                       moe_intermediate_size=64, shared_expert_intermediate_size=96,
                                                       **{k: v for k, v in COMMON.items() if k not in ('rope_theta', 'intermediate_size')},
                                                       rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.25}),
                        'Qwen3_5MoeForCausalLM'),
        'qwen3_next': (lambda: T.Qwen3NextConfig(head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                                                 linear_value_head_dim=16, linear_conv_kernel_dim=4, tie_word_embeddings=False,
                                                 layer_types=['linear_attention', 'full_attention'], num_experts=4, num_experts_per_tok=2,
                                                 moe_intermediate_size=64, shared_expert_intermediate_size=96, norm_topk_prob=True,
                                                 decoder_sparse_step=1, mlp_only_layers=[],
                                                 **{k: v for k, v in COMMON.items() if k != 'rope_theta'},
                                                 rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.25}),
                       'Qwen3NextForCausalLM'),
        # GLM-4 family: rotary on half the head with (2i, 2i+1) pairs, biased q|k|v, fused gate_up; glm4 adds post-sub-layer norms
        'glm': (lambda: T.GlmConfig(head_dim=32, pad_token_id=0, tie_word_embeddings=False, **{k: v for k, v in COMMON.items() if k != 'rope_theta'},
                                    rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.5}), 'GlmForCausalLM'),
        'glm4': (lambda: T.Glm4Config(head_dim=32, pad_token_id=0, tie_word_embeddings=False, **{k: v for k, v in COMMON.items() if k != 'rope_theta'},
                                      rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.5}), 'Glm4ForCausalLM'),
        # Phi-3: q|k|v and gate|up fused in the checkpoint, rotary on three quarters of the head; the long-context variant
        # divides the frequencies by per-dimension factors (short ones up to the original window, long ones beyond)
        'phi3': (lambda: T.Phi3Config(pad_token_id=0, tie_word_embeddings=False, **{k: v for k, v in COMMON.items() if k != 'rope_theta'},
                                      rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.75}), 'Phi3ForCausalLM'),
        'phi3_longrope': (lambda: T.Phi3Config(pad_token_id=0, tie_word_embeddings=False, original_max_position_embeddings=64,
                                               **{k: v for k, v in COMMON.items() if k != 'rope_theta'},
                                               rope_parameters={'rope_type': 'longrope', 'rope_theta': 10000.0, 'original_max_position_embeddings': 64,
                                                                'short_factor': [1.0 + 0.05 * i for i in range(16)],
                                                                'long_factor': [1.5 + 0.2 * i for i in range(16)]}), 'Phi3ForCausalLM'),
        # Gemma: "1 + w" norms, tanh-GELU gate, embeddings times √hidden, tied head
        'gemma': (lambda: T.GemmaConfig(head_dim=32, **COMMON), 'GemmaForCausalLM'),
        # Gemma-2: sliding-window layers alternate with global ones, scores and output logits soft-capped, four norms per layer,
        # softmax scale from query_pre_attn_scalar.  Gemma-3 (text): q/k norms, five local layers per global one, local layers with a
        # rotary base of their own, linear position scaling on the global layers
        'gemma2': (lambda: T.Gemma2Config(head_dim=32, sliding_window=16, query_pre_attn_scalar=24, **COMMON), 'Gemma2ForCausalLM'),
        'gemma3': (lambda: T.Gemma3TextConfig(head_dim=32, sliding_window=16, query_pre_attn_scalar=24,
                                              **{**{k: v for k, v in COMMON.items() if k != 'rope_theta'}, 'num_hidden_layers': 6},
                                              rope_parameters={'full_attention': {'rope_type': 'linear', 'factor': 8.0, 'rope_theta': 1000000.0},
                                                               'sliding_attention': {'rope_type': 'default', 'rope_theta': 10000.0}}), 'Gemma3ForCausalLM'),
        'mistral_window': (lambda: T.MistralConfig(sliding_window=16, **COMMON), 'MistralForCausalLM'),
        # OLMo-2: norms on the sub-layer outputs only, q / k norms over the whole projection
        'olmo2': (lambda: T.Olmo2Config(tie_word_embeddings=False, **COMMON), 'Olmo2ForCausalLM'),
        'olmo3': (lambda: T.Olmo3Config(tie_word_embeddings=False, sliding_window=16, **{**COMMON, 'num_hidden_layers': 4}), 'Olmo3ForCausalLM'),
        # ERNIE-4.5: rotary pairs (2i, 2i+1) over the whole head; SmolLM3: every fourth layer without position information
        'ernie4_5': (lambda: T.Ernie4_5Config(head_dim=32, tie_word_embeddings=False, use_bias=False, **COMMON), 'Ernie4_5ForCausalLM'),
        'smollm3': (lambda: T.SmolLM3Config(tie_word_embeddings=True, pad_token_id=0, **{**COMMON, 'num_hidden_layers': 4}), 'SmolLM3ForCausalLM'),
        # Granite: Llama with four constants (embeddings ×, softmax scale, residual ×, logits ÷)
        'granite': (lambda: T.GraniteConfig(tie_word_embeddings=True, embedding_multiplier=12.0, attention_multiplier=0.0078125 * 4, residual_multiplier=0.22,
                                            logits_scaling=8.0, **COMMON), 'GraniteForCausalLM'),
        'llama_dynamic_ntk': (lambda: T.LlamaConfig(tie_word_embeddings=False, **{**COMMON, 'max_position_embeddings': 64},
                                                    rope_scaling={'rope_type': 'dynamic', 'factor': 2.0}), 'LlamaForCausalLM'),
        # DeepSeek-V3: latent attention (query bottleneck, shared rotary key head, 48-wide scores / 24-wide values), a dense first
        # layer, sigmoid router with selection bias and expert groups, ungated shared expert
        'deepseek_v3': (lambda: T.DeepseekV3Config(moe_intermediate_size=64, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, n_group=4,
                                                   topk_group=2, first_k_dense_replace=1, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=32,
                                                   qk_rope_head_dim=16, v_head_dim=24, routed_scaling_factor=2.5, norm_topk_prob=True,
                                                   tie_word_embeddings=False, **{**COMMON, 'num_hidden_layers': 3, 'num_key_value_heads': 4}),
                        'DeepseekV3ForCausalLM'),
        # DeepSeek-V2 (Lite form: plain query projection): softmax scores, groups ranked by their best expert, weights scaled but not renormalised
        'deepseek_v2': (lambda: T.DeepseekV2Config(moe_intermediate_size=64, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=2, n_group=4,
                                                   topk_group=2, topk_method='group_limited_greedy', first_k_dense_replace=1, q_lora_rank=None,
                                                   kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=24, routed_scaling_factor=16.0,
                                                   tie_word_embeddings=False, **{**COMMON, 'num_hidden_layers': 3, 'num_key_value_heads': 4}),
                        'DeepseekV2ForCausalLM'),
        'deepseek_v3_yarn': (lambda: T.DeepseekV3Config(moe_intermediate_size=64, n_routed_experts=4, n_shared_experts=2, num_experts_per_tok=2, n_group=1,
                                                        topk_group=1, first_k_dense_replace=0, q_lora_rank=None, kv_lora_rank=32, qk_nope_head_dim=32,
                                                        qk_rope_head_dim=16, v_head_dim=32, routed_scaling_factor=1.0, norm_topk_prob=False,
                                                        tie_word_embeddings=False, **{**COMMON, 'num_key_value_heads': 4, 'max_position_embeddings': 4096},
                                                        rope_scaling={'rope_type': 'yarn', 'factor': 40.0, 'beta_fast': 32, 'beta_slow': 1, 'mscale': 1.0,
                                                                      'mscale_all_dim': 1.0, 'original_max_position_embeddings': 64}),
                             'DeepseekV3ForCausalLM'),
        # GLM-4.5: DeepSeek-V3's routing over grouped-query attention with q/k norms, biased q|k|v and rotary on half the head
        'glm4_moe': (lambda: T.Glm4MoeConfig(head_dim=32, moe_intermediate_size=64, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, n_group=2,
                                             topk_group=1, first_k_dense_replace=1, routed_scaling_factor=1.5, norm_topk_prob=True, use_qk_norm=True,
                                             attention_bias=True, tie_word_embeddings=False, pad_token_id=0,
                                             **{**{k: v for k, v in COMMON.items() if k != 'rope_theta'}, 'num_hidden_layers': 3},
                                             rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.5}),
                     'Glm4MoeForCausalLM'),
        # GPT-OSS: sink logits in the softmax, alternating sliding-window layers, biases on every projection, the router and the
        # experts, softmax over the top-k router logits, clamped gated unit, YaRN without truncation
        'gpt_oss': (lambda: T.GptOssConfig(head_dim=32, num_local_experts=4, num_experts_per_tok=2, sliding_window=16, tie_word_embeddings=False,
                                           **{**{k: v for k, v in COMMON.items() if k != 'rope_theta'}, 'intermediate_size': 64, 'num_hidden_layers': 4},
                                           rope_parameters={'rope_type': 'yarn', 'factor': 8.0, 'beta_fast': 32.0, 'beta_slow': 1.0, 'truncate': False,
                                                            'original_max_position_embeddings': 64, 'rope_theta': 150000.0}), 'GptOssForCausalLM'),
        'qwen2_moe_shared': (lambda: T.Qwen2MoeConfig(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=96,
                                                      norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], **COMMON), 'Qwen2MoeForCausalLM'),
    }


def _hf_model(name):
    make, cls = _cases()[name]
    try:
        cfg = make()
        hf = getattr(transformers, cls)(cfg).float().eval()
    except Exception as e:  # a transformers build without this family or with other argument names
        pytest.skip(f'{name}: {type(e).__name__}: {e}')
    torch.manual_seed(0)
    for n, p in hf.named_parameters():  # non-trivial norms and biases, so that a swapped or dropped tensor shows
        if 'norm' in n:
            torch.nn.init.normal_(p, 1.0, 0.1)
        elif p.dim() == 1:
            torch.nn.init.normal_(p, 0.0, 0.1)
    for mod in hf.modules():       # this transformers build's DeepSeek-V2 group routing reads an attribute its constructor never sets
        if hasattr(mod, 'topk_method') and not hasattr(mod, 'num_experts'):
            mod.num_experts = hf.config.n_routed_experts
    for n, b in hf.named_buffers():
        if n.endswith('e_score_correction_bias'):      # the selection bias is a buffer there; non-zero, so that it matters
            torch.nn.init.normal_(b, 0.0, 0.2)
    return hf


def _ours(path, ids):
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.decoder import PackedBatch
    m = TransformersModel(model_id=path)
    n = ids.shape[0]
    with torch.no_grad():
        return m, m.model.logits(m.model(PackedBatch(ids, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))).float()


@pytest.mark.parametrize('name', list(_cases()))
def test_hf_checkpoint_gives_the_same_logits_here(name, tmp_path):
    hf = _hf_model(name)
    hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
    ids = torch.randint(0, 512, (1, 150 if name in ('llama3_rope', 'phi3_longrope', 'llama_dynamic_ntk', 'deepseek_v3_yarn', 'gpt_oss') else 37), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits[0]
    _, got = _ours(str(tmp_path / 'hf'), ids[0])
    # Gemma-2 / 3 multiply the stream by "1 + w" ≈ 2 four times per layer: the same fp32 rounding shows up a few times larger
    assert torch.allclose(got, want, atol=6e-5 if name in ('gemma2', 'gemma3') else 2e-5), float((got - want).abs().max())


@pytest.mark.parametrize('name', ['qwen3', 'qwen3_moe', 'mixtral', 'qwen2_moe_shared', 'qwen3_5', 'qwen3_5_moe', 'qwen3_next', 'glm', 'glm4', 'phi3',
                                  'phi3_longrope', 'gemma', 'deepseek_v2', 'deepseek_v3', 'deepseek_v3_yarn', 'glm4_moe', 'gemma2', 'gemma3', 'gpt_oss', 'granite', 'olmo2', 'olmo3', 'ernie4_5', 'smollm3'])
def test_checkpoint_saved_here_loads_in_transformers(name, tmp_path):
    hf = _hf_model(name)
    hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
    ids = torch.randint(0, 512, (1, 29), generator=torch.Generator().manual_seed(2))
    m, ours = _ours(str(tmp_path / 'hf'), ids[0])
    out = m.save('export', str(tmp_path / 'ours'))
    back = getattr(transformers, _cases()[name][1]).from_pretrained(out).float().eval()
    for mod in back.modules():
        if hasattr(mod, 'topk_method') and not hasattr(mod, 'num_experts'):
            mod.num_experts = back.config.n_routed_experts
    with torch.no_grad():
        theirs = back(ids).logits[0]
    assert torch.allclose(ours, theirs, atol=6e-5 if name in ('gemma2', 'gemma3') else 2e-5), float((ours - theirs).abs().max())


@pytest.mark.parametrize('name', ['qwen3', 'qwen3_moe'])
def test_adapter_saved_in_peft_layout_merges_into_the_hf_model(name, tmp_path):
    """PEFT key names and the split of fused projections: merging ``scale · B @ A`` of every saved adapter tensor into
    the Hugging Face weight it names must reproduce the logits of the adapted model here."""
    from safetensors.torch import load_file
    from twinkle_b200.model import LoraConfig
    from twinkle_b200.models.decoder import PackedBatch
    hf = _hf_model(name)
    hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
    ids = torch.randint(0, 512, (1, 33), generator=torch.Generator().manual_seed(3))
    m, base = _ours(str(tmp_path / 'hf'), ids[0])
    m.add_adapter_to_model('a', LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    m.set_optimizer('AdamW', lr=5e-2, adapter_name='a')
    batch = [{'input_ids': ids[0, :-1].tolist(), 'labels': ids[0, 1:].tolist()}]
    for _ in range(2):                                       # B starts at zero: two steps make the adapter matter
        m.forward_backward(inputs=batch, adapter_name='a')
        m.clip_grad_and_step(adapter_name='a')
    out = m.save('adapter', str(tmp_path / 'ad'), adapter_name='a')
    n = ids.shape[1]
    with torch.no_grad():
        adapted = torch.as_tensor(m.forward_only(inputs=[{'input_ids': ids[0].tolist(), 'labels': ids[0].tolist()}], adapter_name='a', return_logits=True)['logits']).float()
    adapted = adapted.reshape(-1, adapted.shape[-1])[:n]
    assert float((adapted - base).abs().max()) > 1e-3         # the adapter changed the model
    import json
    cfg = json.load(open(out + '/adapter_config.json'))
    assert cfg['peft_type'] == 'LORA' and cfg['r'] == 4
    scale = cfg['lora_alpha'] / cfg['r']
    sd = load_file(out + '/adapter_model.safetensors')
    params = dict(hf.named_parameters())
    merged = 0
    with torch.no_grad():
        for k, a in sd.items():
            if '.lora_A.' not in k:
                continue
            b = sd[k.replace('.lora_A.', '.lora_B.')]
            target = k[len('base_model.model.'):].replace('.lora_A.weight', '')
            if target + '.weight' in params:
                params[target + '.weight'] += scale * (b.float() @ a.float())
                merged += 1
            else:                                             # fused expert tensors of newer transformers: [E, out, in] per expert index
                pytest.skip(f'{target}: this transformers build stores the module differently')
    assert merged > 0
    with torch.no_grad():
        theirs = hf(ids).logits[0]
    assert torch.allclose(adapted, theirs, atol=5e-5), float((adapted - theirs).abs().max())


def test_unknown_architectures_are_refused_not_guessed(tmp_path, monkeypatch):
    """Cohere's Command models share their config fields with Llama but run attention and feed-forward block in parallel from
    one LayerNorm and scale their logits: loading one as a Llama would run and be wrong.  Unknown ``model_type`` values are
    refused unless explicitly allowed."""
    from twinkle_b200.models.config import DecoderConfig
    cfg = {'model_type': 'cohere', 'hidden_size': 128, 'num_attention_heads': 4, 'num_hidden_layers': 2, 'vocab_size': 512}
    with pytest.raises(NotImplementedError, match='cohere'):
        DecoderConfig.from_hf(cfg)
    monkeypatch.setenv('TWINKLE_ALLOW_UNKNOWN_ARCH', '1')
    assert DecoderConfig.from_hf(cfg).hidden_size == 128
    monkeypatch.delenv('TWINKLE_ALLOW_UNKNOWN_ARCH')
    with pytest.raises(NotImplementedError):
        DecoderConfig.from_hf({'model_type': 'qwen2_vl', 'text_config': {'model_type': 'qwen2_vl_text'}, 'vision_config': {'model_type': 'siglip'}})


@pytest.mark.parametrize('name', ['qwen3', 'glm4', 'qwen3_5'])
def test_adapter_trained_here_merges_into_the_hf_model(name, tmp_path):
    """PEFT-shaped adapter tensors exported here, merged by hand into the Hugging Face model's own projections
    (``W += α/r · B A``), give the logits this package computes with the adapter active — also where the checkpoint orders
    rows differently (GLM's rotary pairing, Qwen3.5's query | gate interleave)."""
    from twinkle_b200.model import MultiLoraTransformersModel
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.models.layers import lora_batch
    hf = _hf_model(name)
    hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
    m = MultiLoraTransformersModel(model_id=str(tmp_path / 'hf'), device='cpu', max_loras=2, max_r=8, seed=0)
    m.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8, 'target_modules': ['q_proj', 'k_proj', 'v_proj', 'o_proj', 'gate_proj', 'up_proj', 'down_proj']})
    m.set_optimizer('AdamW', lr=2e-2, adapter_name='a')
    g = torch.Generator().manual_seed(5)
    batch = [{'input_ids': (ids := torch.randint(0, 512, (33, ), generator=g))[:-1].tolist(), 'labels': ids[1:].tolist()}]
    for _ in range(3):
        m.forward_backward(inputs=batch, adapter_name='a')
        m.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
    ids = torch.randint(0, 512, (29, ), generator=torch.Generator().manual_seed(6))
    n = ids.shape[0]
    with torch.no_grad(), lora_batch(m.multi_lora.batch_for('a', n, 'cpu')):
        ours = m.model.logits(m.model(PackedBatch(ids, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))).float()
    with torch.no_grad():
        base = hf(ids[None]).logits[0]
    sd = m.multi_lora.get_state_dict('a')
    params = dict(hf.named_parameters())
    merged = 0
    with torch.no_grad():
        for k, a in sd.items():
            if not k.endswith('lora_A.weight'):
                continue
            b = sd[k.replace('lora_A', 'lora_B')]
            target = k[len('base_model.model.'):-len('.lora_A.weight')] + '.weight'
            if target not in params and target.replace('model.', 'model.language_model.', 1) in params:
                target = target.replace('model.', 'model.language_model.', 1)
            if target not in params:        # a projection the checkpoint keeps fused (GLM's gate_up): the adapter covers its half of the rows
                fused = target.replace('mlp.gate_proj', 'mlp.gate_up_proj').replace('mlp.up_proj', 'mlp.gate_up_proj')
                assert fused in params, target
                w = params[fused]
                half = w.shape[0] // 2
                rows = slice(0, half) if 'gate_proj' in k else slice(half, None)
                w[rows] += (b.float() @ a.float()) * 2.0
            else:
                params[target] += (b.float() @ a.float()) * 2.0
            merged += 1
        theirs = hf(ids[None]).logits[0]
    assert merged >= 7 and not torch.allclose(base, theirs, atol=1e-3)
    assert torch.allclose(ours, theirs, atol=5e-5), float((ours - theirs).abs().max())


def test_internlm2_checkpoint_layout(tmp_path):
    """InternLM2 is the Llama computation under other tensor names, with q, k and v in one ``wqkv`` grouped per key / value
    head.  Its modelling code is not part of ``transformers``, so the checkpoint is built here from a Llama model by that
    renaming; it must give the Llama logits, and saving it again must reproduce the file tensor for tensor."""
    import json
    import os

    from safetensors.torch import load_file, save_file
    hf = _hf_model('llama3_rope')
    cfg = hf.config
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size // cfg.num_attention_heads
    sd, out = hf.state_dict(), {}
    out['model.tok_embeddings.weight'], out['model.norm.weight'], out['output.weight'] = sd['model.embed_tokens.weight'], sd['model.norm.weight'], sd['lm_head.weight']
    for i in range(cfg.num_hidden_layers):
        a, b = f'model.layers.{i}.', f'model.layers.{i}.'
        q, k, v = (sd[a + f'self_attn.{p}_proj.weight'] for p in 'qkv')
        g = hq // hkv
        out[b + 'attention.wqkv.weight'] = torch.cat([q.reshape(hkv, g * d, -1), k.reshape(hkv, d, -1), v.reshape(hkv, d, -1)], 1).reshape(-1, q.shape[1])
        for src, dst in (('self_attn.o_proj', 'attention.wo'), ('mlp.gate_proj', 'feed_forward.w1'), ('mlp.up_proj', 'feed_forward.w3'),
                         ('mlp.down_proj', 'feed_forward.w2'), ('input_layernorm', 'attention_norm'), ('post_attention_layernorm', 'ffn_norm')):
            out[b + dst + '.weight'] = sd[a + src + '.weight']
    path = str(tmp_path / 'internlm2')
    os.makedirs(path)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(path, 'model.safetensors'), metadata={'format': 'pt'})
    conf = {k: v for k, v in cfg.to_dict().items() if k in ('vocab_size', 'hidden_size', 'intermediate_size', 'num_hidden_layers', 'num_attention_heads',
                                                            'num_key_value_heads', 'max_position_embeddings', 'rms_norm_eps', 'tie_word_embeddings')}
    conf.update(model_type='internlm2', architectures=['InternLM2ForCausalLM'], bias=False, rope_theta=10000.0, torch_dtype='float32',
                rope_scaling={'type': 'dynamic', 'factor': 2.0})
    with open(os.path.join(path, 'config.json'), 'w') as f:
        json.dump(conf, f)
    hf.config.rope_parameters = {'rope_type': 'dynamic', 'factor': 2.0, 'rope_theta': 10000.0}          # the Llama twin of that config
    hf = transformers.LlamaForCausalLM(hf.config).float().eval()
    hf.load_state_dict(sd)
    ids = torch.randint(0, 512, (1, 41), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want = hf(ids).logits[0]
    m, got = _ours(path, ids[0])
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    back = load_file(os.path.join(m.save('export', str(tmp_path / 'ours')), 'model.safetensors'))
    assert sorted(back) == sorted(out)
    for k in out:
        assert torch.equal(back[k], out[k]), k


def test_granite_log_probs_carry_the_logit_divisor(tmp_path):
    """The fused head + log-softmax path never forms the scaled logits: it folds Granite's divisor into the temperature."""
    from twinkle_b200.models.decoder import PackedBatch
    hf = _hf_model('granite')
    hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
    ids = torch.randint(0, 512, (1, 33), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = torch.log_softmax(hf(ids).logits[0, :-1].float() / 0.7, -1).gather(-1, ids[0, 1:, None])[:, 0]
    m, _ = _ours(str(tmp_path / 'hf'), ids[0])
    n = ids.shape[1]
    with torch.no_grad():
        hidden = m.model(PackedBatch(ids[0], torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))
        got, _ = m.model.token_logprobs(hidden[:-1], ids[0, 1:], temperature=0.7)
    assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())
