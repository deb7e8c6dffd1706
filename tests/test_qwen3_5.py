"""Qwen3.5 text stack (Gated DeltaNet layers + gated full attention with partial rotary and "1 + w" norms) through the
sharded backend, the multi-LoRA pool and the paged sampler.  Parity with the Hugging Face implementation is in
``test_hf_parity.py``; here: training, the adapter format (query and output gate are one ``q_proj`` for PEFT) and decoding."""
import torch


def _batch(n=2, length=40, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 1024, (length + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


def test_config_round_trip_and_rotary_width():
    from twinkle_b200.models import preset
    from twinkle_b200.models.config import DecoderConfig
    cfg = preset('tiny-qwen3.5')
    assert cfg.rotary_dim == 16 and cfg.attn_output_gate and cfg.rms_norm_offset == 1.0
    hf = cfg.to_hf()
    assert hf['model_type'] == 'qwen3_5_text' and hf['architectures'] == ['Qwen3_5ForCausalLM']
    assert hf['rope_parameters']['partial_rotary_factor'] == 0.25 and hf['layer_types'].count('full_attention') == 1
    back = DecoderConfig.from_hf(hf)
    assert (back.partial_rotary_factor, back.attn_output_gate, back.rms_norm_offset, back.layer_types) == (0.25, True, 1.0, cfg.layer_types)
    assert preset('tiny-dense').rotary_dim == 64            # full rotary everywhere else


def test_full_parameter_training_reduces_the_loss():
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-qwen3.5', seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    losses = []
    for _ in range(4):
        losses.append(m.forward_backward(inputs=_batch())['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < losses[0] - 0.2, losses


def test_adapter_keeps_query_and_gate_in_one_q_proj(tmp_path):
    """The gate part shares the adapter's A with the query part; the exported B interleaves their rows per head the way
    the checkpoint's q_proj does, and loading it into a fresh pool reproduces the tenant's outputs."""
    from twinkle_b200.model import MultiLoraTransformersModel
    from twinkle_b200.models.layers import Linear

    def make():
        m = MultiLoraTransformersModel(model_id='tiny-qwen3.5', seed=0, device='cpu', max_loras=2, max_r=8)
        m.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8, 'target_modules': 'all-linear'})
        m.set_optimizer('AdamW', lr=5e-3, adapter_name='a')
        return m

    m = make()
    attn = next(l for l in m.model.layers if not getattr(l, 'is_linear', False)).self_attn
    qkv: Linear = attn.qkv_proj
    assert qkv.lora_A['q_gate'] is qkv.lora_A['q_proj'] and qkv.gate_head_dim == 64
    for _ in range(3):
        m.forward_backward(inputs=_batch(), adapter_name='a')
        m.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
    sd = m.multi_lora.get_state_dict('a')
    kb = [k for k in sd if k.endswith('self_attn.q_proj.lora_B.weight')]
    assert len(kb) == 1 and sd[kb[0]].shape == (2 * 4 * 64, 4) and not any('q_gate' in k for k in sd)
    assert float(sd[kb[0]].reshape(4, 128, 4)[:, 64:].abs().sum()) > 0          # the gate rows were trained too
    want = m.forward_only(inputs=_batch(seed=9), adapter_name='a')['logps']
    fresh = make()
    unused = fresh.multi_lora.set_state_dict('a', sd)
    assert unused == []
    got = fresh.forward_only(inputs=_batch(seed=9), adapter_name='a')['logps']
    base = fresh.forward_only(inputs=_batch(seed=9), adapter_name='a', disable_lora=True)['logps']
    assert torch.allclose(torch.as_tensor(want), torch.as_tensor(got), atol=1e-5)
    assert not torch.allclose(torch.as_tensor(base), torch.as_tensor(got), atol=1e-4)        # and the adapter does something


def test_sampler_decodes_with_gate_partial_rotary_and_linear_state():
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.sampler import TorchSampler
    s = TorchSampler(model_id='tiny-qwen3.5', weight_seed=0, enable_lora=False, device='cpu')
    prompts = [{'input_ids': [5, 6, 7, 8, 9, 10]}, {'input_ids': [11, 12]}]
    resps = s.sample(prompts, SamplingParams(max_tokens=5, temperature=1.0, seed=4, logprobs=1))
    for p, r in zip(prompts, resps):
        seq = r.sequences[0]
        ids = torch.tensor(p['input_ids'] + seq.tokens)
        n = len(ids)
        with torch.no_grad():
            hidden = s.model(PackedBatch(ids, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))
            lp, _ = s.model.token_logprobs(hidden[:-1], ids[1:])
        assert torch.allclose(torch.tensor(seq.logprobs), lp[len(p['input_ids']) - 1:].float(), atol=2e-4)
