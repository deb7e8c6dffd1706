"""Sliding-window layers, soft-capped scores and logits, per-layer rotary bases (Mistral-v0.1 / Phi-3 windows, Gemma-2,
Gemma-3): the attention forms against an explicit mask, training through the sharded backend, and the paged sampler, which
must apply the same window and cap while decoding.  Parity with Hugging Face is in ``test_hf_parity.py``."""
import torch


def _gemma_like(**kw):
    from twinkle_b200.models import preset
    base = dict(model_type='gemma3_text', num_hidden_layers=4, sliding_window=8, layer_types=['sliding_attention', 'sliding_attention', 'full_attention', 'sliding_attention'],
                sandwich_norm=True, rms_norm_offset=1.0, hidden_act='gelu_pytorch_tanh', embed_scale=16.0, query_pre_attn_scalar=48.0,
                rope_local_theta=1e3, rope_scaling={'rope_type': 'linear', 'factor': 4.0}, qk_norm=True)
    base.update(kw)
    return preset('tiny-dense', **base)


def test_window_and_softcap_against_an_explicit_mask():
    from twinkle_b200 import ops
    g = torch.Generator().manual_seed(0)
    T, H, D, W, cap = 23, 2, 16, 5, 3.0
    q, k, v = (torch.randn(T, H, D, generator=g) for _ in range(3))
    cu = torch.tensor([0, 9, 23], dtype=torch.int32)
    out = ops.flash_attn_varlen(q, k, v, cu, 14, True, 0.3, window=W, softcap=cap)
    ref = torch.empty_like(out)
    for a, b in ((0, 9), (9, 23)):
        s = torch.einsum('ihd,jhd->hij', q[a:b], k[a:b]) * 0.3
        s = torch.tanh(s / cap) * cap
        i, j = torch.arange(b - a)[:, None], torch.arange(b - a)[None, :]
        s = s.masked_fill((j > i) | (i - j >= W), float('-inf'))
        ref[a:b] = torch.einsum('hij,jhd->ihd', torch.softmax(s, -1), v[a:b])
    assert torch.allclose(out, ref, atol=1e-6)
    # a window no row reaches is plain causal attention
    assert torch.equal(ops.flash_attn_varlen(q, k, v, cu, 14, True, 0.3, window=14), ops.flash_attn_varlen(q, k, v, cu, 14, True, 0.3))


def test_config_keeps_per_layer_windows():
    from twinkle_b200.models.config import DecoderConfig
    cfg = _gemma_like()
    assert [cfg.layer_window(i) for i in range(4)] == [8, 8, None, 8] and abs(cfg.attn_scale - 48.0**-0.5) < 1e-12
    back = DecoderConfig.from_hf(cfg.to_hf())
    assert back.layer_types == cfg.layer_types and back.sliding_window == 8 and back.rope_local_theta == 1e3
    assert back.rope_scaling['rope_type'] == 'linear' and back.embed_scale == 16.0 and back.sandwich_norm and back.qk_norm
    mistral = DecoderConfig.from_hf({'model_type': 'mistral', 'hidden_size': 256, 'num_attention_heads': 4, 'sliding_window': 4096})
    assert mistral.layer_window(0) == 4096
    qwen = DecoderConfig.from_hf({'model_type': 'qwen2', 'hidden_size': 256, 'num_attention_heads': 4, 'sliding_window': 4096})
    assert qwen.layer_window(0) is None                  # that family carries a window size that is switched off


def test_training_and_sampling_apply_the_same_window():
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.sampler import TorchSampler
    cfg = _gemma_like(model_type='gemma2', attn_logit_softcapping=20.0, final_logit_softcapping=10.0, rope_local_theta=None, rope_scaling=None, qk_norm=False)
    m = TransformersModel(config=cfg, seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(3)
    feats = []
    for _ in range(2):
        ids = torch.randint(0, 1024, (41, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    losses = []
    for _ in range(4):
        losses.append(m.forward_backward(inputs=feats)['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < losses[0] - 0.1, losses
    for c in (cfg, _gemma_like()):
        s = TorchSampler(config=c, weight_seed=0, enable_lora=False, device='cpu')
        prompts = [{'input_ids': list(range(5, 18))}, {'input_ids': [11, 12]}]       # the first prompt is already longer than the window
        resps = s.sample(prompts, SamplingParams(max_tokens=6, temperature=1.0, seed=4, logprobs=1))
        for p, r in zip(prompts, resps):
            seq = r.sequences[0]
            ids = torch.tensor(p['input_ids'] + seq.tokens)
            n = len(ids)
            with torch.no_grad():
                hidden = s.model(PackedBatch(ids, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))
                lp, _ = s.model.token_logprobs(hidden[:-1], ids[1:])
            assert torch.allclose(torch.tensor(seq.logprobs), lp[len(p['input_ids']) - 1:].float(), atol=2e-4)
