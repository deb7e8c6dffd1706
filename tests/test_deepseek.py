"""DeepSeek-V3 family (multi-head latent attention, sigmoid group-limited routing with a selection bias, dense first layers,
ungated shared expert) through the sharded backend, adapters, expert parallelism and the paged sampler.  Parity with the
Hugging Face implementation is in ``test_hf_parity.py``."""
import torch

from tests.dist_utils import run_ranks


def _batch(n=2, length=40, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 1024, (length + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


def test_config_round_trip():
    from twinkle_b200.models import preset
    from twinkle_b200.models.config import DecoderConfig
    cfg = preset('tiny-deepseek')
    assert cfg.is_mla and cfg.rotary_dim == 16 and not cfg.layer_is_moe(0) and cfg.layer_is_moe(1)
    hf = cfg.to_hf()
    assert hf['model_type'] == 'deepseek_v3' and hf['n_routed_experts'] == 8 and hf['n_shared_experts'] == 1 and hf['kv_lora_rank'] == 32
    back = DecoderConfig.from_hf(hf)
    for f in ('q_lora_rank', 'kv_lora_rank', 'qk_nope_head_dim', 'qk_rope_head_dim', 'v_head_dim', 'n_group', 'topk_group', 'routed_scaling_factor',
              'first_k_dense_replace', 'router_scoring', 'router_bias', 'shared_expert_gate', 'shared_expert_intermediate_size', 'num_experts'):
        assert getattr(back, f) == getattr(cfg, f), f
    assert abs(back.attn_scale - 48**-0.5) < 1e-12


def test_full_parameter_and_adapter_training():
    from twinkle_b200.model import MultiLoraTransformersModel, TransformersModel
    m = TransformersModel(model_id='tiny-deepseek', seed=0, device='cpu')
    bias = [p for n, p in m.model.named_parameters() if n.endswith('e_score_correction_bias')]
    assert len(bias) == 2 and not any(p.requires_grad for p in bias)          # steered outside the loss, never by a gradient
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    losses = []
    for _ in range(4):
        losses.append(m.forward_backward(inputs=_batch())['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < losses[0] - 0.2, losses
    ml = MultiLoraTransformersModel(model_id='tiny-deepseek', seed=0, device='cpu', max_loras=2, max_r=8)
    ml.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8, 'target_modules': 'all-linear',
                                  'target_parameters': ['mlp.experts.gate_up_proj', 'mlp.experts.down_proj']})
    ml.set_optimizer('AdamW', lr=1e-2, adapter_name='a')
    losses = []
    for _ in range(4):
        losses.append(ml.forward_backward(inputs=_batch(), adapter_name='a')['loss'])
        ml.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
    assert losses[-1] < losses[0] - 0.05, losses
    keys = set(ml.multi_lora.get_state_dict('a'))
    for part in ('q_a_proj', 'q_b_proj', 'kv_a_proj_with_mqa', 'kv_b_proj', 'o_proj', 'mlp.experts.gate_up_proj', 'shared_expert'):
        assert any(part in k for k in keys), part


def _ep_worker(rank, world):
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    m = TransformersModel(model_id='tiny-deepseek', seed=0, device='cpu', device_mesh=DeviceMesh.from_sizes(dp_size=world, ep_size=world))
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    feats = _batch(n=2 * world)
    out = []
    for _ in range(3):
        o = m.forward_backward(inputs=feats[rank * 2:(rank + 1) * 2])
        m.clip_grad_and_step(max_grad_norm=1.0)
        out.append(o['loss'])
    return out


def test_expert_parallel_matches_one_process():
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-deepseek', seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    ref = []
    for _ in range(3):
        ref.append(m.forward_backward(inputs=_batch(n=4))['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    res = run_ranks(_ep_worker, 2)
    mean = [sum(r[i] for r in res) / 2 for i in range(3)]
    for a, b in zip(ref, mean):
        assert abs(a - b) < 2e-4, (ref, res)


def test_sampler_decodes_latent_attention_from_the_paged_cache():
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.sampler import TorchSampler
    s = TorchSampler(model_id='tiny-deepseek', weight_seed=0, enable_lora=False, device='cpu')
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


def _pp_worker(rank, world):
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    m = MegatronModel(config=preset('tiny-deepseek'), device_mesh=DeviceMesh.from_sizes(pp_size=world, dp_size=1), seed=0)
    m.set_optimizer('AdamW', lr=2e-3)
    out = []
    for _ in range(3):
        out.append(m.forward_backward(inputs=_batch(n=4), micro_batch_size=1)['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    return out


def test_pipeline_stages_match_one_process_and_tensor_parallel_is_refused():
    import pytest

    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-deepseek', seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=2e-3)
    ref = []
    for _ in range(3):
        ref.append(m.forward_backward(inputs=_batch(n=4), micro_batch_size=1)['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    for curve in run_ranks(_pp_worker, 2):           # the dense first layer and the mixture-of-experts layers land on different stages
        for a, b in zip(ref, curve):
            assert abs(a - b) < 2e-4, (ref, curve)
    from twinkle_b200.models import build_model, preset
    from twinkle_b200.parallel.tensor import apply_tensor_parallel

    class _Two:
        world_size, rank = 2, 0

    with pytest.raises(NotImplementedError):
        apply_tensor_parallel(build_model(preset('tiny-deepseek')), preset('tiny-deepseek'), _Two(), False)


def test_adapter_config_can_exclude_modules():
    """PEFT's ``exclude_modules`` (the reference's DeepSeek cookbook keeps one projection out of ``all-linear`` with it)."""
    from twinkle_b200.model import MultiLoraTransformersModel
    ml = MultiLoraTransformersModel(model_id='tiny-deepseek', seed=0, device='cpu', max_loras=1, max_r=8)
    ml.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8, 'target_modules': 'all-linear', 'exclude_modules': ['kv_b_proj', 'o_proj']})
    keys = set(ml.multi_lora.get_state_dict('a'))
    assert any('q_b_proj' in k for k in keys) and not any('kv_b_proj' in k or '.o_proj.' in k for k in keys)
    assert ml.optimizer_groups['a'].adapter_config.to_peft_dict()['exclude_modules'] == ['kv_b_proj', 'o_proj']
