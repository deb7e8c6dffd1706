"""Behavioural contracts a user of the reference relies on: LoRA slot pool rules, checkpoint directory layout,
sampling contract, Tinker datum mapping."""
import json
import os

import pytest
import torch


def test_multi_lora_slot_pool_rules():
    from twinkle_b200.model.multi_lora import LoraConfig, MultiLora
    from twinkle_b200.models import PackedBatch, build_model, lora_batch, preset
    model = build_model(preset('tiny-dense'), seed=0)
    ml = MultiLora(model, max_loras=2, max_r=8)
    a = ml.acquire_lora('a', LoraConfig(r=4, lora_alpha=8, target_modules=['q_proj', 'v_proj']))
    b = ml.acquire_lora('b', LoraConfig(r=8, lora_alpha=16, target_modules='all-linear', use_rslora=True))
    assert {a, b} == {0, 1}
    with pytest.raises(ValueError):
        ml.acquire_lora('a', LoraConfig(r=4))                     # tenant exists
    with pytest.raises(RuntimeError):
        ml.acquire_lora('c', LoraConfig(r=4))                     # no free slot
    ml.release_lora('b')
    with pytest.raises(ValueError):
        ml.acquire_lora('c', LoraConfig(r=16))                    # rank above the pool rank
    assert ml.tenants['a'].config.scaling == 8 / 4 and LoraConfig(r=16, lora_alpha=32, use_rslora=True).scaling == 32 / 4
    # with B = 0 the adapter is the identity; setting B on a non-target module changes nothing
    ids = torch.arange(1, 33)
    batch = PackedBatch(ids, torch.arange(32), torch.tensor([0, 32], dtype=torch.int32), 32)
    with torch.no_grad():
        base = model(batch)
        with lora_batch(ml.batch_for('a', 32, 'cpu')):
            assert torch.allclose(model(batch), base, atol=1e-6)
        slot = ml.tenants['a'].slot
        for n, p in ml.pool_parameters():
            if 'lora_B' in n and 'o_proj' in n:
                p[slot].fill_(0.5)                                 # o_proj is not targeted by tenant a
        with lora_batch(ml.batch_for('a', 32, 'cpu')):
            assert torch.allclose(model(batch), base, atol=1e-6)
        for n, p in ml.pool_parameters():
            if 'lora_B' in n and 'q_proj' in n:
                p[slot].fill_(0.5)
        with lora_batch(ml.batch_for('a', 32, 'cpu')):
            assert not torch.allclose(model(batch), base, atol=1e-4)
    sd = ml.get_state_dict('a')
    assert all('.lora_A.weight' in k or '.lora_B.weight' in k for k in sd) and all('o_proj' not in k for k in sd)
    ra = next(v for k, v in sd.items() if k.endswith('q_proj.lora_A.weight'))
    assert ra.shape[0] == 4                                        # saved at the tenant's own rank, not the pool rank
    ml.release_lora('a')
    assert ml.free_slots() == 2
    for n, p in ml.pool_parameters():
        if 'lora_B' in n:
            assert float(p.abs().max()) == 0.0                     # release zeroes B (and restores A)


def test_checkpoint_directory_layout_and_resume(tmp_path):
    from twinkle_b200.model import LoraConfig, TransformersModel
    m = TransformersModel(model_id='tiny-dense', seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    m.set_lr_scheduler('LinearWarmupScheduler', num_warmup_steps=1, num_training_steps=10)
    feats = [{'input_ids': list(range(1, 33)), 'labels': list(range(2, 34))}]
    for _ in range(2):
        m.forward_backward(inputs=feats)
        m.clip_grad_and_step()
    path = m.save('step2', str(tmp_path), save_optimizer=True)
    files = set(os.listdir(path))
    assert 'config.json' in files and any(f.endswith('.safetensors') for f in files)
    assert {'optimizer.pt', 'scheduler.pt', 'rng_state.pt', 'trainer_state.json'} <= files
    st = json.load(open(os.path.join(path, 'trainer_state.json')))
    assert st['cur_step'] == 2 and 'consumed_train_samples' in st and 'gradient_accumulation_steps' in st
    before = {k: v.clone() for k, v in m.get_state_dict().items()}
    m2 = TransformersModel(model_id='tiny-dense', seed=1)          # different init
    m2.set_optimizer('AdamW', lr=1e-3)
    m2.load('step2', str(tmp_path), load_optimizer=True)
    info = m2.resume_from_checkpoint(path)
    assert info['cur_step'] == 2
    after = m2.get_state_dict()
    assert all(torch.equal(before[k], after[k]) for k in before)
    # adapter checkpoints: PEFT layout, adapter name stripped from the keys
    l = TransformersModel(model_id='tiny-dense', seed=0)
    l.add_adapter_to_model('t', LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    l.set_optimizer('AdamW', lr=1e-3, adapter_name='t')
    l.forward_backward(inputs=feats, adapter_name='t')
    l.clip_grad_and_step(adapter_name='t')
    ap = l.save('ad', str(tmp_path), adapter_name='t')
    assert {'adapter_config.json', 'adapter_model.safetensors'} <= set(os.listdir(ap))
    from safetensors.torch import load_file
    keys = list(load_file(os.path.join(ap, 'adapter_model.safetensors')))
    assert keys and all(k.startswith('base_model.model.') and '.t.' not in k for k in keys)
    assert json.load(open(os.path.join(ap, 'adapter_config.json')))['r'] == 4


def test_sampling_contract_cpu():
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.sampler import TorchSampler
    s = TorchSampler(model_id='tiny-dense', weight_seed=0, enable_lora=False)
    prompt = {'input_ids': [5, 6, 7, 8]}
    r, = s.sample([prompt], SamplingParams(max_tokens=5, temperature=1.0, top_p=0.9, num_samples=3, seed=1, logprobs=1))
    assert len(r.sequences) == 3
    for seq in r.sequences:
        assert seq.stop_reason in ('stop', 'length') and len(seq.tokens) <= 5 and len(seq.logprobs) == len(seq.tokens)
        f = seq.new_input_feature
        n = len(seq.tokens)
        assert f['input_ids'][:4] == [5, 6, 7, 8] and list(f['input_ids'][4:]) == seq.tokens
        # pre-shifted labels: position p−1 predicts the first sampled token, nothing earlier carries a loss
        assert list(f['labels'][3:3 + n]) == seq.tokens and all(l == -100 for l in f['labels'][:3])
        assert all(lp <= 0 for lp in seq.logprobs)                 # processed-distribution log-probs
    again, = s.sample([prompt], SamplingParams(max_tokens=5, temperature=1.0, top_p=0.9, num_samples=3, seed=1, logprobs=1))
    assert [q.tokens for q in again.sequences] == [q.tokens for q in r.sequences]   # seeded draws repeat
    score, = s.sample([prompt], SamplingParams(max_tokens=0, prompt_logprobs=2))
    assert score.sequences == [] and score.prompt_logprobs[0] is None and len(score.prompt_logprobs) == 4
    assert len(score.topk_prompt_logprobs[1]) == 2
    stop, = s.sample([prompt], SamplingParams(max_tokens=8, temperature=0.0, stop=[r.sequences[0].tokens[0]]))
    assert stop.sequences[0].stop_reason in ('stop', 'length')


def test_tinker_datum_mapping():
    from twinkle_b200.server.backends import datum_to_input_feature
    d = {'model_input': {'tokens': [5, 6, 7, 8]},
         'loss_fn_inputs': {'target_tokens': {'data': [6, 7, 8, 9]}, 'weights': {'data': [0, 1, 0, 1]}, 'logprobs': {'data': [-1.0, -2.0, -3.0, -4.0]},
                            'advantages': {'data': [0.5, 0.5, 0.5, 0.5]}}}
    from twinkle_b200.server.backends import split_loss_inputs
    f = datum_to_input_feature(d)
    assert f['input_ids'] == [5, 6, 7, 8] and f['labels'] == [-100, 7, -100, 9]
    assert f['old_logps'] == [-1.0, -2.0, -3.0, -4.0] and f['advantages'] == [0.5] * 4
    kw = split_loss_inputs([f])
    assert kw['old_logps'] == [[-2.0, -4.0]] and kw['advantages'] == [[0.5, 0.5]]    # only target positions reach the loss
    f2 = datum_to_input_feature({'model_input': {'tokens': [1, 2, 3]}, 'loss_fn_inputs': {'target_tokens': {'data': [2, 0, 4]}}})
    assert f2['labels'] == [2, -100, 4]                             # without weights, token id 0 marks "no target"
    chunks = datum_to_input_feature({'model_input': {'chunks': [{'tokens': [1, 2]}, {'tokens': [3]}]}})
    assert chunks['input_ids'] == [1, 2, 3]
