"""The cookbook scripts run end to end at tiny scale (CPU) and do what they say."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(f'cookbook_{name}', os.path.join(ROOT, 'cookbook', f'{name}.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_sft_lora_loss_falls(tmp_path):
    losses = _load('sft_lora').main(['--steps', '8', '--out', str(tmp_path)])
    assert losses[-1] < losses[0] - 0.1
    assert os.path.isfile(os.path.join(str(tmp_path), 'adapter', 'adapter_model.safetensors'))


def test_grpo_multi_lora_two_tenants():
    hist = _load('grpo_multi_lora').main(['--steps', '1', '--tenants', '2', '--prompts', '2', '--group', '2', '--max-tokens', '6'])
    assert [h['tenant'] for h in hist] == ['tenant0', 'tenant1'] and all(0.0 <= h['reward'] <= 1.0 for h in hist)


def test_dpo_loss_falls():
    losses = _load('dpo').main(['--steps', '4'])
    assert losses[-1] < losses[0]


def test_server_cookbook_native_backend():
    losses = _load('server_tinker_client').main(['--backend', 'native', '--steps', '2'])
    assert losses[1] < losses[0]


def test_gkd_off_and_on_policy():
    off = _load('gkd').main(['--steps', '4'])
    assert off[-1] < off[0]
    on = _load('gkd').main(['--mode', 'on', '--steps', '2', '--max-tokens', '6'])
    assert len(on) == 2 and all(x == x and x >= 0 for x in on)
    topk = _load('gkd').main(['--steps', '3', '--topk', '8'])
    assert topk[-1] < topk[0]


def test_embedding_infonce_learns_retrieval():
    r = _load('embedding_infonce').main(['--steps', '15'])
    assert r['losses'][-1] < 0.2 * r['losses'][0] and r['acc_after'] >= r['acc_before'] and r['acc_after'] == 1.0


def test_moe_routing_replay():
    r = _load('moe_routing_replay').main([])
    assert r['matches_sampler'] and r['replay_kept'] and not r['free_kept']
    assert all(rec == n - 1 for rec, n in zip(r['recorded'], r['lens']))     # every fed token recorded: prompt and decode steps


def test_server_twinkle_client_native_backend():
    r = _load('server_twinkle_client').main(['--backend', 'native', '--epochs', '2'])
    assert r['losses'][-1] < r['losses'][0] and r['path'].startswith('twinkle://') and len(r['tokens']) == 4
    assert any(run.get('training_run_id') or run.get('run_id') or run for run in r['runs'])


def test_http_twin_positional_arguments():
    import pytest
    from twinkle_b200.client import MultiLoraTransformersModel
    seen = {}
    twin = MultiLoraTransformersModel.__new__(MultiLoraTransformersModel)
    twin._call = lambda method, adapter, **kw: seen.update(method=method, adapter=adapter, kw=kw)
    twin.set_optimizer('AdamW', lr=1e-3, adapter_name='a')
    assert seen == dict(method='set_optimizer', adapter='a', kw=dict(optimizer_cls='AdamW', lr=1e-3))
    with pytest.raises(TypeError):
        twin.set_optimizer('AdamW', 'extra')
    with pytest.raises(TypeError):
        twin.set_loss('GRPOLoss', loss_cls='DPOLoss')
    twin.forward_backward([{'input_ids': [1]}], adapter_name='a')          # the reference's HTTP twin takes the batch by position
    assert seen['method'] == 'forward_backward' and seen['kw'] == dict(inputs=[{'input_ids': [1]}])
    with pytest.raises(TypeError):
        twin.forward_backward([{'input_ids': [1]}], [{'input_ids': [2]}])


def test_sft_pipeline_cli_trains_saves_resumes_and_evaluates(tmp_path):
    mod = _load('sft_pipeline_cli')
    common = ['--model', 'tiny-dense', '--use-lora', 'true', '--lr', '2e-3', '--bs', '4', '--output-dir', str(tmp_path)]
    first = mod.main(common + ['--max-steps', '3'])
    assert first['step'] == 3 and first['consumed'] == 12 and os.path.isdir(first['checkpoint'])
    assert float(first['eval']['loss']) > 0.0                                   # forward_only + calculate_loss feed the evaluation metric
    second = mod.main(common + ['--max-steps', '6', '--resume-from-checkpoint', first['checkpoint']])
    assert second['step'] == 6 and len(second['losses']) == 3 and second['consumed'] == 24
    assert second['losses'][0] < first['losses'][0]                             # continues from the trained adapter, not from scratch
    assert float(second['eval']['loss']) < float(first['eval']['loss'])


def test_grpo_pool_disaggregated_trainer_and_sampler_groups():
    """Two FSDP trainer workers and one sampler worker in separate processes; weights cross through the checkpoint
    engine.  After every sync the sampler's log-probs are the trainer's (bf16 transport rounding only)."""
    hist = _load('grpo_pool_disaggregated').main(['--steps', '3', '--device', 'cpu', '--prompts', '2', '--group', '4', '--max-tokens', '6'])
    assert len(hist) == 3 and all(h['samples'] == 8 for h in hist)
    assert hist[0]['sync_bytes'] > 10 * hist[1]['sync_bytes'] > 0          # first sync carries the base weights, later ones the adapter
    assert all(h['logp_drift'] < 0.03 for h in hist), hist


def test_tinker_dpo_then_resume_after_server_restart():
    r = _load('server_tinker_dpo_resume').main(['--steps', '3'])
    assert abs(r['losses'][0] - 0.6931) < 1e-3 and r['losses'][-1] < r['losses'][0]       # starts at log 2: policy == reference
    assert r['metrics']['rewards/accuracies'] >= 0.5 and r['metrics']['rewards/margins'] > 0 and 'grad_norm' in r['metrics']
    assert abs(r['next_uninterrupted'][0] - r['next_resumed'][0]) < 1e-4                  # adapter restored exactly
    assert abs(r['next_uninterrupted'][1] - r['next_resumed'][1]) < 1e-4                  # and the Adam moments and step count
    assert r['info']['is_lora'] and r['info']['lora_rank'] == 8 and r['info']['base_model'] == 'tiny-dense'
    assert len(r['runs']) >= 1 and len(r['tokens']) == 4


def test_vision_language_sft_full_and_lora(tmp_path):
    full = _load('mm_sft').main(['--steps', '6', '--batch', '4', '--out', str(tmp_path)])
    assert full[-1] < 0.7 * full[0] and os.path.isfile(os.path.join(str(tmp_path), 'final', 'config.json'))
    lora = _load('mm_sft').main(['--steps', '4', '--batch', '4', '--lora-rank', '4', '--lr', '1e-2'])
    assert lora[-1] < lora[0]


def test_multimodal_grpo_runs_and_keeps_images_in_training_features():
    hist = _load('mm_grpo').main(['--steps', '2', '--prompts', '2', '--group', '2', '--max-tokens', '4'])
    assert len(hist) == 2 and all(h['sequences'] == 4 and h['loss'] == h['loss'] for h in hist)


def test_deepseek_ep_lora_and_megatron_moe_scripts(tmp_path):
    losses = _load('deepseek_ep_lora').main(['--steps', '4', '--seq-len', '48', '--seqs-per-rank', '2', '--out', str(tmp_path)])
    assert losses[-1] < losses[0]
    from safetensors.torch import load_file
    keys = set(load_file(os.path.join(str(tmp_path), 'adapter', 'adapter_model.safetensors')))
    assert any('mlp.experts.gate_up_proj' in k for k in keys) and any('q_b_proj' in k for k in keys) and not any('kv_a_proj_with_mqa' in k for k in keys)
    losses = _load('megatron_tp_moe').main(['--steps', '3', '--seq-len', '48', '--micro-batches', '2'])
    assert losses[-1] < losses[0]


def test_server_config_examples_validate():
    import glob

    from twinkle_b200.server.config import ServerConfig
    files = sorted(glob.glob(os.path.join(ROOT, 'cookbook', 'server_configs', '*.yaml')))
    assert len(files) >= 3
    for f in files:
        cfg = ServerConfig.from_yaml(f)
        assert cfg.applications[0].name == 'gateway'
        for app in cfg.applications:
            assert app.typed_args is not None     # arguments parsed against the schema of that kind of application
