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
