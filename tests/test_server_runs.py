"""Training-run and checkpoint records of the server (reference ``server/checkpoint/training_run_manager.py``,
``checkpoint_manager.py``): paging newest-first, client save directories behind a pointer record, last-checkpoint
bookkeeping, transient sampler weights, per-token isolation."""
import os
import time

import pytest

from twinkle_b200.server.checkpoint import CheckpointManager, TrainingRunManager, dir_size, token_dir


def _fill(d, n=10):
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, 'adapter_model.safetensors'), 'wb') as f:
        f.write(b'x' * n)


def test_runs_are_paged_newest_first_and_isolated_per_token(tmp_path):
    runs = TrainingRunManager(str(tmp_path))
    for i in range(5):
        runs.save('tok-a', f'run{i}', 'Qwen/Qwen3-8B', lora_config={'rank': 8 + i, 'train_mlp': True}, user_metadata={'i': i})
        os.utime(os.path.join(runs.run_dir('tok-a', f'run{i}'), 'run.json'), (1000 + i, 1000 + i))
    runs.save('tok-b', 'other', 'Qwen/Qwen3-8B')
    page = runs.list_runs('tok-a', limit=2, offset=1)
    assert [r['training_run_id'] for r in page['training_runs']] == ['run3', 'run2']
    assert page['cursor'] == {'offset': 1, 'limit': 2, 'total_count': 5}
    r = runs.get('tok-a', 'run4')
    assert r['lora_rank'] == 12 and r['is_lora'] and r['train_mlp'] is True and r['model_owner'] == token_dir('tok-a')
    assert r['user_metadata'] == {'i': 4} and not r['corrupted']
    assert runs.get('tok-b', 'run4') is None and [x['training_run_id'] for x in runs.list_runs('tok-b')['training_runs']] == ['other']
    assert 'tok-a' not in ''.join(os.listdir(tmp_path))          # the token itself never names a directory
    # an unreadable record is reported, not hidden
    with open(os.path.join(runs.run_dir('tok-a', 'run0'), 'run.json'), 'w') as f:
        f.write('{not json')
    assert runs.get('tok-a', 'run0')['corrupted'] is True
    assert runs.update('tok-a', 'run0', {'x': 1}) is None
    assert runs.get('tok-a', '../run1') is None


def test_client_save_dir_is_reached_through_a_pointer_and_must_be_allowed(tmp_path, monkeypatch):
    root, mine, elsewhere = tmp_path / 'root', tmp_path / 'mine', tmp_path / 'elsewhere'
    for d in (root, mine, elsewhere):
        d.mkdir()
    runs = TrainingRunManager(str(root))
    with pytest.raises(PermissionError):
        runs.save('tok', 'r1', 'base', save_dir=str(mine))
    with pytest.raises(ValueError):
        runs.save('tok', 'r1', 'base', save_dir=str(tmp_path / 'missing'))
    monkeypatch.setenv('TWINKLE_ALLOWED_SAVE_DIRS', str(mine))
    rec = runs.save('tok', 'r1', 'base', save_dir=str(mine))
    assert rec['save_dir'] == os.path.realpath(mine)
    assert runs.run_dir('tok', 'r1').startswith(os.path.realpath(mine))
    assert os.path.isfile(os.path.join(root, token_dir('tok'), 'r1', 'run.json'))       # pointer in the default place
    assert runs.get('tok', 'r1')['base_model'] == 'base'
    assert [r['training_run_id'] for r in runs.list_runs('tok')['training_runs']] == ['r1']
    ck = CheckpointManager(str(root), runs)
    _fill(ck.path_for('tok', 'r1', 'step1'))
    meta = ck.register('tok', 'r1', 'step1')
    assert ck.resolve_load_path('tok', meta['path']).startswith(os.path.realpath(mine))
    with pytest.raises(PermissionError):
        runs.save('tok', 'r2', 'base', user_metadata={'save_dir': str(elsewhere)})


def test_checkpoint_records_and_last_checkpoint_bookkeeping(tmp_path):
    ck = CheckpointManager(str(tmp_path))
    ck.create_run('tok', 'run', 'Qwen/Qwen3-8B', lora_config={'rank': 16, 'train_attn': True}, user_metadata={'who': 'me'})
    _fill(ck.path_for('tok', 'run', 'a'), 100)
    a = ck.register('tok', 'run', 'a')
    time.sleep(0.01)
    _fill(ck.path_for('tok', 'run', 'b'), 50)
    b = ck.register('tok', 'run', 'b', public=True)
    assert a['size_bytes'] >= 100 and a['checkpoint_type'] == 'training' and a['is_lora'] and a['lora_rank'] == 16
    assert a['train_attn'] is True and a['user_metadata'] == {'who': 'me'} and b['public'] is True and a['public'] is False
    assert [m['name'] for m in ck.list_checkpoints('tok', 'run')] == ['a', 'b']
    assert ck.get_run('tok', 'run')['last_checkpoint']['name'] == 'b'
    assert ck.get('tok', 'run', 'weights/a')['path'] == 'twinkle://run/weights/a'
    # sampler weights: only the newest set stays on disk
    _fill(ck.path_for('tok', 'run', 's1', 'sampler_weights'))
    ck.register('tok', 'run', 's1', 'sampler_weights')
    outside = tmp_path / 'outside'
    _fill(str(outside))
    os.symlink(outside, os.path.join(ck.run_dir('tok', 'run'), 'sampler_weights', 'link'))
    _fill(ck.path_for('tok', 'run', 's2', 'sampler_weights'))
    s2 = ck.register('tok', 'run', 's2', 'sampler_weights')
    assert os.listdir(os.path.join(ck.run_dir('tok', 'run'), 'sampler_weights')) == ['s2']
    assert os.path.isfile(outside / 'adapter_model.safetensors')               # the link was removed, not followed
    run = ck.get_run('tok', 'run')
    assert run['last_sampler_checkpoint']['name'] == 's2' and s2['checkpoint_type'] == 'sampler' and run['last_checkpoint']['name'] == 'b'
    # deleting the newest training checkpoint rolls last_checkpoint back
    assert ck.delete('tok', 'run', 'weights/b') and not ck.delete('tok', 'run', 'weights/b') and not ck.delete('tok', 'run', '../x')
    assert ck.get_run('tok', 'run')['last_checkpoint']['name'] == 'a'
    assert ck.delete('tok', 'run', 'a') and ck.get_run('tok', 'run')['last_checkpoint'] is None
    assert ck.parse_path('twinkle://run/sampler_weights/s2') == {'path': 'twinkle://run/sampler_weights/s2', 'training_run_id': 'run',
                                                                 'checkpoint_type': 'sampler', 'checkpoint_id': 'sampler_weights/s2'}
    assert ck.parse_path('/etc/passwd') is None
    info = ck.weights_info('tok', 'twinkle://run/sampler_weights/s2')
    assert info['training_run_id'] == 'run' and info['base_model'] == 'Qwen/Qwen3-8B' and info['lora_rank'] == 16
    assert dir_size(str(outside)) == 10
