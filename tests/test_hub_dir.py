"""The hub interface against a hub that needs no network: repositories as directories (``dir://``).  Create, push
(synchronous and queued), status, download with and without the weight files, single-file download, token check, the
alias table (reference ``src/twinkle/hub/hub.py:31-657``)."""
import os
import time

import pytest


@pytest.fixture()
def hub(tmp_path, monkeypatch):
    root, cache = tmp_path / 'hub', tmp_path / 'cache'
    root.mkdir()
    monkeypatch.setenv('TWINKLE_DIR_HUB', str(root))
    monkeypatch.setenv('TWINKLE_HUB_CACHE', str(cache))
    return root


def _checkpoint(d):
    os.makedirs(d / 'sub', exist_ok=True)
    (d / 'config.json').write_text('{"a": 1}')
    (d / 'tokenizer.json').write_text('{}')
    (d / 'model.safetensors').write_bytes(b'\x00' * 1024)
    (d / 'sub' / 'notes.txt').write_text('x')
    return d


def test_push_download_and_queue(hub, tmp_path):
    from twinkle_b200.hub import MODEL_ALIASES, HubOperation
    src = _checkpoint(tmp_path / 'ckpt')
    HubOperation.create_model_repo('dir://team/model-a')
    assert (hub / 'team' / 'model-a').is_dir()
    HubOperation.push_to_hub('dir://team/model-a', str(src))
    got = HubOperation.download_model('dir://team/model-a')
    assert sorted(os.listdir(got)) == ['config.json', 'model.safetensors', 'sub', 'tokenizer.json'] and os.path.isfile(os.path.join(got, 'sub', 'notes.txt'))
    # tokenizer-only download leaves the weights out
    light = HubOperation.download_model('dir://team/model-a', ignore_model=True, cache_dir=str(tmp_path / 'light'))
    assert 'model.safetensors' not in os.listdir(light) and 'tokenizer.json' in os.listdir(light)
    only = HubOperation.download_file('dir://team/model-a', allow_patterns='config.json', cache_dir=str(tmp_path / 'one'))
    assert [f for _, _, fs in os.walk(only) for f in fs] == ['config.json']
    # queued upload: status moves from running / completed, wait_for returns the result
    fut = HubOperation.push_to_hub('dir://team/model-b', str(src), async_upload=True)
    assert HubOperation.upload_status('dir://team/model-b') in ('running', 'completed')
    res = HubOperation.wait_for('dir://team/model-b', timeout=30)
    assert res['dir://team/model-b'].endswith('model-b') and HubOperation.upload_status('dir://team/model-b') == 'completed' and fut.done()
    # a failing upload is reported, not raised on the caller's thread
    HubOperation.push_to_hub('dir://../escape', str(src), async_upload=True)
    for _ in range(100):
        if HubOperation.upload_status('dir://../escape') != 'running':
            break
        time.sleep(0.01)
    assert HubOperation.upload_status('dir://../escape') == 'failed'
    assert HubOperation.upload_status('dir://never') == 'unknown'
    # aliases resolve before anything else
    MODEL_ALIASES['short'] = 'dir://team/model-a'
    try:
        assert HubOperation.download_model('short') == got
    finally:
        MODEL_ALIASES.pop('short')
    with pytest.raises(FileNotFoundError):
        HubOperation.download_model('dir://team/missing')


def test_token_check(hub, tmp_path):
    from twinkle_b200.hub import HubOperation
    (hub / '.tokens').write_text('good-token\n')
    src = _checkpoint(tmp_path / 'ckpt')
    assert HubOperation.try_login('good-token') and not HubOperation.try_login('bad')
    with pytest.raises(PermissionError):
        HubOperation.push_to_hub('dir://team/m', str(src), token='bad')
    HubOperation.push_to_hub('dir://team/m', str(src), token='good-token')
    assert (hub / 'team' / 'm' / 'config.json').is_file()
