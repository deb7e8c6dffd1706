"""Two tenants on one server-side base model: interleaving their steps must give each the loss curve it gets alone
(separate adapter slots, gradients, optimizer state and loss settings), and one tenant cannot touch the other's model."""
import os
import tempfile

import pytest
import torch


def _server():
    from twinkle_b200.server import ServerLauncher
    return ServerLauncher({
        'persistence': {'mode': 'memory'},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': ['tiny-dense']}},
            {'name': 'model', 'route_prefix': '/model/tiny-dense', 'import_path': 'model',
             'args': {'model_id': 'tiny-dense', 'backend': 'transformers', 'max_loras': 2}},
        ],
    })


def _data(seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(3):
        ids = torch.randint(3, 512, (21, ), generator=g).tolist()
        out.append({'model_input': {'tokens': ids[:-1]}, 'loss_fn_inputs': {'target_tokens': {'data': ids[1:]}, 'weights': {'data': [1.0] * 20}}})
    return out


def _step(tc, data, lr):
    out = tc.forward_backward(data, 'cross_entropy').result()
    tc.optim_step({'learning_rate': lr}).result()
    m = out['metrics']
    return m.get('loss', m.get('loss:sum'))


def test_interleaved_tenants_match_solo_runs(monkeypatch):
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_mt_'))
    monkeypatch.setenv('TWINKLE_POLL_INTERVAL', '0.01')
    from twinkle_b200.client import HttpError, TinkerClient
    solo = {}
    for name, seed, lr in (('alice', 1, 2e-3), ('bob', 2, 5e-3)):
        c = TinkerClient(app=_server().root, token=name)
        if name == 'bob':                        # bob gets the second slot when he shares the server; give him the same one here
            c.create_lora_training_client('tiny-dense', rank=8)
        tc = c.create_lora_training_client('tiny-dense', rank=8)
        solo[name] = [_step(tc, _data(seed), lr) for _ in range(3)]
    server = _server()
    a = TinkerClient(app=server.root, token='alice').create_lora_training_client('tiny-dense', rank=8)
    b = TinkerClient(app=server.root, token='bob').create_lora_training_client('tiny-dense', rank=8)
    mixed = {'alice': [], 'bob': []}
    for _ in range(3):
        # forward_backward of one tenant sits between forward_backward and optim_step of the other
        fa = a.forward_backward(_data(1), 'cross_entropy').result()
        fb = b.forward_backward(_data(2), 'cross_entropy').result()
        a.optim_step({'learning_rate': 2e-3}).result()
        b.optim_step({'learning_rate': 5e-3}).result()
        mixed['alice'].append(fa['metrics'].get('loss', fa['metrics'].get('loss:sum')))
        mixed['bob'].append(fb['metrics'].get('loss', fb['metrics'].get('loss:sum')))
    for name in solo:
        assert solo[name][-1] < solo[name][0]
        assert mixed[name] == pytest.approx(solo[name], abs=2e-4), (name, solo[name], mixed[name])
    # bob cannot drive alice's model
    from twinkle_b200.client import TrainingClient
    intruder = TrainingClient(b.t, a.model_id, b.session_id)
    with pytest.raises(HttpError) as e:
        intruder.forward_backward(_data(2), 'cross_entropy').result()
    assert e.value.status in (403, 404)
    # a third tenant does not fit (max_loras = 2) until one leaves
    c = TinkerClient(app=server.root, token='carol')
    with pytest.raises((HttpError, RuntimeError)):
        r = c.create_lora_training_client('tiny-dense', rank=8)
        _step(r, _data(3), 1e-3)
    a.unload().result()
    tc = c.create_lora_training_client('tiny-dense', rank=8)
    assert _step(tc, _data(3), 1e-3) > 0
