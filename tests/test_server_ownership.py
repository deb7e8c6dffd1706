"""Ownership rules of the served model application, checked with two tokens on CPU, and the resume route end to end.

One tenant must not reach another's adapter by guessing its server-side name, by re-creating its model id, through
``get_info``, or by naming a server-local directory to load; ``resume_from_checkpoint`` over HTTP must take the path
``save`` returned and restore the progress counters (reference ``src/twinkle/server/model/twinkle_handlers.py``)."""
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
             'args': {'model_id': 'tiny-dense', 'backend': 'transformers', 'max_loras': 3}},
        ],
    })


def _feats(seed, n=2):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(3, 512, (17, ), generator=g).tolist()
        out.append({'input_ids': ids, 'labels': ids[1:] + [-100]})
    return out


def test_one_token_cannot_reach_anothers_adapter(monkeypatch):
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_own_'))
    monkeypatch.setenv('TWINKLE_POLL_INTERVAL', '0.01')
    from twinkle_b200.client import HttpError, MultiLoraTransformersModel, TinkerClient, TwinkleClient
    server = _server()
    alice = TwinkleClient(app=server.root, token='alice', heartbeat_interval=60)
    bob = TwinkleClient(app=server.root, token='bob', heartbeat_interval=60)
    ma = MultiLoraTransformersModel('tiny-dense', client=alice)
    ma.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8})
    ma.set_optimizer('AdamW', lr=1e-3, adapter_name='a')
    ma.forward_backward(inputs=_feats(0), adapter_name='a')
    model_id = ma.adapters['a']
    model_app = server.model_apps[0]
    internal = model_app.adapters[model_id]['adapter']          # the backend-side adapter name
    mb = MultiLoraTransformersModel('tiny-dense', client=bob)
    # (1) bob names alice's model id, then the backend's internal adapter name: neither reaches the backend
    for name in (model_id, internal):
        with pytest.raises(HttpError) as e:
            mb._call('clip_grad_and_step', adapter_name=name)
        assert e.value.status in (403, 404), (name, e.value.status)
        with pytest.raises(HttpError) as e:
            mb._call('get_state_dict', adapter_name=name)
        assert e.value.status in (403, 404)
    # (2) re-creating an existing model id is refused, by the owner and by anyone else
    tb = TinkerClient(app=server.root, token='bob')
    with pytest.raises(HttpError) as e:
        tb.t.post('/model/tiny-dense/tinker/create_model', {'model_id': model_id, 'session_id': tb.session_id, 'lora_config': {'rank': 4}},
                  model_id=model_id)
    assert e.value.status == 409
    assert model_app.adapters[model_id]['token'] == 'alice'
    # (3) get_info checks the token
    with pytest.raises(HttpError) as e:
        bob.t.post('/model/tiny-dense/tinker/get_info', {'model_id': model_id}, model_id=model_id)
    assert e.value.status == 403
    assert alice.t.post('/model/tiny-dense/tinker/get_info', {'model_id': model_id}, model_id=model_id)['lora_rank'] == 4
    # (4) a server-local directory outside the token's root is not loadable; alice's own checkpoint is
    outside = tempfile.mkdtemp(prefix='tk_outside_')
    with pytest.raises(HttpError) as e:
        alice.t.post('/model/tiny-dense/twinkle/load', {'adapter_name': model_id, 'name': outside}, model_id=model_id)
    assert e.value.status == 403
    path = ma.save(name='c1', adapter_name='a', save_optimizer=True)
    assert path.startswith('twinkle://')
    alice.t.post('/model/tiny-dense/twinkle/load', {'adapter_name': model_id, 'name': path}, model_id=model_id)
    mb.add_adapter_to_model('b', {'r': 4, 'lora_alpha': 8})
    with pytest.raises(HttpError) as e:    # bob cannot load alice's checkpoint by its URI either
        bob.t.post('/model/tiny-dense/twinkle/load', {'adapter_name': mb.adapters['b'], 'name': path}, model_id=mb.adapters['b'])
    assert e.value.status in (403, 404)
    alice.close()
    bob.close()


def test_resume_from_checkpoint_over_http_restores_progress(monkeypatch):
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_res_'))
    from twinkle_b200.client import MultiLoraTransformersModel, TwinkleClient
    server = _server()
    c = TwinkleClient(app=server.root, token='alice', heartbeat_interval=60)
    m = MultiLoraTransformersModel('tiny-dense', client=c)
    m.add_adapter_to_model('a', {'r': 4, 'lora_alpha': 8})
    m.set_optimizer('AdamW', lr=1e-3, adapter_name='a')
    for i in range(3):
        m.forward_backward(inputs=_feats(i), adapter_name='a')
        m.clip_grad_and_step(adapter_name='a')
    path = m.save(name='step3', adapter_name='a', save_optimizer=True)
    for i in range(2):                                   # move past the checkpoint
        m.forward_backward(inputs=_feats(10 + i), adapter_name='a')
        m.clip_grad_and_step(adapter_name='a')
    info = m.resume_from_checkpoint(path, adapter_name='a')    # positional argument = the request record's ``name``
    assert info['cur_step'] == 3 and info['consumed_train_samples'] == 6, info
    only = m.resume_from_checkpoint(name=path, adapter_name='a', resume_only_model=True)
    assert only['cur_step'] == 0
    c.close()
