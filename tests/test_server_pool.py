"""The HTTP server in front of worker groups: a 2-rank model group (gloo, sharded base + LoRA tenants) and a 1-rank
sampler group, both as pool workers.  Two tenants train over the Tinker routes, save weights for the sampler and
sample from them; ``/healthz`` reaches the workers; per-datum results come back in request order (reference
``src/twinkle/server/model/app.py:50-234``)."""
import tempfile

import pytest
import torch


def _datums(seed, n=4):
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        L = 12 + 3 * i                      # different lengths: the order of the per-datum outputs is checkable
        ids = torch.randint(3, 512, (L + 1, ), generator=g).tolist()
        out.append({'model_input': {'tokens': ids[:-1]}, 'loss_fn_inputs': {'target_tokens': {'data': ids[1:]}, 'weights': {'data': [1.0] * L}}})
    return out


@pytest.fixture()
def server(monkeypatch):
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_pool_'))
    monkeypatch.setenv('TWINKLE_POLL_INTERVAL', '0.01')
    from twinkle_b200.server import ServerLauncher
    s = ServerLauncher({
        'persistence': {'mode': 'memory'},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': ['tiny-dense']}},
            {'name': 'model', 'route_prefix': '/model/tiny-dense', 'import_path': 'model',
             'args': {'model_id': 'tiny-dense', 'backend': 'transformers', 'max_loras': 2, 'max_r': 8,
                      'device_group': {'name': 'model', 'ranks': 2, 'device_type': 'cpu'}, 'device_mesh': {'dp_size': None, 'fsdp_size': 2}}},
            {'name': 'sampler', 'route_prefix': '/sampler/tiny-dense', 'import_path': 'sampler',
             'args': {'model_id': 'tiny-dense', 'sampler_type': 'torch', 'workers': 'pool', 'max_loras': 2,
                      'device_group': {'name': 'sampler', 'ranks': 1, 'device_type': 'cpu'}, 'engine_args': {'max_r': 8}}},
        ],
    })
    try:
        yield s
    finally:
        s.shutdown()


def test_two_tenants_train_and_sample_through_worker_groups(server):
    from twinkle_b200 import infra
    from twinkle_b200.client import TinkerClient
    assert infra.get_mode() == 'pool'
    m = server.model_apps[0]
    assert getattr(m.backend, '_remote_proxy', None) is not None and m.backend.data_world_size() == 2
    clients = {n: TinkerClient(app=server.root, token=n) for n in ('alice', 'bob')}
    tcs = {n: c.create_lora_training_client('tiny-dense', rank=8) for n, c in clients.items()}
    losses = {n: [] for n in tcs}
    for step in range(3):
        for i, (n, tc) in enumerate(tcs.items()):
            data = _datums(10 + i)
            out = tc.forward_backward(data, 'cross_entropy').result()
            # one output per datum, in request order (lengths differ per datum)
            assert [len(o['logprobs']['data']) for o in out['loss_fn_outputs']] == [len(d['model_input']['tokens']) for d in data]
            tc.optim_step({'learning_rate': 5e-3}).result()
            m_ = out['metrics']
            losses[n].append(m_.get('loss', m_.get('loss:sum')))
    for n, c in losses.items():
        assert c[-1] < c[0], (n, c)
    # health: a round trip to every worker of the group
    assert clients['alice'].t.get('/model/tiny-dense/healthz')['status'] == 'ok'
    # weights for the sampler, then sampling from them on the sampler group
    for n, tc in tcs.items():
        sc = tc.save_weights_and_get_sampling_client(f'{n}-w')
        r = sc.sample([5, 6, 7, 8], 1, {'max_tokens': 4, 'temperature': 0.0}).result()
        assert len(r['sequences'][0]['tokens']) == 4
