"""The whole HTTP stack on mock backends (no GPU): route set, Tinker future protocol, sessions, admission
control, checkpoint registry, client twins.  Mirrors the reference's mock-mode server tests."""
import os
import time

import pytest


@pytest.fixture()
def server(tmp_path, monkeypatch):
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', str(tmp_path / 'ckpt'))
    monkeypatch.setenv('TWINKLE_LONG_POLL_TIMEOUT', '5')
    monkeypatch.setenv('TWINKLE_POLL_INTERVAL', '0.02')
    from twinkle_b200.server import ServerLauncher
    cfg = {
        'persistence': {'mode': 'file', 'file_path': str(tmp_path / 'state.json')},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': ['mock-base']}},
            {'name': 'model', 'route_prefix': '/model/mock-base', 'import_path': 'model', 'args': {'model_id': 'mock-base', 'backend': 'mock', 'max_loras': 2}},
            {'name': 'sampler', 'route_prefix': '/sampler/mock-base', 'import_path': 'sampler', 'args': {'model_id': 'mock-base', 'sampler_type': 'mock'}},
            {'name': 'processor', 'route_prefix': '/processor', 'import_path': 'processor', 'args': {}},
        ],
    }
    return ServerLauncher(cfg)


CONTRACT = {
    'gateway': ['/asample', '/chat/completions', '/create_model', '/create_sampling_session', '/create_session', '/forward', '/forward_backward',
                '/get_info', '/get_server_capabilities', '/healthz', '/load_weights', '/models', '/optim_step', '/retrieve_future', '/save_weights',
                '/save_weights_for_sampler', '/session_heartbeat', '/telemetry', '/training_runs', '/training_runs/{run_id}',
                '/training_runs/{run_id}/checkpoints', '/twinkle/capacity_info', '/twinkle/create_session', '/twinkle/get_server_capabilities',
                '/twinkle/healthz', '/twinkle/healthz/deep', '/twinkle/session_heartbeat', '/twinkle/status', '/twinkle/training_runs',
                '/twinkle/weights_info', '/unload_model', '/weights_info'],
    'model': ['/healthz'] + [f'/tinker/{e}' for e in ('create_model', 'forward', 'forward_backward', 'get_info', 'load_weights', 'optim_step',
                                                       'save_weights', 'save_weights_for_sampler', 'unload_model')] +
    [f'/twinkle/{e}' for e in ('add_adapter_to_model', 'add_metric', 'apply_patch', 'backward', 'calculate_loss', 'calculate_metric',
                               'clip_grad_and_step', 'clip_grad_norm', 'create', 'forward', 'forward_backward', 'forward_only', 'get_state_dict',
                               'get_train_configs', 'load', 'lr_step', 'resume_from_checkpoint', 'save', 'set_loss', 'set_lr_scheduler',
                               'set_optimizer', 'set_processor', 'set_template', 'step', 'upload_status/{request_id}', 'upload_to_hub', 'zero_grad')],
    'sampler': ['/tinker/asample'] + [f'/twinkle/{e}' for e in ('add_adapter_to_sampler', 'apply_patch', 'create', 'sample', 'sample_stream', 'set_template')],
    'processor': ['/twinkle/call', '/twinkle/create'],
}


def test_route_contract(server):
    apps = {'gateway': server.gateway.app, 'model': server.model_apps[0].app, 'sampler': server.sampler_apps[0].app,
            'processor': server.processor_apps[0].app}
    for name, want in CONTRACT.items():
        have = {r.path for r in apps[name].routes}
        missing = [p for p in want if p not in have]
        assert not missing, (name, missing)


def test_tinker_protocol_end_to_end(server):
    from twinkle_b200.client import HttpError, TinkerClient
    c = TinkerClient(app=server.root, token='alice')
    assert 'mock-base' in [m['model_name'] for m in c.get_server_capabilities()['supported_models']]
    tr = c.create_lora_training_client('mock-base', rank=8)
    datum = {'model_input': {'tokens': [5, 6, 7, 8]}, 'loss_fn_inputs': {'target_tokens': {'data': [6, 7, 8, 9]}, 'weights': {'data': [0, 1, 1, 1]}}}
    out = tr.forward_backward([datum, datum]).result()
    assert len(out['loss_fn_outputs']) == 2 and out['loss_fn_outputs'][0]['logprobs']['data'][0] == 0.0
    assert out == tr.forward_backward([datum, datum]).result()  # deterministic mock
    assert tr.optim_step({'learning_rate': 1e-3}).result()['metrics']['step'] == 1.0
    # optim_step without a new forward_backward is rejected
    with pytest.raises(HttpError):
        tr.optim_step().result()
    path = tr.save_state('step1').result()['path']
    assert path.startswith('twinkle://')
    samp = tr.save_weights_for_sampler('s1').result()
    assert 'sampling_session_id' in samp
    sc = c.create_sampling_client('mock-base', samp['path'])
    res = sc.sample([1, 2, 3], num_samples=2, sampling_params={'max_tokens': 4}).result()
    assert len(res['sequences']) == 2 and len(res['sequences'][0]['tokens']) == 4
    # another token can neither see nor use the model
    other = TinkerClient(app=server.root, token='bob')
    with pytest.raises(HttpError) as e:
        other.t.post('/forward_backward', {'model_id': tr.model_id, 'forward_backward_input': {'data': [datum]}})
    assert e.value.status == 403
    runs = c.t.get('/training_runs')['training_runs']
    assert runs and runs[0]['training_run_id'] == tr.model_id
    assert other.t.get('/training_runs')['training_runs'] == []
    # slot pool: max_loras = 2
    c.create_lora_training_client('mock-base')
    with pytest.raises(HttpError):
        c.create_lora_training_client('mock-base')
    tr.unload().result()
    c.create_lora_training_client('mock-base')


def test_twinkle_client_and_processor(server):
    from twinkle_b200.client import DataLoader, Dataset, MultiLoraTransformersModel, TorchSampler, TwinkleClient
    c = TwinkleClient(app=server.root, token='alice', heartbeat_interval=0.05)
    m = MultiLoraTransformersModel('mock-base', client=c)
    m.add_adapter_to_model('a', {'r': 8, 'lora_alpha': 16})
    out = m.forward_backward(inputs=[{'input_ids': [1, 2, 3], 'labels': [2, 3, -100]}], adapter_name='a')
    assert 'loss' in out
    assert m.clip_grad_and_step(adapter_name='a') == 1.0
    assert 'loss' in m.forward_backward([{'input_ids': [1, 2, 3], 'labels': [2, 3, -100]}], adapter_name='a')       # inputs by position, as against a local model
    assert m.clip_grad_and_step(1.0, 2, adapter_name='a') == 1.0
    assert MultiLoraTransformersModel('ms://mock-base', client=c).model_id == 'mock-base'                          # hub prefixes name the same served model
    s = TorchSampler('ms://mock-base', client=c)
    assert s.model_id == 'mock-base' and s.apply_patch('Qwen3ChatTemplate') == {'status': 'ok'}
    s.set_template('Template')
    r = s.sample([{'messages': [{'role': 'user', 'content': 'hi'}]}], {'max_tokens': 3})
    assert len(r[0]['sequences'][0]['tokens']) == 3 and r[0]['sequences'][0]['new_input_feature']['labels'][-2] != -100
    ds = Dataset({'__class__': 'DatasetMeta', 'kwargs': {'data': [{'messages': [{'role': 'user', 'content': str(i)}]} for i in range(6)]}}, client=c)
    assert len(ds) == 6
    dl = DataLoader(ds, batch_size=2, shuffle=False, client=c)
    assert sum(1 for _ in dl) == 3
    from twinkle_b200.client import LazyDataset, PackingDataset
    meta = {'__class__': 'DatasetMeta', 'kwargs': {'data': [{'messages': [{'role': 'user', 'content': str(i)}, {'role': 'assistant', 'content': 'ok'}]} for i in range(6)]}}
    assert len(LazyDataset(meta, client=c)) == 6 and hasattr(PackingDataset(meta, client=c), 'object_id')      # the other dataset twins of the reference client
    time.sleep(0.15)
    assert c.status()['gauges']['sessions'] >= 1
    # the manager calls of the reference client (``twinkle_client/manager.py``): health, capacity, sessions, paged runs, paths
    from twinkle_b200.client import TwinkleClientError
    assert c.health_check() and 'replicas' in c.get_capacity_info() and c.create_session({'purpose': 'test'}) != c.session_id
    assert c.get_server_capabilities() == c.capabilities()
    m.save(name='ck1', adapter_name='a')
    runs, cursor = c.list_training_runs_with_cursor(limit=5)
    assert runs and cursor['total_count'] == len(c.list_training_runs(limit=100)) and c.list_training_runs(limit=1, offset=len(runs)) == []
    run = runs[0]['training_run_id']
    assert c.get_training_run(run)['training_run_id'] == run and c.find_training_run_by_model(runs[0]['base_model'])
    cks = c.list_checkpoints(run)
    assert cks
    info = c.get_checkpoint_path(run, 'weights/ck1')
    assert info['twinkle_path'] == f'twinkle://{run}/weights/ck1' == c.get_checkpoint_twinkle_path(run, 'ck1') and info['path'].endswith('ck1')
    assert c.get_latest_checkpoint_path(run) == info['path'] and c.get_weights_info(info['twinkle_path']) == c.weights_info(info['twinkle_path'])
    with pytest.raises(TwinkleClientError):
        c.get_training_run('no-such-run')
    c.close()
    from twinkle_b200.client import init_twinkle_client
    c2 = init_twinkle_client(api_key='alice', session_heartbeat_interval=30, app=server.root)      # the reference's argument names
    assert c2.t.token == 'alice' and c2.list_training_runs(limit=1)
    c2.close()


def test_admission_control_and_state(server, tmp_path):
    from twinkle_b200.server.config import ServerConfig, TaskQueueConfig
    from twinkle_b200.server.queue import PreflightError, RateLimiter, TaskQueueMixin
    from twinkle_b200.server.state import FileBackend, MemoryBackend, ServerState
    t = [0.0]
    rl = RateLimiter(rps=2, tps=100, window=1.0, clock=lambda: t[0])
    assert rl.acquire('k', 10)[0] and rl.acquire('k', 10)[0] and not rl.acquire('k', 10)[0]
    t[0] = 1.5
    assert rl.acquire('k', 90)[0] and not rl.acquire('k', 20)[0]

    class Q(TaskQueueMixin):
        pass

    q = Q()
    q._init_task_queue(ServerState(), TaskQueueConfig(max_input_tokens=10))
    with pytest.raises(PreflightError):
        q.preflight('tok', input_tokens=11)
    with pytest.raises(PreflightError):
        q.preflight('tok', batch_size=1, data_world_size=2)
    # leader lease: one leader among replicas sharing a backend; hand-over after expiry
    be = FileBackend(str(tmp_path / 's.json'))
    a, b = ServerState(be, 'A'), ServerState(be, 'B')
    assert a.try_acquire_leadership(now=100.0) and not b.try_acquire_leadership(now=101.0)
    assert a.try_acquire_leadership(now=110.0)  # renew
    assert b.try_acquire_leadership(now=200.0) and not a.try_acquire_leadership(now=201.0)
    # sweep removes what hangs off dead sessions
    st = ServerState(MemoryBackend(), 'X')
    sid = st.create_session('tok')
    st.register_model('m1', 'tok', 'base', sid)
    st.backend.update_atomic(f'session:{sid}', lambda s: {**s, 'heartbeat': time.time() - 100})
    gone = st.sweep(session_timeout=10)
    assert gone['sessions'] == [sid] and gone['models'] == ['m1']
    with pytest.raises(Exception):
        ServerConfig(applications=[{'name': 'x', 'import_path': 'model', 'args': {'model_id': 'a', 'bogus': 1}}])


def test_openai_chat_completions_tools_reasoning_logprobs_and_stream(server):
    import json
    from twinkle_b200.client import Transport
    t = Transport(app=server.root, token='alice')
    backend = server.sampler_apps[0].backend
    backend.script = [{'text': '<think>\nneed the sum\n</think>\n\nLet me add. <tool_call>\n{"name": "add", "arguments": {"a": 2, "b": 3}}\n</tool_call>',
                       'stop_reason': 'stop'}]
    tools = [{'type': 'function', 'function': {'name': 'add', 'description': 'Add.', 'parameters': {'type': 'object', 'properties': {}}}}]
    body = {'model': 'mock-base', 'messages': [{'role': 'user', 'content': [{'type': 'text', 'text': 'what is 2+3?'}]}], 'tools': tools, 'max_tokens': 64,
            'logprobs': True}
    r = t.post('/chat/completions', body)
    ch = r['choices'][0]
    assert r['object'] == 'chat.completion' and ch['finish_reason'] == 'tool_calls'
    assert ch['message']['reasoning_content'] == 'need the sum' and ch['message']['content'] == 'Let me add.'
    call = ch['message']['tool_calls'][0]
    assert call['type'] == 'function' and call['function']['name'] == 'add' and json.loads(call['function']['arguments']) == {'a': 2, 'b': 3}
    assert len(ch['logprobs']['content']) == r['usage']['completion_tokens'] and ch['logprobs']['content'][0]['logprob'] <= 0
    assert r['usage']['total_tokens'] == r['usage']['prompt_tokens'] + r['usage']['completion_tokens']
    # a follow-up in OpenAI wire form (function-style tool call + tool result) is accepted
    backend.script = [{'text': 'The sum is 5.', 'stop_reason': 'stop'}]
    follow = {'model': 'mock-base', 'tools': tools, 'max_tokens': 16, 'messages': body['messages'] + [
        {'role': 'assistant', 'content': None, 'tool_calls': [call]}, {'role': 'tool', 'tool_call_id': call['id'], 'content': '5'}]}
    r2 = t.post('/chat/completions', follow)
    assert r2['choices'][0]['message'] == {'role': 'assistant', 'content': 'The sum is 5.'} and r2['choices'][0]['finish_reason'] == 'stop'
    assert [m['id'] for m in t.get('/models')['data']] == ['mock-base']
