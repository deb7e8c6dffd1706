"""Server building blocks without any HTTP: atomic state updates under contention, cleanup-leader election and
hand-over, session sweep, rate limiter / preflight, config validation, and the hang guards fed with bad payloads
(reference tiers: tests/server/state/*, tests/server/utils/*, tests/server/config/*, nccl-safe e2e payload list)."""
import threading

import pytest
import torch

from twinkle_b200.server.state import FileBackend, MemoryBackend, ServerState


@pytest.mark.parametrize('make', [lambda p: MemoryBackend(), lambda p: FileBackend(str(p / 's.json'))])
def test_update_atomic_under_contention(tmp_path, make):
    b = make(tmp_path)
    n_threads, n_each = 8, 25

    def work():
        for _ in range(n_each):
            b.update_atomic('counter', lambda cur: (cur or 0) + 1)

    ts = [threading.Thread(target=work) for _ in range(n_threads)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert b.get('counter') == n_threads * n_each
    assert b.set_nx('once', 1) and not b.set_nx('once', 2) and b.get('once') == 1
    b.set('a:1', 1)
    b.set('a:2', 2)
    assert sorted(b.keys('a:')) == ['a:1', 'a:2'] and b.count('a:') == 2 and b.mget(['a:1', 'zzz']) == [1, None]
    assert b.delete('a:1') and not b.exists('a:1')


def test_single_leader_and_handover(tmp_path):
    backend = FileBackend(str(tmp_path / 'lease.json'))
    replicas = [ServerState(backend, replica_id=f'r{i}') for i in range(4)]
    now = 1000.0
    got = [r.try_acquire_leadership(now) for r in replicas]
    assert sum(got) == 1
    leader = replicas[got.index(True)]
    assert leader.try_acquire_leadership(now + 1)                      # renewing keeps it
    assert not any(r.try_acquire_leadership(now + 1) for r in replicas if r is not leader)
    leader.release_leadership()
    got2 = [r.try_acquire_leadership(now + 2) for r in replicas if r is not leader]
    assert sum(got2) == 1                                               # hand-over after release
    # an expired lease is taken by whoever asks first
    taker = replicas[0]
    assert taker.try_acquire_leadership(now + 10_000)


def test_sweep_expires_silent_sessions_and_their_resources():
    st = ServerState(MemoryBackend(), replica_id='r0')
    live = st.create_session('alice')
    dead = st.create_session('bob')
    st.register_model('m-live', 'alice', 'base', live)
    st.register_model('m-dead', 'bob', 'base', dead)
    st.create_sampling_session('bob', 'base', None, dead)
    rec = st.backend.get(f'session:{dead}')
    rec['heartbeat'] -= 10_000
    st.backend.set(f'session:{dead}', rec)
    removed = st.sweep(session_timeout=1800)
    assert removed['sessions'] == [dead] and removed['models'] == ['m-dead'] and len(removed['sampling']) == 1
    assert st.get_model('m-live') is not None and st.get_session(live) is not None
    assert st.gauges()['sessions'] == 1


def test_rate_limiter_and_preflight():
    from twinkle_b200.server.config import TaskQueueConfig
    from twinkle_b200.server.queue import PreflightError, RateLimiter, TaskQueueMixin
    clock = [0.0]
    rl = RateLimiter(rps=2, tps=100, window=1.0, clock=lambda: clock[0])
    assert rl.acquire('t', 60)[0] and rl.acquire('t', 30)[0]
    ok, why = rl.acquire('t', 1)
    assert not ok and 'request rate' in why
    clock[0] = 1.5                                                      # window slides
    assert rl.acquire('t', 90)[0]
    ok, why = rl.acquire('t', 50)
    assert not ok and 'token rate' in why
    assert rl.acquire('other', 50)[0]                                   # limits are per key

    class App(TaskQueueMixin):
        pass

    app = App()
    app._init_task_queue(ServerState(MemoryBackend()), TaskQueueConfig(max_input_tokens=100, rps_limit=1000, tps_limit=1e9))
    app.preflight('tok', input_tokens=100, batch_size=4, data_world_size=4)
    with pytest.raises(PreflightError) as e:
        app.preflight('tok', input_tokens=101)
    assert e.value.status_code == 413
    with pytest.raises(PreflightError, match='smaller than the data-parallel world size'):
        app.preflight('tok', batch_size=2, data_world_size=4)
    with pytest.raises(PreflightError, match='multiple of'):
        app.preflight('tok', batch_size=6, data_world_size=2, batch_size_multiple=4)
    with pytest.raises(Exception):
        TaskQueueConfig(rps_limit=0)
    with pytest.raises(Exception):
        TaskQueueConfig(no_such_field=1)


def test_bad_payloads_do_not_break_the_next_step():
    """The payloads of the reference's nccl-safe e2e list, fed straight into the model API with the hang guards on:
    every call returns (zero loss instead of an exception that would leave peers waiting) and the next good step works."""
    import os
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    os.environ['TWINKLE_FAIL_FAST'] = '0'
    try:
        m = MultiLoraTransformersModel(model_id='tiny-dense', max_loras=1, max_r=8, seed=0)
        m.add_adapter_to_model('a', LoraConfig(r=8, lora_alpha=16, target_modules='all-linear'))
        m.set_optimizer('AdamW', lr=1e-3, adapter_name='a')
        m.set_loss('GRPOLoss', adapter_name='a')
        good = [{'input_ids': list(range(1, 33)), 'labels': [-100] * 16 + list(range(18, 34))} for _ in range(2)]
        bad_calls = [
            dict(old_logps=[[0.0] * 3, [0.0] * 3], advantages=[1.0, -1.0]),                       # wrong old_logps length
            dict(old_logps=[[float('nan')] * 16] * 2, advantages=[1.0, -1.0]),                    # NaN log-probs
            dict(advantages=[1e30, -1e30]),                                                       # extreme advantages
        ]
        for kw in bad_calls:
            out = m.forward_backward(inputs=good, adapter_name='a', **kw)
            assert 'loss' in out
            m.clip_grad_and_step(adapter_name='a')
        masked = [{'input_ids': list(range(1, 33)), 'labels': [-100] * 32} for _ in range(2)]    # all labels masked
        m.forward_backward(inputs=masked, adapter_name='a', advantages=[1.0, -1.0])
        m.clip_grad_and_step(adapter_name='a')
        out = m.forward_backward(inputs=good, adapter_name='a', advantages=[1.0, -1.0])
        norm = m.clip_grad_and_step(adapter_name='a')
        assert torch.isfinite(torch.tensor(float(out['loss']))) and norm is not None
        for n, p in m.model.named_parameters():
            if 'lora' in n:
                assert torch.isfinite(p).all(), n
    finally:
        os.environ.pop('TWINKLE_FAIL_FAST', None)


def test_exception_hierarchy_and_status_mapping(tmp_path):
    import pytest
    from twinkle_b200.server.backends import BackendSelector
    from twinkle_b200.server.config import ServerConfig
    from twinkle_b200.server.exceptions import (ConcurrencyError, ConfigError, ConfigParseError, ResourceExhaustedError, StateBackendError,
                                                TwinkleServerError, status_code_of)
    from twinkle_b200.server.queue import PreflightError
    from twinkle_b200.server.state import MemoryBackend, ServerState
    with pytest.raises(ConfigError) as ei:
        BackendSelector.model('hf')
    assert ei.value.field == 'backend' and ei.value.value == 'hf' and 'mock' in ei.value.allowed and "allowed: ['mock'" in str(ei.value)
    assert isinstance(ei.value, ValueError) and status_code_of(ei.value) == 400
    with pytest.raises(ConfigError):
        BackendSelector.sampler('')
    bad = tmp_path / 'bad.yaml'
    bad.write_text('applications: [unclosed')
    with pytest.raises(ConfigParseError):
        ServerConfig.from_yaml(str(bad))
    bad.write_text('- just\n- a list\n')
    with pytest.raises(ConfigParseError):
        ServerConfig.from_yaml(str(bad))
    with pytest.raises(FileNotFoundError):
        ServerConfig.from_yaml(str(tmp_path / 'missing.yaml'))
    st = ServerState(MemoryBackend(), per_token_model_limit=1)
    st.register_model('m1', 'tok', 'base', None)
    with pytest.raises(ResourceExhaustedError) as ei:
        st.register_model('m2', 'tok', 'base', None)
    assert isinstance(ei.value, PermissionError) and status_code_of(ei.value) == 429
    assert issubclass(ConcurrencyError, StateBackendError) and issubclass(PreflightError, TwinkleServerError)
    assert [status_code_of(e) for e in (StateBackendError('x'), ConcurrencyError('x'), PreflightError('x', 413), KeyError('k'), TimeoutError(),
                                        PermissionError(), TypeError(), RuntimeError())] == [503, 409, 413, 404, 504, 403, 400, 500]


def test_wire_types_validate_bodies_and_parse_paths():
    import pytest
    from twinkle_b200.client.types import (REQUESTS, ParsedCheckpointTwinklePath, RequestError, SampleResponseModelList, TrainingRunsResponse,
                                           UploadToHubRequest, validate_request)
    out = validate_request('clip_grad_and_step', {'model_id': 'm1', 'extra_flag': 7}, aliases={'model_id': 'adapter_name'})
    assert out['adapter_name'] == 'm1' and out['max_grad_norm'] == 1.0 and out['norm_type'] == 2 and out['extra_flag'] == 7
    with pytest.raises(RequestError) as ei:
        validate_request('set_loss', {'adapter_name': 'a'})
    assert 'loss_cls' in str(ei.value) and ei.value.status_code == 400
    with pytest.raises(RequestError):
        validate_request('forward', {'adapter_name': 'a'})
    assert validate_request('unknown_route', {'x': 1}) == {'x': 1}
    assert REQUESTS['forward_only'](inputs=[1]).adapter_name is None
    assert UploadToHubRequest(checkpoint_dir={'twinkle_path': 'twinkle://r/weights/c'}, hub_model_id='u/m').checkpoint_dir == 'twinkle://r/weights/c'
    with pytest.raises(Exception):
        UploadToHubRequest(checkpoint_dir={}, hub_model_id='u/m')
    p = ParsedCheckpointTwinklePath.parse('twinkle://run1/sampler_weights/step-3')
    assert (p.training_run_id, p.checkpoint_type, p.checkpoint_id) == ('run1', 'sampler', 'step-3')
    for bad in ('twinkle://run1/weights', '/tmp/x', 'twinkle://run1/other/x'):
        with pytest.raises(ValueError):
            ParsedCheckpointTwinklePath.parse(bad)
    r = SampleResponseModelList(result=[{'sequences': [{'stop_reason': 'stop', 'tokens': [1, 2], 'logprobs': [-0.1, -0.2]}]}])
    assert r.result[0].sequences[0].tokens == [1, 2]
    runs = TrainingRunsResponse(training_runs=[{'training_run_id': 'r', 'last_checkpoint': {'checkpoint_id': 'c'}}], cursor={'total_count': 1})
    assert runs.training_runs[0].last_checkpoint.checkpoint_type == 'training' and runs.cursor.limit == 100


def test_otlp_json_export_of_metrics_and_spans():
    from twinkle_b200.server.telemetry import MetricsRegistry, Tracer
    from twinkle_b200.server.telemetry.otlp import OTLPExporter
    reg, tr = MetricsRegistry(), Tracer()
    reg.inc('twinkle_http_requests_total', app='gateway', status=200)
    reg.inc('twinkle_http_requests_total', app='gateway', status=200)
    reg.set_gauge('twinkle_queue_depth', 3)
    for v in (0.1, 0.2, 0.3, 0.4):
        reg.observe('twinkle_task_execution_seconds', v)
    with tr.span('POST /forward', model_id='m1', app='model'):
        pass
    try:
        with tr.span('POST /boom'):
            raise ValueError('x')
    except ValueError:
        pass
    sent = []
    ex = OTLPExporter('http://collector:4317/', 'svc', post=lambda url, body: sent.append((url, body)))
    assert ex.endpoint == 'http://collector:4318' and ex.export(reg, tr)
    (murl, m), (turl, t) = sent
    assert murl.endswith('/v1/metrics') and turl.endswith('/v1/traces')
    res = m['resourceMetrics'][0]
    assert res['resource']['attributes'][0] == {'key': 'service.name', 'value': {'stringValue': 'svc'}}
    by = {x['name']: x for x in res['scopeMetrics'][0]['metrics']}
    s = by['twinkle_http_requests_total']['sum']
    assert s['isMonotonic'] and s['aggregationTemporality'] == 2 and s['dataPoints'][0]['asDouble'] == 2.0
    assert {'key': 'status', 'value': {'intValue': '200'}} in s['dataPoints'][0]['attributes']
    assert by['twinkle_queue_depth']['gauge']['dataPoints'][0]['asDouble'] == 3.0
    summ = by['twinkle_task_execution_seconds']['summary']['dataPoints'][0]
    assert summ['count'] == '4' and abs(summ['sum'] - 1.0) < 1e-9 and summ['quantileValues'][0] == {'quantile': 0.5, 'value': 0.3}
    spans = t['resourceSpans'][0]['scopeSpans'][0]['spans']
    assert [x['name'] for x in spans] == ['POST /forward', 'POST /boom'] and len(spans[0]['traceId']) == 32 and len(spans[0]['spanId']) == 16
    assert spans[0]['status'] == {'code': 1} and spans[1]['status']['code'] == 2 and 'ValueError' in spans[1]['status']['message']
    assert {'key': 'twinkle.model_id', 'value': {'stringValue': 'm1'}} in spans[0]['attributes']
    assert int(spans[0]['endTimeUnixNano']) >= int(spans[0]['startTimeUnixNano'])
    sent.clear()
    assert ex.export(reg, tr) and [u for u, _ in sent] == ['http://collector:4318/v1/metrics']     # spans are sent once

    def down(url, body):
        raise OSError('unreachable')

    bad = OTLPExporter('http://c:4318', post=down)
    assert bad.export(reg, tr) is False and bad.failures == 1
