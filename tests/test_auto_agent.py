"""twinkle-auto: run store + script runtime round trip through real child processes, tool dispatch, the conversation
loop against a scripted model, monitor verdicts including an automatic fix and the three-fix limit, skills."""
import io
import json
import os
import sys
import textwrap
import time

import pytest

from twinkle_b200.client.auto import (MAX_FIX_ATTEMPTS, AgentLoop, RunStore, ScriptedLLM, ToolExecutor, TrainingMonitor, TrainingRuntime,
                                      local_findings, merge_stream, parse_verdict, server_config, split_gpus)
from twinkle_b200.client.auto.app import AutoApp, header_lines, main, sparkline
from twinkle_b200.client.skills import LocalSkillProvider, SkillManager, default_manager, parse_skill

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

GOOD = textwrap.dedent(f'''
    import sys, time
    sys.path.insert(0, {REPO!r})
    from twinkle_b200.client.auto.runtime import TrainingRuntime
    rt = TrainingRuntime()
    rt.start(model_id='tiny', config=dict(lr=1e-3))
    rt.register_graceful_shutdown(lambda: open('saved.flag', 'w').write('1'))
    start = rt.get_resume_info()['global_step']
    for step in range(start, TOTAL):
        rt.log_metrics(step=step, loss=1.0 / (step + 1), lr=1e-3)
        time.sleep(DELAY)
    rt.finish()
''')
BAD = GOOD.replace("rt.finish()", "raise ValueError('boom: batch size must be >= 2')")


def script(src=GOOD, total=4, delay=0.0):
    return src.replace('TOTAL', str(total)).replace('DELAY', str(delay))


def wait_for(pred, timeout=20.0):
    end = time.time() + timeout
    while time.time() < end:
        if pred():
            return True
        time.sleep(0.05)
    return False


def test_run_lifecycle_and_resume(tmp_path):
    store = RunStore(tmp_path)
    res = store.start('demo run', script(total=3), model_id='tiny', unique=False)
    assert res['status'] == 'running' and res['run_id'] == 'demo-run'
    assert store.wait('demo-run') == 'completed'
    rows = store.metrics('demo-run')
    assert [r['step'] for r in rows] == [0, 1, 2] and 'run demo-run started' in store.log_tail('demo-run')
    assert store.list_runs()[0]['last_step'] == 2
    # a relaunch continues after the last logged step instead of starting over
    up = store.update_script('demo-run', script(total=5))
    assert up['script_version'] == 2 and (tmp_path / 'demo-run' / 'train_v1.py').exists()
    assert store.resume('demo-run')['status'] == 'running' and store.wait('demo-run') == 'completed'
    assert [r['step'] for r in store.metrics('demo-run')] == [0, 1, 2, 3, 4]
    assert store.start('demo run', script(), unique=False)['run_id'] == 'demo-run-2'       # names never collide


def test_stop_saves_and_pause_kills(tmp_path):
    store = RunStore(tmp_path)
    rid = store.start('slow', script(total=10_000, delay=0.02), unique=False)['run_id']
    assert wait_for(lambda: len(store.metrics(rid)) >= 2)
    assert store.resume(rid)['status'] == 'error'                                            # already running
    store.stop(rid)
    assert store.wait(rid) == 'stopped' and (tmp_path / rid / 'saved.flag').exists()         # SIGTERM handler ran
    n = len(store.metrics(rid))
    assert store.resume(rid)['status'] == 'running'
    assert wait_for(lambda: len(store.metrics(rid)) > n)
    first_new = store.metrics(rid)[n]['step']
    assert first_new == store.metrics(rid)[n - 1]['step'] + 1
    store.pause(rid)
    assert store.wait(rid) == 'paused'
    (tmp_path / rid / 'saved.flag').unlink()
    time.sleep(0.1)
    assert not (tmp_path / rid / 'saved.flag').exists()                                      # SIGKILL: no handler


def test_runtime_metric_encoding(tmp_path):
    import torch
    rt = TrainingRuntime('r', tmp_path)
    rt.log_metrics(step=0, loss=torch.tensor(2.5), grad_norm=float('nan'))
    row = json.loads((tmp_path / 'r' / 'metrics.jsonl').read_text())
    assert row['loss'] == 2.5 and row['grad_norm'] == 'nan' and rt.get_resume_info()['global_step'] == 1


def test_tool_executor(tmp_path, monkeypatch):
    store = RunStore(tmp_path)
    ex = ToolExecutor(store)
    assert 'unknown tool' in ex.execute('nope', {})
    assert 'bad arguments' in ex.execute('select_run', dict(wrong=1))
    assert 'does not parse' in ex.execute('start_training', dict(run_id='x', script_content='def ('))
    res = json.loads(ex.execute('start_training', dict(run_id='t', script_content=script(total=2), model_id='tiny')))
    assert res['status'] == 'running' and store.selected == res['run_id']
    store.wait(res['run_id'])
    st = json.loads(ex.execute('get_training_status', dict(run_id=res['run_id'])))
    assert st['status'] == 'completed' and len(st['recent_metrics']) == 2
    assert json.loads(ex.execute('list_training_runs', {}))[0]['run_id'] == res['run_id']
    info = json.loads(ex.execute('get_cluster_info', {}))
    assert info['cpu_count'] >= 1 and 'gpus' in info
    hub = tmp_path / 'hub' / 'models' / 'Qwen' / 'Qwen3-8B'
    hub.mkdir(parents=True)
    monkeypatch.setenv('TWINKLE_LOCAL_HUB', str(tmp_path / 'hub'))
    assert json.loads(ex.execute('search_models', dict(query='qwen3')))['results'][0]['id'] == 'Qwen/Qwen3-8B'
    assert json.loads(ex.execute('shutdown_server', {}))['status'] == 'not_running'


def test_gpu_split_and_server_config():
    assert split_gpus(8) == dict(train=[0, 1, 2, 3, 4, 5], sampler=[6, 7])
    assert split_gpus(2) == dict(train=[0, 1], sampler=[])
    assert split_gpus(4, train=2, sampler=1) == dict(train=[0, 1], sampler=[2])
    assert split_gpus(1, sampler=4) == dict(train=[0], sampler=[])
    assert split_gpus(0) == dict(train=[], sampler=[])
    from twinkle_b200.server.config import ServerConfig
    cfg = ServerConfig(**server_config('Qwen/Qwen3-8B', split_gpus(8), port=8123, persistence_path='/tmp/x.json'))       # the strict schema accepts it
    kinds = [a.import_path for a in cfg.applications]
    assert kinds == ['model', 'processor', 'sampler', 'server'] and cfg.http_options.port == 8123
    assert cfg.applications[0].typed_args.nproc_per_node == 6 and cfg.applications[2].typed_args.nproc_per_node == 2


def test_agent_loop_tool_rounds_and_pruning(tmp_path):
    store = RunStore(tmp_path)
    seen = []
    llm = ScriptedLLM([
        dict(content='', tool_calls=[dict(name='start_training', arguments=json.dumps(dict(run_id='exp', script_content=script(total=2))))]),
        dict(content='', tool_calls=[dict(name='list_training_runs', arguments={})]),
        'Started exp; it is running.',
    ])
    agent = AgentLoop(llm, ToolExecutor(store), on_tool=lambda n, a, r: seen.append(n))
    agent.inject_skills('# Skills\nalways log metrics')
    out = agent.send('train something small')
    assert out == 'Started exp; it is running.' and seen == ['start_training', 'list_training_runs']
    roles = [m['role'] for m in agent.history]
    assert roles == ['user', 'assistant', 'tool', 'assistant', 'tool', 'assistant']
    assert agent.history[2]['tool_call_id'] == agent.history[1]['tool_calls'][0]['id']
    sys_msg = llm.requests[-1]['messages'][0]['content']
    assert 'always log metrics' in sys_msg and 'Currently selected run: exp' in sys_msg
    assert len(llm.requests[0]['tools']) >= 12
    store.wait(store.selected)
    # pruning cuts only in front of user messages
    agent.max_history_chars = 200
    agent.send('x' * 150)
    agent.send('y' * 150)
    assert agent.history[0]['role'] == 'user' and all(m['role'] != 'tool' for m in agent.history[:1])
    # a model that never stops calling tools is cut off
    loop = ScriptedLLM([], default=dict(content='', tool_calls=[dict(name='list_training_runs', arguments={})]))
    a2 = AgentLoop(loop, ToolExecutor(store), max_tool_rounds=3)
    a2.send('go')
    assert len(loop.requests) == 3 and 'too many tool rounds' in a2.history[-1]['content']


def test_stream_merge():
    chunks = [dict(choices=[dict(delta=dict(content='Hel'))]), dict(choices=[dict(delta=dict(content='lo'))]),
              dict(choices=[dict(delta=dict(tool_calls=[dict(index=0, id='c1', function=dict(name='select_run', arguments='{"run'))]))]),
              dict(choices=[dict(delta=dict(tool_calls=[dict(index=0, function=dict(arguments='_id": "a"}'))]))])]
    got = []
    r = merge_stream(chunks, got.append)
    assert r['content'] == 'Hello' and got == ['Hel', 'lo']
    assert r['tool_calls'] == [dict(id='c1', name='select_run', arguments=dict(run_id='a'))]


def test_verdict_parsing_and_findings():
    assert parse_verdict('LGTM - fine')[0] == 'lgtm'
    assert parse_verdict('Loss has plateaued; lower the lr.') == ('warning', 'Loss has plateaued; lower the lr.', '')
    kind, why, code = parse_verdict('```diagnosis\nbatch too small\n```\n```python\nprint(1)\n```')
    assert (kind, why, code) == ('fix', 'batch too small', 'print(1)\n')
    assert parse_verdict('The import is wrong.\n```python\nimport os\n```')[1] == 'The import is wrong.'
    snap = dict(process='exited', status='crashed', stall_seconds=0.0, log_tail='Traceback (most recent call last)\nValueError',
                metrics=[dict(step=3, loss='nan')])
    f = local_findings(snap)
    assert any('never reported completion' in x for x in f) and any('loss is nan' in x for x in f) and any('error marker' in x for x in f)
    rising = dict(process='alive', status='running', stall_seconds=700.0, log_tail='', metrics=[dict(step=i, loss=v) for i, v in enumerate([1, .5, .3, .2, .9, 1.2, 1.5, 2.0])])
    f2 = local_findings(rising)
    assert any('loss rose' in x for x in f2) and any('no new metric' in x for x in f2)


def test_monitor_fix_and_limits(tmp_path):
    store = RunStore(tmp_path)
    msgs = []
    rid = store.start('broken', script(BAD, total=2), unique=False)['run_id']
    assert store.wait(rid) == 'crashed'
    fixed = script(total=4)
    llm = ScriptedLLM([f'```diagnosis\nthe script raises at the end\n```\n```python\n{fixed}\n```'])
    mon = TrainingMonitor(store, llm, msgs.append)
    assert mon.check() == 'fix'
    assert 'boom' in llm.requests[0]['messages'][1]['content'] and 'Current train.py' in llm.requests[0]['messages'][1]['content']
    assert store.wait(rid) == 'completed' and store.meta(rid)['script_version'] == 2
    assert [r['step'] for r in store.metrics(rid)] == [0, 1, 2, 3]                           # resumed, not restarted
    assert any('attempt 1/3' in m for m in msgs) and any('relaunched' in m for m in msgs)
    assert mon.check() == 'idle'                                                              # completed and clean
    # a healthy progressing run costs no model call; an unchanged snapshot is skipped
    rid2 = store.start('fine', script(total=10_000, delay=0.02), unique=False)['run_id']
    assert wait_for(lambda: len(store.metrics(rid2)) >= 1)
    n_calls = len(llm.requests)
    assert mon.check() == 'healthy' and len(llm.requests) == n_calls
    store.pause(rid2)
    store.wait(rid2)
    # warnings are relayed; fixes stop after the limit; an unparsable fix is not applied
    rid3 = store.start('again', script(BAD, total=1), unique=False)['run_id']
    store.wait(rid3)
    llm2 = ScriptedLLM(['KL is exploding; lower the learning rate.'])
    mon2 = TrainingMonitor(store, llm2, msgs.append)
    assert mon2.check() == 'warning' and msgs[-1].startswith('[monitor] KL is exploding')
    assert mon2.check() == 'unchanged'
    mon2.fix_attempts[rid3] = MAX_FIX_ATTEMPTS
    mon2._last_hash = ''
    llm2.replies.append('```python\nprint(1)\n```')
    assert mon2.check() == 'fix-refused' and 'do not answer with a fixed script' in llm2.requests[-1]['messages'][0]['content']
    mon2.fix_attempts[rid3] = 0
    mon2._last_hash = ''
    llm2.replies.append('```python\ndef (\n```')
    assert mon2.check() == 'fix-refused' and store.meta(rid3)['script_version'] == 1


def test_skills(tmp_path):
    s = parse_skill('---\nname: my-skill\ndescription: "does things"\n---\n# Title\nbody', 'fallback')
    assert (s.name, s.description, s.content) == ('my-skill', 'does things', '# Title\nbody')
    assert parse_skill('# Heading line\ntext', 'fallback').name == 'fallback'
    m = default_manager()
    m.load_all()
    assert {'twinkle-training', 'autoresearch'} <= set(m.names())
    prompt = m.format_for_prompt()
    assert 'TrainingRuntime' in prompt and 'get_resume_info' in prompt
    (tmp_path / 'twinkle-training.md').write_text('---\nname: twinkle-training\ndescription: override\n---\nmine')
    m.register(LocalSkillProvider(tmp_path, 'user'))
    m.load_all()
    assert [x for x in m.skills if x.name == 'twinkle-training'][0].content == 'mine'      # later provider wins
    assert '(summary only)' in m.format_for_prompt(max_chars=10)

    class Broken(LocalSkillProvider):
        def load(self):
            raise OSError('offline')

    m2 = SkillManager([Broken(tmp_path, 'bad')])
    assert m2.load_all() == [] and 'offline' in m2.errors['bad']


def test_bundled_skill_skeleton_runs(tmp_path):
    """The skeleton that the bundled skill teaches must itself be valid Python that uses names which exist."""
    import re
    text = open(os.path.join(REPO, 'twinkle_b200', 'client', 'skills', 'bundled', 'twinkle-training.md')).read()
    block = re.search(r'```python\n(import os.*?)```', text, re.S).group(1)
    compile(block, 'skeleton', 'exec')
    from twinkle_b200.client import TinkerClient, TrainingClient
    for name in ('forward_backward', 'optim_step', 'save_state', 'save_weights_for_sampler'):
        assert hasattr(TrainingClient, name)
    assert hasattr(TinkerClient, 'create_lora_training_client') and hasattr(TinkerClient, 'create_sampling_client')


def test_app_commands_and_once(tmp_path, capsys):
    store = RunStore(tmp_path)
    assert sparkline([3, 2, 1, float('nan')]) == '█▄▁' and sparkline([]) == ''
    out = io.StringIO()
    llm = ScriptedLLM([dict(content='', tool_calls=[dict(name='start_training', arguments=dict(run_id='ui', script_content=script(total=3)))]), 'done'])
    app = AutoApp(store, llm, out=out, monitor=False)
    app.run(io.StringIO('please train\n/runs\n/metrics\n/skills\n/bogus\n/quit\n'))
    store.wait(store.selected)
    text = out.getvalue()
    assert 'start_training(' in text and 'agent> done' in text and 'twinkle-training' in text and 'commands:' in text
    assert store.selected and store.selected.startswith('ui_')
    assert header_lines(store)[0].startswith(f'run {store.selected}')
    assert main(['--dry-run', '--once', 'hello', '--base-dir', str(tmp_path)]) == 0
    assert 'dry run' in capsys.readouterr().out
