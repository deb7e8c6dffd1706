"""Agentic package: tool dispatch, multi-turn rollout with a scripted sampler, environments, condensing, router
sampler, rewards and filters (reference tests: tests/agentic/*)."""
import json

from twinkle_b200.agentic import (CoTReward, DeadLoopFilter, DedupFilter, Env, EnvPool, EnvTool, ExtractCondensed, F1Reward, FunctionTool,
                                  HardFilter, KeywordCondenser, MessageSanityFilter, MultiTurnCondenseRollout, MultiTurnRollout, NativeChunker,
                                  PIIFilter, RefuseFilter, RouterSampler, StepResult, TokenSoupFilter, ToolExploreReward, ToolManager,
                                  f1_score, normalize_messages, parse_tool_calls)
from twinkle_b200.data_format.sampling import SampledSequence, SampleResponse, SamplingParams


class ScriptedSampler:
    """Replies with the next scripted text for each trajectory (keyed by its first user message)."""

    def __init__(self, scripts, logprob=-0.1):
        self.scripts, self.turn, self.logprob, self.calls = scripts, {}, logprob, 0

    def sample(self, trajectories, sampling_params=None, **kw):
        self.calls += 1
        out = []
        for t in trajectories:
            key = next(m['content'] for m in t['messages'] if m['role'] == 'user')
            i = self.turn.get(key, 0)
            self.turn[key] = i + 1
            text = self.scripts[key][min(i, len(self.scripts[key]) - 1)]
            toks = list(range(len(text.split())))
            out.append(SampleResponse(sequences=[SampledSequence(stop_reason='stop', tokens=toks, logprobs=[self.logprob] * len(toks), decoded=text)]))
        return out


def _call(name, **args):
    return '<tool_call>' + json.dumps({'name': name, 'arguments': args}) + '</tool_call>'


def test_tool_manager_and_parse():
    def add(a: int, b: int) -> int:
        """Add two integers."""
        return a + b

    tm = ToolManager([FunctionTool(add)])
    assert tm.names() == ['add'] and tm.tool_infos()[0]['parameters']['required'] == ['a', 'b']
    calls = parse_tool_calls('thinking… ' + _call('add', a=2, b=3) + ' and ' + _call('nope'))
    assert [c['tool_name'] for c in calls] == ['add', 'nope']
    assert tm(calls[0]) == '5'
    assert tm(calls[1]).startswith('Error: unknown tool')
    assert 'not valid JSON' in tm({'tool_name': 'add', 'arguments': '{bad'})


def test_multi_turn_rollout_runs_tools_until_answer():
    def lookup(key: str) -> str:
        return {'capital:fr': 'Paris'}.get(key, 'unknown')

    scripts = {'q1': [_call('lookup', key='capital:fr'), 'The answer is <answer>Paris</answer>'],
               'q2': ['<answer>42</answer>']}
    sampler = ScriptedSampler(scripts)
    ro = MultiTurnRollout(sampler, ToolManager([FunctionTool(lookup)]), max_turns=4, sampling_params=SamplingParams(max_tokens=32))
    out = ro([{'messages': [{'role': 'user', 'content': 'q1'}]}, {'messages': [{'role': 'user', 'content': 'q2'}]}])
    roles = [m['role'] for m in out[0]['messages']]
    assert roles == ['user', 'assistant', 'tool', 'assistant']
    assert out[0]['messages'][2]['content'] == 'Paris' and out[0]['messages'][1]['tool_calls'][0]['tool_name'] == 'lookup'
    assert [m['role'] for m in out[1]['messages']] == ['user', 'assistant']
    assert out[0]['user_data']['rollout'] == {'turns': 2, 'tool_calls': 1, 'tokens': out[0]['user_data']['rollout']['tokens'], 'stop': 'answer'}
    assert sampler.calls == 2  # both trajectories share turn 1, only the first needs turn 2
    assert F1Reward()(out, ['Paris', '41']) == [1.0, 0.0]
    assert ToolExploreReward()(out, ['Paris', '42']) == [0.1, 0.0]
    assert CoTReward()([{'messages': [{'role': 'assistant', 'content': 'First this. Then that. <answer>x</answer>'}]}]) == [1.0]


class CountEnv(Env):
    """Reach the target by calling ``inc``; reward 1 when reached."""

    def reset(self, trajectory=None):
        self.v, self.target = 0, int((trajectory or {}).get('user_data', {}).get('target', 2))
        return StepResult('start')

    def step(self, tool_name, arguments):
        self.v += int(arguments.get('by', 1))
        done = self.v >= self.target
        return StepResult(f'value={self.v}', 1.0 if done else 0.0, done)

    def tools(self):
        return [{'tool_name': 'inc', 'description': 'increase', 'parameters': {'type': 'object', 'properties': {'by': {'type': 'integer'}}}}]


def test_env_pool_rollout_stops_when_episode_ends():
    pool = EnvPool(CountEnv, 2)
    scripts = {'go': [_call('inc', by=1)] * 5}
    ro = MultiTurnRollout(ScriptedSampler(scripts), pool.managers, max_turns=6)
    out = ro([{'messages': [{'role': 'user', 'content': 'go'}], 'user_data': {'target': 2}}])
    assert out[0]['user_data']['rollout']['stop'] == 'env_done' and out[0]['user_data']['rollout']['turns'] == 2
    assert out[0]['user_data']['env_reward'] == 1.0


def test_chunk_condense_extract_roundtrip():
    long = ('Quarterly revenue rose sharply in the northern region. ' + 'The warehouse inventory figures were audited again. ' * 40)
    traj = {'messages': [{'role': 'user', 'content': 'summarise'}, {'role': 'tool', 'content': long, 'tool_call_id': 'c1'},
                         {'role': 'assistant', 'content': 'ok'}]}
    chunks = NativeChunker(chunk_size=700)(traj)
    assert all(len(c.content) <= 1400 for c in chunks) and ''.join(c.content for c in chunks if c.role == 'tool') == long
    cond = KeywordCondenser(min_chars=300, budget_chars=160, keep_last=1)(chunks)
    condensed = [c for c in cond if c.condensed]
    assert condensed and all(len(c.content) <= 160 for c in condensed) and 'Quarterly revenue' in condensed[0].content
    view = cond.to_trajectory()
    assert sum(len(m['content']) for m in view['messages']) < len(long) / 2 and '[block 1, condensed]' in view['messages'][1]['content']
    tool = ExtractCondensed(cond)
    assert condensed[0].original in tool('extract_condensed', {'blocks': [1]}) and 'unknown' in tool('extract_condensed', {'blocks': [99]})


def test_condense_rollout_presents_short_view_and_serves_originals():
    long = 'Alpha beta gamma delta. ' * 800
    seen = {}

    class Spy(ScriptedSampler):

        def sample(self, trajectories, sampling_params=None, **kw):
            seen['chars'] = sum(len(m['content']) for m in trajectories[0]['messages'])
            seen['tools'] = [t['tool_name'] for t in trajectories[0].get('tools') or []]
            return super().sample(trajectories, sampling_params, **kw)

    scripts = {'start': [_call('extract_condensed', blocks=[1]), '<answer>done</answer>']}
    ro = MultiTurnCondenseRollout(Spy(scripts), condense_above_chars=2000, condenser=KeywordCondenser(min_chars=500, keep_last=0), max_turns=3)
    out = ro([{'messages': [{'role': 'user', 'content': 'start'}, {'role': 'tool', 'content': long, 'tool_call_id': 'x'}]}])
    assert seen['chars'] < len(long) / 3 and 'extract_condensed' in seen['tools']
    tool_msgs = [m for m in out[0]['messages'] if m['role'] == 'tool']
    assert tool_msgs[0]['content'] == long          # stored trajectory keeps the full text
    assert tool_msgs[1]['content'].startswith('[block 1] Alpha beta')


def test_router_sampler_reroutes_low_confidence():
    cheap, strong = ScriptedSampler({'a': ['weak'], 'b': ['fine']}, logprob=-0.1), ScriptedSampler({'a': ['strong'], 'b': ['strong']})
    cheap_resp = cheap.sample

    def shaky(trajs, sp=None, **kw):
        rs = cheap_resp(trajs, sp, **kw)
        rs[0].sequences[0].logprobs = [-3.0] * 3  # first trajectory looks unreliable
        return rs

    cheap.sample = shaky
    r = RouterSampler(cheap, strong, min_mean_logp=-1.0)
    out = r.sample([{'messages': [{'role': 'user', 'content': 'a'}]}, {'messages': [{'role': 'user', 'content': 'b'}]}], SamplingParams(max_tokens=8))
    assert [o.sequences[0].decoded for o in out] == ['strong', 'fine'] and r.routed == 1


def test_filters_and_normaliser():
    ok = {'messages': [{'role': 'user', 'content': 'hi'}, {'role': 'assistant', 'content': 'A clear and useful reply about sorting algorithms.'}]}
    assert all(f.keep(ok) for f in (RefuseFilter(), DeadLoopFilter(), TokenSoupFilter(), HardFilter(), MessageSanityFilter(), PIIFilter()))
    d = DedupFilter()
    assert d.keep(ok) and not d.keep(json.loads(json.dumps(ok)))
    assert not RefuseFilter().keep({'messages': [{'role': 'assistant', 'content': "I'm sorry, but I can't help with that."}]})
    loop = {'messages': [{'role': 'assistant', 'content': '\n'.join(['the same long line again'] * 6)}]}
    assert not DeadLoopFilter().keep(loop)
    soup = {'messages': [{'role': 'assistant', 'content': ' '.join(['zq'] * 200)}]}
    assert not TokenSoupFilter().keep(soup)
    assert not PIIFilter().keep({'messages': [{'role': 'assistant', 'content': 'mail me at jo@example.com'}]})
    masked = {'messages': [{'role': 'assistant', 'content': 'mail me at jo@example.com'}]}
    assert PIIFilter(mask=True).keep(masked) and masked['messages'][0]['content'] == 'mail me at <email>'
    assert not MessageSanityFilter().keep({'messages': [{'role': 'user', 'content': 'a'}, {'role': 'user', 'content': 'b'}]})
    n = normalize_messages({'messages': [{'role': 'System', 'content': ' '}, {'role': 'user', 'content': [{'type': 'text', 'text': 'x'}]},
                                         {'role': 'assistant', 'content': None, 'tool_calls': [{'id': '1', 'function': {'name': 'f', 'arguments': '{}'}}]}]})
    assert [m['role'] for m in n['messages']] == ['user', 'assistant'] and n['messages'][1]['tool_calls'][0]['tool_name'] == 'f'
    assert abs(f1_score('the cats sat', 'cat sat down') - 2 * (2 / 2) * (2 / 3) / ((2 / 2) + (2 / 3))) < 1e-9


def test_tool_call_formats_round_trip():
    from twinkle_b200.template.tools import get_format, parse_tool_calls, tools_system_prompt
    call = {'tool_name': 'read_file', 'arguments': {'path': 'a.py', 'lines': '1-5'}}
    for name in ('hermes', 'react', 'cline', 'vcp'):
        f = get_format(name)
        text = 'Let me look.\n' + f.render(call) + '\n'
        assert f.detect(text), name
        got = f.parse(text)
        assert len(got) == 1 and got[0]['tool_name'] == 'read_file', (name, got)
        args = got[0]['arguments']
        assert {k: str(v) for k, v in args.items()} == {'path': 'a.py', 'lines': '1-5'}, (name, args)
        assert 'Let me look.' in f.strip(text) and 'read_file' not in f.strip(text), name
    calls, rest, fmt = parse_tool_calls('Thought: need it\nAction: search\nAction Input: {"q": "b200"}\nObservation: …')
    assert fmt == 'react' and calls[0]['arguments'] == {'q': 'b200'}
    calls, rest, fmt = parse_tool_calls('<thinking>hm</thinking> no tools here')
    assert calls == [] and fmt is None
    vcp = get_format('vcp')
    nested = vcp.render({'tool_name': 'echo', 'arguments': {'text': 'has 「末」 inside'}})
    assert vcp.parse(nested)[0]['arguments']['text'] == 'has 「末」 inside'
    assert '<tool_call>' in tools_system_prompt([{'tool_name': 'x', 'description': 'd', 'parameters': {}}])


def test_model_condenser_batches_pads_and_rejects_useless_replies():
    from twinkle_b200.agentic import Chunk, Chunks, ModelCondenser
    from twinkle_b200.data_format import SampledSequence, SampleResponse

    class S:
        template = None

        def __init__(self):
            self.calls = []

        def sample(self, trajs, params, **kw):
            self.calls.append((len(trajs), params.max_tokens, kw))
            out = []
            for t in trajs:
                text = t['messages'][1]['content']
                if 'KEEPME' in text:
                    reply = 'x' * 5000  # longer than the passage → rejected
                elif 'FENCE' in text:
                    reply = '```\nshort fenced digest\n```'
                else:
                    reply = 'digest of ' + text.split('Question the reader cares about: ')[1].split('\n')[0]
                out.append(SampleResponse(sequences=[SampledSequence('stop', [1], decoded=reply)]))
            return out

    long = lambda tag: tag + ' ' + 'lorem ipsum ' * 80  # noqa: E731
    chunks = Chunks([Chunk('user', 'Question: who?', 0), Chunk('tool', long('A'), 1), Chunk('tool', long('KEEPME'), 2), Chunk('tool', long('FENCE'), 3),
                     Chunk('tool', 'short', 4), Chunk('tool', long('SKIP: raw'), 5), Chunk('assistant', long('B'), 6)], {'messages': []})
    s = S()
    cond = ModelCondenser(s, compression_ratio=4.0, batch_size=2, skip_pattern=r'^SKIP:',
                          related_query=lambda c: c.content[len('Question: '):] if c.content.startswith('Question: ') else None)
    out = list(cond(chunks))
    assert [c.condensed for c in out] == [False, True, False, True, False, False, False]
    assert out[1].content == 'digest of who?' and out[1].original.startswith('A lorem') and out[1].block == 1
    assert out[3].content == 'short fenced digest' and out[3].block == 2
    assert [c[0] for c in s.calls] == [2, 2] and s.calls[0][2] == {'use_base_model': True}  # 3 jobs → one full batch + one padded
    assert s.calls[0][1] >= 32
    assert list(cond(Chunks(out, {'messages': []})))[1].content == 'digest of who?'  # idempotent on condensed chunks
    assert ModelCondenser(s, lora_path='/x')._ask([{'text': 't', 'budget': 10, 'query': 'q'}]) and s.calls[-1][2] == {'adapter_path': '/x'}
    import pytest
    with pytest.raises(ValueError):
        ModelCondenser(s, compression_ratio=1.0)
    with pytest.raises(ValueError):
        ModelCondenser(s, user_prompt_template='no slots')


class _Obs:

    def __init__(self, observation, reward=0.0, done=False):
        self.observation, self.reward, self.done = observation, reward, done


class CounterEnvironment:
    """OpenEnv-style environment: counts up by the action's ``by`` and ends at ``limit``."""

    def __init__(self, limit=3):
        self.limit, self.n = limit, 0

    def reset(self):
        self.n = 0
        return _Obs({'text': 'n=0'})

    def step(self, action):
        by = action.by if hasattr(action, 'by') else action['by']
        self.n += by
        return {'observation': f'n={self.n}', 'reward': float(by), 'done': self.n >= self.limit}


class CounterAction:

    def __init__(self, by=1):
        self.by = by


def test_openenv_adapter_and_sharded_pool(monkeypatch):
    from twinkle_b200.agentic import EnvPoolAdapter, EnvTool, OpenEnv, ShardedEnvPool, ToolManager, normalize_result, observation_text
    env = OpenEnv(env_cls=f'{__name__}:CounterEnvironment', env_kwargs={'limit': 2}, action_cls=CounterAction)
    assert env.reset().observation == 'n=0'
    r = env.step('act', {'by': 2})
    assert (r.observation, r.reward, r.done) == ('n=2', 2.0, True)
    mapped = OpenEnv(env_cls=CounterEnvironment, action_mapper=lambda name, args: {'by': 5 if name == 'jump' else 1})
    assert mapped.step('jump', {}).observation == 'n=5' and mapped.tools()[0]['tool_name'] == 'act'
    assert observation_text({'foo': 1}) == '{"foo": 1}' and observation_text(None) == '' and normalize_result('plain')['observation'] == 'plain'
    import pytest
    with pytest.raises(ValueError):
        OpenEnv()
    with pytest.raises(ValueError):
        OpenEnv(env_cls='NoDots')

    # two "workers" built by hand: rank 0 owns slots 0-1, rank 1 owns slot 2
    pools = []
    for rank in (0, 1):
        monkeypatch.setenv('RANK', str(rank))
        monkeypatch.setenv('WORLD_SIZE', '2')
        pools.append(ShardedEnvPool(pool_size=3, env_kwargs={'env_cls': CounterEnvironment, 'env_kwargs': {'limit': 2}}))
    assert [(p._start, p._end) for p in pools] == [(0, 2), (2, 3)]
    assert pools[0].reset(2) is None and pools[1].reset(2)['observation'] == 'n=0'
    parts = [p.step_batch([0, 1, 2], ['act'] * 3, [{'by': 1}, {'by': 2}, {'by': 1}]) for p in pools]
    from twinkle_b200.agentic.openenv import _merge_by_slot
    merged = _merge_by_slot(parts)
    assert [m['observation'] for m in merged] == ['n=1', 'n=2', 'n=1'] and [m['done'] for m in merged] == [False, True, False]
    assert pools[0].step(0, 'act', {'by': 1})['episode_reward'] == 2.0

    monkeypatch.setenv('RANK', '0')
    monkeypatch.setenv('WORLD_SIZE', '1')
    pool = ShardedEnvPool(pool_size=2, env_kwargs={'env_cls': CounterEnvironment})
    a, b = pool.get_adapters(2)
    assert isinstance(a, EnvPoolAdapter) and a.reset().observation == 'n=0'
    assert a.step('act', {'by': 2}).info == {'episode_reward': 2.0} and a.episode_reward == 2.0 and b.episode_reward == 0.0
    bad = a.step('act', {'nope': 1})
    assert bad.done and bad.observation.startswith('Error:')
    tm = ToolManager(EnvTool.from_env(b))
    assert tm({'tool_name': 'act', 'arguments': {'by': 1}}) == 'n=1'
    with pytest.raises(ValueError):
        pool.get_adapters(3)
    pool.close()


def test_client_multi_turn_rollout_token_exact_state():
    import pytest
    from twinkle_b200.agentic import FunctionTool, ToolManager
    from twinkle_b200.client import ClientMultiTurnRollout
    from twinkle_b200.template import Template
    tpl = Template(model_id=None)

    def add(a: int, b: int) -> int:
        """Add two integers."""
        return a + b

    class HttpLikeSampler:
        """Answers like the JSON of ``/twinkle/sample``: first a tool call, then a final answer; one trajectory runs
        into the length limit at once."""

        def __init__(self):
            self.batches = []

        def sample(self, feats, sp):
            self.batches.append(len(feats))
            out = []
            for f in feats:
                text_so_far = tpl.decode(f['input_ids'], skip_special_tokens=False)
                if 'LONG' in text_so_far:
                    reply, reason = 'cut off', 'length'
                elif 'tool_response' in text_so_far or '"role": "tool"' in text_so_far or '5' in text_so_far.split('add')[-1]:
                    reply, reason = 'The sum is 5.', 'stop'
                else:
                    reply, reason = '<tool_call>\n{"name": "add", "arguments": {"a": 2, "b": 3}}\n</tool_call>', 'stop'
                toks = tpl.tokenizer.encode(reply)
                out.append({'sequences': [{'stop_reason': reason, 'tokens': toks, 'logprobs': [-0.1] * len(toks), 'decoded': reply,
                                           'new_input_feature': Template.concat_input_feature(f, toks)}]})
            return out

    s = HttpLikeSampler()
    roll = ClientMultiTurnRollout(s, tpl, ToolManager([FunctionTool(add)]), {'max_tokens': 64}, max_turns=3)
    res = roll([{'messages': [{'role': 'user', 'content': 'what is 2+3? use add'}]}, {'messages': [{'role': 'user', 'content': 'LONG one'}]}])
    assert s.batches == [2, 1]  # the finished trajectory is left out of the second call
    a, b = res
    assert [m['role'] for m in a['messages']] == ['user', 'assistant', 'tool', 'assistant'] and a['messages'][2]['content'] == '5'
    assert a['turns'] == 2 and a['stop_reason'] == 'stop' and not a['truncated']
    assert b['turns'] == 1 and b['stop_reason'] == 'length'
    labels = a['input_feature']['labels']
    assert sum(1 for x in labels if x != -100) == len(a['logprobs']) and len(labels) == len(a['input_feature']['input_ids'])
    # a single allowed turn that ends in a tool call is a truncation
    one = ClientMultiTurnRollout(HttpLikeSampler(), tpl, ToolManager([FunctionTool(add)]), {'max_tokens': 64}, max_turns=1)(
        [{'messages': [{'role': 'user', 'content': 'use add'}]}])[0]
    assert one['truncated'] and one['stop_reason'] == 'max_turns' and one['messages'][-1]['role'] == 'assistant'
    with pytest.raises(ValueError):
        ClientMultiTurnRollout(HttpLikeSampler(), tpl, None, {'max_tokens': 8})([{'messages': [{'role': 'user', 'content': 'use add'}]}])
    with pytest.raises(TypeError):
        roll({'messages': []})
    with pytest.raises(ValueError):
        ClientMultiTurnRollout(s, tpl, sampling_params={'num_samples': 2})
    assert roll([]) == []


def test_template_tool_call_parsing_and_react_rollout():
    from twinkle_b200.agentic import FunctionTool, MultiTurnRollout, ToolManager
    from twinkle_b200.data_format import SampledSequence, SampleResponse
    from twinkle_b200.template import Template
    t = Template(model_id=None)
    msg = t.response_message('ok <tool_call>\n{"name": "add", "arguments": {"a": 1}}\n</tool_call>')
    assert msg['content'] == 'ok' and msg['tool_calls'][0]['tool_name'] == 'add' and msg['tool_calls'][0]['arguments'] == {'a': 1}
    assert t.response_message('plain') == {'role': 'assistant', 'content': 'plain'}
    react = Template(model_id=None, agent_template='react')
    text = 'Thought: add them\nAction: add\nAction Input: {"a": 2, "b": 3}'
    assert react.parse_tool_call(text)[0]['arguments'] == {'a': 2, 'b': 3} and react.clean_tool_call(text) == 'Thought: add them'
    assert react.parse_tool_call('<tool_call>\n{"name": "add", "arguments": {}}\n</tool_call>') == []  # only the configured syntax

    def add(a: int, b: int) -> int:
        """Add."""
        return a + b

    class S:

        def sample(self, trajs, sp, **kw):
            out = []
            for tr in trajs:
                done = any(m['role'] == 'tool' for m in tr['messages'])
                out.append(SampleResponse(sequences=[SampledSequence('stop', [1], decoded='Final Answer: 5' if done else text)]))
            return out

    res = MultiTurnRollout(S(), ToolManager([FunctionTool(add)]), max_turns=3, tool_format='react')([{'messages': [{'role': 'user', 'content': '2+3?'}]}])[0]
    assert [m['role'] for m in res['messages']] == ['user', 'assistant', 'tool', 'assistant'] and res['messages'][2]['content'] == '5'
    assert res['messages'][1]['content'] == 'Thought: add them' and res['user_data']['rollout']['tool_calls'] == 1
