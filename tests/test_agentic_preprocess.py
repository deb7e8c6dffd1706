"""Quality pipeline steps of the agentic package: text operators, allow list, intent classifier, LLM back ends,
log-probability scorers, round filter and the pipeline runner (all CPU, no model: back ends are faked)."""
import json
import math

import pytest

from twinkle_b200.agentic import (ChrMinScorer, DedupFilter, FixUnicodeFilter, IntentClassifier, LLMBackend, MessageNormalizer, ModelFilter,
                                  OpenAIBackend, ParaphraseScorer, PassNScorer, QualityPreprocessor, RemoveRepeatSentencesFilter,
                                  RoundScoreFilter, SamplerBackend, SIFDScorer, SpecialCharsFilter, TokenNumFilter, chr_min_distinct,
                                  count_tokens, ifd_family)
from twinkle_b200.data_format import SampledSequence, SampleResponse, user_data_get
from twinkle_b200.template import Template


def row(*turns, **extra):
    return dict(messages=[{'role': r, 'content': c} for r, c in turns], **extra)


def test_fix_unicode_repairs_mojibake_and_normalises():
    f = FixUnicodeFilter()
    bad = 'cafÃ© â€“ donâ€™t\x07 é'
    kept, dropped = f([row(('user', 'q'), ('assistant', bad))])
    assert dropped == []
    assert kept[0]['messages'][1]['content'] == 'café – don’t é'
    assert kept[0]['messages'][0]['content'] == 'q'
    with pytest.raises(ValueError):
        FixUnicodeFilter('XYZ')


def test_remove_repeat_sentences_keeps_first_occurrence():
    f = RemoveRepeatSentencesFilter(lowercase=True)
    text = 'The answer is 4. Let me check. the answer is 4! Ok.\nThe answer is 4.\nDone.'
    kept, _ = f([row(('assistant', text))])
    assert kept[0]['messages'][0]['content'] == 'The answer is 4. Let me check. Ok.\n\nDone.'


def test_special_chars_and_token_num_filters():
    rows = [row(('assistant', 'plain words only here')), row(('assistant', '#$%^&*()!!@@##$$')), row(('user', 'no assistant text'))]
    kept, dropped = SpecialCharsFilter(0.25)(rows)
    assert len(kept) == 2 and dropped[0]['drop_reason'] == 'special_chars_ratio'
    assert count_tokens('hello, 世界 ok') == 5
    kept, dropped = TokenNumFilter(min_num=3, max_num=5)([row(('assistant', 'a b')), row(('assistant', 'a b c d')), row(('assistant', 'a b c d e f'))])
    assert [r['messages'][0]['content'] for r in kept] == ['a b c d']
    assert all(d['drop_reason'] == 'token_count_out_of_range' for d in dropped)
    tok = Template(model_id=None).tokenizer
    assert count_tokens('abc', tok) == len(tok.encode('abc'))


def test_model_filter_families_and_tails():
    f = ModelFilter()
    ids = ['Qwen/Qwen3-235B-A22B-Thinking-2507', 'deepseek-ai/DeepSeek-R1-Distill-Qwen-7B', 'moonshotai/Kimi-K2-Instruct', 'Qwen/Qwen3-8B',
           'meta/llama-3', None]
    kept, dropped = f([{'model_id': i} for i in ids])
    assert [r['model_id'] for r in kept] == ids[:3]
    assert all(d['drop_reason'] == 'model_not_allowed' for d in dropped)
    assert len(ModelFilter(patterns=['meta/llama'])([{'model_id': 'meta/llama-3'}])[0]) == 1


def test_message_normalizer_step():
    kept, dropped = MessageNormalizer()([{'messages': [{'role': 'USER', 'content': [{'type': 'text', 'text': 'hi'}]},
                                                       {'role': 'assistant', 'content': None}]}, {'messages': 'oops'}])
    assert kept[0]['messages'][0] == {'role': 'user', 'content': 'hi'} and kept[0]['messages'][1]['content'] == ''
    assert dropped[0]['drop_reason'] == 'no_messages'


def test_intent_classifier_detects_and_pairs_rounds():
    think = '<think>' + 'step ' * 60 + '</think> 42'
    rows = [
        {'messages': [{'role': 'user', 'content': 'weather?'}, {'role': 'assistant', 'content': '', 'tool_calls': [{'tool_name': 'w', 'arguments': {}}]},
                      {'role': 'tool', 'content': 'sunny'}, {'role': 'assistant', 'content': '```python\nprint("sunny day")\n```'}]},
        row(('user', 'Write code'), ('assistant', '```python\ndef f(x):\n    return x + 1\n```')),
        row(('user', 'Solve $x^2=4$ with \\frac{1}{2} and \\sqrt{2}, x = 2'), ('assistant', 'ok')),
        row(('user', 'hi'), ('assistant', think)),
        row(('user', 'q'), ('assistant', 'a1'), ('user', 'That is wrong, try again'), ('assistant', 'a2')),
        row(('user', 'That is wrong'), ('assistant', 'fine')),
        row(('user', 'hello'), ('assistant', 'hello there')),
    ]
    kept, dropped = IntentClassifier()(rows)
    assert [r['intent'] for r in kept] == ['tool_call', 'code', 'math', 'reasoning', 'user_dissatisfaction']
    # the tool-call detector is definitive: the fenced code in the same trajectory is not looked at
    assert user_data_get(kept[0]['user_data'], 'key_rounds') == [1]
    assert user_data_get(kept[2]['user_data'], 'key_rounds') == [1]  # signal in the user turn → next assistant turn
    assert user_data_get(kept[4]['user_data'], 'intents') == {'3': 'user_dissatisfaction'}
    assert [d['drop_reason'] for d in dropped] == ['no_key_rounds'] * 2  # a complaint before any answer does not count
    kept, dropped = IntentClassifier(drop_no_key_rounds=False)(rows[-1:])
    assert kept[0]['intent'] == 'other' and not dropped
    # dict-shaped user_data stays a dict
    kept, _ = IntentClassifier()([dict(rows[1], user_data={'src': 'x'})])
    assert kept[0]['user_data'] == {'src': 'x', 'key_rounds': [1], 'intents': {'1': 'code'}}


def test_logprob_metrics_by_hand():
    # prompt of 2 tokens, response tokens [7, 8, 7]; deltas: 7 → +1.0 and −0.5 (min −0.5), 8 → +0.2
    cond_ids, asst_ids = [1, 2, 7, 8, 7], [7, 8, 7]
    cond_lp = [None, -1.0, {7: -1.0}, {'8': {'logprob': -0.8}}, [(7, -2.5)]]
    asst_lp = [None, -1.0, -2.0]
    asst_lp[0] = -2.0
    assert chr_min_distinct(cond_lp, asst_lp, cond_ids, asst_ids, 2) == pytest.approx(0.5)
    fam = ifd_family(cond_lp, asst_lp, cond_ids, asst_ids, 2)
    deltas = [1.0, 0.2, -0.5]
    assert fam['n_tokens'] == 3 and fam['ifd'] == pytest.approx(math.exp(-sum(deltas) / 3))
    assert fam['s_ifd_50'] == pytest.approx(math.exp(-(1.0 - 0.5) / 2))
    assert chr_min_distinct([], [], [], [], 0) is None and ifd_family(None, None, [], [], 0) == {}


class FakeBackend(LLMBackend):
    """Chat replies chosen by a substring of the last message; flat log-probabilities."""

    def __init__(self, hard=(), replies=None):
        self.hard, self.replies, self.calls = set(hard), replies or {}, []

    def chat(self, messages, *, temperature=0.0, max_tokens=16, n=1):
        self.calls.append(messages)
        last = messages[-1]['content']
        for key, val in self.replies.items():
            if key in last:
                return [{'content': v, 'reasoning_content': ''} for v in (val if isinstance(val, list) else [val] * n)]
        return [{'content': 'a reply of several plain words here', 'reasoning_content': ''}] * n

    def prompt_logprobs(self, messages):
        return None

    def prompt_logprobs_ids(self, input_ids_list):
        return [[None] + [-1.0] * (len(ids) - 1) for ids in input_ids_list]


class RuleBackend(FakeBackend):
    """Log-probabilities by rule: a token costs −1 on its own and −0.5 when a prompt precedes it, except token ids in
    ``hard``, which the prompt does not help (−1.5 conditioned)."""

    def prompt_logprobs_ids(self, input_ids_list):
        # the filter asks for the conditioned batch first, then the lone answers
        self._turn = getattr(self, '_turn', 0) + 1
        conditioned = self._turn % 2 == 1
        out = []
        for ids in input_ids_list:
            out.append([(-1.5 if t in self.hard else -0.5) if conditioned else -1.0 for t in ids])
        return out


def test_round_score_filter_keeps_hard_rounds_and_rewrites_key_rounds(tmp_path):
    tpl = Template(model_id=None)
    easy, hard = 'aaaaaaaaaaaa', 'zzzzzzzzzzzz'
    hard_ids = set(tpl.tokenizer.encode('z'))
    backend = RuleBackend(hard=hard_ids)
    rows = [
        dict(row(('user', 'q1'), ('assistant', easy), ('user', 'q2'), ('assistant', hard)), user_data=[('key_rounds', '[1, 3]')]),
        row(('user', 'q'), ('assistant', easy)),
        row(('user', 'q'), ('assistant', hard)),
        row(('user', 'only a question')),
    ]
    f = RoundScoreFilter(tpl, backend, [ChrMinScorer(0.47), SIFDScorer()], trace_dir=str(tmp_path / 'trace'))
    kept, dropped = f(rows)
    # easy answers: every token is helped by the prompt → chr_min 1.0 ≥ 0.47 → fails; hard: 'z' never helped
    assert user_data_get(kept[0]['user_data'], 'key_rounds') == [3]
    assert kept[1] is rows[2] and kept[2] is rows[3]
    assert [d['drop_reason'] for d in dropped] == ['score_round_failed']
    traces = sorted((tmp_path / 'trace').iterdir())
    assert len(traces) == 4
    rec = json.loads(traces[0].read_text())
    assert set(rec['scores']) == {'chr_min', 'sifd'} and rec['scores']['sifd']['extras']['ifd'] == pytest.approx(math.exp(-0.5))
    # intent gate: rounds without a listed intent are not scored, the row then has no context
    kept, dropped = RoundScoreFilter(tpl, backend, [ChrMinScorer()], intents=['math'])(rows[:1])
    assert not kept and dropped[0]['drop_reason'] == 'score_no_context'
    with pytest.raises(TypeError):
        RoundScoreFilter(object(), backend, [])


def test_pass_n_and_paraphrase_scorers():
    tpl = Template(model_id=None)
    rows = [row(('user', 'solved question'), ('assistant', 'the recorded answer one')), row(('user', 'open question'), ('assistant', 'the recorded answer two'))]
    policy = FakeBackend(replies={'solved question': 'good', 'open question': ['good', 'bad', 'bad', 'bad']})
    judge = FakeBackend(replies={'[Candidate]\ngood': 'fine. <verdict>PASS</verdict>', '[Candidate]\nbad': '<verdict>fail</verdict>'})
    f = RoundScoreFilter(tpl, policy, [PassNScorer(policy, judge, n=4, max_pass_rate=0.75)])
    ctx = f.build_contexts(rows)
    res = PassNScorer(policy, judge, n=4, max_pass_rate=0.75).score(ctx)
    assert [r.score for r in res] == [1.0, 0.25] and [r.passed for r in res] == [False, True]
    assert PassNScorer.parse_verdict('I think PASS') is True and PassNScorer.parse_verdict('pass or fail?') is None
    kept, dropped = f(rows)
    assert kept == rows[1:] and dropped[0]['drop_reason'] == 'score_round_failed'

    backend = RuleBackend(hard=set(tpl.tokenizer.encode('z')), replies={'solved question': 'zzzzzzzz', 'open question': 'aaaaaaaa'})
    sc = ParaphraseScorer(backend, tpl, chr_min_threshold=0.47)
    res = sc.score(ctx)
    assert [r.passed for r in res] == [True, False] and res[0].extras['paraphrase_text'] == 'zzzzzzzz'
    assert '<reference_answer>\nthe recorded answer one' in backend.calls[0][-1]['content'] and len(backend.calls[0]) == 1


def test_openai_backend_wire_format():
    seen = []

    def post(url, body):
        seen.append((url, body))
        if url.endswith('/chat/completions') and body.get('max_tokens') == 0:
            return {'prompt_logprobs': [None, {'5': {'logprob': -0.1}}]}
        if url.endswith('/chat/completions'):
            return {'choices': [{'message': {'content': '<think>hm</think> yes'}}, {'message': {'content': 'no', 'reasoning_content': 'r'}}]}
        if url.endswith('/completions'):
            return {'choices': [{'prompt_logprobs': [None, -0.3]}]}
        return {'data': [{'index': 1, 'embedding': [0, 1]}, {'index': 0, 'embedding': [1, 0]}]}

    b = OpenAIBackend('http://h:1', 'm', post=post)
    assert b.chat([{'role': 'user', 'content': 'x'}], n=2) == [{'content': 'yes', 'reasoning_content': 'hm'}, {'content': 'no', 'reasoning_content': 'r'}]
    assert seen[0][0] == 'http://h:1/v1/chat/completions' and seen[0][1]['n'] == 2
    assert b.prompt_logprobs([{'role': 'user', 'content': 'x'}])[1]['5']['logprob'] == -0.1
    assert b.prompt_logprobs_ids([[1, 2]]) == [[None, -0.3]] and seen[-1][1]['echo'] is True
    assert b.embeddings(['a', 'b']).tolist() == [[1.0, 0.0], [0.0, 1.0]]
    assert len(b.chat_batch([[{'role': 'user', 'content': str(i)}] for i in range(3)])) == 3

    def broken(url, body):
        raise OSError('down')

    assert OpenAIBackend('http://h:1/v1', 'm', post=broken).chat([]) == []


def test_sampler_backend_uses_score_only_mode():

    class S:

        def __init__(self):
            self.seen = []

        def sample(self, inputs, params, **kw):
            self.seen.append((inputs, params, kw))
            if params.max_tokens == 0:
                return [SampleResponse(sequences=[], prompt_logprobs=[None] + [-0.5] * (len(i.get('input_ids', [0, 0])) - 1)) for i in inputs]
            return [SampleResponse(sequences=[SampledSequence('stop', [1], decoded='<think>t</think>out') for _ in range(params.num_samples)]) for _ in inputs]

    s = S()
    b = SamplerBackend(s, adapter_name='ad')
    assert b.chat([{'role': 'user', 'content': 'x'}], n=2) == [{'content': 'out', 'reasoning_content': 't'}] * 2
    assert s.seen[0][2] == {'adapter_name': 'ad'} and s.seen[0][1].num_samples == 2
    assert b.prompt_logprobs_ids([[1, 2, 3]]) == [[None, -0.5, -0.5]]
    assert s.seen[-1][1].max_tokens == 0 and s.seen[-1][1].prompt_logprobs == 1
    assert b.prompt_logprobs([{'role': 'user', 'content': 'x'}]) == [None, -0.5]
    with pytest.raises(NotImplementedError):
        b.embeddings(['a'])
    with pytest.raises(ValueError):
        b.prompt_logprobs_ids([])


def test_quality_preprocessor_runs_mixed_steps_and_logs_drops(tmp_path):
    log = tmp_path / 'd' / 'dropped.jsonl'
    rows = [row(('user', 'a'), ('assistant', 'plain answer words')), row(('user', 'a'), ('assistant', 'plain answer words')),
            row(('user', 'b'), ('assistant', '!!!@@@###$$$'))]
    pipe = QualityPreprocessor([MessageNormalizer(), DedupFilter(), SpecialCharsFilter()], dropped_log_path=str(log))
    out = pipe(rows)
    assert len(out) == 1
    assert [(s['step'], s['before'], s['after']) for s in pipe.last_stats] == [('MessageNormalizer', 3, 3), ('DedupFilter', 3, 2), ('SpecialCharsFilter', 2, 1)]
    lines = [json.loads(l) for l in log.read_text().splitlines()]
    assert [l['step'] for l in lines] == ['DedupFilter', 'SpecialCharsFilter'] and lines[1]['row']['drop_reason'] == 'special_chars_ratio'
    assert QualityPreprocessor([lambda rs: []])(rows) == []


def test_pii_rewriter_detects_validates_and_stays_consistent():
    from twinkle_b200.agentic import PIIPresidioFilter, PIIRewriter, Strategy
    from twinkle_b200.agentic.pii import cn_id_ok, hash_short, iban_ok, luhn_ok
    assert luhn_ok('4111 1111 1111 1111') and not luhn_ok('4111 1111 1111 1112') and not luhn_ok('1234')
    assert cn_id_ok('11010519491231002X') and not cn_id_ok('110105194912310021')
    assert iban_ok('GB82 WEST 1234 5698 7654 32') and not iban_ok('GB82 WEST 1234 5698 7654 33')
    text = ('Mail bob.smith@corp.io or call +1 415-555-2671 / 13812345678. Card 4111 1111 1111 1111, not 4111 1111 1111 1112. SSN 123-45-6789. '
            'IP 10.1.2.3, version 1.2.3.4.5, id 11010519491231002X, iban GB82 WEST 1234 5698 7654 32, see https://x.y/z?a=1. bob.smith@corp.io again')
    r = PIIRewriter()
    ents = [e for _, _, e in r.detect(text)]
    assert ents == ['EMAIL_ADDRESS', 'PHONE_NUMBER', 'CN_PHONE', 'CREDIT_CARD', 'US_SSN', 'IP_ADDRESS', 'CN_ID', 'IBAN_CODE', 'URL', 'EMAIL_ADDRESS']
    rows, dropped = r([{'messages': [{'role': 'user', 'content': text}, {'role': 'assistant', 'content': [{'type': 'text', 'text': 'bob.smith@corp.io'}]}]}])
    out = rows[0]['messages'][0]['content']
    assert dropped == [] and 'bob.smith' not in out and '4111 1111 1111 1112' in out and '1.2.3.4.5' in out and out.endswith('@example.com again')
    fake = out.split('Mail ')[1].split(' ')[0]
    assert out.count(fake) == 2 and '192.0.2.' in out and 'https://example.com/' in out and '. ' in out.split('https://example.com/')[1][:12]
    assert '411************1111' in out and '138****5678' in out and r.last_report['EMAIL_ADDRESS'] == 2
    assert rows[0]['messages'][1]['content'][0]['text'] == 'bob.smith@corp.io'  # only string contents are rewritten
    h = PIIRewriter(entity_strategy={'EMAIL_ADDRESS': 'hash', 'US_SSN': Strategy.REDACT}, entities=['EMAIL_ADDRESS', 'US_SSN'], salt='s')
    assert h.rewrite('a@b.co 123-45-6789 10.1.2.3') == f"{hash_short('a@b.co', 's')}  10.1.2.3"
    ner = PIIRewriter(ner_fn=lambda t: [(t.index('Alice'), t.index('Alice') + 5, 'PERSON')] if 'Alice' in t else [])
    assert 'Alice' not in ner.rewrite('Alice wrote to alice@x.org') and ' wrote to ' in ner.rewrite('Alice wrote to alice@x.org')
    with pytest.raises(ValueError):
        PIIRewriter(entity_strategy={'URL': 'scramble'})
    assert PIIPresidioFilter is PIIRewriter
