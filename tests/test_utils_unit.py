"""Small utilities: truncation strategies, quantised-checkpoint dequantisers, streaming safetensors writer / lazy
reader, single-winner notification claim, rewards, model-hub alias handling."""
import json
import os
import uuid

import pytest
import torch


def test_template_truncation_strategies():
    from twinkle_b200.template import Template
    msgs = {'messages': [{'role': 'user', 'content': 'x' * 60}, {'role': 'assistant', 'content': 'y' * 60}]}
    full = Template(model_id=None, max_length=None).encode(msgs)
    n = len(full['input_ids'])
    assert n > 40
    with pytest.raises(ValueError):
        Template(model_id=None, max_length=32, truncation_strategy='raise').encode(msgs)
    left = Template(model_id=None, max_length=32, truncation_strategy='left').encode(msgs)
    right = Template(model_id=None, max_length=32, truncation_strategy='right').encode(msgs)
    assert len(left['input_ids']) == 32 and len(right['input_ids']) == 32
    assert left['input_ids'] == full['input_ids'][-32:] or left['input_ids'][-5:] == full['input_ids'][-5:]
    assert right['input_ids'][:5] == full['input_ids'][:5]
    parts = Template(model_id=None, max_length=32, truncation_strategy='split').encode(msgs)
    assert isinstance(parts, list) and sum(len(p['input_ids']) for p in parts) == n
    gone = Template(model_id=None, max_length=32, truncation_strategy='delete').batch_encode([msgs])
    assert gone == []


def test_dequantizers():
    from twinkle_b200.utils.dequantizer import Dequantizer, dequant_fp8_block, dequant_mxfp4
    w = torch.randn(200, 300)
    scale = torch.rand(2, 3) + 0.5                                   # one scale per 128×128 block
    q = (w / scale.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]).to(torch.float8_e4m3fn)
    back = dequant_fp8_block(q, scale, dtype=torch.float32)
    assert back.shape == w.shape and float((back - w).abs().max()) < 0.2 * float(w.abs().max())
    got = Dequantizer.maybe_dequantize('layer.weight', q, lambda n: scale if n == 'layer.weight_scale_inv' else None)
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float(), back, atol=0.05, rtol=0.05)
    assert Dequantizer.maybe_dequantize('x', w, lambda n: None) is w
    # mxfp4: nibble 2 = 1.0, nibble 10 = -1.0 (sign bit set); scale byte 128 → ×2
    blocks = torch.full((1, 16), (10 << 4) | 2, dtype=torch.uint8)
    vals = dequant_mxfp4(blocks, torch.tensor([128], dtype=torch.uint8), dtype=torch.float32)
    assert vals.shape == (32, ) and vals[0] == 2.0 and vals[1] == -2.0


def test_streaming_safetensors_roundtrip(tmp_path):
    from twinkle_b200.utils.safetensors_io import SafetensorLazyLoader, StreamingSafetensorSaver
    saver = StreamingSafetensorSaver(str(tmp_path), max_shard_bytes=4096)   # tiny shards → several files + an index
    tensors = {f'layer.{i}.weight': torch.randn(32, 16) for i in range(6)}
    saver.add_many(tensors.items())
    files = saver.finalize()
    assert len(files) > 1 and os.path.isfile(os.path.join(str(tmp_path), 'model.safetensors.index.json'))
    idx = json.load(open(os.path.join(str(tmp_path), 'model.safetensors.index.json')))
    assert set(idx['weight_map']) == set(tensors)
    loader = SafetensorLazyLoader(str(tmp_path))
    assert sorted(loader.keys()) == sorted(tensors) and 'layer.3.weight' in loader
    assert all(torch.equal(loader.get(k), v) for k, v in tensors.items())
    assert torch.equal(loader.get_slice('layer.2.weight')[4:8], tensors['layer.2.weight'][4:8])
    loader.close()
    peft = StreamingSafetensorSaver(str(tmp_path / 'ad'), peft=True)
    peft.add('base_model.model.x.lora_A.weight', torch.zeros(2, 2))
    assert [os.path.basename(f) for f in peft.finalize()] == ['adapter_model.safetensors']


def test_claim_once_and_notifier(monkeypatch):
    from twinkle_b200.notifier import Notifier
    from twinkle_b200.utils.parallel import claim_once
    key = f'test-{uuid.uuid4().hex}'
    assert claim_once(key, ttl=60) is True and claim_once(key, ttl=60) is False   # one winner per key and window
    sent = []

    class Capture(Notifier):
        def _send(self, text):
            sent.append(text)

    n = Capture(dedup_ttl=60)
    msg = f'boom {uuid.uuid4().hex}'
    assert n.notify(msg) and not n.notify(msg) and sent == [msg]                   # the same report goes out once
    n.to_env()
    back = Notifier.from_env()
    assert back is not None and type(back).__name__ in ('Capture', 'Notifier')


def test_rewards():
    from twinkle_b200.reward import CountdownReward, FormatReward, GSM8KAccuracyReward, MathReward, extract_boxed
    t = lambda text: {'messages': [{'role': 'user', 'content': 'q'}, {'role': 'assistant', 'content': text}]}
    assert GSM8KAccuracyReward()([t('so 6*7 #### 42'), t('#### 41'), t('the answer is 1,000')], ['42', '42', '1000']) == [1.0, 0.0, 1.0]
    assert extract_boxed(r'thus \\boxed{\\frac{1}{2}} done') == r'\\frac{1}{2}'
    assert MathReward()([t(r'\\boxed{3.50}'), t(r'\\boxed{4}')], ['3.5', '5']) == [1.0, 0.0]
    fmt = FormatReward()([t('<think>a</think><answer>b</answer>'), t('no tags')])
    assert fmt[0] > fmt[1]
    cd = CountdownReward()([t('<answer>(3+4)*2</answer>'), t('<answer>3+4+2</answer>')], [{'target': 14, 'nums': [3, 4, 2]}] * 2)
    assert cd == [1.0, 0.0] or cd[0] > cd[1]


def test_hub_local_paths_and_aliases(tmp_path):
    from twinkle_b200.hub import HubOperation
    d = tmp_path / 'model'
    d.mkdir()
    (d / 'config.json').write_text('{}')
    assert HubOperation.download_model(str(d)) == str(d)                          # local directories pass through
    with pytest.raises(Exception):
        HubOperation.download_model('ms://definitely/not-cached-anywhere')        # offline: no silent network access


def test_geglu_reference_path_and_kernel_bundle_covers_gemma():
    import torch
    import torch.nn.functional as F
    from twinkle_b200 import ops
    from twinkle_b200.kernel import b200_builtin
    x = torch.randn(2, 5, 16, requires_grad=True)
    y = ops.geglu(x)
    g, u = x.chunk(2, -1)
    assert torch.allclose(y, F.gelu(g, approximate='tanh') * u, atol=1e-6)
    y.sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape
    names = {k.__name__ for k in b200_builtin()}
    assert {'Qwen3RMSNorm', 'Qwen3MLP', 'LlamaRMSNorm'} <= names
    assert not ({'Gemma2RMSNorm', 'Gemma2MLP'} & names) or {'Gemma2RMSNorm', 'Gemma2MLP'} <= names  # both or neither


def test_misc_helpers(tmp_path):
    import base64
    import torch
    from twinkle_b200.models.decoder import DecoderConfig, build_model
    from twinkle_b200.utils.misc import (align_logps_to_mask, call_with_supported_kwargs, copy_files_by_pattern, deep_getattr, find_all_linears,
                                         get_llm_model, get_runtime_meta, has_signature_parameter, load_mm_file)

    class A:
        b = {'c': type('C', (), {'d': 5})()}

    assert deep_getattr(A(), 'b.c.d') == 5 and deep_getattr(A(), 'b.x.d', 'dflt') == 'dflt'

    def f(a, b=2):
        return a + b

    assert call_with_supported_kwargs(f, 1, b=3, zzz=9) == 4 and call_with_supported_kwargs(lambda **kw: sorted(kw), x=1, y=2) == ['x', 'y']
    assert has_signature_parameter(f, 'b') and not has_signature_parameter(f, 'c')
    src, dst = tmp_path / 's', tmp_path / 'd'
    (src / 'sub').mkdir(parents=True)
    for name in ('tokenizer.json', 'config.json', 'model.safetensors', 'sub/vocab.txt', 'sub/skip.bin'):
        (src / name).write_text('x')
    assert copy_files_by_pattern(str(src), str(dst), ['*.json', '*.txt'], exclude_patterns='config*') == ['sub/vocab.txt', 'tokenizer.json']
    assert copy_files_by_pattern(str(src), str(dst), '*.json') == ['config.json']  # existing files are not copied again
    assert 'rank=' in get_runtime_meta() and 'pid=' in get_runtime_meta()

    from twinkle_b200.models.config import PRESETS
    m = build_model(DecoderConfig(**PRESETS['tiny-dense']))
    wrapper = type('W', (), {'model': type('V', (), {'model': m})()})()
    assert get_llm_model(wrapper) is m
    assert find_all_linears(wrapper) == ['down_proj', 'gate_proj', 'k_proj', 'o_proj', 'q_proj', 'up_proj', 'v_proj']
    moe = find_all_linears(build_model(DecoderConfig(**PRESETS['tiny-moe'])))
    assert 'gate' not in moe and {'gate_up_proj', 'down_proj', 'q_proj'} <= set(moe)

    mask = torch.tensor([[0, 1, 1, 0], [1, 1, 1, 1], [0, 0, 0, 0]], dtype=torch.bool)
    out = align_logps_to_mask([[0.5, 0.25, 9.0], 2.0, [1.0]], mask, torch.float32)
    assert out.tolist() == [[0, 0.5, 0.25, 0], [2, 2, 2, 2], [0, 0, 0, 0]]
    dense = torch.ones(3, 4)
    assert align_logps_to_mask(dense, mask, torch.float32) is not None and align_logps_to_mask('x', mask, torch.float32) is None
    assert align_logps_to_mask(torch.tensor([[1.0, 2.0]]), mask, torch.float32)[0].tolist() == [0, 1, 2, 0]

    assert load_mm_file(b'abc').read() == b'abc' and load_mm_file('data:image/png;base64,' + base64.b64encode(b'xyz').decode()).read() == b'xyz'
    p = tmp_path / 'f.bin'
    p.write_bytes(b'123')
    assert load_mm_file(str(p)).read() == b'123' and load_mm_file(7) == 7
    import pytest
    with pytest.raises(FileNotFoundError):
        load_mm_file('/no/such/file!!')


def test_safe_arithmetic_rejects_everything_but_arithmetic():
    import pytest
    from twinkle_b200.reward import CountdownReward, safe_arithmetic
    assert safe_arithmetic('(1+2)*3/ -3') == -3.0 and safe_arithmetic('2.5*4') == 10.0
    for bad in ('__import__("os").system("true")', '2**10', 'a+1', '1/0', '(' * 300, '[1][0]', 'True+1'):
        with pytest.raises(ValueError):
            safe_arithmetic(bad)
    t = lambda c: {'messages': [{'role': 'assistant', 'content': c}]}  # noqa: E731
    assert CountdownReward()([t('<answer>(3+5)*2 = 16</answer>'), t('<answer>3+5</answer>')], [{'nums': [2, 3, 5], 'target': 16}] * 2) == [1.0, 0.0]


def test_reasoning_split_and_qwen3_chat_template_patches():
    import jinja2
    from twinkle_b200.patch import apply_context, apply_patch
    from twinkle_b200.template import Template
    t = Template(model_id=None)
    traj = {'messages': [{'role': 'assistant', 'content': '<think>\nhm\n</think>\n\nans </think> tail'},
                         {'role': 'assistant', 'content': 'no opening tag </think> rest'}]}
    out = t._to_standard_reasoning_content(traj)['messages']
    assert out[0]['reasoning_content'] == 'hm' and out[0]['content'] == 'ans </think> tail'
    assert 'reasoning_content' not in out[1] and out[1]['content'] == 'no opening tag </think> rest'

    shipped = ("{%- for message in messages %}{%- set content = message.content %}{%- set reasoning_content = '' %}\n"
               "            {%- if '</think>' in content %}\n"
               "                {%- set reasoning_content = content.split('</think>')[0].rstrip('\\n').split('<think>')[-1].lstrip('\\n') %}\n"
               "                {%- set content = content.split('</think>')[-1].lstrip('\\n') %}\n"
               "            {%- endif %}\n"
               "[R={{ reasoning_content }}|C={{ content }}]{%- endfor %}\n"
               "{%- if multi %}\n    {{- raise_exception('No user query found in messages.') }}\n{%- endif %}")

    class Tok:
        chat_template = shipped

    tok, env = Tok(), jinja2.Environment()
    render = lambda src, **kw: env.from_string(src).render(**kw).replace('\n', '')  # noqa: E731
    msgs = [{'content': '<think>\nhm\n</think>\n\nans </think> tail'}, {'content': 'no open </think> rest'}]
    assert render(shipped, messages=msgs, multi=False) == '[R=hm|C= tail][R=no open |C= rest]'  # the defect
    with apply_context(tok, 'Qwen3ChatTemplate') as p:
        assert p.applied
        assert render(tok.chat_template, messages=msgs, multi=False) == '[R=hm|C=ans </think> tail][R=|C=no open </think> rest]'
        q = apply_patch(tok, 'Qwen3AllowToolTailTemplate')
        assert q.applied and render(tok.chat_template, messages=[], multi=True) == ''
        q.unpatch(tok)
    assert tok.chat_template == shipped

    class Other:
        chat_template = '{{ messages }}'

    assert not apply_patch(Other(), 'Qwen3ChatTemplate').applied


def test_rope_scaling_matches_transformers_and_travels_in_config():
    import pytest
    import torch
    from twinkle_b200.models.config import DecoderConfig
    from twinkle_b200.ops.reference import rope_inv_freq, rope_tables
    variants = ({'rope_type': 'llama3', 'factor': 8.0, 'low_freq_factor': 1.0, 'high_freq_factor': 4.0, 'original_max_position_embeddings': 8192},
                {'rope_type': 'yarn', 'factor': 4.0, 'original_max_position_embeddings': 32768}, {'rope_type': 'linear', 'factor': 2.0})
    try:
        from transformers import LlamaConfig
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        for rs in variants:
            c = LlamaConfig(hidden_size=4096, num_attention_heads=32, max_position_embeddings=131072, rope_parameters={**rs, 'rope_theta': 500000.0})
            want, att = ROPE_INIT_FUNCTIONS[rs['rope_type']](c, 'cpu')
            got, a = rope_inv_freq(128, 500000.0, rs)
            assert torch.allclose(want, got, rtol=1e-6, atol=0) and a == pytest.approx(att)
    except (ImportError, TypeError, KeyError):  # other transformers versions spell the config differently
        pass
    plain, _ = rope_inv_freq(128, 1e6)
    lin, _ = rope_inv_freq(128, 1e6, {'type': 'linear', 'factor': 4.0})
    assert torch.allclose(lin * 4, plain)
    l3, _ = rope_inv_freq(128, 5e5, variants[0])
    base, _ = rope_inv_freq(128, 5e5)
    assert torch.equal(l3[:8], base[:8]) and torch.allclose(l3[-1], base[-1] / 8)       # fast dims untouched, slowest ÷ factor
    cos, sin = rope_tables(torch.arange(4), 128, 5e5, variants[1])
    assert cos[0, 0] == pytest.approx(0.1 * torch.log(torch.tensor(4.0)).item() + 1.0)   # yarn scales cos/sin
    with pytest.raises(NotImplementedError):
        rope_inv_freq(128, 1e6, {'rope_type': 'su', 'factor': 2.0})            # an unknown variant is refused, not approximated
    cfg = DecoderConfig.from_hf({'model_type': 'llama', 'hidden_size': 256, 'num_attention_heads': 4, 'max_position_embeddings': 131072,
                                 'rope_scaling': {'rope_type': 'llama3', 'factor': 8.0, 'low_freq_factor': 1.0, 'high_freq_factor': 4.0,
                                                  'original_max_position_embeddings': 8192}, 'rope_theta': 5e5})
    assert cfg.rope_scaling['rope_type'] == 'llama3' and not cfg.qk_norm
    assert DecoderConfig.from_hf(cfg.to_hf()).rope_scaling == cfg.rope_scaling
    assert DecoderConfig.from_hf({'model_type': 'qwen3', 'rope_scaling': None}).rope_scaling is None
    assert DecoderConfig.from_hf({'model_type': 'qwen3', 'rope_parameters': {'rope_type': 'default', 'rope_theta': 1e6}}).rope_scaling is None


def test_image_sources_can_be_restricted(tmp_path, monkeypatch):
    import base64
    import pytest
    from twinkle_b200.utils.misc import load_mm_file
    f = tmp_path / 'x.bin'
    f.write_bytes(b'abc')
    assert load_mm_file(str(f)).read() == b'abc'
    monkeypatch.setenv('TWINKLE_MM_SOURCES', 'data')
    with pytest.raises(PermissionError):
        load_mm_file(str(f))
    with pytest.raises(PermissionError):
        load_mm_file('http://example.invalid/a.png')
    assert load_mm_file('data:image/png;base64,' + base64.b64encode(b'xyz').decode()).read() == b'xyz'


def test_safe_mode_refuses_callables_for_remote_calls(monkeypatch):
    """``TWINKLE_TRUST_REMOTE_CODE=0``: classes and callables are refused as arguments of remote classes and of calls
    that go to workers (reference ``utils/unsafe.py``); unset or ``1`` lets them through."""
    import twinkle_b200 as tw
    from twinkle_b200.utils import any_callable, check_unsafe
    assert any_callable({'a': [1, (2, len)]}) and any_callable(int) and not any_callable({'a': [1, 'x', {'b': 2.0}]})
    monkeypatch.delenv('TWINKLE_TRUST_REMOTE_CODE', raising=False)
    check_unsafe(len, cls=int)
    monkeypatch.setenv('TWINKLE_TRUST_REMOTE_CODE', '0')
    check_unsafe('CrossEntropyLoss', lr=1e-3)
    with pytest.raises(ValueError):
        check_unsafe(loss_cls=int)

    @tw.remote_class()
    class Box:

        def __init__(self, x=None):
            self.x = x

    assert Box('name').x == 'name'
    with pytest.raises(ValueError):
        Box(lambda: 1)
    monkeypatch.setenv('TWINKLE_TRUST_REMOTE_CODE', '1')
    assert callable(Box(len).x)
    for name in ('exists', 'requires', 'find_free_port', 'find_node_ip', 'trust_remote_code', 'check_unsafe', 'framework_util', 'torch_util',
                 'Plugin', 'is_master', 'init_twinkle_client', 'init_tinker_client', '__release_datetime__'):
        assert hasattr(tw, name), name


def test_loader_expands_block_quantised_fp8_weights(tmp_path):
    """A checkpoint that stores a weight in fp8 with a grid of inverse scales (one per 128 x 128 block) beside it reads as
    bf16 through the lazy loader."""
    from safetensors.torch import save_file

    from twinkle_b200.utils.safetensors_io import SafetensorLazyLoader
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 384, generator=g)
    scale_inv = w.reshape(2, 128, 3, 128).abs().amax(dim=(1, 3)) / 448.0
    q = (w.reshape(2, 128, 3, 128) / scale_inv[:, None, :, None]).reshape(256, 384).to(torch.float8_e4m3fn)
    save_file({'model.layers.0.mlp.down_proj.weight': q, 'model.layers.0.mlp.down_proj.weight_scale_inv': scale_inv.contiguous(),
               'model.norm.weight': torch.ones(8)}, str(tmp_path / 'model.safetensors'))
    loader = SafetensorLazyLoader(str(tmp_path))
    got = loader.get('model.layers.0.mlp.down_proj.weight')
    assert got.dtype == torch.bfloat16 and got.shape == w.shape
    assert float((got.float() - w).abs().max()) < 0.08 * float(w.abs().max())        # fp8 e4m3 keeps three mantissa bits
    assert loader.get('model.norm.weight').dtype == torch.float32


def test_hub_kernel_references():
    """``kernel.hub``: 'repo:Layer' with exactly one of revision / version, immutable, resolved per device by ``resolve_value``."""
    import dataclasses

    from twinkle_b200.kernel import HubRef, hub, resolve_value
    r = hub('org/repo:SiluAndMul', version=2)
    assert (r.repo_id, r.layer_name, r.version, r.revision, r.backend) == ('org/repo', 'SiluAndMul', 2, None, None)
    assert hub('ms://org/repo:Layer', revision='main', backend='cuda') == HubRef('ms://org/repo', 'Layer', 'main', None, 'cuda')   # colons in the repo id stay there
    assert hub('org/repo', 'Layer', 'v1').revision == 'v1'
    for bad in (dict(), dict(revision='a', version=1)):
        with pytest.raises(ValueError):
            hub('org/repo:Layer', **bad)
    with pytest.raises(ValueError):
        hub('org/repo', version=1)
    with pytest.raises(dataclasses.FrozenInstanceError):
        r.version = 3
    assert resolve_value({'cuda': {'cuda': int}, 'npu': str}, 'cuda') is int and resolve_value({'npu': str}, 'cuda') is None


def test_device_placement_of_explicit_groups():
    import numpy as np

    from twinkle_b200 import DeviceGroup, DeviceMesh
    from twinkle_b200.infra import get_device_placement
    groups = [DeviceGroup(name='training_cluster', ranks=list(range(16)), device_type='cuda',
                          _device_mesh={'main': DeviceMesh(device_type='cuda', mesh=np.arange(16).reshape(2, 2, 4), mesh_dim_names=('pp', 'dp', 'tp'))}),
              DeviceGroup(name='inference_cluster', ranks=list(range(8)), device_type='cuda',
                          _device_mesh={'inference': DeviceMesh(device_type='cuda', mesh=np.arange(8).reshape(2, 4), mesh_dim_names=('dp', 'tp'))})]
    text = get_device_placement(groups)
    assert "group 'training_cluster'" in text and "('pp', 'dp', 'tp')" in text and 'inference' in text
    assert 'rank 13: coord (1, 1, 1) data_rank 1' in text          # pp 1, dp 1, tp 1
    assert get_device_placement([]) == 'No device group provided.'


def test_tensor_helpers_of_the_utils_namespace():
    import twinkle_b200.utils as u
    moved = u.to_device({'a': torch.ones(2), 'b': [torch.zeros(1), 'text'], 'c': 3}, 'cpu')
    assert moved['b'][1] == 'text' and moved['c'] == 3 and moved['a'].device.type == 'cpu'
    sd = u.clone_state_dict_to_cpu({'w': torch.ones(2, requires_grad=True), 'step': 4})
    assert not sd['w'].requires_grad and sd['step'] == 4
    assert u.pad_sequence_to_length(torch.ones(2, 3), 5, -1.0).tolist()[0] == [1, 1, 1, -1, -1]
    assert u.pad_sequence_to_length(torch.ones(2, 3), 5, -1.0, left_pad=True).tolist()[0] == [-1, -1, 1, 1, 1]
    cat = u.pad_and_stack_tensors([torch.ones(2, 3), torch.ones(1, 5)])
    assert cat.shape == (3, 5) and cat[0, 3:].tolist() == [-200, -200] and cat[2].tolist() == [1] * 5
    assert u.pad_and_stack_tensors([torch.ones(2, 3), torch.ones(1, 5)], pad_value=0, concat=False).shape == (2, 2, 5)
    for name in ('SafetensorLazyLoader', 'StreamingSafetensorSaver', 'selective_log_softmax', 'framework_util', 'torch_util', 'processing_lock', 'Dequantizer'):
        assert hasattr(u, name), name
