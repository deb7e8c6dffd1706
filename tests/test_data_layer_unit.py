"""Pure unit tests for the data layer and small runtime utilities: processor collation, datasets, data loaders,
packing, preprocessors, template labelling, kernel registry, patches, CLI layering, component loader
(reference tiers: tests/processor, tests/dataset, tests/dataloader, tests/preprocessor, tests/template, tests/kernel,
tests/patch, tests/cli, tests/pluger)."""
import json
import os

import pytest
import torch

from twinkle_b200.dataset import Dataset, DatasetMeta
from twinkle_b200.utils.device_mesh import DeviceMesh


# ------------------------------------------------------------------------------------------------------ processor
def test_processor_packs_and_splits():
    from twinkle_b200.processor import InputProcessor, zigzag_indices
    feats = [{'input_ids': list(range(10, 17)), 'labels': list(range(11, 18))}, {'input_ids': [1, 2, 3], 'labels': [2, 3, -100]}]
    mb, = InputProcessor()(feats)
    assert mb.input_ids.tolist() == list(range(10, 17)) + [1, 2, 3]
    assert mb.position_ids.tolist() == list(range(7)) + [0, 1, 2]
    assert mb.cu_seqlens.tolist() == [0, 7, 10] and mb.max_seqlen == 7 and mb.seq_lens == [7, 3]
    # fixed micro-batches
    mbs = InputProcessor(micro_batch_size=1)(feats)
    assert [m.seq_lens for m in mbs] == [[7], [3]]
    # Ulysses: sequences are padded so the packed row divides by sp, each rank keeps a contiguous slice
    parts = [InputProcessor(sp_size=2, sp_rank=r)(feats)[0] for r in range(2)]
    total = sum(parts[0].seq_lens)
    assert total % 2 == 0 and all(p.input_ids.numel() == total // 2 for p in parts)
    assert torch.cat([p.local_index for p in parts]).tolist() == list(range(total))
    # context parallel: zig-zag halves, every rank the same number of tokens, the union covers the row once
    cps = [InputProcessor(cp_size=2, cp_rank=r)(feats)[0] for r in range(2)]
    assert all(n % 4 == 0 for n in cps[0].seq_lens)
    idx = torch.cat([p.local_index for p in cps])
    assert sorted(idx.tolist()) == list(range(sum(cps[0].seq_lens)))
    assert zigzag_indices(8, 2, 0).tolist() == [0, 1, 6, 7] and zigzag_indices(8, 2, 1).tolist() == [2, 3, 4, 5]
    rows = InputProcessor.unpack_packed_sequences(torch.arange(10), [7, 3], -1)
    assert rows.shape == (2, 7) and rows[1].tolist() == [7, 8, 9, -1, -1, -1, -1]


# -------------------------------------------------------------------------------------------------------- dataset
def test_dataset_sources_map_filter_mix_save(tmp_path):
    p = tmp_path / 'rows.jsonl'
    p.write_text('\n'.join(json.dumps({'q': f'q{i}', 'a': f'a{i}'}) for i in range(6)))
    ds = Dataset(DatasetMeta(dataset_id=str(p)))
    assert len(ds) == 6 and ds[2]['q'] == 'q2'
    ds.map(lambda r: {'messages': [{'role': 'user', 'content': r['q']}, {'role': 'assistant', 'content': r['a']}]})
    ds.filter(lambda r: r['messages'][0]['content'] != 'q3')
    assert len(ds) == 5 and 'messages' in ds[0]
    # wrap-around slice and in-memory columns
    mem = Dataset(DatasetMeta(data={'x': [1, 2, 3]}, data_slice=range(5)))
    assert [r['x'] for r in mem] == [1, 2, 3, 1, 2]
    # mixing: interleave vs concat
    a = Dataset(DatasetMeta(data=[{'v': 'a'}] * 3))
    a.add_dataset(DatasetMeta(data=[{'v': 'b'}] * 3))
    a.mix_dataset(interleave=True)
    assert [r['v'] for r in a][:4] == ['a', 'b', 'a', 'b']
    out = tmp_path / 'out.jsonl'
    ds.save_as(str(out))
    assert len(out.read_text().strip().splitlines()) == 5
    with pytest.raises(ValueError):
        DatasetMeta()


def test_packing_and_template_labels():
    from twinkle_b200.dataset.packing import PackingDataset, pack_to_constant_volume
    bins = pack_to_constant_volume([5, 4, 3, 3, 2, 1], 6)
    assert sorted(sum(([5, 4, 3, 3, 2, 1][i] for i in b)) for b in bins) == sorted([6, 6, 6]) or all(
        sum([5, 4, 3, 3, 2, 1][i] for i in b) <= 6 for b in bins)
    assert sorted(i for b in bins for i in b) == list(range(6))
    from twinkle_b200.template import Template
    t = Template(model_id=None, max_length=64)
    f = t.encode({'messages': [{'role': 'user', 'content': 'hi'}, {'role': 'assistant', 'content': 'yo'}]})
    n = len(f['input_ids'])
    assert len(f['labels']) == n and f['labels'][-1] == -100           # pre-shifted: nothing to predict after the last token
    first = next(i for i, l in enumerate(f['labels']) if l != -100)
    assert f['labels'][first] == f['input_ids'][first + 1]              # labels[t] is the target of position t
    assert all(l == -100 for l in f['labels'][:first])                  # the prompt carries no loss
    rows = [{'input_ids': list(range(i + 3)), 'labels': list(range(i + 3))} for i in range(5)]
    pk = PackingDataset(DatasetMeta(data=rows))
    pk.pack_dataset(max_length=8)
    assert sum(len(r['input_ids']) for r in pk) == sum(i + 3 for i in range(5)) and all(len(r['input_ids']) <= 8 for r in pk)
    assert all(r['position_ids'][0] == 0 for r in pk)


def test_dataloader_slices_resumes_and_retries():
    from twinkle_b200.dataloader import DataLoader, RetrySampler
    rows = [{'i': i} for i in range(16)]
    mesh = DeviceMesh.from_sizes(dp_size=1)
    dl = DataLoader(Dataset(DatasetMeta(data=rows)), batch_size=4, device_mesh=mesh, shuffle=False)
    batches = list(dl)
    assert len(batches) == 4 and [r['i'] for r in batches[0]] == [0, 1, 2, 3] and dl.get_state()['consumed_train_samples'] == 16
    dl2 = DataLoader(Dataset(DatasetMeta(data=rows)), batch_size=4, device_mesh=mesh, shuffle=False)
    dl2.skip_consumed_samples(8)
    assert [r['i'] for r in next(iter(dl2))] == [8, 9, 10, 11]
    with pytest.raises(ValueError):
        DataLoader(Dataset(DatasetMeta(data=rows)), batch_size=1, device_mesh=DeviceMesh.from_sizes(dp_size=2))

    class Flaky:
        def __len__(self):
            return 6

        def __getitem__(self, i):
            if i == 2:
                raise RuntimeError('bad row')
            return i

    got = list(RetrySampler(Flaky(), shuffle=False))
    assert 2 not in got and len(got) == 6  # the bad row is replaced, the epoch keeps its length


def test_preprocessors():
    from twinkle_b200 import preprocessor as P
    row = P.AlpacaProcessor().preprocess({'instruction': 'Add', 'input': '1+1', 'output': '2'})
    assert [m['role'] for m in row['messages']] == ['user', 'assistant'] and '1+1' in row['messages'][0]['content']
    g = P.GSM8KProcessor().preprocess({'question': 'q', 'answer': 'work #### 42'})
    assert g['messages'][0]['role'] in ('system', 'user') and str(g.get('user_data', {}).get('ground_truth', g.get('user_data'))).find('42') >= 0


# ------------------------------------------------------------------------------------------- kernels / patches / cli
def test_kernelize_swaps_and_restores():
    from twinkle_b200.kernel import kernelize, resolve_value

    class Norm(torch.nn.Module):
        def forward(self, x):
            return x + 1

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.n = Norm()

        def forward(self, x):
            return self.n(x)

    net = Net()
    _, undo = kernelize(net, {Norm: {'cpu': lambda self, x: x + 100, 'cuda': lambda self, x: x + 200}}, device='cpu')
    assert float(net(torch.zeros(1))) == 100.0 and type(net.n).__name__ == 'NormKernelized' and isinstance(net.n, Norm)
    undo()
    assert float(net(torch.zeros(1))) == 1.0 and type(net.n) is Norm
    assert resolve_value({'default': 3}, 'cuda') == 3 and resolve_value({'npu': 1}, 'cuda') is None
    import math as _m
    _, undo = kernelize(None, {'math.sqrt': lambda x: -1.0})
    assert _m.sqrt(4) == -1.0
    undo()
    assert _m.sqrt(4) == 2.0


def test_fused_ce_patch_is_reversible():
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.patch import EmbeddingPatch, FusedCEPatch, apply_context, apply_patch
    m = TransformersModel(model_id='tiny-dense', seed=0)
    task = m.task
    before = {k: v.clone() for k, v in m.model.state_dict().items()}
    p = apply_patch(m, FusedCEPatch)
    assert m.task == 'fused_lm_ce'
    p.unpatch(m)
    with apply_context(m, EmbeddingPatch):
        assert m.task == 'embedding'
    after = m.model.state_dict()
    assert m.task == task and before.keys() == after.keys() and all(torch.equal(before[k], after[k]) for k in before)


def test_cli_layering(tmp_path, monkeypatch):
    from twinkle_b200.cli.cli import CLI
    env = tmp_path / '.env'
    env.write_text('TWINKLE_LEARNING_RATE=1e-3\nTWINKLE_BATCH_SIZE=4\n')
    y = tmp_path / 'c.yaml'
    y.write_text('training:\n  batch_size: 8\noptimizer:\n  weight_decay: 0.5\nsomething_else: 7\n')
    monkeypatch.setenv('TWINKLE_BATCH_SIZE', '6')
    a = CLI.from_args(['--config', str(y), '--lr', '2e-4', '--unknown-flag', 'x'], env_file=str(env))
    assert a.learning_rate == pytest.approx(2e-4)       # flag beats .env
    assert a.batch_size == 8                             # YAML beats environment beats .env
    assert a.weight_decay == 0.5 and a.extra['something_else'] == 7 and a.extra['unknown_flag'] == 'x'


def test_construct_class_and_plugin_guard(tmp_path, monkeypatch):
    from twinkle_b200 import loss as loss_mod
    from twinkle_b200.utils.loader import construct_class
    obj = construct_class('GRPOLoss', None, loss_mod, epsilon=0.3)
    assert type(obj).__name__ == 'GRPOLoss' and obj.epsilon == 0.3
    inst = loss_mod.CrossEntropyLoss()
    assert construct_class(inst, None, loss_mod) is inst
    with pytest.raises(ValueError):
        construct_class('NoSuchLoss', None, loss_mod)
    plug = tmp_path / 'plug'
    plug.mkdir()
    (plug / '__init__.py').write_text('class MyLoss:\n    pass\n')
    monkeypatch.delenv('TWINKLE_TRUST_REMOTE_CODE', raising=False)
    with pytest.raises(Exception):
        construct_class(str(plug), None, loss_mod)     # refused unless remote code is trusted


def test_arrow_and_feather_files_load_like_the_other_formats(tmp_path):
    import pyarrow as pa
    import pyarrow.feather as feather

    from twinkle_b200.dataset import Dataset, DatasetMeta
    table = pa.table({'query': ['a', 'b', 'c'], 'response': ['x', 'y', 'z']})
    with pa.OSFile(str(tmp_path / 'file.arrow'), 'wb') as sink, pa.ipc.new_file(sink, table.schema) as w:
        w.write_table(table)
    with pa.OSFile(str(tmp_path / 'stream.arrow'), 'wb') as sink, pa.ipc.new_stream(sink, table.schema) as w:     # what `datasets` writes
        w.write_table(table)
    feather.write_feather(table, str(tmp_path / 'rows.feather'))
    for fn in ('file.arrow', 'stream.arrow', 'rows.feather'):
        ds = Dataset(DatasetMeta(str(tmp_path / fn)))
        assert len(ds) == 3 and ds[1] == {'query': 'b', 'response': 'y'}
    import pytest
    os.makedirs(tmp_path / 'set.lance')
    with pytest.raises(ImportError):          # the Lance reader is an optional package; the error says which
        Dataset(DatasetMeta(str(tmp_path / 'set.lance')))


def test_dataloader_collates_with_a_processor_when_one_is_set():
    from twinkle_b200.dataloader import DataLoader
    from twinkle_b200.dataset import Dataset, DatasetMeta
    rows = [{'input_ids': list(range(3, 3 + n)), 'labels': list(range(4, 4 + n))} for n in (5, 7, 6, 4)]
    dl = DataLoader(Dataset(DatasetMeta(data=rows)), batch_size=2, shuffle=False)
    assert isinstance(next(iter(dl)), list)                              # rows as they are: the model collates
    dl.set_processor('InputProcessor')
    batch = next(iter(dl))
    assert len(batch) == 1 and batch[0].cu_seqlens.tolist() == [0, 5, 12] and batch[0].max_seqlen == 7        # the two rows packed into one micro-batch
    dl.set_processor(lambda rows: len(rows))
    assert next(iter(dl)) == 2


def test_image_columns_switch_between_bytes_and_decoded_images(tmp_path):
    from PIL import Image

    from twinkle_b200.dataset import Dataset, DatasetMeta
    rows = [{'images': [Image.new('RGB', (4, 3), (255, 0, 0))], 'text': 'a'}, {'images': Image.new('RGB', (2, 2), (0, 255, 0)), 'text': 'b'}]
    ds = Dataset(DatasetMeta(data=rows))
    ds.cast_column('images', decode=False)
    assert isinstance(ds[0]['images'][0]['bytes'], bytes) and isinstance(ds[1]['images']['bytes'], bytes) and ds[0]['text'] == 'a'
    ds.cast_column('images', decode=True)
    assert ds[0]['images'][0].size == (4, 3) and ds[1]['images'].getpixel((0, 0)) == (0, 255, 0)
    ds.save_as(str(tmp_path / 'seen.jsonl'), mode='training')
    ds.cast_column('images', decode=False)
    _ = ds[1]
    ds.flush_save()
    _ = ds[0]                                                        # read after the writer was closed: not recorded
    assert len(open(tmp_path / 'seen.jsonl').read().strip().splitlines()) == 1
