"""Host-side helpers of the op layer that need no GPU: split-K chunking, LoRA rank masks, segment starts."""
import torch

from twinkle_b200 import ops


def test_split_k_offsets_cover_the_rows_in_64_row_multiples():
    for n in (8192, 8193, 40000, 262144, 1000003):
        off = ops._split_k_offsets(n, 'cpu').tolist()
        assert off[0] == 0 and off[-1] == n and len(off) - 1 <= 33
        sizes = [b - a for a, b in zip(off, off[1:])]
        assert all(s > 0 for s in sizes) and all(s % 64 == 0 for s in sizes[:-1]) and min(sizes[:-1] or [1024]) >= 1024
    assert ops._split_k_offsets(8192, 'cpu') is ops._split_k_offsets(8192, 'cpu')          # cached per size


def test_rank_mask_scales_the_leading_rank_columns_and_repeats_per_stacked_pool():
    segs = [(0, 3, 0, 2, 2.0), (3, 5, -1, 4, 1.0), (5, 6, 1, 4, 0.5)]
    m = ops._sgmv_rowmask(segs, 4, 'cpu', torch.float32)
    assert m.shape == (6, 4)
    assert m[0].tolist() == [2.0, 2.0, 0.0, 0.0] and m[3].tolist() == [0.0] * 4 and m[5].tolist() == [0.5] * 4
    m2 = ops._sgmv_rowmask(segs, 4, 'cpu', torch.float32, 3)                               # three projections' pools side by side
    assert m2.shape == (6, 12) and torch.equal(m2, m.repeat(1, 3))
    assert ops._sgmv_rowmask(segs, 4, 'cpu', torch.float32, 3) is m2


def test_segment_starts_name_the_first_token_of_every_packed_sequence():
    cu = torch.tensor([0, 3, 3, 7], dtype=torch.int32)
    assert ops._segment_starts(cu, 7).tolist() == [0, 0, 0, 3, 3, 3, 3]


def test_adapter_options_that_are_not_implemented_are_refused_not_dropped(caplog):
    import logging

    import pytest

    from twinkle_b200.model.multi_lora import LoraConfig
    ok = LoraConfig.from_any({'r': 4, 'lora_alpha': 8, 'modules_to_save': None, 'use_dora': False, 'rank_pattern': {}, 'init_lora_weights': True, 'bias': 'none',
                              'exclude_modules': ('o_proj', ), 'target_modules': {'q_proj', 'v_proj'}})
    assert ok.r == 4 and ok.exclude_modules == ['o_proj'] and ok.target_modules == ['q_proj', 'v_proj']
    for bad in ({'use_dora': True}, {'rank_pattern': {'q_proj': 4}}, {'modules_to_save': ['lm_head']}, {'layers_to_transform': [0, 1]}):
        with pytest.raises(NotImplementedError):
            LoraConfig.from_any({'r': 4, **bad})
    assert LoraConfig.from_any(LoraConfig(r=4).to_peft_dict()).r == 4          # what this package writes, it reads
    with caplog.at_level(logging.WARNING, logger='twinkle_b200'):
        LoraConfig.from_any({'r': 4, 'lora_dropout': 0.05})
    assert any('not applied' in r.getMessage() for r in caplog.records)
