"""The copy jobs of the receive-side Ulysses exchange, checked on CPU: executing every rank's jobs on byte arrays gives
exactly the all-to-all of the reference (``sequence_parallel/utils.py:269-401``) in both directions, for q-like and
k/v-like head counts and every group size, and the debug bounds check accepts them and rejects a corrupted job."""
import numpy as np
import pytest
import torch

from twinkle_b200.parallel.symm import check_jobs, exchange_jobs


def _run_jobs(staged, me, seq_to_head):
    """Executes rank ``me``'s jobs against the ranks' staged tensors (numpy byte views)."""
    sp = len(staged)
    x = staged[me]
    out_shape, jobs = exchange_jobs(tuple(x.shape), x.element_size(), sp, me, seq_to_head)
    check_jobs(jobs, x.numel() * x.element_size(), int(np.prod(out_shape)) * x.element_size())
    out = np.zeros(int(np.prod(out_shape)) * x.element_size(), dtype=np.uint8)
    for r, s_off, s_stride, d_off, d_stride, chunk, n in jobs:
        src = staged[r].contiguous().view(torch.uint8).reshape(-1).numpy()
        for row in range(n):
            out[d_off + row * d_stride:d_off + row * d_stride + chunk] = src[s_off + row * s_stride:s_off + row * s_stride + chunk]
    return torch.from_numpy(out).view(x.dtype).reshape(out_shape)


@pytest.mark.parametrize('sp', [2, 4, 8])
@pytest.mark.parametrize('heads', [32, 8])
def test_jobs_equal_all_to_all(sp, heads):
    t, D = 6, 16
    g = torch.Generator().manual_seed(sp * 100 + heads)
    xs = [torch.randn(t, heads, D, generator=g).bfloat16() for _ in range(sp)]       # rank r: its tokens, all heads
    hl = heads // sp
    # seq → head: rank m ends up with all tokens (rank-major) of heads [m·hl, (m+1)·hl)
    got = [_run_jobs(xs, m, True) for m in range(sp)]
    for m in range(sp):
        want = torch.cat([xs[r][:, m * hl:(m + 1) * hl] for r in range(sp)], 0)
        assert torch.equal(got[m], want)
    # head → seq brings every rank's tokens back with all heads in order
    back = [_run_jobs(got, m, False) for m in range(sp)]
    for m in range(sp):
        assert torch.equal(back[m], xs[m])


def test_bounds_check_rejects_bad_jobs():
    shape, es, sp = (8, 8, 16), 2, 4
    out_shape, jobs = exchange_jobs(shape, es, sp, 1, True)
    src_bytes, dst_bytes = 8 * 8 * 16 * 2, int(np.prod(out_shape)) * 2
    check_jobs(jobs, src_bytes, dst_bytes)
    r, s_off, s_stride, d_off, d_stride, chunk, n = jobs[0]
    with pytest.raises(AssertionError):
        check_jobs([(r, s_off + src_bytes, s_stride, d_off, d_stride, chunk, n)] + jobs[1:], src_bytes, dst_bytes)       # reads past the source
    with pytest.raises(AssertionError):
        check_jobs([(r, s_off, s_stride, jobs[1][3], d_stride, chunk, n)] + jobs[1:], src_bytes, dst_bytes)              # two jobs, same bytes
    with pytest.raises(AssertionError):
        check_jobs(jobs[1:], src_bytes, dst_bytes)                                                                        # a hole in the output
    with pytest.raises(AssertionError):
        check_jobs([(r, s_off + 8, s_stride, d_off, d_stride, chunk, n)] + jobs[1:], src_bytes, dst_bytes)                # misaligned
    with pytest.raises(ValueError):
        exchange_jobs((8, 6, 16), 2, 4, 0, True)                                                                          # heads do not divide


def test_guard_zones_around_symmetric_tensors_catch_a_stray_write():
    """Placement with guard zones keeps 256-byte alignment and disjoint zones; a byte written just past a tensor (what a
    peer kernel with a wrong extent would do) is reported next to that tensor."""
    import torch
    from twinkle_b200.parallel.symm import GUARD_PATTERN, damaged_guards, fill_guards, place_guarded
    raw = torch.zeros(1 << 16, dtype=torch.uint8)
    used, records = 0, []
    for i, nbytes in enumerate((1000, 4096, 24)):
        start, used = place_guarded(used, nbytes, 512)
        assert start % 256 == 0 and used % 256 == 0 and start >= 512
        fill_guards(raw, start, nbytes, 512)
        records.append((f't{i}', start, nbytes, 512))
    for (_, s0, n0, g0), (_, s1, _, g1) in zip(records, records[1:]):
        assert s0 + n0 + g0 <= s1 - g1                       # zones of neighbours do not overlap
    assert place_guarded(0, 100, 0) == (0, 256)              # without guards: plain aligned bump allocation
    assert damaged_guards(raw, records) == []
    _, s1, n1, _ = records[1]
    raw[s1:s1 + n1].fill_(7)                                 # writing the tensor itself is fine
    assert damaged_guards(raw, records) == []
    raw[s1 + n1] = 0                                         # one byte past its end
    bad = damaged_guards(raw, records)
    assert len(bad) == 1 and bad[0].startswith('t1') and 'above' in bad[0]
    raw[s1 + n1] = GUARD_PATTERN
    raw[records[2][1] - 1] = 1                               # one byte before the next tensor
    assert damaged_guards(raw, records)[0].startswith('t2 (below')
