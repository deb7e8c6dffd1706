"""Hang guards on 2 CPU ranks (gloo) with ``TWINKLE_FAIL_FAST=0``: a payload that breaks the loss on ONE rank must not
leave the other rank alone in a collective.  Every call returns on both ranks, the ranks stay in step, and the next
regular step works (reference ``tests/server/integration/test_nccl_safe_twinkle_e2e.py:88-125, 167-210``)."""
import os

import torch

from tests.dist_utils import run_ranks


def _feats(seed, n=2, length=24):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(3, 512, (length + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


class _RaisesOnRankOne:
    """A loss that fails on one rank only (a tenant-specific bug, a corrupt shard of the batch…)."""
    reduction = 'sum'

    def __init__(self, inner, rank):
        self.inner, self.rank = inner, rank

    def __call__(self, inputs, outputs, **kw):
        if self.rank == 1:
            raise RuntimeError('synthetic failure on rank 1')
        return self.inner(inputs, outputs, **kw)


def _scenario(rank, world):
    import torch.distributed as dist
    os.environ['TWINKLE_FAIL_FAST'] = '0'
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None)
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.0)
    m.set_loss('GRPOLoss')
    report = {}
    good = _feats(100 + rank)
    n_tok = 24

    def kw(bad=None):
        old = [[-1.0] * n_tok for _ in good]
        adv = [0.5, -0.5]
        if bad == 'short' and rank == 1:
            old = [[-1.0] * 5 for _ in good]                 # wrong length on one rank
        if bad == 'nan' and rank == 1:
            old = [[float('nan')] * n_tok for _ in good]
        return {'old_logps': old, 'advantages': adv}

    # 1) ragged old_logps of the wrong length, 2) NaN log-probs: rank 1's loss fails, rank 0's is fine
    for case in ('short', 'nan'):
        out = m.forward_backward(inputs=good, **kw(case))
        m.clip_grad_and_step(max_grad_norm=1.0)
        report[case] = float(out['loss']) if out.get('loss') is not None else None
    # 3) every label masked on rank 1
    masked = [dict(f, labels=[-100] * len(f['labels'])) for f in good] if rank == 1 else good
    out = m.forward_backward(inputs=masked, **kw())
    m.clip_grad_and_step(max_grad_norm=1.0)
    report['masked'] = float(out['loss'])
    # 4) an exception on one rank only, raised by the loss object itself
    og = m._group(None)
    inner = og.loss_instance
    og.loss_instance = type(inner)(_RaisesOnRankOne(getattr(inner, 'loss', inner), rank)) if hasattr(inner, 'loss') else _RaisesOnRankOne(inner, rank)
    out = m.forward_backward(inputs=good, **kw())
    m.clip_grad_and_step(max_grad_norm=1.0)
    report['raises'] = float(out['loss'])
    og.loss_instance = inner
    # 5) a regular step afterwards: both ranks still hold the same model (equal loss on equal data) and it is finite
    same = _feats(7)
    m.set_loss('CrossEntropyLoss')
    out = m.forward_backward(inputs=same)
    norm = m.clip_grad_and_step(max_grad_norm=1.0)
    report['after'] = float(out['loss'])
    t = torch.tensor([report['after']], dtype=torch.float64)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report['spread'] = float(hi - lo)
    report['norm'] = float(norm)
    return report


def test_bad_payload_on_one_rank_keeps_ranks_in_step():
    r0, r1 = run_ranks(_scenario, 2, timeout=240.0)
    for r in (r0, r1):
        assert r['spread'] < 1e-6, (r0, r1)                       # ranks agree on the model after four failures
        assert r['after'] == r['after'] and 0.0 < r['after'] < 20.0
        assert r['norm'] == r['norm']
    for case in ('short', 'nan', 'raises'):
        assert r1[case] == 0.0 or r1[case] == r1[case], (case, r1)   # the failing rank answered (zero loss), no hang
    assert r0['short'] == r0['short'] and r0['masked'] == r0['masked']
