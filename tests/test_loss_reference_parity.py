"""Loss formulas pinned against the reference's own implementations on CPU (``baseline/_ref``, installed offline from
the reference checkout; skipped where it is absent).  Same inputs, same keyword arguments, same number out."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, 'baseline', '_ref')
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, 'twinkle')), reason='reference package not installed under baseline/_ref')


@pytest.fixture(scope='module')
def ref():
    for p in (os.path.join(ROOT, 'baseline', 'shims'), REF):
        if p not in sys.path:
            sys.path.insert(0, p)
    import twinkle.loss as L
    return L


def _pref_batch(seed=0, pairs=3, S=12):
    g = torch.Generator().manual_seed(seed)
    logps = -torch.rand(2 * pairs, S, generator=g) * 3
    labels = torch.randint(5, 100, (2 * pairs, S), generator=g)
    for b in range(2 * pairs):
        labels[b, :2 + b % 3] = -100                     # prompts of different lengths
    ref_logps = -torch.rand(2 * pairs, S, generator=g) * 3
    return logps, labels, ref_logps


def _mine_and_theirs(cls_mine, cls_ref, kwargs, call_kwargs_mine, call_kwargs_ref, logps, labels):
    mine = cls_mine(**kwargs)({'labels': labels}, {'logps': logps.clone().requires_grad_(True)}, **call_kwargs_mine)
    theirs = cls_ref(**kwargs)({'labels': labels}, {'logps': logps.clone().requires_grad_(True)}, **call_kwargs_ref)
    a = mine['loss'] if isinstance(mine, dict) else mine.loss
    b = theirs['loss'] if isinstance(theirs, dict) else theirs.loss
    return float(a), float(b)


@pytest.mark.parametrize('kwargs', [dict(loss_type='sigmoid'), dict(loss_type='ipo', beta=0.25), dict(loss_type='hinge'),
                                    dict(loss_type='sigmoid', sft_weight=0.5), dict(loss_type='sigmoid', label_smoothing=0.1)])
def test_dpo_matches_reference(ref, kwargs):
    from twinkle_b200.loss import DPOLoss
    logps, labels, ref_logps = _pref_batch()
    a, b = _mine_and_theirs(DPOLoss, ref.DPOLoss, kwargs, {'ref_logps': ref_logps}, {'ref_outputs': {'logps': ref_logps}}, logps, labels)
    assert a == pytest.approx(b, rel=1e-5, abs=1e-6), kwargs
    # the two sequence-level vectors are an equivalent way to hand over the reference policy
    mask = (labels != -100).float()
    seq = (ref_logps * mask).sum(-1)
    c, d = _mine_and_theirs(DPOLoss, ref.DPOLoss, kwargs, {'ref_chosen_logps': seq[0::2], 'ref_rejected_logps': seq[1::2]},
                            {'ref_chosen_logps': seq[0::2], 'ref_rejected_logps': seq[1::2]}, logps, labels)
    assert c == pytest.approx(d, rel=1e-5, abs=1e-6) and c == pytest.approx(a, rel=1e-5, abs=1e-6)


def test_cpo_orpo_simpo_match_reference(ref):
    from twinkle_b200.loss import CPOLoss, ORPOLoss, SimPOLoss
    logps, labels, _ = _pref_batch(seed=2)
    for mine, theirs, kw in ((CPOLoss, ref.CPOLoss, dict(beta=0.1, bc_coef=0.7)), (ORPOLoss, ref.ORPOLoss, dict(lambda_orpo=0.2)),
                             (SimPOLoss, ref.SimPOLoss, dict(beta=2.0, gamma=0.3))):
        a, b = _mine_and_theirs(mine, theirs, kw, {}, {}, logps, labels)
        assert a == pytest.approx(b, rel=1e-5, abs=1e-6), mine.__name__


@pytest.mark.parametrize('name,kwargs', [('GRPOLoss', dict(epsilon=0.2, epsilon_high=0.3)), ('GSPOLoss', dict(epsilon=0.1)),
                                         ('SAPOLoss', dict()), ('SAPOLoss', dict(tau_pos=1.2, tau_neg=0.8)),
                                         ('CISPOLoss', dict(epsilon=0.2, epsilon_high=0.5)), ('BNPOLoss', dict()), ('DRGRPOLoss', dict())])
def test_policy_gradient_losses_match_reference(ref, name, kwargs):
    import twinkle_b200.loss as M
    g = torch.Generator().manual_seed(4)
    B, S = 4, 10
    logps = -torch.rand(B, S, generator=g) * 2
    old = logps + torch.randn(B, S, generator=g) * 0.4            # some ratios beyond every clipping range
    labels = torch.randint(5, 100, (B, S), generator=g)
    labels[:, :3] = -100
    adv = torch.tensor([1.0, -0.5, 0.25, -2.0])
    call = {'old_logps': old, 'advantages': adv}
    a, b = _mine_and_theirs(getattr(M, name), getattr(ref, name), kwargs, call, call, logps, labels)
    assert a == pytest.approx(b, rel=1e-5, abs=1e-6), (name, kwargs)
    # default constructor arguments agree as well
    mine, theirs = getattr(M, name)(), getattr(ref, name)()
    for attr in ('epsilon', 'epsilon_high', 'beta', 'tau_pos', 'tau_neg'):
        if hasattr(theirs, attr):
            assert getattr(mine, attr) == getattr(theirs, attr), (name, attr)


def test_padding_garbage_does_not_reach_the_loss():
    from twinkle_b200.loss.grpo import align_to_mask
    mask = torch.tensor([[False, True, True, False]])
    vals = [[float('nan'), 1.0, 2.0, float('inf')]]
    out = align_to_mask(vals, mask)
    assert torch.isfinite(out).all() and out.tolist() == [[0.0, 1.0, 2.0, 0.0]]
