"""Pure unit tests on tiny tensors: losses, advantages, metrics, device-mesh arithmetic (reference tiers:
tests/loss/*, tests/advantage/*, tests/metric/*, tests/DeviceMesh/*)."""
import math

import pytest
import torch

from twinkle_b200.advantage import GRPOAdvantage, RLOOAdvantage
from twinkle_b200.loss import (BNPOLoss, CISPOLoss, CPOLoss, ChunkedCrossEntropyLoss, CrossEntropyLoss, DFTLoss, DPOLoss, DRGRPOLoss, GKDLoss,
                               GRPOLoss, GSPOLoss, MSELoss, ORPOLoss, SAPOLoss, SimPOLoss)
from twinkle_b200.loss.gkd import generalized_jsd
from twinkle_b200.utils.device_mesh import DeviceMesh


def _val(out):
    return out['loss'] if isinstance(out, dict) else out


def test_cross_entropy_sum_and_mean_and_dft():
    logps = torch.tensor([[-1.0, -2.0, -3.0, -0.5]])
    labels = torch.tensor([[5, -100, 7, 9]])
    out = CrossEntropyLoss()({'labels': labels}, {'logps': logps})
    assert float(out['loss']) == pytest.approx(1.0 + 3.0 + 0.5) and int(out['num_tokens']) == 3
    mean = CrossEntropyLoss(reduction='mean')({'labels': labels}, {'logps': logps})
    assert float(mean['loss']) == pytest.approx(4.5 / 3) and int(mean['num_tokens'] or 0) == 0
    dft = DFTLoss()({'labels': labels}, {'logps': logps})
    want = sum(-lp * math.exp(lp) for lp in (-1.0, -3.0, -0.5))
    assert float(dft['loss']) == pytest.approx(want, rel=1e-5)


def test_chunked_ce_matches_plain_and_its_gradient():
    torch.manual_seed(0)
    logits = torch.randn(2, 7, 11, requires_grad=True)
    labels = torch.randint(0, 11, (2, 7))
    labels[0, 2] = -100
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 11), labels.reshape(-1), ignore_index=-100, reduction='sum')
    g_ref, = torch.autograd.grad(ref, logits)
    out = ChunkedCrossEntropyLoss(chunk_size=3)({'labels': labels}, {'logits': logits})
    g, = torch.autograd.grad(out['loss'], logits)
    assert float(out['loss']) == pytest.approx(float(ref), rel=1e-5) and torch.allclose(g, g_ref, atol=1e-5)


def test_mse():
    out = MSELoss()({'labels': torch.tensor([[1.0, 2.0]])}, {'logits': torch.tensor([[0.0, 4.0]])})
    assert float(_val(out)) == pytest.approx((1 + 4) / 2)


def _pref_batch():
    # rows alternate chosen / rejected; two pairs
    labels = torch.tensor([[1, 2, 3], [1, 2, -100], [4, 5, 6], [4, -100, -100]])
    logps = torch.tensor([[-0.1, -0.2, -0.3], [-1.0, -1.0, 0.0], [-0.5, -0.5, -0.5], [-0.2, 0.0, 0.0]])
    return {'labels': labels}, {'logps': logps.clone().requires_grad_(True)}


def test_dpo_variants_against_hand_computation():
    inputs, outputs = _pref_batch()
    ref = torch.tensor([-0.9, -1.5, -1.2, -0.4])  # per-sequence reference log-probs
    pol = (outputs['logps'] * (inputs['labels'] != -100)).sum(-1)
    margin = 0.1 * ((pol[0::2] - ref[0::2]) - (pol[1::2] - ref[1::2]))
    want = -torch.nn.functional.logsigmoid(margin).mean()
    out = DPOLoss(beta=0.1)(inputs, outputs, ref_logps=ref)
    assert float(_val(out)) == pytest.approx(float(want), rel=1e-5)
    hinge = DPOLoss(beta=0.1, loss_type='hinge')(inputs, outputs, ref_logps=ref)
    assert float(_val(hinge)) == pytest.approx(float(torch.relu(1 - margin).mean()), rel=1e-5)
    ipo = DPOLoss(beta=0.1, loss_type='ipo')(inputs, outputs, ref_logps=ref)
    assert torch.isfinite(_val(ipo))
    with pytest.raises(ValueError):
        DPOLoss(loss_type='nope')
    with pytest.raises(AssertionError):
        DPOLoss()({'labels': inputs['labels'][:3]}, {'logps': outputs['logps'][:3]}, ref_logps=ref[:3])
    for cls in (SimPOLoss, CPOLoss, ORPOLoss):  # reference-free family: finite and differentiable
        o = _val(cls()(inputs, outputs))
        g, = torch.autograd.grad(o, outputs['logps'], allow_unused=True)
        assert torch.isfinite(o) and g is not None and torch.isfinite(g).all()


def _rl_batch():
    labels = torch.tensor([[-100, 3, 4, 5], [-100, -100, 6, 7]])
    logps = torch.tensor([[0.0, -0.5, -0.6, -0.7], [0.0, 0.0, -1.0, -1.2]], requires_grad=True)
    old = torch.tensor([[0.0, -0.6, -0.6, -0.9], [0.0, 0.0, -0.7, -1.2]])
    return {'labels': labels}, {'logps': logps}, old, torch.tensor([1.0, -0.5])


def test_grpo_family():
    inputs, outputs, old, adv = _rl_batch()
    mask = inputs['labels'] != -100
    ratio = torch.exp(outputs['logps'] - old)
    a = adv[:, None].expand_as(ratio)
    per_tok = -torch.min(ratio * a, ratio.clamp(0.8, 1.2) * a)
    want = ((per_tok * mask).sum(-1) / mask.sum(-1)).mean()
    out = GRPOLoss(epsilon=0.2)(inputs, outputs, old_logps=old, advantages=adv)
    assert float(_val(out)) == pytest.approx(float(want), rel=1e-5)
    # no advantages → zero loss that still touches the graph (keeps collectives aligned)
    z = GRPOLoss()(inputs, outputs)
    assert float(_val(z)) == 0.0 and _val(z).requires_grad
    # ragged python lists (one list of completion-token values per row) are aligned to the label mask
    ragged = GRPOLoss(epsilon=0.2)(inputs, outputs, old_logps=[[-0.6, -0.6, -0.9], [-0.7, -1.2]], advantages=[1.0, -0.5])
    assert float(_val(ragged)) == pytest.approx(float(want), rel=1e-5)
    bnpo = BNPOLoss(epsilon=0.2)(inputs, outputs, old_logps=old, advantages=adv)
    assert float(_val(bnpo)) == pytest.approx(float((per_tok * mask).sum() / mask.sum()), rel=1e-5)
    dr = DRGRPOLoss(epsilon=0.2, max_completion_length=10)(inputs, outputs, old_logps=old, advantages=adv)
    assert float(_val(dr)) == pytest.approx(float((per_tok * mask).sum() / (2 * 10)), rel=1e-5)
    gspo = GSPOLoss(epsilon=0.2)(inputs, outputs, old_logps=old, advantages=adv)
    seq_lr = ((outputs['logps'] - old) * mask).sum(-1) / mask.sum(-1)
    r = torch.exp(seq_lr)
    want_g = (-torch.min(r * adv, r.clamp(0.8, 1.2) * adv)).mean()
    assert float(_val(gspo)) == pytest.approx(float(want_g), rel=1e-5)
    for cls in (SAPOLoss, CISPOLoss):
        o = _val(cls()(inputs, outputs, old_logps=old, advantages=adv))
        g, = torch.autograd.grad(o, outputs['logps'])
        assert torch.isfinite(o) and torch.isfinite(g).all()
    kl = GRPOLoss(beta=0.5)(inputs, outputs, old_logps=old, advantages=adv, ref_logps=old)
    assert float(_val(kl)) > float(_val(GRPOLoss(beta=0.0)(inputs, outputs, old_logps=old, advantages=adv)))


def test_gkd_and_jsd():
    torch.manual_seed(1)
    s, t = torch.log_softmax(torch.randn(4, 9), -1), torch.log_softmax(torch.randn(4, 9), -1)
    assert torch.allclose(generalized_jsd(s, t, 0.0), torch.nn.functional.kl_div(s, t, log_target=True, reduction='none').sum(-1), atol=1e-6)
    assert torch.allclose(generalized_jsd(s, t, 1.0), torch.nn.functional.kl_div(t, s, log_target=True, reduction='none').sum(-1), atol=1e-6)
    assert float(generalized_jsd(s, s, 0.5).abs().max()) < 1e-6
    logits = torch.randn(1, 5, 9, requires_grad=True)
    labels = torch.tensor([[-100, 1, 2, -100, 3]])
    teacher = torch.randn(1, 5, 9)
    full = GKDLoss(beta=0.5)({'labels': labels}, {'logits': logits}, teacher_logits=teacher)
    assert torch.isfinite(_val(full)) and float(_val(full)) > 0
    same = GKDLoss(beta=0.5)({'labels': labels}, {'logits': logits}, teacher_logits=logits.detach())
    assert float(_val(same)) == pytest.approx(0.0, abs=1e-6)
    tl, ti = torch.log_softmax(teacher, -1).topk(4, -1)
    topk = GKDLoss(beta=0.0, topk=4)({'labels': labels}, {'logits': logits}, teacher_topk_logprobs=tl, teacher_topk_indices=ti)
    g, = torch.autograd.grad(_val(topk), logits)
    assert torch.isfinite(g).all() and float(g[0, 0].abs().sum()) == 0.0  # masked position gets no gradient


def test_advantages():
    r = [1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0]
    a = GRPOAdvantage()(r, num_generations=4, scale='group')
    assert a.shape == (8, ) and float(a[:4].sum()) == pytest.approx(0.0, abs=1e-6) and float(a[4:].abs().max()) == 0.0
    b = GRPOAdvantage()(r, num_generations=4, scale='none')
    assert b.tolist()[:4] == [0.5, -0.5, -0.5, 0.5]
    c = GRPOAdvantage()(r, num_generations=4, scale='batch')
    assert float(c[0]) == pytest.approx(0.5 / (torch.tensor(r).std() + 1e-8), rel=1e-5)
    l = RLOOAdvantage()(r, num_generations=4)
    assert float(l[0]) == pytest.approx(1.0 - (0 + 0 + 1) / 3)
    with pytest.raises(ValueError):
        GRPOAdvantage()(r, num_generations=4, scale='bogus')


def test_metrics_accumulate():
    from twinkle_b200.metric import Accuracy, LossMetric
    m = LossMetric()
    m.accumulate(None, {'loss': 2.0, 'num_tokens': 10}, grad_norm=1.5)
    m.accumulate(None, {'loss': 1.0, 'num_tokens': 30}, grad_norm=0.5)
    res = m.calculate()
    assert float(str(res['loss'])) == pytest.approx((2.0 + 1.0) / 40, rel=1e-3)  # sum-losses over summed token counts
    assert float(str(res['grad_norm'])) == 1.5
    acc = Accuracy()
    logits = torch.tensor([[[0.1, 0.9], [0.8, 0.2], [0.3, 0.7]]])
    acc.accumulate({'labels': torch.tensor([[1, 1, -100]])}, {'logits': logits})
    assert float(str(acc.calculate()['accuracy']).rstrip('%')) in (50.0, 0.5)


def test_device_mesh_arithmetic():
    m = DeviceMesh.from_sizes(fsdp_size=4, dp_size=2)
    assert m.world_size == 8 and m.data_world_size == 8
    assert sorted({m.get_data_rank_from_global_rank(r) for r in range(8)}) == list(range(8))
    sp = DeviceMesh.from_sizes(fsdp_size=8, dp_size=None, ulysses_size=4)
    assert sp.data_world_size == 2 and [sp.get_data_rank_from_global_rank(r) for r in range(8)] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert sp.get_slice(16, 1) == slice(8, 16)
    tp = DeviceMesh.from_sizes(tp_size=2, pp_size=2, dp_size=2)
    assert tp.world_size == 8 and tp.data_world_size == 2
    # ranks that differ only in tp / pp position read the same data
    groups = {}
    for r in range(8):
        groups.setdefault(tp.get_data_rank_from_global_rank(r), []).append(r)
    assert sorted(len(v) for v in groups.values()) == [4, 4]
    last = tp.get_pp_last_ranks()
    assert len(last) == 4
    with pytest.raises(Exception):
        DeviceMesh.from_sizes(fsdp_size=3, dp_size=None, ulysses_size=2).data_world_size


def test_graded_math_and_multimodal_rewards():
    import math
    from twinkle_b200.preprocessor import CompetitionMathGRPOProcessor
    from twinkle_b200.reward import (MultiModalAccuracyReward, OlympiadBenchAccuracyReward, OlympiadBenchFormatReward, OlympiadBenchQualityReward,
                                     all_boxed, normalize_math_answer, reward_mapping, split_answers)
    a = lambda c, **ud: {'messages': [{'role': 'assistant', 'content': c}], 'user_data': ud}  # noqa: E731
    assert all_boxed('a \\boxed{\\frac{1}{2}} b \\boxed{x}') == ['\\frac{1}{2}', 'x']
    assert normalize_math_answer('$\\dfrac{1}{2}$') == '0.5' and normalize_math_answer('1,000.50') == '1000.5' and normalize_math_answer('\\text{Yes}.') == 'yes'
    assert split_answers('(1,2),(3,4), 5') == ['(1,2)', '(3,4)', '5']
    acc = OlympiadBenchAccuracyReward()
    got = acc([a('so \\boxed{\\frac{1}{2}}', ground_truth='0.5'), a('x \\boxed{10}', ground_truth='11'),
               a('\\boxed{1}, \\boxed{(3,4)}', ground_truth='(3,4),2', is_multiple_answer=True), a('no box', ground_truth='1'),
               a('\\boxed{7}', ground_truth=[('unused', 0)])])
    assert got[0] == 1.0 and got[1] == pytest.approx(0.99 * math.exp(-5 / 11)) and got[2] == 0.5 and got[3] == 0.0
    assert acc([{'messages': [{'role': 'assistant', 'content': '\\boxed{1,000}'}], 'user_data': [('ground_truth', '$1000$')]}]) == [1.0]  # pair-list user_data
    assert acc([a('\\boxed{3}')], ground_truths=['the answer is \\boxed{3}']) == [1.0]
    fmt = OlympiadBenchFormatReward()([a('\\boxed{3}'), a('\\boxed{1} \\boxed{2} \\boxed{3}'), a('\\boxed{1}' + 'x' * 300), a('nothing')])
    assert fmt == [1.0, pytest.approx(0.4), 0.7, 0.0]
    q = OlympiadBenchQualityReward()
    txt = 'Step 1: x = 1 + 2 = 3. Then y = x * 2 = 6, z = y / 3 - 1 ^ 2. Therefore the answer is \\boxed{6}'
    assert q.reasoning(txt) == 1.0 and q.reasoning('hello') == 0.0
    assert [q.length(n) for n in (50, 200, 1000, 6000)] == [pytest.approx(0.15), pytest.approx(0.65), 1.0, 0.25] and q.length(3000) == pytest.approx(0.5)
    assert q.non_repetition('ab ' * 100) < 0.2 and q.non_repetition('short') == 1.0
    assert q([a(txt)])[0] == pytest.approx(0.4 + 0.3 * q.length(len(txt)) + 0.3 * q.non_repetition(txt))
    mm = MultiModalAccuracyReward()([a('<think>..</think><answer> 3 </answer>', ground_truth='3'),
                                     a('<answer>Yes</answer>', ground_truth='no', solution='<answer> yes </answer>'), a('3', ground_truth='3'),
                                     a('<answer>3.0</answer>', ground_truth=3), a('<answer>4</answer>', ground_truth=3)])
    assert mm == [1.0, 1.0, 0.0, 1.0, 0.0]
    assert {'OlympiadBenchAccuracyReward', 'MultiModalAccuracyReward'} <= set(reward_mapping)
    row = CompetitionMathGRPOProcessor()([{'problem': '1+1?', 'solution': 'It is \\boxed{2}.'}])[0]
    assert [m['role'] for m in row['messages']] == ['system', 'user'] and row['user_data'] == {'solution': 'It is \\boxed{2}.', 'ground_truth': '2'}


def test_torch_schedulers_resolve_by_name():
    """``set_lr_scheduler`` takes the names of this package's schedulers and of ``torch.optim.lr_scheduler`` classes."""
    import pytest

    from twinkle_b200.model import TransformersModel
    from twinkle_b200.module.scheduler import resolve_scheduler
    assert resolve_scheduler('cosine').__name__ == 'CosineWarmupScheduler' and resolve_scheduler('StepLR').__name__ == 'StepLR'
    with pytest.raises(KeyError):
        resolve_scheduler('NoSuchScheduler')
    m = TransformersModel(model_id='tiny-dense', seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=1e-2)
    m.set_lr_scheduler('StepLR', step_size=1, gamma=0.5)
    ids = list(range(3, 40))
    lrs = []
    for _ in range(3):
        m.forward_backward(inputs=[{'input_ids': ids[:-1], 'labels': ids[1:]}])
        m.clip_grad_and_step(max_grad_norm=1.0)
        lrs.append(m._group(None).optimizer.param_groups[0]['lr'])
    assert lrs == pytest.approx([5e-3, 2.5e-3, 1.25e-3])
