"""Tensor × pipeline parallel backend on CPU/gloo: schedules, parity with one process, bitwise HF round trip
(the Qwen3-32B tensor × pipeline configuration in miniature: TP=2 × PP=2, sequence-parallel activations, interleaved 1F1B with 2 virtual
stages)."""
import os

import pytest
import torch

from tests.dist_utils import run_ranks


def test_schedules_are_complete_and_ordered():
    from twinkle_b200.parallel.pipeline import build_schedule
    for P, V, M in [(2, 1, 4), (4, 1, 8), (2, 2, 4), (4, 2, 8), (2, 3, 6)]:
        for r in range(P):
            ops = build_schedule(P, V, M, r)
            assert len(ops) == 2 * M * V
            seen_f = set()
            for op in ops:
                if op.kind == 'F':
                    seen_f.add((op.chunk, op.micro))
                else:
                    assert (op.chunk, op.micro) in seen_f  # backward only after its forward
            assert len(seen_f) == M * V
            # in-flight forwards never exceed the warm-up depth + 1
            live = peak = 0
            for op in ops:
                live += 1 if op.kind == 'F' else -1
                peak = max(peak, live)
            bound = (P - r - 1) + 1 if V == 1 else (P - r - 1) * 2 + (V - 1) * P + 1
            assert peak <= min(bound, M * V)


def _feats():
    g = torch.Generator().manual_seed(11)
    out = []
    for n in (64, 48, 32, 64):
        ids = torch.randint(0, 1024, (n + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


def _single_curve(steps):
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-dense', num_hidden_layers=4)
    m = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    curve = []
    for _ in range(steps):
        o = m.forward_backward(inputs=_feats(), micro_batch_size=1)
        m.clip_grad_and_step(max_grad_norm=1.0)
        curve.append(o['loss'])
    return curve, {k: v.clone() for k, v in m.get_state_dict().items()}


def _worker(rank, world, tmp, tp, pp, vpp, steps):
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-dense', num_hidden_layers=4)
    mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=world // (tp * pp), vpp_size=vpp, sequence_parallel=tp > 1)
    m = MegatronModel(config=cfg, device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    curve = []
    for _ in range(steps):
        o = m.forward_backward(inputs=_feats(), micro_batch_size=1)
        m.clip_grad_and_step(max_grad_norm=1.0)
        curve.append(o['loss'])
    path = m.save('ckpt', tmp)
    before = {k: v.clone() for k, v in m.get_state_dict().items()}
    # perturb, reload, compare bitwise
    with torch.no_grad():
        for _, p in m.named_parameters():
            p.add_(1.0)
    m.load('ckpt', tmp)
    after = m.get_state_dict()
    same = all(torch.equal(before[k], after[k]) for k in before)
    return curve, same, path


@pytest.mark.parametrize('tp,pp,vpp', [(2, 2, 2), (1, 2, 1), (2, 1, 1)])
def test_tp_pp_matches_single_and_roundtrips(tmp_path, tp, pp, vpp):
    steps = 3
    single, single_sd = _single_curve(steps)
    res = run_ranks(_worker, tp * pp, str(tmp_path), tp, pp, vpp, steps)
    for curve, same, path in res:
        assert same
        for a, b in zip(single, curve):
            assert abs(a - b) < 2e-4, (single, curve)
    # the merged checkpoint is a plain HF directory holding every tensor of the single-process model
    from twinkle_b200.utils.safetensors_io import SafetensorLazyLoader
    loader = SafetensorLazyLoader(res[0][2])
    for k, v in single_sd.items():
        if k == 'lm_head.weight':
            continue
        assert k in loader, k
        assert torch.allclose(loader.get(k), v, atol=2e-4), k


def _resume_worker(rank, world, tmp, tp, pp, dp, recompute):
    """Trains 2 steps, saves everything, trains 2 more (reference continuation); a second model of the same layout resumes
    from the checkpoint and must produce the same two losses, bit for bit, and the same counters."""
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-dense', num_hidden_layers=4)
    mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=dp, sequence_parallel=tp > 1)

    def make():
        m = MegatronModel(config=cfg, device_mesh=mesh, seed=0, recompute=recompute)
        m.set_optimizer('AdamW', lr=2e-3)
        m.set_lr_scheduler('CosineWarmupScheduler', num_warmup_steps=1, num_training_steps=8)
        return m

    feats = _feats()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))

    def run(m, n):
        out = []
        for _ in range(n):
            o = m.forward_backward(inputs=feats[sl], micro_batch_size=1)
            m.clip_grad_and_step(max_grad_norm=1.0)
            out.append(o['loss'])
        return out

    a = make()
    first = run(a, 2)
    a.save('mid', tmp, save_optimizer=True)
    cont = run(a, 2)
    sharded = {n: tuple(st['master'].shape) for n, st in a._state.items()}
    full = {n: p.numel() for n, p in a.named_parameters()}
    b = make()
    info = b.resume_from_checkpoint(os.path.join(tmp, 'mid'))
    resumed = run(b, 2)
    return {'first': first, 'cont': cont, 'resumed': resumed, 'info': info, 'state_numel': {n: s[0] for n, s in sharded.items()}, 'full': full}


@pytest.mark.parametrize('tp,pp,dp,recompute', [(1, 2, 2, 'full'), (2, 1, 2, None)])
def test_resume_restores_optimizer_scheduler_and_counters(tmp_path, tp, pp, dp, recompute):
    res = run_ranks(_resume_worker, tp * pp * dp, str(tmp_path), tp, pp, dp, recompute)
    for r in res:
        assert r['info']['cur_step'] == 2 and r['info']['consumed_train_samples'] == 2 * len(_feats())
        assert r['resumed'] == r['cont'], (r['cont'], r['resumed'])          # same optimizer moments, schedule position and weights
        # distributed optimizer: a rank keeps fp32 master + moments for 1/dp of every parameter it holds
        for n, k in r['state_numel'].items():
            assert k <= -(-r['full'][n] // dp)


def test_layer_recompute_does_not_change_the_numbers(tmp_path):
    a = run_ranks(_resume_worker, 4, str(tmp_path / 'a'), 1, 2, 2, 'full')
    b = run_ranks(_resume_worker, 4, str(tmp_path / 'b'), 1, 2, 2, None)
    for ra, rb in zip(a, b):
        for x, y in zip(ra['first'] + ra['cont'], rb['first'] + rb['cont']):
            assert abs(x - y) < 1e-5, (ra, rb)


def _cp_worker(rank, world, tp, pp, cp, steps):
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-dense', num_hidden_layers=4)
    mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, cp_size=cp, dp_size=world // (tp * pp * cp), sequence_parallel=tp > 1)
    m = MegatronModel(config=cfg, device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    curve = []
    for _ in range(steps):
        o = m.forward_backward(inputs=_feats(), micro_batch_size=2)
        n = m.clip_grad_and_step(max_grad_norm=1.0)
        curve.append((o['loss'], n))
    return curve


@pytest.mark.parametrize('tp,pp,cp', [(1, 1, 2), (2, 1, 2), (1, 2, 2)])
def test_context_parallel_axis_matches_single(tp, pp, cp):
    """Zig-zag context parallelism on the tensor / pipeline backend: keys and values gathered per layer, whole sequences
    for the loss, context-parallel ranks reduced like data ranks (reference ``megatron/strategy/megatron.py:90-107``:
    ``context_parallel_size``)."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-dense', num_hidden_layers=4)
    one = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0)
    one.set_optimizer('AdamW', lr=1e-3)
    single = []
    for _ in range(3):
        o = one.forward_backward(inputs=_feats(), micro_batch_size=2)
        n = one.clip_grad_and_step(max_grad_norm=1.0)
        single.append((o['loss'], n))
    for curve in run_ranks(_cp_worker, tp * pp * cp, tp, pp, cp, 3):
        for (a, na), (b, nb) in zip(single, curve):
            assert abs(a - b) < 3e-4 and abs(na - nb) < 3e-3 * max(na, 1.0), (single, curve)


def _moe_feats():
    g = torch.Generator().manual_seed(21)
    out = []
    for n in (64, 48, 64, 32):
        ids = torch.randint(0, 1024, (n + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


def _ep_worker(rank, world, tmp, tp, pp, ep, steps, etp=1, sp=None):
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe', router_aux_loss_coef=0.0, num_hidden_layers=2 * pp)
    dp = world // (tp * pp)
    mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=dp, ep_size=ep, etp_size=etp,
                                 sequence_parallel=(tp > 1) if sp is None else sp)
    m = MegatronModel(config=cfg, device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    feats = _moe_feats()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    curve = []
    for _ in range(steps):
        o = m.forward_backward(inputs=feats[sl], micro_batch_size=1)
        n = m.clip_grad_and_step(max_grad_norm=1.0)
        import torch.distributed as dist
        t = torch.tensor([o['loss'] * o['num_tokens'], o['num_tokens']], dtype=torch.float64)
        dist.all_reduce(t, group=m.dp_comm.group)
        curve.append((float(t[0] / t[1]), n))
    path = m.save('moe', tmp)
    before = {k: v.clone() for k, v in m.get_state_dict().items()}
    with torch.no_grad():
        for _, p in m.named_parameters():
            p.add_(1.0)
    m.load('moe', tmp)
    same = all(torch.equal(before[k], v) for k, v in m.get_state_dict().items())
    n_experts_local = m.chunks[0].layers[0].mlp.experts.gate_up_proj.shape[0]
    if etp > 1:
        return curve, same, tuple(m.chunks[0].layers[0].mlp.experts.gate_up_proj.shape), sorted(before)
    return curve, same, n_experts_local, sorted(before)


@pytest.mark.parametrize('tp,pp,ep,world', [(1, 1, 2, 2), (2, 1, 2, 4), (1, 2, 2, 4)])
def test_expert_parallel_axis_matches_single(tmp_path, tp, pp, ep, world):
    """Experts split over the data-parallel ranks of the tensor / pipeline backend: loss curve and gradient norm of one
    process, bitwise HF round trip with all experts gathered, expert optimizer state not sliced by the distributed
    optimizer (reference ``megatron/strategy/megatron.py:90-107``: ``expert_model_parallel_size``)."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe', router_aux_loss_coef=0.0, num_hidden_layers=2 * pp)
    one = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0)
    one.set_optimizer('AdamW', lr=1e-3)
    single = []
    for _ in range(3):
        o = one.forward_backward(inputs=_moe_feats(), micro_batch_size=1)
        n = one.clip_grad_and_step(max_grad_norm=1.0)
        single.append((o['loss'], n))
    keys = sorted(one.get_state_dict().keys())
    for curve, same, el, saved in run_ranks(_ep_worker, world, str(tmp_path), tp, pp, ep, 3):
        assert same and el == cfg.num_experts // ep
        for (a, na), (b, nb) in zip(single, curve):
            assert abs(a - b) < 5e-4 and abs(na - nb) < 5e-3 * max(na, 1.0), (single, curve)
    from twinkle_b200.utils.safetensors_io import SafetensorLazyLoader
    loader = SafetensorLazyLoader(os.path.join(str(tmp_path), 'moe'))
    for k in keys:
        if k != 'lm_head.weight':
            assert k in loader, k


@pytest.mark.parametrize('tp,pp,ep,world,sp', [(2, 1, 1, 2, True), (2, 1, 1, 2, False), (2, 1, 2, 4, True)])
def test_expert_tensor_parallel_matches_single(tmp_path, tp, pp, ep, world, sp):
    """Every expert's intermediate dimension split over the tensor-parallel group (reference
    ``megatron/strategy/megatron.py:90-107``: ``expert_tensor_parallel_size``), with and without sequence-parallel
    activations and together with expert parallelism: loss curve and gradient norm of one process, shard shapes, and
    a bitwise round trip through the HF checkpoint (expert slices gathered over both groups)."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe', router_aux_loss_coef=0.0, num_hidden_layers=2 * pp)
    one = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0)
    one.set_optimizer('AdamW', lr=1e-3)
    single = []
    for _ in range(3):
        o = one.forward_backward(inputs=_moe_feats(), micro_batch_size=1)
        n = one.clip_grad_and_step(max_grad_norm=1.0)
        single.append((o['loss'], n))
    want = (cfg.num_experts // ep, 2 * cfg.moe_intermediate_size // tp, cfg.hidden_size)
    for curve, same, shape, saved in run_ranks(_ep_worker, world, str(tmp_path), tp, pp, ep, 3, tp, sp):
        assert same and shape == want, (shape, want)
        for (a, na), (b, nb) in zip(single, curve):
            assert abs(a - b) < 5e-4 and abs(na - nb) < 5e-3 * max(na, 1.0), (single, curve)
    from twinkle_b200.utils.safetensors_io import SafetensorLazyLoader
    loader = SafetensorLazyLoader(os.path.join(str(tmp_path), 'moe'))
    ref = one.get_state_dict()
    assert loader.get('model.layers.0.mlp.experts.3.down_proj.weight').shape == ref['model.layers.0.mlp.experts.3.down_proj.weight'].shape


def _aux_worker(rank, world, tp, pp, steps):
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe', router_aux_loss_coef=0.05, num_hidden_layers=2 * pp)
    mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=world // (tp * pp), sequence_parallel=tp > 1)
    m = MegatronModel(config=cfg, device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    curve = []
    for _ in range(steps):
        o = m.forward_backward(inputs=_moe_feats(), micro_batch_size=2)
        curve.append((o['loss'], m.clip_grad_and_step(max_grad_norm=1.0)))
    return curve


@pytest.mark.parametrize('tp,pp', [(1, 2), (2, 1)])
def test_router_load_balance_loss_on_the_pipeline_backend(tp, pp):
    """The router's auxiliary loss of every pipeline stage's own layers enters that stage's backward and the reported
    loss.  Without tensor parallelism the numbers are those of one process; with sequence-parallel activations every
    rank balances its own token slice, which changes the term slightly but must still train."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    single = {}
    for coef in (0.05, 0.0):
        cfg = preset('tiny-moe', router_aux_loss_coef=coef, num_hidden_layers=2 * pp)
        one = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0)
        one.set_optimizer('AdamW', lr=1e-3)
        single[coef] = []
        for _ in range(3):
            o = one.forward_backward(inputs=_moe_feats(), micro_batch_size=2)
            single[coef].append((o['loss'], one.clip_grad_and_step(max_grad_norm=1.0)))
    assert abs(single[0.05][0][1] - single[0.0][0][1]) > 1e-3      # the term is there at all: it changes the gradient
    for curve in run_ranks(_aux_worker, 2, tp, pp, 3):
        for (a, na), (b, nb) in zip(single[0.05], curve):
            if tp == 1:
                assert abs(a - b) < 5e-4 and abs(na - nb) < 5e-3 * max(na, 1.0), (single[0.05], curve)
            else:
                assert abs(a - b) < 2e-2 and abs(na - nb) < 5e-2 * max(na, 1.0), (single[0.05], curve)
        assert curve[-1][0] < curve[0][0]


def _reshard_worker(rank, world, tmp, src, dst, moe=False):
    """Trains 2 steps under layout ``src`` = (tp, pp, dp[, ep]), saves weights and optimizer state, trains 2 more; a model of
    layout ``dst`` resumes from the files of the first and must continue on the same curve."""
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe', num_hidden_layers=2, router_aux_loss_coef=0.0) if moe else preset('tiny-dense', num_hidden_layers=4)
    g = torch.Generator().manual_seed(13)
    feats = []          # rows of one length: the mean over data-parallel ranks is then the mean over tokens at every dp size
    for _ in range(4):
        ids = torch.randint(0, 1024, (65, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})

    def make(tp, pp, dp, ep=1):
        mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=dp, ep_size=ep if ep > 1 else None, sequence_parallel=tp > 1)
        m = MegatronModel(config=cfg, device_mesh=mesh, seed=0)
        m.set_optimizer('AdamW', lr=2e-3)
        m.set_lr_scheduler('CosineWarmupScheduler', num_warmup_steps=1, num_training_steps=8)
        return m, mesh

    def run(m, mesh, n):
        dr = mesh.get_data_rank_from_global_rank(rank)
        sl = mesh.get_slice(len(feats), dr)
        out = []
        for _ in range(n):
            o = m.forward_backward(inputs=feats[sl], micro_batch_size=1)
            m.clip_grad_and_step(max_grad_norm=1.0)
            out.append(o['loss'])
        return dr, out

    a, mesh_a = make(*src)
    run(a, mesh_a, 2)
    a.save('mid', tmp, save_optimizer=True)
    cont = run(a, mesh_a, 2)
    weights_a = {k: v.float().cpu().numpy() for k, v in a.get_state_dict().items()}     # by value through the result queue
    b, mesh_b = make(*dst)
    info = b.resume_from_checkpoint(os.path.join(tmp, 'mid'))
    resumed = run(b, mesh_b, 2)
    weights_b = {k: v.float().cpu().numpy() for k, v in b.get_state_dict().items()}
    return {'cont': cont, 'resumed': resumed, 'info': info, 'wa': weights_a, 'wb': weights_b}


@pytest.mark.parametrize('src,dst', [((2, 1, 2), (1, 2, 2)), ((1, 2, 2), (2, 2, 1)), ((2, 2, 1), (1, 1, 4)),
                                     ((1, 1, 4, 2), (1, 2, 2, 2)), ((1, 1, 4, 4), (2, 1, 2, 1)), ((1, 2, 2, 1), (1, 1, 4, 2))])
def test_optimizer_state_loads_into_another_layout(tmp_path, src, dst):
    """The last three cases move a mixture-of-experts model between expert-parallel layouts (ep 2 → ep 2 beside pipeline
    stages, ep 4 → whole experts beside tensor parallelism, whole experts → ep 2)."""
    res = run_ranks(_reshard_worker, 4, str(tmp_path), src, dst, len(src) == 4)
    cont, resumed, wa, wb = {}, {}, {}, {}
    for r in res:
        assert r['info']['cur_step'] == 2
        cont.setdefault(r['cont'][0], r['cont'][1])
        resumed.setdefault(r['resumed'][0], r['resumed'][1])
        wa.update(r['wa'])
        wb.update(r['wb'])
    # per-rank losses depend on which rows a rank got; their mean over the data-parallel ranks does not
    mean = lambda d: [sum(v[i] for v in d.values()) / len(d) for i in range(2)]     # noqa: E731
    for x, y in zip(mean(cont), mean(resumed)):
        assert abs(x - y) < 2e-5, (cont, resumed)
    # two more optimizer steps from resharded moments end on the same weights
    for k in wa:
        if k in wb:
            assert abs(wa[k] - wb[k]).max() < 2e-5, k
