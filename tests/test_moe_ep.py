"""MoE: local grouped path vs the dense-math oracle, and expert parallel (gloo, world 2) vs one process —
logits-level outputs, loss and gradients (reference model: tests/moe/test_ep_fsdp_vs_single.py)."""
import torch

from tests.dist_utils import run_ranks


def _inputs():
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 1024, (96, ), generator=g)
    labels = torch.randint(0, 1024, (96, ), generator=g)
    pos = torch.cat([torch.arange(64), torch.arange(32)])
    cu = torch.tensor([0, 64, 96], dtype=torch.int32)
    return ids, labels, pos, cu


def _run(model):
    from twinkle_b200.models import PackedBatch
    ids, labels, pos, cu = _inputs()
    h = model(PackedBatch(ids, pos, cu, 64, labels))
    lp, _ = model.token_logprobs(h, labels)
    loss = -lp.mean()
    aux = model.aux_loss()
    if aux is not None:
        loss = loss + aux
    loss.backward()
    return loss.detach(), h.detach()


def test_local_moe_matches_dense_oracle():
    from twinkle_b200.models import build_model, preset
    from twinkle_b200.ops import reference as ref
    cfg = preset('tiny-moe')
    m = build_model(cfg, seed=1)
    blk = m.layers[0].mlp
    x = torch.randn(50, cfg.hidden_size)
    w, idx, _ = blk.route(x, None)
    want = ref.moe_experts(x, w, idx, blk.experts.gate_up_proj, blk.experts.down_proj)
    got = blk(x)
    assert torch.allclose(got, want, atol=1e-5), float((got - want).abs().max())


def _ep_worker(rank, world):
    from twinkle_b200.models import build_model, preset
    from twinkle_b200.parallel.expert import apply_expert_parallel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-moe')
    m = build_model(cfg, seed=1)
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ep_size=world)
    apply_expert_parallel(m, mesh, cfg)
    loss, h = _run(m)
    g = m.layers[0].mlp.experts.down_proj.grad
    return float(loss), h, g, m.layers[0].mlp.gate.weight.grad


def test_expert_parallel_matches_single():
    from twinkle_b200.models import build_model, preset
    cfg = preset('tiny-moe')
    single = build_model(cfg, seed=1)
    loss, h = _run(single)
    res = run_ranks(_ep_worker, 2)
    for r, (l, hh, g, gg) in enumerate(res):
        assert abs(l - float(loss)) < 1e-5
        assert torch.allclose(hh, h, atol=1e-5)
        # both ranks fed the same tokens: every expert sees each token twice → expert grads are 2x, router grads equal
        full = single.layers[0].mlp.experts.down_proj.grad
        El = cfg.num_experts // 2
        assert torch.allclose(g, 2 * full[r * El:(r + 1) * El], atol=1e-5)
        assert torch.allclose(gg, single.layers[0].mlp.gate.weight.grad, atol=1e-5)


def _train_curve(rank, world, steps):
    import torch.distributed as dist
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    torch.manual_seed(0)
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ep_size=world) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    from twinkle_b200.models import preset
    # the load-balance loss is a non-linear function of the tokens a rank sees, so it is switched off for the comparison
    m = TransformersModel(config=preset('tiny-moe', router_aux_loss_coef=0.0), device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(21)
    feats = []
    for n in (48, 80, 64, 32):
        ids = torch.randint(0, 1024, (n + 1, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    curve = []
    for _ in range(steps):
        out = m.forward_backward(inputs=feats[sl])
        norm = m.clip_grad_and_step(max_grad_norm=1.0)
        t = torch.tensor([out['loss'] * out['num_tokens'], out['num_tokens']], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        curve.append((float(t[0] / t[1]), float(norm) if norm is not None else 0.0))
    return curve


def test_expert_parallel_training_matches_single_process():
    """Full-parameter steps through the engine: expert gradients stay on their owner rank, the clip norm counts
    every expert once, so loss and gradient-norm curves equal the single-process ones."""
    single = _train_curve(0, 1, 4)
    multi = run_ranks(_train_curve, 2, 4)
    assert single[0][0] > single[-1][0]
    for c in multi:
        for (l1, n1), (l2, n2) in zip(single, c):
            assert abs(l1 - l2) < 2e-4, (single, c)
            assert abs(n1 - n2) < 2e-3 * max(1.0, n1), (single, c)


def test_shared_expert_math_and_hf_round_trip(tmp_path):
    """MoE block with an always-on gated expert: output = routed + sigmoid(gate·x)·MLP(x); the HF checkpoint written
    by ``save`` (shared expert split into gate/up/down, config field kept) loads back to the same loss."""
    import torch.nn.functional as F
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import DecoderConfig
    m = TransformersModel(model_id='tiny-moe-shared', seed=0)
    blk = m.model.layers[0].mlp
    assert blk.shared_expert is not None and blk.shared_expert_gate.weight.shape == (1, 256)
    x = torch.randn(12, 256)
    with torch.no_grad():
        full = blk(x)
        shared, gate = blk.shared_expert, blk.shared_expert_gate
        blk.shared_expert = blk.shared_expert_gate = None
        routed = blk(x)
        blk.shared_expert, blk.shared_expert_gate = shared, gate
        g, u = F.linear(x, shared.gate_up_proj.weight).chunk(2, -1)
        want = routed + torch.sigmoid(F.linear(x, gate.weight)) * F.linear(F.silu(g) * u, shared.down_proj.weight)
    assert torch.allclose(full, want, atol=1e-5)
    ids = torch.randint(0, 1024, (33, ), generator=torch.Generator().manual_seed(1))
    batch = [{'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()}]
    m.set_optimizer('AdamW', lr=1e-2)
    first = m.forward_backward(inputs=batch)['loss']
    before = gate.weight.detach().clone()
    m.clip_grad_and_step(max_grad_norm=1.0)
    assert not torch.equal(before, gate.weight.detach())          # the shared path trains
    out = m.save('ck', str(tmp_path))
    cfg = DecoderConfig.from_pretrained(out)
    assert cfg.shared_expert_intermediate_size == 192 and cfg.num_experts == 8
    from safetensors import safe_open
    import glob
    names = set()
    for f in glob.glob(out + '/*.safetensors'):
        with safe_open(f, 'pt') as fh:
            names |= set(fh.keys())
    assert {'model.layers.0.mlp.shared_expert.gate_proj.weight', 'model.layers.0.mlp.shared_expert.up_proj.weight',
            'model.layers.0.mlp.shared_expert.down_proj.weight', 'model.layers.0.mlp.shared_expert_gate.weight'} <= names
    m2 = TransformersModel(model_id=out, seed=5)
    a, b = m.forward_only(inputs=batch, return_logits=False), m2.forward_only(inputs=batch, return_logits=False)
    assert torch.allclose(torch.as_tensor(a['logps']).float(), torch.as_tensor(b['logps']).float(), atol=1e-5)
    assert float(first) > 0
