"""The smallest end-to-end configuration: tiny dense decoder, LoRA SFT, fp32, CPU, gloo world_size=2
with sharded base weights; the 5-step loss curve must match a plain-PyTorch
oracle (no engine, autograd + torch.optim.AdamW on the same LoRA slices)."""
import torch

from tests.dist_utils import run_ranks


def _batch():
    g = torch.Generator().manual_seed(1234)
    feats = []
    for _ in range(4):
        ids = torch.randint(0, 1024, (129, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return feats


def _oracle_curve(steps=5):
    from twinkle_b200.model.multi_lora import LoraConfig, MultiLora
    from twinkle_b200.models import build_model, preset, PackedBatch, lora_batch
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(42)
    cfg = preset('tiny-dense')
    model = build_model(cfg, seed=0)
    ml = MultiLora(model, 1, 8)
    ml.acquire_lora('a', LoraConfig(r=8, lora_alpha=16))
    params = [p for n, p in model.named_parameters() if 'lora' in n]
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.01)
    feats = _batch()
    ids = torch.cat([torch.tensor(f['input_ids']) for f in feats])
    labels = torch.cat([torch.tensor(f['labels']) for f in feats])
    pos = torch.cat([torch.arange(128) for _ in feats])
    cu = torch.arange(0, 5, dtype=torch.int32) * 128
    curve = []
    for _ in range(steps):
        batch = PackedBatch(ids, pos, cu, 128, labels)
        with lora_batch(ml.batch_for('a', ids.numel(), 'cpu')):
            h = model(batch)
        logits = h @ model.head_weight().t()
        lp, _ = ref.logprob_from_logits(logits, labels)
        loss = -lp.sum() / labels.numel()
        opt.zero_grad()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        curve.append(float(loss))
    return curve


def _engine_curve(rank, world, steps):
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    torch.manual_seed(42)
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0)
    m.add_adapter_to_model('a', LoraConfig(r=8, lora_alpha=16, target_modules='all-linear'))
    m.set_optimizer('AdamW', lr=1e-4, weight_decay=0.01, adapter_name='a')
    feats = _batch()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    curve = []
    for _ in range(steps):
        out = m.forward_backward(inputs=feats[sl], adapter_name='a')
        m.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
        # global loss = Σ loss_sum / Σ tokens
        t = torch.tensor([out['loss'] * out['num_tokens'], out['num_tokens']], dtype=torch.float64)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t)
        curve.append(float(t[0] / t[1]))
    return curve


def test_single_process_matches_oracle():
    oracle = _oracle_curve()
    mine = _engine_curve(0, 1, 5)
    assert oracle[0] > oracle[-1]
    for a, b in zip(oracle, mine):
        assert abs(a - b) < 1e-4, (oracle, mine)


def test_gloo_world2_fsdp_matches_oracle():
    oracle = _oracle_curve()
    curves = run_ranks(_engine_curve, 2, 5)
    assert curves[0] == curves[1]
    for a, b in zip(oracle, curves[0]):
        assert abs(a - b) < 1e-4, (oracle, curves[0])
