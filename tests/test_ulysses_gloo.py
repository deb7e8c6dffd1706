"""Full-parameter SFT on 4 CPU ranks (gloo): flat-bucket FSDP over all 4, Ulysses SP = 2 inside it, so two data
groups of two sequence-parallel ranks each.  The global loss curve must match one process on the whole batch."""
import torch

from tests.dist_utils import run_ranks


def _batch():
    g = torch.Generator().manual_seed(7)
    feats = []
    for n in (96, 64, 128, 32):
        ids = torch.randint(0, 1024, (n + 1, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return feats


def _curve(rank, world, steps, sp):
    import torch.distributed as dist
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    torch.manual_seed(0)
    if world > 1:
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=sp)
    else:
        mesh = DeviceMesh.from_sizes(dp_size=1)
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.0)
    feats = _batch()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    curve = []
    for _ in range(steps):
        out = m.forward_backward(inputs=feats[sl])
        m.clip_grad_and_step(max_grad_norm=1.0)
        t = torch.tensor([out['loss'] * out['num_tokens'], out['num_tokens']], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
            t = t / sp  # sequence-parallel peers report the same data group's numbers
        curve.append(float(t[0] / t[1]))
    return curve


def test_fsdp4_ulysses2_matches_single_process():
    single = _curve(0, 1, 4, 1)
    multi = run_ranks(_curve, 4, 4, 2)
    assert single[0] > single[-1]
    for c in multi:
        for a, b in zip(single, c):
            assert abs(a - b) < 2e-4, (single, c)
