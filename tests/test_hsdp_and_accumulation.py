"""Hybrid sharding (shard inside ``fsdp``, replicate over ``dp``) on 4 CPU ranks, and gradient accumulation of
replicated LoRA pools over several micro-batches on 2: both must reproduce the single-process numbers (reference
``src/twinkle/model/transformers/strategy/accelerate.py:106-110``)."""
import torch

from tests.dist_utils import run_ranks


def _batch(n=4, seed=5):
    g = torch.Generator().manual_seed(seed)
    feats = []
    for L in (96, 64, 128, 80)[:n]:
        ids = torch.randint(0, 1024, (L + 1, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return feats


def _full_curve(rank, world, hybrid):
    import torch.distributed as dist
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    if world > 1:
        mesh = DeviceMesh.from_sizes(dp_size=2, fsdp_size=2)
        kw = {'strategy': 'accelerate'} if hybrid else {}
    else:
        mesh, kw = DeviceMesh.from_sizes(dp_size=1), {}
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0, **kw)
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.0)
    feats = _batch()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    out = []
    for _ in range(4):
        o = m.forward_backward(inputs=feats[sl])
        gn = m.clip_grad_and_step(max_grad_norm=1.0)
        t = torch.tensor([o['loss'] * o['num_tokens'], o['num_tokens']], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        out.append((float(t[0] / t[1]), float(gn)))
    info = {'curve': out, 'hybrid': m.engine.replica_comm is not None, 'shard_world': m.engine.comm.world_size}
    if world > 1:
        # shards are replicated across the dp axis: rank r and the rank with the same fsdp coordinate agree bit for bit
        b = m.engine.trainable_buckets()[0]
        mine = b.master.double().sum().reshape(1)
        allv = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allv, mine)
        info['master_sums'] = [float(v) for v in allv]
        ax = list(mesh.mesh_dim_names).index('fsdp')
        info['fsdp_coord'] = [mesh.coord_of(r)[ax] for r in range(world)]
    return info


def test_hybrid_sharding_matches_single_process():
    single = _full_curve(0, 1, False)['curve']
    for hybrid in (True, False):
        res = run_ranks(_full_curve, 4, hybrid)
        for r in res:
            assert r['hybrid'] is hybrid and r['shard_world'] == (2 if hybrid else 4)
            for (a, ga), (b, gb) in zip(single, r['curve']):
                assert abs(a - b) < 2e-4 and abs(ga - gb) < 2e-3 * max(ga, 1.0), (single, r['curve'])
        if hybrid:
            sums, coords = res[0]['master_sums'], res[0]['fsdp_coord']
            by_fsdp = {}
            for r, c in enumerate(coords):
                by_fsdp.setdefault(c, []).append(sums[r])                  # same fsdp coordinate = same shard
            for vals in by_fsdp.values():
                assert len(vals) == 2 and vals[0] == vals[1], (coords, sums)
            assert len({v[0] for v in by_fsdp.values()}) == 2, 'the two shards of a group differ'


def _lora_curve(rank, world, micro):
    import torch.distributed as dist
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None)
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0)
    m.add_adapter_to_model('a', LoraConfig(r=8, lora_alpha=16, target_modules='all-linear'))
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.01, adapter_name='a')
    feats = _batch()
    sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
    out = []
    for _ in range(3):
        o = m.forward_backward(inputs=feats[sl], adapter_name='a', micro_batch_size=micro)
        gn = m.clip_grad_and_step(max_grad_norm=1e9, adapter_name='a')
        t = torch.tensor([o['loss'] * o['num_tokens'], o['num_tokens']], dtype=torch.float64)
        dist.all_reduce(t)
        out.append((float(t[0] / t[1]), float(gn)))
    return out


def test_lora_gradients_over_micro_batches_are_summed_once():
    one = run_ranks(_lora_curve, 2, 2)[0]        # both sequences of a rank in one micro-batch
    two = run_ranks(_lora_curve, 2, 1)[0]        # one sequence per micro-batch: two backward passes per step
    for (a, ga), (b, gb) in zip(one, two):
        assert abs(a - b) < 1e-4 and abs(ga - gb) < 1e-4 * max(ga, 1.0), (one, two)
