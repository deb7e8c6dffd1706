"""Two pieces that had no test of their own: the two-phase gradient norm of expert-parallel parameters
(``utils/grad_clip.py``; reference ``src/twinkle/utils/grad_clip.py:208-285``) against the norm of the assembled
gradient, and the gateway's sticky adapter router (reference ``src/twinkle/server/routing/sticky_lora_router.py``)."""
import math

import torch

from tests.dist_utils import run_ranks


def _full_grads():
    g = torch.Generator().manual_seed(3)
    dense = torch.randn(16, generator=g)
    experts = [torch.randn(8, generator=g), torch.randn(8, generator=g)]      # two expert sets, one per EP rank
    return dense, experts


def _norm_worker(rank, world, max_norm, norm_type):
    import torch.distributed as dist
    from twinkle_b200.utils.grad_clip import normalize_and_clip_grad_norm
    dense, experts = _full_grads()
    ep, f = divmod(rank, 2)                                                    # rank = ep * 2 + ep_fsdp
    ep_group = fs_group = None
    for grp in ([0, 2], [1, 3]):
        h = dist.new_group(grp)
        if rank in grp:
            ep_group = h
    for grp in ([0, 1], [2, 3]):
        h = dist.new_group(grp)
        if rank in grp:
            fs_group = h
    pd = torch.nn.Parameter(torch.zeros(4))
    pd.grad = dense[rank * 4:(rank + 1) * 4].clone() * 10.0                     # sharded over all 4 ranks; 10 = token count
    pe = torch.nn.Parameter(torch.zeros(4))
    pe.grad = experts[ep][f * 4:(f + 1) * 4].clone() * 10.0                     # expert set `ep`, sharded over its ep_fsdp pair
    n = normalize_and_clip_grad_norm([pd, pe], num_tokens=10.0, max_grad_norm=max_norm, norm_type=norm_type, group=None, sharded=True,
                                     ep_params=[pe], ep_group=ep_group, ep_fsdp_group=fs_group)
    return n, pd.grad.tolist(), pe.grad.tolist()


def test_expert_parallel_two_phase_norm_equals_assembled_norm():
    dense, experts = _full_grads()
    whole = torch.cat([dense] + experts)
    for norm_type, want in ((2.0, float(whole.norm(2))), (math.inf, float(whole.abs().max()))):
        res = run_ranks(_norm_worker, 4, 1.0, norm_type)
        coef = min(1.0, 1.0 / (want + 1e-6))
        for rank, (n, gd, ge) in enumerate(res):
            assert abs(n - want) < 1e-4 * want, (norm_type, n, want)
            ep, f = divmod(rank, 2)
            assert torch.allclose(torch.tensor(gd), dense[rank * 4:(rank + 1) * 4] * coef, atol=1e-5)
            assert torch.allclose(torch.tensor(ge), experts[ep][f * 4:(f + 1) * 4] * coef, atol=1e-5)


class _Replica:
    """The part of a model application the router looks at."""

    def __init__(self, rid, base, max_loras):
        class A:
            model_id, max_loras = base, 0
        self.args = A()
        self.args.max_loras = max_loras
        self.replica_id, self.adapters = rid, {}

    class worker:
        @staticmethod
        def depth():
            return 0


def test_sticky_router_keeps_an_adapter_on_its_replica_and_fills_the_emptiest():
    from twinkle_b200.server.apps.gateway import Router
    r = Router()
    a, b = _Replica('A', 'base', 2), _Replica('B', 'base', 4)
    other = _Replica('C', 'other-base', 8)
    for x in (a, b, other):
        r.add_model(x)
    # new adapters go to the replica of that base with the most free slots
    first = r.model_for('base', None)
    assert first is b
    b.adapters['m1'] = {}
    b.adapters['m2'] = {}
    b.adapters['m3'] = {}                                            # B now has 1 free slot, A has 2
    assert r.model_for('base', None) is a
    a.adapters['m4'] = {}
    # an existing adapter always resolves to the replica that holds it, however full that one is
    assert r.model_for('base', 'm1') is b and r.model_for('base', 'm4') is a
    assert r.model_for('other-base', None) is other
    # unknown base: nothing to route to
    import pytest
    with pytest.raises(Exception):
        r.model_for('missing', None)
