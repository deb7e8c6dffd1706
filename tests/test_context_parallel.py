"""Context parallelism: key-index construction and a 2-rank gloo run (zig-zag shards + gathered keys with a
bottom-right causal offset) against one process on the whole sequences."""
import torch

from tests.dist_utils import run_ranks


def test_key_index_reproduces_full_causal_attention():
    """Emulate cp ranks in one process: every local chunk attends to exactly its causal prefix."""
    from twinkle_b200.ops import reference as ref
    from twinkle_b200.parallel.context import cp_key_index
    from twinkle_b200.processor import zigzag_indices
    torch.manual_seed(0)
    cp, seq_lens, Hq, Hkv, D = 2, [16, 8], 4, 2, 8
    T = sum(seq_lens)
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    cu = torch.tensor([0, 16, 24], dtype=torch.int32)
    want = ref.attention_varlen(q, k, v, cu, True)
    local_idx = []
    for r in range(cp):
        idx, off = [], 0
        for n in seq_lens:
            idx.append(zigzag_indices(n, cp, r) + off)
            off += n
        local_idx.append(torch.cat(idx))
    gathered_k = torch.cat([k[i] for i in local_idx])  # rank-major, as an all-gather returns it
    gathered_v = torch.cat([v[i] for i in local_idx])
    for r in range(cp):
        rows, cu_q, cu_k, max_q, max_k = cp_key_index(seq_lens, cp, r, 'cpu')
        out = ref.attention_varlen(q[local_idx[r]], gathered_k[rows], gathered_v[rows], cu_q, True, None, False, cu_k)
        assert torch.allclose(out, want[local_idx[r]], atol=1e-5)
        assert int(cu_k[-1]) == (2 * cp + 1) * sum(n // (2 * cp) for n in seq_lens)  # same key volume on every rank


def _curve(rank, world, steps):
    import torch.distributed as dist
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    torch.manual_seed(0)
    mesh = DeviceMesh.from_sizes(dp_size=1, cp_size=world) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    m = TransformersModel(model_id='tiny-dense', device_mesh=mesh, seed=0)
    m.set_optimizer('AdamW', lr=1e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(5)
    feats = []
    for n in (64, 32, 96):  # multiples of 2·cp
        ids = torch.randint(0, 1024, (n + 1, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    curve = []
    for _ in range(steps):
        out = m.forward_backward(inputs=feats)
        m.clip_grad_and_step(max_grad_norm=1.0)
        t = torch.tensor([out['loss'] * out['num_tokens'], out['num_tokens']], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        curve.append(float(t[0] / t[1]))
    return curve


def test_cp2_training_matches_single_process():
    single = _curve(0, 1, 4)
    multi = run_ranks(_curve, 2, 4)
    assert single[0] > single[-1]
    for c in multi:
        for a, b in zip(single, c):
            assert abs(a - b) < 2e-4, (single, c)


def test_ulysses_kv_replication_keeps_gqa_pairing_for_any_group_size():
    """Emulated head exchange: after repeating every K/V head ``sp/gcd(kv, sp)`` times, rank r's slice of query heads
    attends to its slice of K/V heads and the concatenation equals full GQA attention."""
    import torch.nn.functional as F
    from twinkle_b200.parallel.ulysses import kv_replication
    assert [kv_replication(8, s) for s in (1, 2, 4, 8, 16, 3, 6, 12)] == [1, 1, 1, 1, 2, 3, 3, 3]
    torch.manual_seed(0)
    t, d = 10, 8
    for hq, hkv, sp in ((24, 8, 3), (24, 8, 6), (12, 4, 6), (12, 6, 4), (32, 8, 16), (8, 8, 4), (6, 2, 3)):
        q, k, v = torch.randn(t, hq, d), torch.randn(t, hkv, d), torch.randn(t, hkv, d)
        grp = hq // hkv
        full = F.scaled_dot_product_attention(q.transpose(0, 1), k.repeat_interleave(grp, 1).transpose(0, 1),
                                              v.repeat_interleave(grp, 1).transpose(0, 1), is_causal=True).transpose(0, 1)
        rep = kv_replication(hkv, sp)
        kr, vr = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        assert kr.shape[1] % sp == 0 and (hq // sp) % (kr.shape[1] // sp) == 0
        parts = []
        for r in range(sp):
            ql = q[:, r * hq // sp:(r + 1) * hq // sp]
            kl, vl = (x[:, r * x.shape[1] // sp:(r + 1) * x.shape[1] // sp] for x in (kr, vr))
            g = ql.shape[1] // kl.shape[1]
            parts.append(F.scaled_dot_product_attention(ql.transpose(0, 1), kl.repeat_interleave(g, 1).transpose(0, 1),
                                                        vl.repeat_interleave(g, 1).transpose(0, 1), is_causal=True).transpose(0, 1))
        assert torch.allclose(torch.cat(parts, 1), full, atol=1e-6), (hq, hkv, sp)
