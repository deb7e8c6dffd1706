"""Index bookkeeping of the peer-memory expert-parallel path, with every rank emulated in one CPU process: the
"peer buffers" are plain per-rank tensors, the pulls are the torch restatements of the CUDA kernels."""
import torch

from twinkle_b200.ops import reference as ref
from twinkle_b200.parallel.expert_symm import ep_metadata, pull_combine, pull_rows, pull_wgrad


def _setup(ep=4, E=8, k=2, H=16, I=8, Ts=(13, 7, 20, 16), align=4, cap=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(T, H, generator=g) for T in Ts]
    idx = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]) for T in Ts]
    ws = [torch.rand(T, k, generator=g) for T in Ts]
    gate_up = torch.randn(E, 2 * I, H, generator=g) * 0.3
    down = torch.randn(E, H, I, generator=g) * 0.3
    counts_all = torch.stack([torch.bincount(i.reshape(-1), minlength=E) for i in idx]).to(torch.int32)
    metas = [ep_metadata(idx[r].reshape(-1), counts_all, r, k, cap, align) for r in range(ep)]
    return xs, idx, ws, gate_up, down, counts_all, metas


def test_dispatch_experts_combine_match_dense_reference():
    ep, E, k, H = 4, 8, 2, 16
    xs, idx, ws, gate_up, down, counts_all, metas = _setup()
    El = E // ep
    toks = [m.tok_sorted for m in metas]
    ys = []
    for d in range(ep):
        m = metas[d]
        rows = pull_rows(xs, toks, None, m, H)
        assert int(m.total_rows) <= rows.shape[0]
        # every local expert's segment holds exactly the rows routed to it, in (source rank, sorted position) order
        off = m.offsets.tolist()
        for e in range(El):
            want = int(counts_all[:, d * El + e].sum())
            seg = rows[off[e]:off[e + 1]]
            assert off[e] % 4 == 0 and off[e + 1] - off[e] >= want
            assert float(seg[want:].abs().sum()) == 0.0
        y = ref.swiglu(ref.grouped_gemm(rows, gate_up[d * El:(d + 1) * El], m.offsets))
        ys.append(ref.grouped_gemm(y, down[d * El:(d + 1) * El], m.offsets))
    for s in range(ep):
        out = pull_combine(ys, metas[s], ws[s], H)
        want = ref.moe_experts(xs[s], ws[s], idx[s], gate_up, down)
        assert torch.allclose(out, want, atol=1e-5), float((out - want).abs().max())


def test_backward_pulls_are_the_adjoints():
    ep, H = 4, 16
    xs, idx, ws, gate_up, down, counts_all, metas = _setup(seed=1)
    toks = [m.tok_sorted for m in metas]
    g = torch.Generator().manual_seed(5)
    cap = metas[0].src_rank.numel()
    ys = [torch.randn(cap, H, generator=g) for _ in range(ep)]
    for d in range(ep):
        ys[d][metas[d].src_rank < 0] = 0  # padding rows carry nothing
    gouts = [torch.randn(x.shape[0], H, generator=g) for x in xs]

    # combine: out_s = Σ_j w·y_d[row]; its adjoint wrt y is the weighted pull of the output gradients
    ys_req = [y.clone().requires_grad_(True) for y in ys]
    ws_req = [w.clone().requires_grad_(True) for w in ws]
    total = sum((pull_combine(ys_req, metas[s], ws_req[s], H) * gouts[s]).sum() for s in range(ep))
    total.backward()
    w_sorted = [ws[s].reshape(-1)[metas[s].order] for s in range(ep)]
    for d in range(ep):
        gy = pull_rows(gouts, toks, w_sorted, metas[d], H)
        assert torch.allclose(gy, ys_req[d].grad, atol=1e-5)
    for s in range(ep):
        assert torch.allclose(pull_wgrad(gouts[s], ys, metas[s]), ws_req[s].grad, atol=1e-4)

    # dispatch: rows_d = x_s[tok]; its adjoint wrt x is the unweighted combine of the row gradients
    xs_req = [x.clone().requires_grad_(True) for x in xs]
    grows = [torch.randn(cap, H, generator=g) for _ in range(ep)]
    total = sum((pull_rows(xs_req, toks, None, metas[d], H) * grows[d]).sum() for d in range(ep))
    total.backward()
    for s in range(ep):
        assert torch.allclose(pull_combine(grows, metas[s], None, H), xs_req[s].grad, atol=1e-5)


def test_rows_over_capacity_are_dropped_not_misplaced():
    xs, idx, ws, gate_up, down, counts_all, metas = _setup(cap=16, seed=2)
    for r, m in enumerate(metas):
        assert int(m.offsets[-1]) <= 16
        kept = m.dst_rank >= 0
        assert bool((m.dst_row[kept] < 16).all())
    assert any(int(m.total_rows) > 16 for m in metas)
