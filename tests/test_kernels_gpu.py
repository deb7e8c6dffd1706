"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op.
Tolerances follow the reference's distributed tests (logits 1e-2 / 5e-3, grads 2e-2 / 1e-2) expressed
as relative Frobenius error, which for bf16 outputs sits near 2e-3."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def E():
    from twinkle_b200 import ops
    e = ops.ext()
    e.read_and_clear_error()
    yield e
    assert e.read_and_clear_error() == 0


def rel(a, b):
    """Error of ``a`` against the reference ``b`` as one number that a norm alone cannot hide things from: the
    relative Frobenius error, the worst row's error (against that row's own norm plus the typical row norm, weighted
    1/4) and the worst element's error (against its own magnitude plus the reference's RMS, weighted 1/16).  A single
    wrong 16-byte vector in a 4096 x 4096 output moves the Frobenius term by 1e-3 but the element term by ~5e-2, so
    ragged-tail and stray-store bugs fail the same bounds that rounding passes; the per-row / per-element scales keep
    heavy-tailed tensors (a softmax gradient with one large entry per row) from tripping on ordinary rounding."""
    a, b = a.detach().float(), b.detach().float()
    d = a - b
    fro = float(d.norm() / (b.norm() + 1e-12))
    if b.dim() < 1 or b.numel() == 0:
        return fro
    rms = float(b.pow(2).mean().sqrt()) + 1e-12
    elem = float((d.abs() / (b.abs() + rms)).max())
    rows_d = d.reshape(-1, d.shape[-1]) if d.dim() > 1 else d.reshape(1, -1)
    rows_b = b.reshape(-1, b.shape[-1]) if b.dim() > 1 else b.reshape(1, -1)
    typical_row = rms * math.sqrt(rows_b.shape[-1])
    row = float((rows_d.norm(dim=-1) / (rows_b.norm(dim=-1) + typical_row)).max())
    return max(fro, row / 4.0, elem / 16.0)


@pytest.mark.parametrize('layout', ['nt', 'nn', 'tn'])
@pytest.mark.parametrize('shape', [(128, 256, 64), (304, 520, 200), (1024, 4096, 4096), (4096, 1024, 2048), (72, 8, 64)])
def test_gemm(E, layout, shape):
    M, N, K = shape
    torch.manual_seed(0)
    if layout == 'nt':
        a, b = torch.randn(M, K, device='cuda').bfloat16(), torch.randn(N, K, device='cuda').bfloat16()
        r = a.float() @ b.float().t()
    elif layout == 'nn':
        a, b = torch.randn(M, K, device='cuda').bfloat16(), torch.randn(K, N, device='cuda').bfloat16()
        r = a.float() @ b.float()
    else:
        a, b = torch.randn(K, M, device='cuda').bfloat16(), torch.randn(K, N, device='cuda').bfloat16()
        r = a.float().t() @ b.float()
    assert rel(E.gemm(a, b, layout), r) < 4e-3
    assert rel(E.gemm(a, b, layout, None, False, torch.float32), r) < 1e-5
    acc = torch.ones(M, N, device='cuda')
    E.gemm(a, b, layout, acc, True)
    assert rel(acc - 1, r) < 1e-5
    assert E.read_and_clear_error() == 0


@pytest.mark.parametrize('layout', ['nt', 'nn', 'tn'])
@pytest.mark.parametrize('shape', [(4096, 2048, 512), (4000, 2504, 200), (2304, 4096, 4096)])
def test_gemm_sm_pair(E, layout, shape):
    """256x256 tiles on SM pairs (cta_group::2) against fp32, including ragged M / N / K and accumulate."""
    M, N, K = shape
    torch.manual_seed(0)
    if layout == 'nt':
        a, b = torch.randn(M, K, device='cuda').bfloat16(), torch.randn(N, K, device='cuda').bfloat16()
        r = a.float() @ b.float().t()
    elif layout == 'nn':
        a, b = torch.randn(M, K, device='cuda').bfloat16(), torch.randn(K, N, device='cuda').bfloat16()
        r = a.float() @ b.float()
    else:
        a, b = torch.randn(K, M, device='cuda').bfloat16(), torch.randn(K, N, device='cuda').bfloat16()
        r = a.float().t() @ b.float()
    E.set_gemm_pair(1)
    try:
        n0 = E.launch_count()
        o = E.gemm(a, b, layout)
        acc = torch.ones(M, N, device='cuda', dtype=torch.float32)
        E.gemm(a, b, layout, acc, True)
        torch.cuda.synchronize()
    finally:
        E.set_gemm_pair(0)
    assert E.launch_count() - n0 == 2
    assert rel(o, r) < 4e-3
    assert rel(acc - 1, r) < 1e-4
    try:
        single = E.gemm(a, b, layout)  # single-CTA tiles
    finally:
        E.set_gemm_pair(1)
    assert rel(o, single) < 1e-6  # same products, same fp32 accumulation order per k-step


def test_grouped_gemm(E):
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    Eg, K, N = 4, 256, 512
    counts = [100, 0, 300, 128]
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + (c + 127) // 128 * 128)
    x = torch.zeros(offs[-1], K, device='cuda').bfloat16()
    for e, c in enumerate(counts):
        x[offs[e]:offs[e] + c] = torch.randn(c, K, device='cuda').bfloat16()
    w = torch.randn(Eg, N, K, device='cuda').bfloat16()
    off = torch.tensor(offs, device='cuda', dtype=torch.int32)
    want = ref.grouped_gemm(x, w, off)
    assert rel(E.grouped_gemm(x, w, off, 'nt'), want) < 4e-3
    assert rel(E.grouped_gemm(x, w.transpose(1, 2).contiguous(), off, 'nn'), want) < 4e-3
    dy = torch.randn(offs[-1], N, device='cuda').bfloat16()
    gw = E.grouped_gemm_wgrad(dy, x, off, Eg)
    gr = torch.stack([dy[offs[e]:offs[e + 1]].float().t() @ x[offs[e]:offs[e + 1]].float() for e in range(Eg)])
    assert rel(gw, gr) < 1e-5 and float(gw[1].abs().max()) == 0.0
    # second operand pair (a rank-16 and a rank-72 low-rank term summed in tensor memory with the base product): both
    # layouts, with the narrow operand far below / just above the kernel's 64-wide k-tile
    for r in (16, 72):
        x2 = torch.zeros(offs[-1], r, device='cuda').bfloat16()
        for e, c in enumerate(counts):
            x2[offs[e]:offs[e] + c] = torch.randn(c, r, device='cuda').bfloat16()
        w2 = torch.randn(Eg, N, r, device='cuda').bfloat16()
        both = want.float() + ref.grouped_gemm(x2, w2, off).float()
        got = E.grouped_gemm(x, w, off, 'nt', None, None, False, x2, w2)
        assert rel(got, both) < 4e-3
        got = E.grouped_gemm(x, w.transpose(1, 2).contiguous(), off, 'nn', None, None, False, x2, w2.transpose(1, 2).contiguous())
        assert rel(got, both) < 4e-3
    assert E.read_and_clear_error() == 0


@pytest.mark.parametrize('rows,H', [(1000, 4096), (333, 1000), (257, 5120), (64, 8192), (33, 9216), (1, 128)])
def test_rmsnorm(E, rows, H):
    """Widths served by one / two column vectors per thread of the row-block backward (with a ragged last warp), wider
    than it serves (one warp per row), and row counts that leave the last row group incomplete."""
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    x = torch.randn(rows, H, device='cuda').bfloat16().requires_grad_(True)
    w = (torch.randn(H, device='cuda') * 0.1 + 1).bfloat16().requires_grad_(True)
    y = ops.rmsnorm(x, w, 1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = ref.rmsnorm(xr, wr, 1e-6)
    yr.backward(g.float())
    assert rel(y, yr) < 4e-3 and rel(x.grad, xr.grad) < 4e-3 and rel(w.grad, wr.grad) < 4e-3


def test_add_rmsnorm_fused(E):
    """Residual add inside the norm kernel (forward) and the residual-stream gradient inside its backward kernel,
    against the two-step fp32 reference; ``h`` must equal the bf16 sum bit for bit."""
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    for rows, H in ((515, 4096), (77, 5120), (9, 9216)):
        x = torch.randn(rows, H, device='cuda').bfloat16().requires_grad_(True)
        r = torch.randn(rows, H, device='cuda').bfloat16().requires_grad_(True)
        w = (torch.randn(H, device='cuda') * 0.1 + 1).bfloat16().requires_grad_(True)
        y, h = ops.add_rmsnorm(x, r, w, 1e-6)
        gy, gh = torch.randn_like(y), torch.randn_like(h)
        torch.autograd.backward([y, h], [gy, gh])
        assert torch.equal(h, x.detach() + r.detach())
        xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, r, w))
        hr = (xr + rr) + ((xr + rr).bfloat16().float() - (xr + rr)).detach()
        yr = ref.rmsnorm(hr, wr, 1e-6)
        torch.autograd.backward([yr, hr], [gy.float(), gh.float()])
        assert rel(y, yr) < 4e-3 and rel(w.grad, wr.grad) < 4e-3
        assert rel(x.grad, xr.grad) < 4e-3 and torch.equal(x.grad, r.grad)


@pytest.mark.parametrize('hq,hkv', [(8, 2), (5, 2), (3, 1), (32, 8)])
def test_qk_norm_rope(E, hq, hkv):
    """Head counts that fill the kernel's 8-heads-per-round walk exactly, leave a ragged last round, and put a q/k or
    k/v boundary inside one warp's head pair."""
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    T, d = 777, 128
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device='cuda').bfloat16().requires_grad_(True)
    qw = (torch.randn(d, device='cuda') * 0.1 + 1).bfloat16().requires_grad_(True)
    kw = (torch.randn(d, device='cuda') * 0.1 + 1).bfloat16().requires_grad_(True)
    cos, sin = ops.rope_tables(torch.arange(T, device='cuda'), d, 1e6)
    q, k, v = ops.qkv_norm_rope(qkv, qw, kw, cos, sin, hq, hkv, d)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    qkvr, qwr, kwr = (t.detach().float().requires_grad_(True) for t in (qkv, qw, kw))
    q_, k_, v_ = qkvr.split([hq * d, hkv * d, hkv * d], -1)
    q_, k_, v_ = q_.reshape(T, hq, d), k_.reshape(T, hkv, d), v_.reshape(T, hkv, d)
    q2, k2 = ref.qk_norm_rope(q_, k_, qwr, kwr, cos, sin)
    torch.autograd.backward([q2, k2, v_], [gq.float(), gk.float(), gv.float()])
    assert rel(q, q2) < 5e-3 and rel(k, k2) < 5e-3 and rel(v, v_) == 0
    assert rel(qkv.grad, qkvr.grad) < 5e-3 and rel(qw.grad, qwr.grad) < 5e-3 and rel(kw.grad, kwr.grad) < 5e-3


def test_swiglu_adamw_sumsq(E):
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    gu = torch.randn(513, 2 * 1536, device='cuda').bfloat16().requires_grad_(True)
    y = ops.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gur = gu.detach().float().requires_grad_(True)
    yr = ref.swiglu(gur)
    yr.backward(g.float())
    assert rel(y, yr) < 4e-3 and rel(gu.grad, gur.grad) < 4e-3
    # tanh-GELU gate (Gemma MLPs): same kernels with the other activation; 3-D input goes through as rows
    gu3 = torch.randn(3, 171, 2 * 1536, device='cuda').bfloat16().requires_grad_(True)
    y3 = ops.geglu(gu3)
    g3 = torch.randn_like(y3)
    y3.backward(g3)
    gu3r = gu3.detach().float().requires_grad_(True)
    y3r = ref.geglu(gu3r)
    y3r.backward(g3.float())
    assert y3.shape == (3, 171, 1536) and rel(y3, y3r) < 4e-3 and rel(gu3.grad, gu3r.grad) < 4e-3
    n = 1 << 20
    m0 = torch.randn(n, device='cuda')
    m, ea, es = m0.clone(), torch.zeros(n, device='cuda'), torch.zeros(n, device='cuda')
    mr, ear, esr = m0.clone(), torch.zeros(n, device='cuda'), torch.zeros(n, device='cuda')
    gr = torch.randn(n, device='cuda').bfloat16()
    out = torch.empty(n, device='cuda', dtype=torch.bfloat16)
    for step in (1, 2, 3):
        ops.adamw_step(m, ea, es, gr, out, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
        ref.adamw_step(mr, ear, esr, gr, None, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
    assert rel(m, mr) < 1e-5 and rel(out, mr) < 4e-3
    assert abs(float(ops.sumsq(gr)) / float(gr.float().pow(2).sum()) - 1) < 1e-4
    # a length that leaves a tail after the 4-element vectors, and views that start off the 16-byte grid (scalar path)
    for lo, hi in ((0, 100003), (1, 100004)):
        a = [t[lo:hi].clone() if lo == 0 else t[lo:hi] for t in (m0.clone(), torch.zeros(n, device='cuda'), torch.zeros(n, device='cuda'))]
        b = [t[lo:hi].clone() for t in (m0, torch.zeros(n, device='cuda'), torch.zeros(n, device='cuda'))]
        g32 = torch.randn(n, device='cuda')[lo:hi]
        o32 = torch.empty(n, device='cuda')[lo:hi]
        ops.adamw_step(a[0], a[1], a[2], g32, o32, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0)
        ref.adamw_step(b[0], b[1], b[2], g32.clone(), None, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0)
        assert rel(a[0], b[0]) < 1e-5 and rel(a[1], b[1]) < 1e-5 and rel(a[2], b[2]) < 1e-5 and torch.equal(o32, a[0])
        assert abs(float(ops.sumsq(g32)) / float(g32.pow(2).sum()) - 1) < 1e-4
        assert abs(float(ops.sumsq(gr[lo:hi])) / float(gr[lo:hi].float().pow(2).sum()) - 1) < 1e-4


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_logprob(E, dtype):
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    x = (torch.randn(200, 151936, device='cuda') * 2).to(dtype).requires_grad_(True)
    y = torch.randint(0, 151936, (200, ), device='cuda')
    lp, ent = ops.logprob_from_logits(x, y, 0.7, True)
    glp, ge = torch.randn_like(lp), torch.randn_like(lp)
    torch.autograd.backward([lp, ent], [glp, ge])
    xr = x.detach().float().requires_grad_(True)
    lpr, entr = ref.logprob_from_logits(xr, y, 0.7, True)
    torch.autograd.backward([lpr, entr], [glp, ge])
    assert rel(lp, lpr) < 1e-5 and rel(ent, entr) < 1e-5 and rel(x.grad, xr.grad) < (4e-3 if dtype == torch.bfloat16 else 1e-5)


def test_fused_linear_logprob(E):
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    torch.manual_seed(0)
    h = (torch.randn(1000, 512, device='cuda') * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(3000, 512, device='cuda') * 0.05).bfloat16().requires_grad_(True)
    y = torch.randint(0, 3000, (1000, ), device='cuda')
    lp, _ = ops.fused_linear_logprob(h, w, y, chunk=256)
    (-lp.sum()).backward()
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lpr, _ = ref.fused_linear_logprob(hr, wr, y)
    (-lpr.sum()).backward()
    assert rel(lp, lpr) < 1e-3 and rel(h.grad, hr.grad) < 5e-3 and rel(w.grad, wr.grad) < 5e-3


@pytest.mark.parametrize('case', [([128], 1, 1), ([256], 2, 1), ([100, 300, 77], 4, 2), ([1024, 512, 1], 8, 2), ([2048], 32, 8)])
def test_flash_attention(E, case):
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    lens, hq, hkv = case
    torch.manual_seed(0)
    T, d = sum(lens), 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device='cuda', dtype=torch.int32)
    q, k, v = (torch.randn(T, h, d, device='cuda').bfloat16().requires_grad_(True) for h in (hq, hkv, hkv))
    o = ops.flash_attn_varlen(q, k, v, cu, max(lens))
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = ref.attention_varlen(qr, kr, vr, cu)
    assert rel(o, orf) < 5e-3
    g = torch.randn_like(o)
    o.backward(g)
    orf.backward(g.float())
    assert rel(q.grad, qr.grad) < 8e-3 and rel(k.grad, kr.grad) < 8e-3 and rel(v.grad, vr.grad) < 8e-3
    assert E.read_and_clear_error() == 0


def test_flash_attention_long_packed_row(E):
    """One 32768-token row packed from documents of up to 8192 tokens (the shape of the training benchmark), forward and
    backward against fp32, with the per-row and per-element terms of ``rel`` guarding the tile edges of long documents."""
    from twinkle_b200 import ops
    from twinkle_b200.ops import reference as ref
    lens, hq, hkv, d = [8192, 6000, 8192, 2192, 8192], 4, 2, 128
    assert sum(lens) == 32768
    torch.manual_seed(1)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device='cuda', dtype=torch.int32)
    q, k, v = (torch.randn(T, h, d, device='cuda').bfloat16().requires_grad_(True) for h in (hq, hkv, hkv))
    o = ops.flash_attn_varlen(q, k, v, cu, max(lens))
    g = torch.randn_like(o)
    o.backward(g)
    # fp32 reference one document at a time (an 8192 x 8192 score matrix per head fits easily)
    for i, n in enumerate(lens):
        a, b = int(cu[i]), int(cu[i + 1])
        qr, kr, vr = (t.detach()[a:b].float().requires_grad_(True) for t in (q, k, v))
        one = torch.tensor([0, n], device='cuda', dtype=torch.int32)
        orf = ref.attention_varlen(qr, kr, vr, one)
        orf.backward(g[a:b].float())
        assert rel(o[a:b], orf) < 5e-3, i
        assert rel(q.grad[a:b], qr.grad) < 8e-3 and rel(k.grad[a:b], kr.grad) < 8e-3 and rel(v.grad[a:b], vr.grad) < 8e-3, i
    assert E.read_and_clear_error() == 0


def test_tiny_model_matches_cpu_reference(E):
    """Whole decoder layer stack on the GPU kernels vs the same weights in fp32 on CPU."""
    from twinkle_b200.models import PackedBatch, build_model, preset
    cfg = preset('qwen3-8b', num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                 num_key_value_heads=2, vocab_size=2048)
    ref_model = build_model(cfg, device='cpu', dtype=torch.float32, seed=3)
    gpu_model = build_model(cfg, device='cuda', dtype=torch.bfloat16, seed=3)
    with torch.no_grad():
        for (n, p), (_, pc) in zip(gpu_model.named_parameters(), ref_model.named_parameters()):
            p.copy_(pc)
            pc.copy_(p.float().cpu())
    g = torch.Generator().manual_seed(0)
    lens = [200, 120]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens), ), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])
    cu = torch.tensor([0, 200, 320], dtype=torch.int32)
    labels = torch.randint(0, cfg.vocab_size, (sum(lens), ), generator=g)

    def run(m, dev):
        b = PackedBatch(ids.to(dev), pos.to(dev), cu.to(dev), 200, labels.to(dev))
        h = m(b)
        lp, _ = m.token_logprobs(h, b.labels)
        loss = -lp.mean()
        loss.backward()
        return loss.detach().float().cpu(), m.layers[0].mlp.down_proj.weight.grad.float().cpu()

    lc, gc = run(ref_model, 'cpu')
    lg, gg = run(gpu_model, 'cuda')
    assert abs(float(lc) - float(lg)) < 2e-2, (lc, lg)
    assert rel(gg, gc) < 3e-2


def test_flash_attention_separate_key_ranges(E):
    """Queries of an entry attend to a longer key range of their own, causal diagonal aligned bottom-right
    (what context parallelism feeds the kernel): forward and all three gradients vs fp32."""
    from twinkle_b200 import ops
    torch.manual_seed(3)
    hq, hkv, d = 8, 2, 128
    q_lens, k_lens = [128, 200, 64, 300], [384, 200, 640, 428]
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device='cuda')
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device='cuda')
    q = torch.randn(sum(q_lens), hq, d, device='cuda').bfloat16().requires_grad_(True)
    k = torch.randn(sum(k_lens), hkv, d, device='cuda').bfloat16().requires_grad_(True)
    v = torch.randn(sum(k_lens), hkv, d, device='cuda').bfloat16().requires_grad_(True)
    o = ops.flash_attn_varlen(q, k, v, cu_q, max(q_lens), True, cu_seqlens_k=cu_k, max_seqlen_k=max(k_lens))
    g = torch.randn_like(o)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = ops.ref.attention_varlen(qr, kr, vr, cu_q, True, None, False, cu_k)
    orf.backward(g.float())
    assert rel(o, orf) < 6e-3
    assert rel(q.grad, qr.grad) < 1.5e-2 and rel(k.grad, kr.grad) < 1.5e-2 and rel(v.grad, vr.grad) < 1.5e-2


@pytest.mark.parametrize('layout', ['nt', 'nn', 'tn'])
def test_gemm_sm_pair_staged_epilogue(E, layout):
    """bf16 outputs written through the shared-memory staged epilogue equal the direct-store epilogue bit for bit."""
    M, N, K = 4000, 2504, 520
    torch.manual_seed(1)
    shapes = {'nt': ((M, K), (N, K)), 'nn': ((M, K), (K, N)), 'tn': ((K, M), (K, N))}[layout]
    a, b = (torch.randn(s, device='cuda').bfloat16() for s in shapes)
    staged = E.gemm(a, b, layout)          # default
    E.set_gemm_staged(0)
    try:
        direct = E.gemm(a, b, layout)
        torch.cuda.synchronize()
    finally:
        E.set_gemm_staged(1)
    assert torch.equal(direct, staged)


@pytest.mark.parametrize('sp,t', [(2, 600), (4, 256)])
def test_gemm_head_scatter_epilogue(E, sp, t):
    """q|k|v projection whose epilogue stores every 128-column block into the buffer of the rank owning those heads.
    The ranks of the group run one after another on this GPU with local buffers standing in for the peers' memory
    (the kernel waits on nothing), and are compared with an fp32 matmul sliced the same way."""
    K, qb, kb = 520, 2 * sp, sp                       # q blocks and kv blocks of 128 columns; N = (qb + 2 kb) * 128
    N = (qb + 2 * kb) * 128
    torch.manual_seed(2)
    w = (torch.randn(N, K, device='cuda') / K ** 0.5).bfloat16()
    xs = [torch.randn(t, K, device='cuda').bfloat16() for _ in range(sp)]
    bufs = [torch.full((sp * t, N // sp), float('nan'), device='cuda', dtype=torch.bfloat16) for _ in range(sp)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(sp):
        E.gemm_head_scatter(xs[r], w, ptrs, r, t, qb, kb)
    torch.cuda.synchronize()
    assert E.read_and_clear_error() == 0
    ql, kl = qb // sp * 128, kb // sp * 128
    for c in range(sp):
        rows = []
        for r in range(sp):
            y = xs[r].float() @ w.float().t()
            q, k, v = y[:, :qb * 128], y[:, qb * 128:(qb + kb) * 128], y[:, (qb + kb) * 128:]
            rows.append(torch.cat([q[:, c * ql:(c + 1) * ql], k[:, c * kl:(c + 1) * kl], v[:, c * kl:(c + 1) * kl]], -1))
        want = torch.cat(rows, 0)
        got = bufs[c].float()
        assert not torch.isnan(got).any(), 'a block was not written'
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), float((got - want).abs().max())


def test_ep_peer_kernels_refuse_out_of_range_indices(E):
    """The expert-parallel pull kernels turn every index into a peer address only after a range check: a position or a
    token outside the peers' buffers yields a zero row and ERR_BOUNDS in the error word, and while the word is set the
    kernels touch no peer memory at all.  One GPU stands in for the group (the 'peers' are local buffers)."""
    torch.manual_seed(0)
    H, T, n = 64, 16, 32
    x = torch.randn(T, H, device='cuda').bfloat16()
    tok = torch.randint(0, T, (n, ), device='cuda', dtype=torch.int32)
    src_rank = torch.zeros(8, dtype=torch.int32, device='cuda')
    src_pos = torch.arange(8, dtype=torch.int32, device='cuda')
    total = torch.tensor([8], dtype=torch.int32, device='cuda')
    good = E.ep_rows_gather([x.data_ptr()], [tok.data_ptr()], [], src_rank, src_pos, H, total, n, T)
    assert torch.equal(good, x[tok[:8].long()]) and E.read_and_clear_error() == 0
    # a token id beyond the activation buffer, a position beyond the token list, a rank beyond the group
    tok_bad = tok.clone()
    tok_bad[3] = T + 5
    pos_bad = src_pos.clone()
    pos_bad[5] = n + 7
    rank_bad = src_rank.clone()
    rank_bad[6] = 3
    out = E.ep_rows_gather([x.data_ptr()], [tok_bad.data_ptr()], [], rank_bad, pos_bad, H, total, n, T)
    torch.cuda.synchronize()
    for r in (3, 5, 6):
        assert float(out[r].float().abs().sum()) == 0.0
    for r in (0, 1, 2, 4, 7):
        assert torch.equal(out[r], x[tok[r].long()])
    # the word is still set here: the next launch must not read anything (the output is left as it was allocated)
    E.ep_rows_gather([x.data_ptr()], [tok.data_ptr()], [], src_rank, src_pos, H, total, n, T)
    assert E.read_and_clear_error() == 7
    # combine: a row past the peers' capacity is skipped and reported
    y = torch.randn(10, H, device='cuda').bfloat16()
    dst_rank = torch.zeros(4, 2, dtype=torch.int32, device='cuda')
    dst_row = torch.tensor([[0, 1], [2, 3], [4, 99], [5, 6]], dtype=torch.int32, device='cuda')
    w = torch.ones(4, 2, device='cuda')
    out = E.ep_rows_combine([y.data_ptr()], dst_rank, dst_row, w, H, 10)
    torch.cuda.synchronize()
    assert rel(out[2], y[4].float()) < 1e-2 and rel(out[0], (y[0].float() + y[1].float())) < 1e-2
    assert E.read_and_clear_error() == 7
    dw = E.ep_combine_wgrad(out.contiguous(), [y.data_ptr()], dst_rank, dst_row, 10)
    torch.cuda.synchronize()
    assert float(dw[2, 1]) == 0.0 and E.read_and_clear_error() == 7


def test_sharded_engine_training_matches_cpu(E):
    """Full-parameter training through the flat-bucket engine on the GPU kernels (bf16, weight gradients accumulated by the
    dW GEMM straight into the flat bucket, fp32 master + fused AdamW) against the same engine in fp32 on the CPU: loss curve
    and gradient norm over four steps."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('qwen3-8b', num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2,
                 vocab_size=4096)
    g = torch.Generator().manual_seed(7)
    feats = []
    for n in (257, 193, 301, 129):
        ids = torch.randint(0, cfg.vocab_size, (n, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(device):
        m = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0, device=device)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(4):
            o = m.forward_backward(inputs=feats, micro_batch_size=2)       # two micro-batches: gradients accumulate in the bucket
            n = m.clip_grad_and_step(max_grad_norm=1.0)
            out.append((float(o['loss']), float(n)))
        return out

    cpu, gpu = curve('cpu'), curve('cuda')
    assert cpu[0][0] > cpu[-1][0]
    for (a, na), (b, nb) in zip(cpu, gpu):
        assert abs(a - b) < 3e-2 and abs(na - nb) < 5e-2 * max(na, 1.0), (cpu, gpu)
    assert E.read_and_clear_error() == 0


def test_qwen3_5_stack_trains_on_gpu_like_on_cpu(E):
    """The Qwen3.5 text stack on the GPU (Gated DeltaNet kernels with 128-wide key heads, gated full attention with
    partial rotary on the PyTorch attention path, LoRA over the four-part q|k|v|gate projection) against fp32 on the CPU."""
    from twinkle_b200.model import MultiLoraTransformersModel, TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('tiny-qwen3.5', hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                 linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128, vocab_size=2048)
    g = torch.Generator().manual_seed(11)
    feats = []
    for n in (161, 97, 130):
        ids = torch.randint(0, cfg.vocab_size, (n, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(device):
        m = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0, device=device)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(3):
            o = m.forward_backward(inputs=feats, micro_batch_size=3)
            out.append((float(o['loss']), float(m.clip_grad_and_step(max_grad_norm=1.0))))
        return out

    cpu, gpu = curve('cpu'), curve('cuda')
    assert cpu[0][0] > cpu[-1][0]
    for (a, na), (b, nb) in zip(cpu, gpu):
        assert abs(a - b) < 4e-2 and abs(na - nb) < 8e-2 * max(na, 1.0), (cpu, gpu)

    def lora_curve(device):
        m = MultiLoraTransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0, device=device, max_loras=2, max_r=8)
        m.add_adapter_to_model('a', {'r': 8, 'lora_alpha': 16, 'target_modules': 'all-linear'})
        m.set_optimizer('AdamW', lr=5e-3, adapter_name='a')
        out = []
        for _ in range(3):
            o = m.forward_backward(inputs=feats, micro_batch_size=3, adapter_name='a')
            m.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
            out.append(float(o['loss']))
        return out

    lc, lg = lora_curve('cpu'), lora_curve('cuda')
    assert lc[-1] < lc[0]
    for a, b in zip(lc, lg):
        assert abs(a - b) < 4e-2, (lc, lg)
    assert E.read_and_clear_error() == 0


def test_gated_delta_rule_and_conv_kernels(E):
    """Linear-attention kernels against the fp32 recurrence / convolution on PyTorch: packed sequences (one of them a
    single token, one empty), grouped heads, both key widths, state hand-over to a second call, gradients through the
    autograd wrapper."""
    import torch.nn.functional as F
    from twinkle_b200 import ops
    from twinkle_b200.models.linear_attention import causal_conv1d_varlen_torch, gated_delta_rule_recurrent
    torch.manual_seed(0)
    for dk, dv, hk, hv in ((128, 128, 2, 4), (64, 96, 3, 3)):
        lens = [37, 1, 0, 150]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device='cuda')
        T = sum(lens)
        qkv = torch.randn(T, 2 * hk * dk + hv * dv, device='cuda').bfloat16()       # slices of one fused row, as the layer passes them
        q, k = qkv[:, :hk * dk].view(T, hk, dk), qkv[:, hk * dk:2 * hk * dk].view(T, hk, dk)
        v = qkv[:, 2 * hk * dk:].view(T, hv, dv)
        g = -torch.rand(T, hv, device='cuda') * 0.2
        beta = torch.rand(T, hv, device='cuda')
        o, fin = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu, return_states=True)
        assert fin.shape == (4, hv, dk, dv) and float(fin[2].abs().max()) == 0.0
        rep = hv // hk
        from twinkle_b200.models.linear_attention import l2norm
        qn = l2norm(q).repeat_interleave(rep, 1)
        kn = l2norm(k).repeat_interleave(rep, 1)
        b = cu.tolist()
        for i, (a_, b_) in enumerate(zip(b[:-1], b[1:])):
            if b_ == a_:
                continue
            o_r, s_r = gated_delta_rule_recurrent(qn[a_:b_], kn[a_:b_], v[a_:b_].float(), g[a_:b_], beta[a_:b_])
            assert rel(o[a_:b_], o_r) < 8e-3, (dk, i)
            assert rel(fin[i], s_r) < 2e-3, (dk, i)
        # continue sequence 3 in two calls: second call starts from the first one's state
        a_, b_ = b[3], b[4]
        mid = a_ + 70
        cu1 = torch.tensor([0, 70], dtype=torch.int32, device='cuda')
        cu2 = torch.tensor([0, b_ - mid], dtype=torch.int32, device='cuda')
        o1, s1 = ops.gated_delta_rule_varlen(q[a_:mid], k[a_:mid], v[a_:mid], g[a_:mid].contiguous(), beta[a_:mid].contiguous(), cu1,
                                             return_states=True)
        o2, s2 = ops.gated_delta_rule_varlen(q[mid:b_], k[mid:b_], v[mid:b_], g[mid:b_].contiguous(), beta[mid:b_].contiguous(), cu2,
                                             init_state=s1, return_states=True)
        assert rel(torch.cat([o1, o2]), o[a_:b_]) < 1e-3 and rel(s2[0], fin[3]) < 1e-5
    # gradients: kernel forward + PyTorch backward against the all-PyTorch fp32 function
    T, hk, hv, dk, dv = 96, 2, 2, 64, 64
    cu = torch.tensor([0, 40, 96], dtype=torch.int32, device='cuda')
    ins = [torch.randn(T, hk, dk, device='cuda').bfloat16(), torch.randn(T, hk, dk, device='cuda').bfloat16(),
           torch.randn(T, hv, dv, device='cuda').bfloat16(), -torch.rand(T, hv, device='cuda') * 0.2, torch.rand(T, hv, device='cuda')]
    a = [t.clone().requires_grad_(True) for t in ins]
    o = ops.gated_delta_rule_varlen(*a, cu)
    go = torch.randn_like(o)
    o.backward(go)
    from twinkle_b200.models.linear_attention import gated_delta_rule_varlen_torch
    r = [t.float().clone().requires_grad_(True) for t in ins]
    o_ref = gated_delta_rule_varlen_torch(*r, cu.cpu(), None, chunk=32)
    o_ref.backward(go.float())
    assert rel(o, o_ref) < 8e-3
    for x_, y_ in zip(a, r):
        assert rel(x_.grad, y_.grad) < 2e-2
    # convolution + SiLU, window never crossing a boundary; input is a column slice of a wider row
    C, W = 256, 4
    wide = torch.randn(T, C + 64, device='cuda').bfloat16()
    x = wide[:, :C].requires_grad_(False)
    w = (torch.randn(C, W, device='cuda') * 0.5).bfloat16()
    for act in (True, False):
        y = ops.causal_conv1d_varlen(x, w, cu, act)
        y_ref = causal_conv1d_varlen_torch(x.float(), w.float(), cu, act)
        assert rel(y, y_ref) < 6e-3
    xg = x.clone().contiguous().requires_grad_(True)
    wg = w.clone().requires_grad_(True)
    ops.causal_conv1d_varlen(xg, wg, cu, True).backward(torch.ones(T, C, device='cuda').bfloat16())
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    causal_conv1d_varlen_torch(xr, wr, cu, True).sum().backward()
    assert rel(xg.grad, xr.grad) < 1e-2 and rel(wg.grad, wr.grad) < 1e-2


def test_latent_attention_and_windowed_stacks_train_on_gpu_like_on_cpu(E):
    """Two of the families that leave the plain Llama computation, in bf16 on the GPU against fp32 on the CPU: a DeepSeek-V3
    shaped stack (latent attention with 128-wide score and value heads, so it runs the flash kernels; sigmoid group-limited
    routing feeding the grouped expert GEMMs; frozen selection bias beside trained tensors) and a Gemma-2 shaped one (rows longer
    than the attention window, capped scores and logits, GeGLU kernel, scaled embeddings, four norms per layer)."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    deepseek = preset('tiny-deepseek', hidden_size=512, intermediate_size=1024, q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=64,
                      qk_rope_head_dim=64, v_head_dim=128, head_dim=128, moe_intermediate_size=256, shared_expert_intermediate_size=256, vocab_size=2048)
    gemma = preset('tiny-dense', model_type='gemma2', hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=128, vocab_size=2048, sliding_window=64, qk_norm=False,
                   layer_types=['sliding_attention', 'full_attention', 'sliding_attention', 'full_attention'], sandwich_norm=True, rms_norm_offset=1.0,
                   hidden_act='gelu_pytorch_tanh', embed_scale=512**0.5, query_pre_attn_scalar=128.0, attn_logit_softcapping=50.0,
                   final_logit_softcapping=30.0)
    g = torch.Generator().manual_seed(11)
    feats = []
    for n in (161, 97, 130):
        ids = torch.randint(0, 2048, (n, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(cfg, device):
        m = TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0, device=device)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(3):
            o = m.forward_backward(inputs=feats, micro_batch_size=3)
            m.clip_grad_and_step(max_grad_norm=1.0)
            out.append(float(o['loss']))
        return out

    for cfg in (deepseek, gemma):
        cpu, gpu = curve(cfg, 'cpu'), curve(cfg, 'cuda')
        assert cpu[0] > cpu[-1] and gpu[0] > gpu[-1], (cpu, gpu)
        for a, b in zip(cpu, gpu):
            assert abs(a - b) < 8e-2, (cfg.model_type, cpu, gpu)
    assert E.read_and_clear_error() == 0
