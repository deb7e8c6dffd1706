"""GPU numerics of the multi-LoRA, sampler and router kernels against their fp32 PyTorch restatements, plus the
native sampler and a LoRA training step end to end on the device."""
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
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _tiny():
    from twinkle_b200.models import preset
    return preset('qwen3-8b', num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                  num_key_value_heads=2, vocab_size=1024)


def test_grouped_gemm_group_map(E):
    torch.manual_seed(1)
    G, N, K = 5, 96, 256
    w = (torch.randn(G, N, K, device='cuda') * 0.1).bfloat16()
    lens = [130, 0, 257, 64, 33]
    gmap = [3, 0, 1, 4, 3]  # segment i multiplies by weight gmap[i]; a weight may serve two segments
    off = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device='cuda')
    x = torch.randn(sum(lens), K, device='cuda').bfloat16()
    y = E.grouped_gemm(x, w, off, 'nt', torch.tensor(gmap, dtype=torch.int32, device='cuda'))
    lo = 0
    for n, g in zip(lens, gmap):
        if n:
            assert rel(y[lo:lo + n], x[lo:lo + n].float() @ w[g].float().t()) < 4e-3
        lo += n


@pytest.mark.parametrize('T', [777, 4096, 40000])     # 40000: segments long enough for the split-K weight gradients
def test_sgmv_forward_backward(E, T):
    from twinkle_b200 import ops
    torch.manual_seed(2)
    S, R, K, N = 4, 32, 512, 384
    a = (torch.randn(S, R, K, device='cuda') * 0.05).bfloat16().requires_grad_(True)
    b = (torch.randn(S, N, R, device='cuda') * 0.05).bfloat16().requires_grad_(True)
    cuts = sorted({0, T} | {int(v) for v in torch.randint(1, T, (4, ))})
    nseg = len(cuts) - 1
    slots = [2, -1, 0, 2, 3][:nseg]
    ranks = [32, 0, 8, 32, 16][:nseg]
    scales = [2.0, 0.0, 0.5, 2.0, 1.0][:nseg]
    dev = dict(device='cuda')
    st = torch.tensor(cuts, dtype=torch.int32, **dev)
    sl = torch.tensor(slots, dtype=torch.int32, **dev)
    rk = torch.tensor(ranks, dtype=torch.int32, **dev)
    sc = torch.tensor(scales, dtype=torch.float32, **dev)
    x = torch.randn(T, K, device='cuda').bfloat16().requires_grad_(True)
    y = ops.sgmv(x, a, b, st, sl, rk, sc)
    g = torch.randn_like(y)
    y.backward(g)

    xr, ar, br = (t.detach().float().requires_grad_(True) for t in (x, a, b))
    yr = ops._sgmv_autograd_cpu(xr, ar, br, st, sl, rk, sc)
    yr.backward(g.float())
    assert rel(y, yr) < 6e-3
    assert rel(x.grad, xr.grad) < 8e-3
    assert rel(a.grad, ar.grad) < 8e-3
    assert rel(b.grad, br.grad) < 8e-3
    # rows of slots nobody used and rank rows beyond a segment's rank get no gradient
    assert float(a.grad[1].abs().max()) == 0.0 and float(b.grad[1].abs().max()) == 0.0


def test_sgmv_into_base_output_with_rank_stacked_pools(E):
    """The form the fused q|k|v projection uses: pools of two projections stacked along the rank axis (block-diagonal
    ``B``), the delta accumulated into the base output in place; against base + per-projection deltas in fp32."""
    import torch.nn.functional as F
    from twinkle_b200 import ops
    torch.manual_seed(5)
    T, S, R, K, n1, n2 = 1500, 3, 16, 256, 384, 128
    a1, a2 = ((torch.randn(S, R, K, device='cuda') * 0.05).bfloat16().requires_grad_(True) for _ in range(2))
    b1 = (torch.randn(S, n1, R, device='cuda') * 0.05).bfloat16().requires_grad_(True)
    b2 = (torch.randn(S, n2, R, device='cuda') * 0.05).bfloat16().requires_grad_(True)
    cuts, slots, ranks, scales = [0, 400, 900, T], [1, -1, 2], [16, 0, 8], [2.0, 0.0, 0.5]
    st = torch.tensor(cuts, dtype=torch.int32, device='cuda')
    sl = torch.tensor(slots, dtype=torch.int32, device='cuda')
    rk = torch.tensor(ranks, dtype=torch.int32, device='cuda')
    sc = torch.tensor(scales, dtype=torch.float32, device='cuda')
    host = [(cuts[i], cuts[i + 1], slots[i], ranks[i], scales[i]) for i in range(3)]
    x = torch.randn(T, K, device='cuda').bfloat16().requires_grad_(True)
    base = torch.randn(T, n1 + n2, device='cuda').bfloat16().requires_grad_(True)
    y0 = base * 1.0                                            # a non-leaf, as the projection's output is
    a = torch.cat([a1, a2], 1)
    b = torch.cat([F.pad(b1, (0, R)), F.pad(b2, (R, 0))], 1)
    y = ops.sgmv(x, a, b, st, sl, rk, sc, host, out=y0, repeat=2)
    assert y.data_ptr() == y0.data_ptr()
    g = torch.randn_like(y)
    y.backward(g)
    xr, a1r, a2r, b1r, b2r, baser = (t.detach().float().requires_grad_(True) for t in (x, a1, a2, b1, b2, base))
    yr = baser + torch.cat([ops._sgmv_autograd_cpu(xr, a1r, b1r, st, sl, rk, sc), ops._sgmv_autograd_cpu(xr, a2r, b2r, st, sl, rk, sc)], 1)
    yr.backward(g.float())
    assert rel(y, yr) < 6e-3 and rel(base.grad, baser.grad) == 0.0
    for got, want in ((x.grad, xr.grad), (a1.grad, a1r.grad), (a2.grad, a2r.grad), (b1.grad, b1r.grad), (b2.grad, b2r.grad)):
        assert rel(got, want) < 8e-3
    assert torch.equal(y[400:900], base.detach()[400:900])      # the segment without an adapter keeps the base rows


def test_paged_decode(E):
    from twinkle_b200 import ops
    torch.manual_seed(3)
    B, Hq, Hkv, D, bs, nblocks = 5, 16, 4, 128, 16, 64
    kc = torch.randn(nblocks, bs, Hkv, D, device='cuda').bfloat16()
    vc = torch.randn(nblocks, bs, Hkv, D, device='cuda').bfloat16()
    lens = torch.tensor([1, 17, 160, 33, 200], dtype=torch.int32, device='cuda')
    perm = torch.randperm(nblocks, device='cuda').int()
    tables = torch.zeros(B, 13, dtype=torch.int32, device='cuda')
    used = 0
    for i in range(B):
        nb = (int(lens[i]) + bs - 1) // bs
        tables[i, :nb] = perm[used:used + nb]
        used += nb
    q = torch.randn(B, Hq, D, device='cuda').bfloat16()
    o = ops.paged_attention_decode(q, kc, vc, tables, lens)
    r = ops.ref.paged_attention_decode(q, kc, vc, tables, lens)
    assert rel(o, r) < 6e-3


def test_router(E):
    from twinkle_b200 import ops
    torch.manual_seed(4)
    for (T, Ex, k, renorm) in [(1000, 128, 8, True), (257, 8, 2, False), (64, 64, 6, True)]:
        lg = torch.randn(T, Ex, device='cuda').bfloat16().requires_grad_(True)
        w, idx, probs, hist = ops.moe_router(lg, k, renorm)
        lr = lg.detach().float().requires_grad_(True)
        wr, ir, pr = ops.ref.moe_router(lr, k, renorm)
        assert torch.equal(idx.sort(-1).values, ir.sort(-1).values)
        order, order_r = idx.argsort(-1), ir.argsort(-1)
        assert torch.allclose(w.gather(-1, order), wr.gather(-1, order_r), atol=1e-5, rtol=1e-4)
        assert torch.allclose(probs, pr, atol=1e-6, rtol=1e-4)
        assert torch.equal(hist.long(), torch.bincount(ir.flatten(), minlength=Ex))
        gw, gp = torch.randn_like(w), torch.randn_like(probs)
        ((w.gather(-1, order) * gw).sum() + (probs * gp).sum()).backward()
        ((wr.gather(-1, order_r) * gw).sum() + (pr * gp).sum()).backward()
        assert rel(lg.grad, lr.grad) < 1e-2  # bf16 gradient storage


def test_sampling(E):
    from twinkle_b200 import ops
    torch.manual_seed(5)
    B, V = 64, 50000
    lg = torch.randn(B, V, device='cuda') * 3
    seeds = torch.arange(B, device='cuda', dtype=torch.int64) + 11
    # greedy
    tok, lp = ops.sample_tokens(lg, 0.0, -1, 1.0, seeds=seeds)
    assert torch.equal(tok, lg.argmax(-1))
    # top-k: every draw inside the k largest, log-prob renormalised over them
    k = 20
    tok, lp = ops.sample_tokens(lg, 0.8, k, 1.0, seeds=seeds)
    topv, topi = (lg / 0.8).topk(k, -1)
    assert bool((topi == tok[:, None]).any(-1).all())
    want = torch.log_softmax(topv, -1).gather(-1, (topi == tok[:, None]).float().argmax(-1, keepdim=True)).squeeze(-1)
    assert torch.allclose(lp, want, atol=2e-3)
    # same seeds → same tokens; other seeds → some differ
    tok2, _ = ops.sample_tokens(lg, 0.8, k, 1.0, seeds=seeds)
    tok3, _ = ops.sample_tokens(lg, 0.8, k, 1.0, seeds=seeds + 1000)
    assert torch.equal(tok, tok2) and not torch.equal(tok, tok3)
    # top-p: draws stay inside the nucleus
    p = 0.5
    tok, lp = ops.sample_tokens(lg, 1.0, -1, p, seeds=seeds)
    probs = torch.softmax(lg, -1)
    sp, si = probs.sort(-1, descending=True)
    inside = (sp.cumsum(-1) - sp) < p
    nucleus = torch.zeros_like(probs, dtype=torch.bool).scatter(-1, si, inside)
    assert bool(nucleus.gather(-1, tok[:, None]).all())
    # the empirical distribution of one row follows softmax (chi-square-free check on the top entries)
    row = torch.randn(1, 32, device='cuda') * 2
    n = 20000
    draws, _ = ops.sample_tokens(row.expand(n, -1).contiguous(), 1.0, -1, 1.0, seeds=torch.arange(n, device='cuda', dtype=torch.int64))
    freq = torch.bincount(draws, minlength=32).float() / n
    assert float((freq - torch.softmax(row[0], -1)).abs().max()) < 0.015


def test_sampler_greedy_matches_full_forward(E):
    """Greedy decode through the paged-KV engine equals argmax of a full-sequence forward at every step."""
    from twinkle_b200.models import build_model, preset
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.sampler.engine import NativeEngine
    torch.manual_seed(6)
    cfg = _tiny()
    model = build_model(cfg, device='cuda', dtype=torch.bfloat16, seed=0)
    eng = NativeEngine(model, cfg, num_blocks=64, block_size=16)
    prompts = [[5, 9, 33, 2, 17], [7, 7, 100, 42, 3, 1, 250, 11, 90]]
    outs = eng.generate(prompts, [SamplingParams(max_tokens=6, temperature=0.0) for _ in prompts])
    for prompt, resp in zip(prompts, outs):
        toks = list(prompt)
        for t in resp.sequences[0].tokens:
            n = len(toks)
            batch = PackedBatch(torch.tensor(toks, device='cuda'), torch.arange(n, device='cuda'),
                                torch.tensor([0, n], dtype=torch.int32, device='cuda'), n)
            with torch.no_grad():
                logits = model.logits(model(batch))[-1].float()
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 0.05:  # ties within bf16 noise may legitimately flip
                assert int(logits.argmax()) == t
            toks.append(t)


def test_lora_training_step_on_gpu(E):
    """Two tenants, different ranks, one fused step each: losses fall and the base weights stay untouched."""
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    torch.manual_seed(7)
    m = MultiLoraTransformersModel(config=_tiny(), device='cuda', max_loras=3, max_r=16)
    base = {k: v.detach().clone() for k, v in m.model.named_parameters() if 'lora' not in k}
    for name, r in (('a', 8), ('b', 16)):
        m.add_adapter_to_model(name, LoraConfig(r=r, lora_alpha=2 * r, target_modules='all-linear'))
        m.set_optimizer('AdamW', lr=5e-3, adapter_name=name)
    g = torch.Generator().manual_seed(0)
    feats = []
    for _ in range(4):
        ids = torch.randint(0, 256, (49, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    first, last = {}, {}
    for it in range(6):
        for name in ('a', 'b'):
            out = m.forward_backward(inputs=feats, adapter_name=name)
            m.clip_grad_and_step(adapter_name=name)
            (first if it == 0 else last)[name] = float(out['loss'])
    for name in ('a', 'b'):
        assert last[name] < first[name] - 0.05, (name, first, last)
    for k, v in m.model.named_parameters():
        if 'lora' not in k:
            assert torch.equal(v, base[k]), k


def _tiny_moe():
    from twinkle_b200.models import preset
    return preset('qwen3-30b-a3b', num_hidden_layers=2, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                  vocab_size=1024, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256)


def test_moe_model_matches_cpu_reference(E):
    """Router kernel + 128-aligned expert layout + grouped tcgen05 GEMMs (fwd, dgrad, per-expert wgrad) vs fp32 CPU."""
    from twinkle_b200.models import PackedBatch, build_model
    cfg = _tiny_moe()
    ref_model = build_model(cfg, device='cpu', dtype=torch.float32, seed=5)
    gpu_model = build_model(cfg, device='cuda', dtype=torch.bfloat16, seed=5)
    with torch.no_grad():
        for (_, p), (_, pc) in zip(gpu_model.named_parameters(), ref_model.named_parameters()):
            p.copy_(pc)
            pc.copy_(p.float().cpu())
    g = torch.Generator().manual_seed(0)
    lens = [150, 106]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens), ), generator=g)
    labels = torch.randint(0, cfg.vocab_size, (sum(lens), ), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])
    cu = torch.tensor([0, 150, 256], dtype=torch.int32)
    # pin the routing to the CPU model's choice so a bf16 near-tie in the router cannot send a token elsewhere
    ref_model.set_record_routing(True)

    def run(m, dev, routed=None):
        b = PackedBatch(ids.to(dev), pos.to(dev), cu.to(dev), 150, labels.to(dev), routed_experts=routed)
        h = m(b)
        lp, _ = m.token_logprobs(h, b.labels)
        loss = -lp.mean()
        loss.backward()
        ex = m.layers[1].mlp.experts
        return float(loss), ex.down_proj.grad.float().cpu(), ex.gate_up_proj.grad.float().cpu(), m.layers[0].mlp.gate.weight.grad.float().cpu()

    lc, gdc, gguc, ggc = run(ref_model, 'cpu')
    routed = [r.to('cuda') for r in ref_model.collect_routed_experts()]
    lg, gdg, ggug, ggg = run(gpu_model, 'cuda', routed)
    assert abs(lc - lg) < 3e-2, (lc, lg)
    assert rel(gdg, gdc) < 4e-2 and rel(ggug, gguc) < 4e-2 and rel(ggg, ggc) < 6e-2


def test_moe_expert_lora_trains_on_gpu(E):
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    torch.manual_seed(9)
    m = MultiLoraTransformersModel(config=_tiny_moe(), device='cuda', max_loras=2, max_r=16)
    m.add_adapter_to_model('t', LoraConfig(r=16, lora_alpha=32, target_modules='all-linear'))
    m.set_optimizer('AdamW', lr=5e-3, adapter_name='t')
    g = torch.Generator().manual_seed(0)
    feats = []
    for _ in range(4):
        ids = torch.randint(0, 256, (65, ), generator=g)
        feats.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    losses = []
    for _ in range(6):
        out = m.forward_backward(inputs=feats, adapter_name='t')
        m.clip_grad_and_step(adapter_name='t')
        losses.append(float(out['loss']))
    assert losses[-1] < losses[0] - 0.05, losses
    ex = m.model.layers[0].mlp.experts
    assert float(ex.lora['down_B'][0].abs().max()) > 0  # the expert adapters actually moved


def test_decode_cuda_graph_matches_eager(E):
    """The captured decode step (bucketed batch, static inputs) generates the same greedy tokens and log-probs as the
    eager step, across a batch that shrinks as sequences finish."""
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.models import build_model
    from twinkle_b200.sampler.engine import NativeEngine
    cfg = _tiny()
    model = build_model(cfg, device='cuda', dtype=torch.bfloat16, seed=0)
    prompts = [[5, 9, 33, 2, 17], [7, 7, 100, 42, 3, 1, 250, 11, 90], [1, 2, 3]]
    params = [SamplingParams(max_tokens=n, temperature=0.0, logprobs=1) for n in (20, 7, 12)]  # crosses a 16-token block boundary
    outs = {}
    for graphs in (True, False):
        eng = NativeEngine(model, cfg, num_blocks=64, block_size=16)
        eng.use_cuda_graphs = graphs
        res = eng.generate(prompts, params)
        outs[graphs] = [(r.sequences[0].tokens, r.sequences[0].logprobs) for r in res]
        assert bool(eng._graphs) == graphs
    for (t1, l1), (t0, l0) in zip(outs[True], outs[False]):
        assert t1 == t0
        assert max(abs(a - b) for a, b in zip(l1, l0)) < 1e-3
