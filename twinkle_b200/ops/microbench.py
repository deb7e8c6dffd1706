"""Kernel micro-benchmarks: ``python -m twinkle_b200.ops.microbench --op gemm --m 8192 --n 4096 --k 4096``.

Each op is timed with CUDA events on the launching stream after warm-up, with a write over a buffer larger
than L2 between iterations, and reported as achieved TFLOP/s or GB/s next to the fraction of the measured
device peaks (``MEASURED_PEAKS.json`` at the repository root when present; the stated fallback otherwise).
``--iters 1 --warmup 0 --no-flush`` gives a minimal launch sequence suitable for a profiler capture of one kernel.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Dict, Tuple

import torch


def peaks() -> Dict[str, float]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d['hbm_gbs']), tflops=float(d['bf16_tflops']), source='measured')
    return dict(hbm_gbs=6650.0, tflops=1590.0, source='fallback')


def time_op(fn: Callable[[], None], iters: int, warmup: int, flush: bool) -> float:
    """Median milliseconds per call."""
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def make(op: str, a) -> Tuple[Callable[[], None], float, float]:
    """(callable, flops, algorithmic bytes)."""
    from twinkle_b200 import ops
    E = ops.ext()
    dev = 'cuda'
    bf = torch.bfloat16
    if op == 'gemm':
        M, N, K = a.m, a.n, a.k
        shapes = {'nt': ((M, K), (N, K)), 'nn': ((M, K), (K, N)), 'tn': ((K, M), (K, N))}[a.layout]
        x, w = (torch.randn(s, device=dev, dtype=bf) for s in shapes)
        return (lambda: E.gemm(x, w, a.layout)), 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    if op == 'torch_gemm':
        x, w = torch.randn(a.m, a.k, device=dev, dtype=bf), torch.randn(a.n, a.k, device=dev, dtype=bf)
        return (lambda: torch.nn.functional.linear(x, w)), 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    if op in ('attn_fwd', 'attn_bwd'):
        T, hq, hkv, d = a.tokens, a.heads, a.kv_heads, 128
        n_seq = max(T // a.seq, 1)
        cu = torch.arange(0, n_seq + 1, device=dev, dtype=torch.int32) * a.seq
        q = torch.randn(T, hq, d, device=dev, dtype=bf, requires_grad=True)
        k = torch.randn(T, hkv, d, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(T, hkv, d, device=dev, dtype=bf, requires_grad=True)
        flops_fwd = 4.0 * n_seq * a.seq * a.seq * hq * d / 2  # causal
        byts = 2.0 * (2 * T * hq * d + 2 * T * hkv * d)
        if op == 'attn_fwd':
            def f():
                with torch.no_grad():
                    ops.flash_attn_varlen(q, k, v, cu, a.seq, True)
            return f, flops_fwd, byts
        o = ops.flash_attn_varlen(q, k, v, cu, a.seq, True)
        g = torch.randn_like(o)
        return (lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True)), 2.5 * flops_fwd, 2.5 * byts
    if op in ('rope', 'rope_bwd'):
        T, hq, hkv = a.tokens, a.heads, a.kv_heads
        qkv = torch.randn(T, (hq + 2 * hkv) * 128, device=dev, dtype=bf)
        qw, kw = torch.ones(128, device=dev, dtype=bf), torch.ones(128, device=dev, dtype=bf)
        pos = torch.arange(T, device=dev) % 8192
        cos, sin = ops.rope_tables(pos, 128, 1e6)
        byts = 2.0 * 2 * T * (hq + 2 * hkv) * 128
        if op == 'rope':
            return (lambda: E.qk_norm_rope_fwd(qkv, qw, kw, cos, sin, hq, hkv, 128, 1e-6)), 0.0, byts
        q, k, v, rstd = E.qk_norm_rope_fwd(qkv, qw, kw, cos, sin, hq, hkv, 128, 1e-6)
        gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
        return (lambda: E.qk_norm_rope_bwd(gq, gk, gv, qkv, qw, kw, cos, sin, rstd, hq, hkv, 128)), 0.0, 1.5 * byts
    if op == 'rmsnorm':
        x, w = torch.randn(a.tokens, a.hidden, device=dev, dtype=bf), torch.ones(a.hidden, device=dev, dtype=bf)

        def f():
            with torch.no_grad():
                ops.rmsnorm(x, w, 1e-6)
        return f, 0.0, 4.0 * a.tokens * a.hidden
    if op == 'rmsnorm_bwd':
        x, w = torch.randn(a.tokens, a.hidden, device=dev, dtype=bf), torch.ones(a.hidden, device=dev, dtype=bf)
        g = torch.randn_like(x)
        _, rstd = E.rmsnorm_fwd(x, w, 1e-6, 0.0)
        return (lambda: E.rmsnorm_bwd(g, x, w, rstd, 0.0)), 0.0, 6.0 * a.tokens * a.hidden
    if op == 'swiglu':
        gu = torch.randn(a.tokens, 2 * a.hidden, device=dev, dtype=bf)

        def f():
            with torch.no_grad():
                ops.swiglu(gu)
        return f, 0.0, 6.0 * a.tokens * a.hidden
    if op == 'logprob':
        x = torch.randn(a.tokens, a.vocab, device=dev, dtype=bf)
        y = torch.randint(0, a.vocab, (a.tokens, ), device=dev)

        def f():
            with torch.no_grad():
                ops.logprob_from_logits(x, y)
        return f, 0.0, 2.0 * a.tokens * a.vocab
    if op == 'adamw':
        n = a.numel
        p, g = torch.randn(n, device=dev), torch.randn(n, device=dev, dtype=bf)
        m, v, lo = torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.empty(n, device=dev, dtype=bf)
        return (lambda: ops.adamw_step(p, m, v, g, lo, 1e-4, 0.9, 0.95, 1e-8, 0.01, 1, 1.0)), 0.0, float(n) * (4 * 3 * 2 + 2 + 2)
    if op == 'sgmv':
        # four tenants share the batch: equal token segments, each on its own adapter slot (rank a.rank of a pool of 16)
        T, H, N, r = a.tokens, a.hidden, a.n, a.rank
        x = torch.randn(T, H, device=dev, dtype=bf)
        A = torch.randn(4, 16, H, device=dev, dtype=bf) * 0.02
        B = torch.randn(4, N, 16, device=dev, dtype=bf) * 0.02
        cuts = [T * i // 4 for i in range(5)]
        host = [(cuts[i], cuts[i + 1], i, r, 2.0) for i in range(4)]
        st = torch.tensor(cuts, dtype=torch.int32, device=dev)
        sl = torch.arange(4, dtype=torch.int32, device=dev)
        rk = torch.full((4, ), r, dtype=torch.int32, device=dev)
        sc = torch.full((4, ), 2.0, dtype=torch.float32, device=dev)

        def f():
            with torch.no_grad():
                ops.sgmv(x, A, B, st, sl, rk, sc, host)
        return f, 2.0 * T * r * (H + N), 2.0 * T * (H + N)
    if op == 'paged_decode':
        B, bs, ctx = a.batch, 16, a.seq
        nb = B * ((ctx + bs - 1) // bs)
        kc = torch.randn(nb, bs, a.kv_heads, 128, device=dev, dtype=bf)
        vc = torch.randn_like(kc)
        tables = torch.arange(nb, device=dev, dtype=torch.int32).view(B, -1)
        lens = torch.full((B, ), ctx, device=dev, dtype=torch.int32)
        q = torch.randn(B, a.heads, 128, device=dev, dtype=bf)
        return (lambda: ops.paged_attention_decode(q, kc, vc, tables, lens)), 0.0, 2.0 * 2 * B * ctx * a.kv_heads * 128
    if op == 'sample':
        lg = torch.randn(a.batch, a.vocab, device=dev)
        seeds = torch.arange(a.batch, device=dev, dtype=torch.int64)
        return (lambda: ops.sample_tokens(lg, 0.8, 50, 0.95, seeds=seeds)), 0.0, 4.0 * a.batch * a.vocab
    if op in ('expert_lora', 'expert_lora_split', 'expert_base'):
        # one expert projection of the Qwen3-30B-A3B block: rows = tokens x top-8 over 128 experts (128-row aligned
        # segments), 2048 -> 1536, rank-16 LoRA pair per expert.  expert_base: the grouped GEMM alone; expert_lora: the
        # low-rank term as a second operand pair of the same GEMM; expert_lora_split: shrink, base, then a separate
        # rank-16 GEMM accumulating into the output
        Eg, K, N, r = 128, 2048, 1536, 16
        per = (a.tokens * 8 // Eg + 127) // 128 * 128
        rows = per * Eg
        off = torch.arange(0, Eg + 1, device=dev, dtype=torch.int32) * per
        x = torch.randn(rows, K, device=dev, dtype=bf)
        w = torch.randn(Eg, N, K, device=dev, dtype=bf) * 0.02
        la = torch.randn(Eg, r, K, device=dev, dtype=bf) * 0.02
        lb = torch.randn(Eg, N, r, device=dev, dtype=bf) * 0.02
        flops = 2.0 * rows * K * N + (0.0 if op == 'expert_base' else 2.0 * rows * r * (K + N))
        byts = 2.0 * (rows * K + rows * N + Eg * N * K)
        if op == 'expert_base':
            return (lambda: E.grouped_gemm(x, w, off, 'nt', None)), flops, byts
        if op == 'expert_lora':
            def f():
                h = E.grouped_gemm(x, la, off, 'nt', None)
                E.grouped_gemm(x, w, off, 'nt', None, None, False, h, lb)
            return f, flops, byts

        def f2():
            y = E.grouped_gemm(x, w, off, 'nt', None)
            h = E.grouped_gemm(x, la, off, 'nt', None)
            E.grouped_gemm(h, lb, off, 'nt', None, y, True)
        return f2, flops, byts
    if op in ('gdn', 'gdn_torch'):
        # Gated DeltaNet forward: 16 key / 32 value heads of 128, packed documents of --seq tokens
        T, hk, hv, d = a.tokens, 16, 32, 128
        n_seq = max(T // a.seq, 1)
        cu = torch.arange(0, n_seq + 1, device=dev, dtype=torch.int32) * a.seq
        q, k = torch.randn(T, hk, d, device=dev, dtype=bf), torch.randn(T, hk, d, device=dev, dtype=bf)
        v = torch.randn(T, hv, d, device=dev, dtype=bf)
        g, beta = -torch.rand(T, hv, device=dev) * 0.1, torch.rand(T, hv, device=dev)
        byts = 2.0 * T * d * (2 * hk + 2 * hv) + 8.0 * T * hv
        flops = 2.0 * T * hv * d * d * 3            # S·k, S·q and the rank-1 update
        if op == 'gdn':
            def f():
                with torch.no_grad():
                    ops.gated_delta_rule_varlen(q, k, v, g, beta, cu)
        else:
            from twinkle_b200.models.linear_attention import gated_delta_rule_varlen_torch

            def f():
                with torch.no_grad():
                    gated_delta_rule_varlen_torch(q, k, v, g, beta, cu)
        return f, flops, byts
    if op == 'router':
        lg = torch.randn(a.tokens, 128, device=dev, dtype=bf)

        def f():
            with torch.no_grad():
                ops.moe_router(lg, 8, True)
        return f, 0.0, a.tokens * 128 * (2 + 4) + a.tokens * 8 * 12
    raise SystemExit(f'unknown op {op}')


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--op', required=True)
    ap.add_argument('--m', type=int, default=8192)
    ap.add_argument('--n', type=int, default=4096)
    ap.add_argument('--k', type=int, default=4096)
    ap.add_argument('--layout', default='nt')
    ap.add_argument('--tokens', type=int, default=32768)
    ap.add_argument('--seq', type=int, default=8192)
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--kv-heads', type=int, default=8)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--vocab', type=int, default=151936)
    ap.add_argument('--batch', type=int, default=256)
    ap.add_argument('--rank', type=int, default=16)
    ap.add_argument('--numel', type=int, default=1 << 28)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--no-flush', action='store_true')
    ap.add_argument('--staged', type=int, default=None, help='1: staged epilogue of the SM-pair GEMM (bf16 outputs)')
    ap.add_argument('--pair', type=int, default=None, help='1: SM-pair GEMM kernel, 0: single-CTA tiles (default: library setting)')
    a = ap.parse_args()
    torch.manual_seed(0)
    if a.staged is not None:
        from twinkle_b200 import ops as _ops2
        _ops2.ext().set_gemm_staged(a.staged)
    if a.pair is not None:
        from twinkle_b200 import ops as _ops
        _ops.ext().set_gemm_pair(a.pair)
    fn, flops, byts = make(a.op, a)
    ms = time_op(fn, a.iters, a.warmup, not a.no_flush)
    pk = peaks()
    from twinkle_b200 import ops
    err = ops.ext().read_and_clear_error()
    out = dict(op=a.op, ms=round(ms, 4), error_word=err, peaks=pk['source'])
    if flops:
        out['tflops'] = round(flops / ms / 1e9, 1)
        out['frac_of_gemm_peak'] = round(flops / ms / 1e9 / pk['tflops'], 3)
    out['gbs'] = round(byts / ms / 1e6, 1)
    out['frac_of_hbm_peak'] = round(byts / ms / 1e6 / pk['hbm_gbs'], 3)
    out['args'] = {k: v for k, v in vars(a).items() if k != 'op'}
    print(json.dumps(out))


if __name__ == '__main__':
    main()
