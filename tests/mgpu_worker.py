"""Multi-GPU checks, run under torchrun (one rank per GPU).  Prints one JSON line per check on rank 0 and
exits non-zero on the first failure.  Launched by tests/test_multigpu.py."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def ep_checks(rank, world, dev, report):
    """Expert parallel over all ranks (NCCL all-to-all and peer-memory pulls) vs the single-GPU curve."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('qwen3-30b-a3b', num_hidden_layers=2, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                 vocab_size=1024, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, router_aux_loss_coef=0.0)
    g = torch.Generator().manual_seed(11)
    feats = []
    for _ in range(2 * world):
        ids = torch.randint(0, cfg.vocab_size, (129, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(mesh, backend, my_feats):
        m = TransformersModel(config=cfg, device_mesh=mesh, seed=0, comm_backend=backend, device=dev)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(4):
            o = m.forward_backward(inputs=my_feats)
            m.clip_grad_and_step(max_grad_norm=1.0)
            t = torch.tensor([o['loss'] * o['num_tokens'], o['num_tokens']], device=dev, dtype=torch.float64)
            if mesh.world_size > 1:
                dist.all_reduce(t)
            out.append(float(t[0] / t[1]))
        return out

    single = [curve(DeviceMesh.from_sizes(dp_size=1), 'nccl', feats) if rank == 0 else None]
    dist.broadcast_object_list(single, src=0)
    single = single[0]
    for backend in ('nccl', 'symm'):
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ep_size=world)
        sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
        c = curve(mesh, backend, feats[sl])
        diff = max(abs(a - b) for a, b in zip(single, c))
        report(f'ep{world}_{backend}_matches_single', diff < 4e-2, single=single, multi=c)


def tp_fused_checks(rank, world, dev, report):
    """GEMM+collective kernels against NCCL collectives around torch matmuls, with device-side timing."""
    from twinkle_b200 import ops
    from twinkle_b200.parallel.symm import SymmCommunicator
    from twinkle_b200.parallel.tensor_fused import FusedTP
    E = ops.ext()
    f = FusedTP(SymmCommunicator(None, dev))
    tp = world
    torch.manual_seed(100 + rank)

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))

    def timeit(fn, iters=8):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    T, H, I = 8192, 5120, 25600
    rows = T // tp
    # column-parallel: gather(x) @ W_col^T, W_col [I/tp, H]
    x = torch.randn(rows, H, device=dev).bfloat16()
    wc = (torch.randn(I // tp, H, device=dev) * 0.02).bfloat16()
    full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, x)
    want = full.float() @ wc.float().t()
    y, gathered = f.ag_gemm(x, wc, 'nt')
    torch.cuda.synchronize()
    report('ag_gemm_nt', torch.equal(gathered, full) and rel(y, want) < 4e-3, rel=rel(y, want))
    # row-parallel: reduce_scatter(a @ W_row^T), a [T, I/tp], W_row [H, I/tp]
    a = torch.randn(T, I // tp, device=dev).bfloat16()
    wr = (torch.randn(H, I // tp, device=dev) * 0.02).bfloat16()
    part = (a.float() @ wr.float().t())
    dist.all_reduce(part)
    want_rs = part[rank * rows:(rank + 1) * rows]
    out = f.gemm_rs(a, wr, 'nt')
    torch.cuda.synchronize()
    report('gemm_rs_nt', rel(out, want_rs) < 6e-3, rel=rel(out, want_rs))
    # dgrad forms ('nn')
    gy = torch.randn(T, I // tp, device=dev).bfloat16()
    part = gy.float() @ wc.float()
    dist.all_reduce(part)
    out = f.gemm_rs(gy, wc, 'nn')
    torch.cuda.synchronize()
    report('gemm_rs_nn', rel(out, part[rank * rows:(rank + 1) * rows]) < 6e-3)
    gl = torch.randn(rows, H, device=dev).bfloat16()
    gfull = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(gfull, gl)
    gx, gg = f.ag_gemm(gl, wr, 'nn')
    torch.cuda.synchronize()
    report('ag_gemm_nn', torch.equal(gg, gfull) and rel(gx, gfull.float() @ wr.float()) < 4e-3)

    # timing against NCCL + library GEMM (device events, max over ranks)
    def nccl_col():
        dist.all_gather_into_tensor(full, x)
        return torch.nn.functional.linear(full, wc)

    def nccl_row():
        p_ = torch.nn.functional.linear(a, wr)
        o = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o, p_)
        return o

    t_ag, t_ag_ref = timeit(lambda: f.ag_gemm(x, wc, 'nt')), timeit(nccl_col)
    t_gemm_only = timeit(lambda: torch.nn.functional.linear(full, wc))
    t_rs, t_rs_ref = timeit(lambda: f.gemm_rs(a, wr, 'nt')), timeit(nccl_row)
    flops = 2.0 * T * H * (I // tp)
    link = 770e9
    ag_bytes = (tp - 1) * rows * H * 2          # what one rank must pull
    rs_bytes = (tp - 1) * rows * H * 2          # what one rank must push
    roof_ag = max(flops / 1722.5e12, ag_bytes / link) * 1e3
    roof_rs = max(flops / 1722.5e12, rs_bytes / link) * 1e3
    report('tp_fused_timing', True, tp=tp, shape=[T, H, I // tp], ag_gemm_ms=t_ag, nccl_ag_plus_gemm_ms=t_ag_ref, gemm_rs_ms=t_rs,
           gemm_plus_nccl_rs_ms=t_rs_ref, library_gemm_only_ms=t_gemm_only, copier_ctas=f.copier_ctas(T, H, I // tp), roofline_ms_ag=roof_ag, roofline_ms_rs=roof_rs, frac_of_roofline_ag=roof_ag / t_ag,
           frac_of_roofline_rs=roof_rs / t_rs)
    report('tp_fused_error_word', E.read_and_clear_error() == 0)


def megatron_checks(rank, world, dev, report):
    """Tensor × pipeline parallel backend on GPUs (NCCL p2p + TP collectives) vs the single-GPU curve."""
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.models.config import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('qwen3-8b', num_hidden_layers=4, hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                 num_key_value_heads=2, vocab_size=4096)
    g = torch.Generator().manual_seed(13)
    feats = []
    for n in (1024, 512, 768, 1024):  # multiples of 256 rows per TP rank: the fused GEMM+collective kernels take these
        ids = torch.randint(0, cfg.vocab_size, (n + 1, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(m):
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(3):
            o = m.forward_backward(inputs=feats, micro_batch_size=1)
            m.clip_grad_and_step(max_grad_norm=1.0)
            out.append(float(o['loss']))
        return out

    single = [curve(TransformersModel(config=cfg, device_mesh=DeviceMesh.from_sizes(dp_size=1), seed=0, comm_backend='nccl', device=dev))
              if rank == 0 else None]
    dist.broadcast_object_list(single, src=0)
    single = single[0]
    layouts = [(2, 1, 1), (1, 2, 1)] if world == 2 else [(2, 2, 2), (2, 2, 1)]
    for tp, pp, vpp in layouts:
        mesh = DeviceMesh.from_sizes(tp_size=tp, pp_size=pp, dp_size=world // (tp * pp), vpp_size=vpp, sequence_parallel=tp > 1)
        c = curve(MegatronModel(config=cfg, device_mesh=mesh, seed=0, device=dev))
        vals = [None] * world
        dist.all_gather_object(vals, c)
        c = next(v for v in vals if v and v[0] == v[0] and v[0] != 0.0)  # a rank that holds the loss (last stage)
        diff = max(abs(a - b) for a, b in zip(single, c))
        report(f'megatron_tp{tp}_pp{pp}_vpp{vpp}_matches_single', diff < 5e-2, single=single, multi=c)


def ulysses_fused_checks(rank, world, dev, report):
    """q|k|v projection with the sequence → head exchange in its epilogue: the kernel against GEMM + all-to-all, then
    Ulysses training with the fused projection against the same run with the separate exchange kernels."""
    from twinkle_b200 import ops
    from twinkle_b200.parallel import ulysses as U
    from twinkle_b200.parallel.comm import Communicator
    from twinkle_b200.parallel.symm import SymmCommunicator
    sc = SymmCommunicator(None, dev)
    plain = Communicator(None, dev)
    t, K, hq, hkv, d = 384, 512, 4 * world, 2 * world, 128  # 384 rows: one full 256-row tile and a partial one
    g = torch.Generator(device='cpu').manual_seed(3)
    w = (torch.randn((hq + 2 * hkv) * d, K, generator=g) / K ** 0.5).to(dev).bfloat16()
    x = torch.randn(t, K, generator=torch.Generator(device='cpu').manual_seed(10 + rank)).to(dev).bfloat16()
    n_local = (hq + 2 * hkv) * d // world
    for it in range(3):  # both buffers of the pair are used and reused
        out = U._symm_out(sc, (world * t, n_local), torch.bfloat16, 'qkv_test')
        sc.head_scatter_gemm(x, w, out, t, hq * d // 128, hkv * d // 128)
        y = ops.gemm(x, w, 'nt')
        secs = [y[:, :hq * d].reshape(t, hq, d), y[:, hq * d:(hq + hkv) * d].reshape(t, hkv, d), y[:, (hq + hkv) * d:].reshape(t, hkv, d)]
        want = torch.cat([U._seq_to_head(s_.contiguous(), plain).reshape(world * t, -1) for s_ in secs], dim=-1)
        torch.cuda.synchronize()
        report(f'head_scatter_gemm_{it}', bool(torch.equal(out, want)), max_err=float((out.float() - want.float()).abs().max()))
        x = x + 1
    # training parity
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('qwen3-8b', num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4 * world,
                 num_key_value_heads=world, vocab_size=4096)
    gg = torch.Generator().manual_seed(7)
    feats = []
    for n in (257, 193, 301, 257):
        ids = torch.randint(0, cfg.vocab_size, (n, ), generator=gg)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(fused):
        os.environ['TWINKLE_ULYSSES_FUSED'] = '1' if fused else '0'
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=world)
        m = TransformersModel(config=cfg, device_mesh=mesh, seed=0, comm_backend='symm', device=dev)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(3):
            o = m.forward_backward(inputs=feats, micro_batch_size=2)
            gn = m.clip_grad_and_step(max_grad_norm=1.0)
            out.append((float(o['loss']), float(gn) if gn is not None else 0.0))
        return out

    before = ops.ext().launch_count()
    a = curve(False)
    mid = ops.ext().launch_count()
    b = curve(True)
    after = ops.ext().launch_count()
    os.environ['TWINKLE_ULYSSES_FUSED'] = '0'
    diff = max(abs(p - q) for ra, rb in zip(a, b) for p, q in zip(ra, rb))
    report('ulysses_fused_matches_separate', diff < 2e-2, separate=a, fused=b, launches_separate=mid - before, launches_fused=after - mid)


def main():
    rank, world, local = int(os.environ['RANK']), int(os.environ['WORLD_SIZE']), int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    import datetime
    dist.init_process_group('nccl', device_id=torch.device('cuda', local), timeout=datetime.timedelta(seconds=90))
    from twinkle_b200 import ops
    from twinkle_b200.parallel.comm import Communicator
    from twinkle_b200.parallel.symm import SymmCommunicator
    E = ops.ext()
    dev = torch.device('cuda', local)
    results = {}

    def report(name, ok, **kw):
        t = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({'check': name, 'ok': bool(t.item()), **kw}), flush=True)
        if not t.item():
            dist.destroy_process_group()
            sys.exit(1)

    only = os.environ.get('TK_MGPU_ONLY', '')
    stop_after_kernels = only == 'peer'
    if only in ('peer', 'fsdp'):
        only = ''
    if only in ('ep', 'megatron', 'tp_fused', 'ulysses_fused'):
        {'ep': ep_checks, 'megatron': megatron_checks, 'tp_fused': tp_fused_checks, 'ulysses_fused': ulysses_fused_checks}[only](rank, world, dev, report)
        report('error_word_end', E.read_and_clear_error() == 0)
        dist.barrier()
        dist.destroy_process_group()
        return

    # ---- 1. peer all-gather / reduce-scatter kernels against NCCL (guard zones around every symmetric tensor: a kernel
    # that writes past its destination on a peer shows up in check_canaries)
    os.environ['TWINKLE_SYMM_CANARIES'] = '1'
    sc = SymmCommunicator(None, dev)
    os.environ.pop('TWINKLE_SYMM_CANARIES')
    n = 1 << 20
    shard = sc.alloc(n, torch.bfloat16)
    shard.copy_(torch.randn(n, device=dev).bfloat16() + rank)
    full = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
    dist.barrier()
    sc.wait(sc.all_gather_async(full, shard))
    want = torch.empty_like(full)
    dist.all_gather_into_tensor(want, shard)
    torch.cuda.synchronize()
    report('peer_all_gather', bool(torch.equal(full, want)))
    fg = sc.alloc(n * world, torch.bfloat16)
    fg.copy_(torch.randn(n * world, device=dev).bfloat16())
    gs = torch.ones(n, dtype=torch.float32, device=dev)
    sc.reduce_scatter_accumulate(gs, fg, 0.5)
    tmp = fg.float()
    dist.all_reduce(tmp)
    wantg = 1 + 0.5 * tmp[rank * n:(rank + 1) * n]
    torch.cuda.synchronize()
    err = float((gs - wantg).abs().max())
    report('peer_reduce_scatter', err < 0.05 * world, max_err=err)
    # ---- 2. Ulysses exchange against all_to_all
    from twinkle_b200.parallel import ulysses as U
    t, H, D = 256, 8, 128
    x = torch.randn(t, H, D, device=dev).bfloat16()
    plain = Communicator(None, dev)
    a = U._seq_to_head(x, plain)
    b = U._seq_to_head(x, sc)
    c = U._head_to_seq(a, plain)
    d = U._head_to_seq(a, sc)
    torch.cuda.synchronize()
    report('ulysses_exchange', bool(torch.equal(a, b) and torch.equal(c, d) and torch.equal(c, x)))
    # receive-side exchange of several tensors at once (q, k, v with different head counts), both directions, repeated so
    # that both staging buffers of each pair are used and reused, and its first-generation (push) twin
    for it in range(3):
        xs = [torch.randn(t, h, D, device=dev).bfloat16() for h in (8 * world, 2 * world, 2 * world)]
        want = [U._seq_to_head(z, plain) for z in xs]
        got = sc.exchange_heads(xs, True)
        back = sc.exchange_heads(got, False)
        torch.cuda.synchronize()
        report(f'ulysses_pull_{it}', all(torch.equal(g_, w_) for g_, w_ in zip(got, want)) and all(torch.equal(b_, z) for b_, z in zip(back, xs)))
    sc.legacy_kernels = True
    b2 = U._seq_to_head(x, sc)
    torch.cuda.synchronize()
    sc.legacy_kernels = False
    report('ulysses_push_legacy', bool(torch.equal(a, b2)))
    dist.barrier()
    try:
        sc.check_canaries()
        report('symmetric_guard_zones_intact', len(sc._guards) >= 2)
    except RuntimeError as e:
        report('symmetric_guard_zones_intact', False, detail=str(e))
    report('error_word', E.read_and_clear_error() == 0)
    if stop_after_kernels:
        dist.barrier()
        dist.destroy_process_group()
        return

    # ---- 3. training parity: FSDP(+Ulysses) on W GPUs vs the single-GPU curve of the same global batch
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh
    cfg = preset('qwen3-8b', num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                 num_key_value_heads=2, vocab_size=4096)
    g = torch.Generator().manual_seed(7)
    feats = []
    for _ in range(4):
        ids = torch.randint(0, cfg.vocab_size, (257, ), generator=g)
        feats.append({'input_ids': ids[:-1], 'labels': ids[1:]})

    def curve(mesh, backend, my_feats, group_all=True):
        m = TransformersModel(config=cfg, device_mesh=mesh, seed=0, comm_backend=backend, device=dev)
        m.set_optimizer('AdamW', lr=1e-3)
        out = []
        for _ in range(4):
            o = m.forward_backward(inputs=my_feats, micro_batch_size=2)
            m.clip_grad_and_step(max_grad_norm=1.0)
            t = torch.tensor([o['loss'] * o['num_tokens'], o['num_tokens']], device=dev, dtype=torch.float64)
            if mesh.world_size > 1:
                dist.all_reduce(t)
                t = t / (mesh.ulysses_size or 1)
            out.append(float(t[0] / t[1]))
        return out

    single = None
    if rank == 0:
        single = curve(DeviceMesh.from_sizes(dp_size=1), 'nccl', feats)
    single = [single]
    dist.broadcast_object_list(single, src=0)
    single = single[0]
    for backend in ('nccl', 'symm'):
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None)
        sl = mesh.get_slice(len(feats), mesh.get_data_rank_from_global_rank(rank))
        c = curve(mesh, backend, feats[sl])
        diff = max(abs(a - b) for a, b in zip(single, c))
        report(f'fsdp{world}_{backend}_matches_single', diff < 3e-2, single=single, multi=c)
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=world)
        c = curve(mesh, backend, feats)
        diff = max(abs(a - b) for a, b in zip(single, c))
        report(f'ulysses{world}_{backend}_matches_single', diff < 3e-2, single=single, multi=c)
    # context parallelism (zig-zag shards, keys / values gathered per layer) on the GPUs against the same single-GPU curve
    mesh = DeviceMesh.from_sizes(dp_size=1, cp_size=world)
    c = curve(mesh, 'nccl', feats)
    diff = max(abs(a - b) for a, b in zip(single, c))
    report(f'context_parallel{world}_matches_single', diff < 3e-2, single=single, multi=c)
    report('error_word_end', E.read_and_clear_error() == 0)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
