"""Device-timed micro-benchmarks of the peer-memory data plane, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m twinkle_b200.parallel.microbench

Measures, at the sizes of the Qwen3-8B training step (one decoder layer's parameters = 385 MB in bf16; q / k / v of
65536 tokens per rank), every kernel the sharded engine puts between two GEMMs, and prints one JSON line on rank 0:
the cross-GPU flag barrier, the parameter all-gather, the gradient reduce-scatter (+cast, scale, accumulate), the
Ulysses head↔sequence exchange as one receive-side pull of q, k and v, the first-generation kernels of the same
operations for comparison (``*_legacy``), the NCCL collective each one replaces, and the trainer → sampler weight push
(one rank writing a bucket into a peer's landing zone, with and without the fp32 → bf16 cast).  Times are CUDA events on the
launching stream after warm-up, maximum over ranks; ``gbs`` is the bytes a rank must receive over NVLink divided by
that time, to be read against the measured peer-copy bandwidth of 770 GB/s per direction.
"""
from __future__ import annotations

import datetime
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    rank, world, local = int(os.environ['RANK']), int(os.environ['WORLD_SIZE']), int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev, timeout=datetime.timedelta(seconds=120))
    from twinkle_b200 import ops
    from twinkle_b200.parallel.symm import SymmCommunicator
    sc = SymmCommunicator(None, dev)
    E = ops.ext()
    out = {'n_gpus': world, 'peer_copy_reference_gbs': 770.0}

    from twinkle_b200.utils.profiling import DeviceTimer
    timer = DeviceTimer()

    def timeit(fn, iters=10, warm=3):
        """Mean milliseconds per call: CUDA events around ``iters`` back-to-back calls, maximum over ranks."""
        for _ in range(warm):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        with timer('op'):
            for _ in range(iters):
                fn()
        return timer.summary()['op'] / iters

    def entry(ms, recv_bytes):
        return {'ms': round(ms, 4), 'gbs': round(recv_bytes / ms / 1e6, 1)}

    # ---- barrier
    out['barrier'] = {'ms': round(timeit(sc.barrier_kernel, iters=50), 4)}
    # ---- parameter all-gather: one Qwen3-8B layer (192.9 M bf16 parameters), shard = 1/N
    numel = 192_937_984 // (64 * world) * (64 * world)
    shard = sc.alloc(numel // world, torch.bfloat16)
    shard.normal_()
    full = torch.empty(numel, dtype=torch.bfloat16, device=dev)
    sc.sync_all()
    recv = numel * 2 * (world - 1) // world
    for legacy in (False, True):
        sc.legacy_kernels = legacy
        for blocks in ((8, 16, 32) if not legacy else (16, )):
            sc.copy_blocks = blocks
            ms = timeit(lambda: sc.wait(sc.all_gather_async(full, shard)))
            out[f'all_gather{"_legacy" if legacy else ""}_b{blocks}'] = entry(ms, recv)
    sc.legacy_kernels, sc.copy_blocks = False, 16
    out['all_gather_nccl'] = entry(timeit(lambda: dist.all_gather_into_tensor(full, shard)), recv)
    # ---- gradient reduce-scatter + cast + scale + accumulate
    fg = sc.alloc(numel, torch.bfloat16)
    fg.normal_()
    gs = torch.zeros(numel // world, dtype=torch.float32, device=dev)
    sc.sync_all()
    def symm_rs():
        sc.reduce_scatter_accumulate(gs, fg, 1.0)   # runs on the communicator's side stream
        sc.wait_reduce_scatters()

    out['reduce_scatter_acc'] = entry(timeit(symm_rs), recv)
    tmp = torch.empty(numel // world, dtype=torch.bfloat16, device=dev)

    def nccl_rs():
        dist.reduce_scatter_tensor(tmp, fg)
        gs.add_(tmp.float())

    out['reduce_scatter_nccl_plus_add'] = entry(timeit(nccl_rs), recv)
    # ---- Ulysses exchange: q [t, 32, 128], k and v [t, 8, 128] with t = 65536 / N tokens per rank
    if 32 % world == 0 and 8 % world == 0:
        from twinkle_b200.parallel import ulysses as U
        t = 65536 // world
        q = torch.randn(t, 32, 128, device=dev).bfloat16()
        k = torch.randn(t, 8, 128, device=dev).bfloat16()
        v = torch.randn(t, 8, 128, device=dev).bfloat16()
        recv = (q.numel() + k.numel() + v.numel()) * 2 * (world - 1) // world
        out['ulysses_qkv_pull'] = entry(timeit(lambda: sc.exchange_heads([q, k, v], True)), recv)
        qh, kh, vh = sc.exchange_heads([q, k, v], True)
        out['ulysses_qkv_pull_back'] = entry(timeit(lambda: sc.exchange_heads([qh, kh, vh], False)), recv)
        sc.legacy_kernels = True
        out['ulysses_qkv_push_legacy'] = entry(timeit(lambda: [U._seq_to_head(x, sc) for x in (q, k, v)]), recv)
        sc.legacy_kernels = False

        def nccl_a2a():
            for x in (q, k, v):
                tt, h, d = x.shape
                send = x.view(tt, world, h // world, d).transpose(0, 1).contiguous()
                recv_ = torch.empty_like(send)
                dist.all_to_all_single(recv_, send)

        out['ulysses_qkv_nccl_all_to_all'] = entry(timeit(nccl_a2a), recv)
    # ---- trainer → sampler weight push: rank 0 writes a 512 MiB bf16 bucket into rank 1's landing zone (and the same
    # bucket from fp32 masters, cast on the way); only the sender works, the others wait at the barrier
    n_w = 256 << 20
    landing = sc.alloc(n_w, torch.bfloat16)
    torch.manual_seed(1234)  # the same values on every rank, so that the receiver can check what landed
    src16 = torch.randn(n_w, device=dev, dtype=torch.bfloat16)
    src32 = torch.randn(n_w, device=dev, dtype=torch.float32)
    sc.sync_all()
    dst = [sc.peer_ptrs(landing)[1 % world]]
    for tag, src in (('weight_push_bf16', src16), ('weight_push_fp32_cast', src32)):
        out[tag] = entry(timeit((lambda s_=src: E.peer_copy_cast(s_, dst, 0)) if rank == 0 else (lambda: None), iters=5), n_w * 2)
    sc.sync_all()
    ok = torch.tensor([1.0 if (rank != 1 % world or torch.equal(landing, src32.bfloat16())) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    out['weight_push_received_ok'] = bool(ok.item() > 0.5)
    out['kernel_error_word'] = E.read_and_clear_error()
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
