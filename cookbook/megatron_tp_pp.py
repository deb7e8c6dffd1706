"""Tensor × pipeline parallel SFT (sequence-parallel activations, interleaved 1F1B) and export to a Hugging Face directory.

    python -m torch.distributed.run --nproc-per-node 8 cookbook/megatron_tp_pp.py --model qwen3-32b --tp 4 --pp 2 --vpp 2

The benchmark form of the tensor × pipeline configuration (Qwen3-32B architecture, TP 4 × PP 2, two virtual stages, 16 micro-batches of 8192
tokens, random-init weights, synthetic token ids): device-timed steps (CUDA events, maximum over ranks) printed as one JSON
line, then the weights written through the bridge to Hugging Face safetensors, reloaded and compared bit for bit:

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 cookbook/megatron_tp_pp.py --model qwen3-32b \
        --tp 4 --pp 2 --vpp 2 --seq-len 8192 --micro-batches 16 --warmup 2 --steps 3 --recompute full --roundtrip --json
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--tp', type=int, default=1)
    ap.add_argument('--pp', type=int, default=1)
    ap.add_argument('--vpp', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--seq-len', type=int, default=256)
    ap.add_argument('--micro-batches', type=int, default=4)
    ap.add_argument('--out', default=None)
    ap.add_argument('--warmup', type=int, default=0, help='un-timed steps before the timed ones')
    ap.add_argument('--recompute', default=None, choices=[None, 'full'])
    ap.add_argument('--comm', default='auto', choices=['auto', 'nccl', 'symm'], help='nccl: library collectives around the GEMMs instead of the fused kernels')
    ap.add_argument('--roundtrip', action='store_true', help='save to HF safetensors, perturb, reload, compare bit for bit')
    ap.add_argument('--json', action='store_true', help='print one JSON line with the device-timed throughput')
    a = ap.parse_args(argv)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        dist.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(tp_size=a.tp, pp_size=a.pp, dp_size=max(world // (a.tp * a.pp), 1), vpp_size=a.vpp, sequence_parallel=a.tp > 1)
    model = MegatronModel(model_id=a.model, device_mesh=mesh, seed=0, recompute=a.recompute, comm_backend=a.comm)
    model.set_optimizer('AdamW', lr=1e-4)
    g = torch.Generator().manual_seed(3)
    vocab = model.config.vocab_size
    batch = []
    for _ in range(a.micro_batches):
        ids = torch.randint(0, vocab, (a.seq_len + 1, ), generator=g)
        batch.append({'input_ids': ids[:-1], 'labels': ids[1:]})
    losses = []
    rank = int(os.environ.get('RANK', '0'))
    cuda = torch.cuda.is_available()

    def one_step():
        out = model.forward_backward(inputs=batch, micro_batch_size=1)
        model.clip_grad_and_step(max_grad_norm=1.0)
        return float(out['loss'])

    for _ in range(a.warmup):
        one_step()
    if world > 1:
        dist.barrier()
    if cuda:
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
    for step in range(a.steps):
        losses.append(one_step())
        if rank == 0 and not a.json:
            print(f'step {step} loss {losses[-1]:.4f}')
    ms = None
    if cuda:
        t1.record()
        torch.cuda.synchronize()
        t = torch.tensor([t0.elapsed_time(t1)], device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / max(a.steps, 1)
    result = {'config': f'{a.model} tp{a.tp} x pp{a.pp} x vpp{a.vpp} x dp{max(world // (a.tp * a.pp), 1)}', 'seq_len': a.seq_len,
              'micro_batches': a.micro_batches, 'recompute': a.recompute, 'comm': a.comm, 'losses': losses, 'ms_per_step': ms,
              'tokens_per_s': (a.seq_len * a.micro_batches * max(world // (a.tp * a.pp), 1)) / (ms / 1e3) if ms else None,
              'peak_mem_gib': round(torch.cuda.max_memory_allocated() / 2**30, 1) if cuda else None}
    out_dir = a.out
    if out_dir is None:  # one directory for all ranks
        box = [tempfile.mkdtemp(prefix='tk_hf_') if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        out_dir = box[0]
    if rank == 0 and a.json:   # the timing first: the round trip below needs disk space and minutes at full size
        import json
        print(json.dumps(dict(result, stage='timed')), flush=True)
    if a.roundtrip:
        import time
        t_save = time.time()
        path = model.save('hf', out_dir)
        t_save = time.time() - t_save
        before = {k: v.clone() for k, v in model.get_state_dict().items()}
        with torch.no_grad():
            for _, p in model.named_parameters():
                p.add_(1.0)
        model.load('hf', out_dir)
        after = model.get_state_dict()
        same = torch.tensor([1 if all(torch.equal(before[k], after[k]) for k in before) else 0], device='cuda' if cuda else 'cpu')
        if world > 1:
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
        result.update(roundtrip_bitwise=bool(same.item()), tensors_checked_on_rank0=len(before), save_seconds=round(t_save, 1), hf_dir=path)
    elif not a.json:
        path = model.save('hf', out_dir)
        if rank == 0:
            print('HF directory:', path)
    if rank == 0 and a.json:
        import json
        print(json.dumps(result), flush=True)
    return losses


if __name__ == '__main__':
    main()
