#!/usr/bin/env python
"""Headline benchmark: training tokens/s of Qwen3-8B-architecture full-parameter SFT, and of Qwen3-30B-A3B LoRA SFT.

By default (``--config both``) the two halves of the headline metric run one after the other, each in a process of
its own: the dense result fills the top-level fields of the printed line, the mixture-of-experts result sits under
``"moe"`` (the Qwen3-30B-A3B expert-parallel LoRA configuration: 48 layers, hidden 2048, 128 experts top-8, LoRA r=16 on attention and expert linears,
8 sequences of 4096 tokens per GPU, experts split over all ranks).  ``--config dense`` / ``--config moe`` run one half.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Dense configuration (Qwen3-8B full-parameter SFT): 36 layers, hidden 4096, 32 q / 8 kv heads (head_dim 128), q/k RMSNorm,
SwiGLU 12288, vocab 151936, RoPE θ=1e6, random-init N(0, 0.02), bf16 compute, fp32 master weights +
AdamW, sequences of 32768 tokens packed from documents with lengths uniform in [512, 8192], token ids
uniform, varlen causal attention, activation recompute per layer.  Sharding: flat-bucket FSDP over all N
ranks, Ulysses SP = min(4, N).  Weak scaling: 2 sequences (65536 tokens) per GPU per step, i.e. the named
global batch of 16 sequences at N = 8.

Timing: W un-timed warm-up steps, then K steps bracketed by barrier + synchronize, CUDA events on the
launching stream, max over ranks.  ``value`` times steps whose inputs already sit on the device;
``e2e`` times the same steps through the public API (``forward_backward`` + ``clip_grad_and_step``) with
inputs taken from pinned host memory every step and the loss read back to the host.  Inputs of one step
(65536 tokens × hidden activations) exceed the 126 MB L2 many times over, so no explicit flush is needed.

``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` through its own public API
(``baseline/reference_arm.py``; nothing of this repository's package is imported on that path) for the dense half and
prints the same line with ``"impl": "reference"``.  After the timed regions one more step runs with the phase clock on
and its per-phase device times are printed as ``phases_ms_per_step``; ``config.data_plane`` says which transport each
sharded path resolved to, and a silent fall-back of ``--comm auto`` to library collectives ends the run with an error.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--model', default='qwen3-8b')
    ap.add_argument('--seq-len', type=int, default=32768)
    ap.add_argument('--seqs-per-gpu', type=int, default=2)
    ap.add_argument('--layers', type=int, default=None, help='debug only: overrides the layer count (result marked invalid)')
    ap.add_argument('--comm', default='auto', choices=['auto', 'nccl', 'symm'])
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--sp', type=int, default=None, help='Ulysses degree (default min(4, gpus))')
    ap.add_argument('--ref-micro', type=int, default=1, help='reference arm: sequences per forward_backward call')
    ap.add_argument('--cpu-debug', action='store_true', help='reference arm: run on CPU/gloo (debug only, result invalid)')
    ap.add_argument('--config', default='both', choices=['both', 'dense', 'moe'],
                    help="dense: Qwen3-8B full-parameter SFT; moe: Qwen3-30B-A3B LoRA r=16 SFT with expert parallel = gpus; "
                         "both (default): the two halves of the headline metric one after the other, each in a process of its own, "
                         "printed as one line (the dense fields at top level, the mixture-of-experts result under 'moe')")
    ap.add_argument('--moe-steps', type=int, default=10, help="cap on timed steps of the 'moe' half when --config both")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int = 0):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={self.index}', f'--query-gpu={q}', '--format=csv,noheader,nounits',
                                          '-lms', '200'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), parts[3:7]):
                if v.lower().startswith('active'):
                    reasons.add(name)
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': mx, 'reasons': sorted(reasons), 'samples': len(sm)}


def synthetic_sequences(n_seqs: int, seq_len: int, vocab: int, seed: int, pack: bool = True):
    """Each sequence = documents of length U[512, 8192] packed to exactly ``seq_len`` tokens (``pack``), or one
    document of ``seq_len`` tokens."""
    import torch
    g = torch.Generator().manual_seed(seed)
    feats = []
    for _ in range(n_seqs):
        lens, total = [], 0
        while total < seq_len:
            L = int(torch.randint(512, 8193, (1, ), generator=g)) if pack else seq_len
            L = min(L, seq_len - total)
            lens.append(L)
            total += L
        ids = torch.randint(0, vocab, (seq_len, ), generator=g, dtype=torch.int64)
        pos = torch.cat([torch.arange(L) for L in lens])
        labels = torch.roll(ids, -1)
        ends = torch.tensor(lens).cumsum(0) - 1
        labels[ends] = -100  # no target across document boundaries
        feats.append({'input_ids': ids.pin_memory() if torch.cuda.is_available() else ids,
                      'labels': labels.pin_memory() if torch.cuda.is_available() else labels,
                      'position_ids': pos.pin_memory() if torch.cuda.is_available() else pos})
    return feats


def run_reference(args):
    """The unmodified reference through its own public API (``baseline/reference_arm.py``); nothing of this
    repository's package is imported on that path."""
    sys.path.insert(0, os.path.join(ROOT, 'baseline'))
    try:
        import reference_arm
    except Exception as e:
        if int(os.environ.get('RANK', '0')) == 0:
            print(json.dumps({'impl': 'reference', 'unavailable': f'baseline/reference_arm.py cannot be imported: {type(e).__name__}: {e}'}))
        return
    reference_arm.run(args, synthetic_sequences, ClockSampler)


def run_both(args):
    """Runs ``--config dense`` and then ``--config moe`` as child processes of this rank (the parent never touches the
    GPU, so each half starts from an empty device and a failure of the second cannot lose the first) and prints the
    dense line with the mixture-of-experts result under ``'moe'``.  Children rendezvous on ports next to the launcher's;
    ``TORCHELASTIC_USE_AGENT_STORE`` is cleared so that their rank 0 hosts the store."""
    rank = int(os.environ.get('RANK', '0'))
    base_port = int(os.environ.get('MASTER_PORT', '29500'))
    results = {}
    for k, (cfg, steps, warmup) in enumerate((('dense', args.steps, args.warmup),
                                              ('moe', min(args.steps, args.moe_steps), min(args.warmup, 3)))):
        env = dict(os.environ)
        env['MASTER_PORT'] = str(base_port + 17 + k)
        env['MASTER_ADDR'] = env.get('MASTER_ADDR', '127.0.0.1')
        env.pop('TORCHELASTIC_USE_AGENT_STORE', None)
        cmd = [sys.executable, os.path.abspath(__file__), '--config', cfg, '--gpus', str(args.gpus), '--steps', str(steps), '--warmup', str(max(warmup, 3)),
               '--comm', args.comm, '--impl', args.impl, '--ref-micro', str(args.ref_micro)]
        if args.no_e2e:
            cmd.append('--no-e2e')
        if args.layers is not None:
            cmd += ['--layers', str(args.layers)]
        if args.sp is not None and cfg == 'dense':
            cmd += ['--sp', str(args.sp)]
        try:
            r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, text=True, timeout=2400 if cfg == 'dense' else 1200)
            line = None
            for ln in r.stdout.splitlines():
                if ln.startswith('{'):
                    try:
                        line = json.loads(ln)
                    except ValueError:
                        pass
            if line is None:
                line = {'unavailable': f'{cfg} half exited with code {r.returncode} and printed no result line'}
        except subprocess.TimeoutExpired:
            line = {'unavailable': f'{cfg} half did not finish within its time limit'}
        results[cfg] = line
    if rank != 0:
        return
    out = dict(results['dense'])
    moe = results['moe']
    out['moe'] = moe if 'unavailable' in moe else {k: moe.get(k) for k in ('metric', 'value', 'unit', 'steps', 'warmup', 'ms_per_step', 'config', 'e2e',
                                                                            'gpu_launches', 'peak_mem_gib', 'clocks', 'phases_ms_per_step',
                                                                            'kernel_error_word', 'impl') if k in moe}
    if 'gpu_launches' in out and isinstance(moe.get('gpu_launches'), int):
        out['gpu_launches_by_config'] = {'dense': out['gpu_launches'], 'moe': moe['gpu_launches']}
    print(json.dumps(out), flush=True)


def main():
    args = parse()
    if args.config == 'both':
        run_both(args)
        return
    if args.impl == 'reference':
        run_reference(args)
        return
    os.environ.setdefault('PYTORCH_CUDA_ALLOC_CONF', 'expandable_segments:True')
    import torch
    import torch.distributed as dist
    from twinkle_b200 import ops
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import preset
    from twinkle_b200.utils.device_mesh import DeviceMesh

    rank, world = int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    assert world == args.gpus, f'--gpus {args.gpus} but WORLD_SIZE={world}'
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        import datetime
        dist.init_process_group('nccl', device_id=torch.device('cuda', local), timeout=datetime.timedelta(seconds=300))
    moe = args.config == 'moe'
    if moe:
        # Qwen3-30B-A3B expert-parallel LoRA configuration: 48 layers, hidden 2048, 32 q / 4 kv heads, 128 experts top-8 (FFN 768), aux loss 1e-3,
        # LoRA r=16 on attention and expert linears, sequences of 4096 tokens, 8 sequences per GPU (64 at N=8),
        # experts split over all ranks (EP = N), everything else flat-bucket FSDP over the same ranks.
        if args.model == 'qwen3-8b':
            args.model = 'qwen3-30b-a3b'
        if args.seq_len == 32768:
            args.seq_len = 4096
        if args.seqs_per_gpu == 2:
            args.seqs_per_gpu = 8
        sp = 1
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ep_size=world) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    else:
        sp = args.sp or min(4, world)
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=sp) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    over = {} if args.layers is None else {'num_hidden_layers': args.layers}
    if moe:
        over['router_aux_loss_coef'] = 1e-3
    cfg = preset(args.model, **over)
    if moe:
        from twinkle_b200.model import LoraConfig
        model = TransformersModel(config=cfg, device_mesh=mesh, seed=0, comm_backend=args.comm, grad_dtype='fp32', max_loras=1, max_r=16)
        model.add_adapter_to_model('sft', LoraConfig(r=16, lora_alpha=32, target_modules='all-linear'))
        model.set_optimizer('AdamW', lr=1e-4, weight_decay=0.01, adapter_name='sft')
        akw = {'adapter_name': 'sft'}
    else:
        model = TransformersModel(config=cfg, device_mesh=mesh, seed=0, comm_backend=args.comm, grad_dtype='fp32')
        model.set_optimizer('AdamW', lr=1e-5, weight_decay=0.01)
        akw = {}
    data_ws = mesh.data_world_size
    n_local_seqs = args.seqs_per_gpu * sp          # sequences this rank's data group processes per step
    data_rank = mesh.data_rank or 0
    tokens_per_step_global = args.seqs_per_gpu * world * args.seq_len
    feats = synthetic_sequences(n_local_seqs, args.seq_len, cfg.vocab_size, seed=1000 + data_rank, pack=not moe)
    dev_feats = [{k: v.cuda(non_blocking=True) for k, v in f.items()} for f in feats]
    h2d_bytes = sum(v.numel() * v.element_size() for f in feats for v in f.values()) // sp

    # one micro-batch holds 65536 tokens per rank when the sharded state leaves room for it (N >= 2): parameters are
    # gathered and gradients reduce-scattered once per step instead of once per sequence
    micro = n_local_seqs if (world > 1 or moe) else 1

    def step(batch, read_loss: bool):
        out = model.forward_backward(inputs=batch, micro_batch_size=micro, **akw)
        model.clip_grad_and_step(max_grad_norm=1.0, **akw)
        return float(out['loss']) if read_loss else None

    def timed(batch, steps, read_loss):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ops.ext().launch_count()
        a.record()
        loss = None
        for _ in range(steps):
            loss = step(batch, read_loss)
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = a.elapsed_time(b)
        t = torch.tensor([ms], device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), ops.ext().launch_count() - l0, loss

    for _ in range(args.warmup):
        step(dev_feats, False)
    sampler = ClockSampler(local)
    sampler.start()      # every rank samples its own GPU: the slowest clock of the job paces a synchronous step
    ms, launches, _ = timed(dev_feats, args.steps, False)
    e2e = None
    if not args.no_e2e:
        ms_e, _, loss = timed(feats, args.steps, True)
        e2e = {'value': tokens_per_step_global * args.steps / (ms_e / 1e3), 'unit': 'tokens/s', 'h2d_bytes_per_step': h2d_bytes,
               'd2h_bytes_per_step': 8, 'ms_per_step': ms_e / args.steps, 'loss': loss}
    clocks = sampler.stop()
    if world > 1:
        mine = torch.tensor([float(clocks.get('sm_mhz') or 0.0)], device='cuda')
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        reasons = [None] * world
        dist.all_gather_object(reasons, clocks.get('reasons') or [])
        clocks['sm_mhz_per_rank'] = [float(t.item()) for t in every]
        clocks['reasons'] = sorted({r for rs in reasons for r in rs})
    # one more step with the phase clock on (outside both timed regions): device time per communication phase
    from twinkle_b200.utils.profiling import PHASES
    PHASES.start()
    step(dev_feats, False)
    phases = PHASES.stop()
    plane = model.data_plane()
    if world > 1 and args.comm == 'auto' and any(v in ('nccl', 'gloo') for v in plane.values()):
        raise SystemExit(f'--comm auto fell back to library collectives on {plane}; the peer-memory data plane did not come up')
    err = ops.ext().read_and_clear_error()
    if rank == 0:
        value = tokens_per_step_global * args.steps / (ms / 1e3)
        peak = torch.cuda.max_memory_allocated() / 2**30
        line = {
            'metric': ('train tokens/s/box Qwen3-30B-A3B EP LoRA SFT' if moe else 'train tokens/s/box Qwen3-8B FSDP2 (+Ulysses SP) full-parameter SFT'), 'value': value, 'unit': 'tokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms / args.steps, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
            'data': (f'synthetic (uniform token ids, {args.seqs_per_gpu} full sequences of {args.seq_len} tokens per GPU, random-init weights)' if moe
                     else 'synthetic (uniform token ids, packed docs U[512,8192], random-init weights)'),
            'impl': 'ours',
            'config': {'model': ('Qwen3-30B-A3B architecture, LoRA r=16' if moe else 'Qwen3-8B architecture') if args.layers is None else f'INVALID-debug-{args.layers}-layers',
                       'global_batch': args.seqs_per_gpu * world, 'seq_len': args.seq_len,
                       'parallelism': f'fsdp{world}' + (f'+ulysses{sp}' if sp > 1 else '') + (f'+ep{world}' if moe else ''), 'optimizer': 'AdamW fp32 master',
                       'recompute': 'per-layer', 'micro_batches_per_step': n_local_seqs // micro, 'l2': 'inputs per step exceed the 126 MB L2 (65536 tokens x 4096 hidden bf16 = 512 MiB per activation)',
                       'comm': args.comm, 'data_plane': plane},
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': int(launches), 'peak_mem_gib': round(peak, 1),
            'model_flops_per_token': cfg.flops_per_token(avg_context=0.0), 'kernel_error_word': err,
            'phases_ms_per_step': phases,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
