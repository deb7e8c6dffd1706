"""Full-parameter SFT with flat-bucket FSDP and Ulysses sequence parallel — the loop behind the headline benchmark.

    python -m torch.distributed.run --nproc-per-node 8 cookbook/sft_full_fsdp_ulysses.py --model qwen3-8b --sp 4
    python cookbook/sft_full_fsdp_ulysses.py --model tiny-dense --steps 5           # one process, CPU or one GPU
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--sp', type=int, default=1)
    ap.add_argument('--seq-len', type=int, default=256)
    ap.add_argument('--seqs-per-rank', type=int, default=2)
    ap.add_argument('--lr', type=float, default=1e-4)
    a = ap.parse_args(argv)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        dist.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=a.sp) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    model = TransformersModel(model_id=a.model, device_mesh=mesh, seed=0)
    model.set_optimizer('AdamW', lr=a.lr, weight_decay=0.01)
    vocab = model.config.vocab_size
    g = torch.Generator().manual_seed(1000 + (mesh.data_rank or 0))
    n_seqs = a.seqs_per_rank * max(a.sp, 1)  # sequence-parallel peers share their data group's sequences
    batch = []
    for _ in range(n_seqs):
        ids = torch.randint(0, vocab, (a.seq_len + 1, ), generator=g)
        batch.append({'input_ids': ids[:-1], 'labels': ids[1:]})
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=batch, micro_batch_size=n_seqs)
        norm = model.clip_grad_and_step(max_grad_norm=1.0)
        losses.append(float(out['loss']))
        if int(os.environ.get('RANK', '0')) == 0:
            print(f'step {step} loss {losses[-1]:.4f} grad_norm {float(norm or 0):.3f}')
    return losses


if __name__ == '__main__':
    main()
