"""Mixture-of-experts SFT on the tensor / pipeline backend: attention split over the tensor-parallel group with
sequence-parallel activations, experts split over an expert-parallel group carved out of the data-parallel ranks, and —
with ``--etp`` — every expert's intermediate dimension split over the tensor-parallel group as well.

    python -m torch.distributed.run --nproc-per-node 8 cookbook/megatron_tp_moe.py --model qwen3-30b-a3b --tp 2 --ep 4
    python -m torch.distributed.run --nproc-per-node 8 cookbook/megatron_tp_moe.py --model qwen3-30b-a3b --tp 2 --ep 2 --etp
    python cookbook/megatron_tp_moe.py --model tiny-moe --steps 3
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-moe')
    ap.add_argument('--tp', type=int, default=1)
    ap.add_argument('--pp', type=int, default=1)
    ap.add_argument('--ep', type=int, default=1)
    ap.add_argument('--etp', action='store_true', help='split every expert over the tensor-parallel group')
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--seq-len', type=int, default=256)
    ap.add_argument('--micro-batches', type=int, default=4)
    ap.add_argument('--out', default=None, help='write a Hugging Face checkpoint here after training')
    a = ap.parse_args(argv)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        dist.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    dp = max(world // (a.tp * a.pp), 1)
    mesh = DeviceMesh.from_sizes(tp_size=a.tp, pp_size=a.pp, dp_size=dp, ep_size=a.ep if a.ep > 1 else None,
                                 etp_size=a.tp if (a.etp and a.tp > 1) else None, sequence_parallel=a.tp > 1)
    model = MegatronModel(model_id=a.model, device_mesh=mesh, seed=0)
    model.set_optimizer('AdamW', lr=1e-4)
    data_rank = mesh.get_data_rank_from_global_rank(int(os.environ.get('RANK', '0')))
    g = torch.Generator().manual_seed(3 + data_rank)
    batch = []
    for _ in range(a.micro_batches):
        ids = torch.randint(0, model.config.vocab_size, (a.seq_len + 1, ), generator=g)
        batch.append({'input_ids': ids[:-1], 'labels': ids[1:]})
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=batch, micro_batch_size=1)
        model.clip_grad_and_step(max_grad_norm=1.0)
        losses.append(float(out['loss']))
        if int(os.environ.get('RANK', '0')) == 0:
            print(f'step {step} loss {losses[-1]:.4f}')
    if a.out:
        model.save('checkpoint', a.out)
    return losses


if __name__ == '__main__':
    main()
