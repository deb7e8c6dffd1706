"""Tensor × pipeline parallel SFT (sequence-parallel activations, interleaved 1F1B) and export to a Hugging Face directory.

    python -m torch.distributed.run --nproc-per-node 8 cookbook/megatron_tp_pp.py --model qwen3-32b --tp 4 --pp 2 --vpp 2
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
    a = ap.parse_args(argv)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        dist.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from twinkle_b200.model.megatron import MegatronModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(tp_size=a.tp, pp_size=a.pp, dp_size=max(world // (a.tp * a.pp), 1), vpp_size=a.vpp, sequence_parallel=a.tp > 1)
    model = MegatronModel(model_id=a.model, device_mesh=mesh, seed=0)
    model.set_optimizer('AdamW', lr=1e-4)
    g = torch.Generator().manual_seed(3)
    vocab = model.config.vocab_size
    batch = []
    for _ in range(a.micro_batches):
        ids = torch.randint(0, vocab, (a.seq_len + 1, ), generator=g)
        batch.append({'input_ids': ids[:-1], 'labels': ids[1:]})
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=batch, micro_batch_size=1)
        model.clip_grad_and_step(max_grad_norm=1.0)
        losses.append(float(out['loss']))
        if int(os.environ.get('RANK', '0')) == 0:
            print(f'step {step} loss {losses[-1]:.4f}')
    out_dir = a.out or tempfile.mkdtemp(prefix='tk_hf_')
    path = model.save('hf', out_dir)
    if int(os.environ.get('RANK', '0')) == 0:
        print('HF directory:', path)
    return losses


if __name__ == '__main__':
    main()
