"""DeepSeek-V3-shaped LoRA SFT: multi-head latent attention, sigmoid group-limited routing, experts split over the ranks
(expert parallel) with adapters on the attention / shared-expert linears and on the fused expert tensors.

    python -m torch.distributed.run --nproc-per-node 8 cookbook/deepseek_ep_lora.py --model /path/to/DeepSeek-V3-checkpoint
    python cookbook/deepseek_ep_lora.py --model tiny-deepseek --steps 5

The adapter leaves one projection out of ``all-linear`` (PEFT's ``exclude_modules``) and names the expert tensors as
``target_parameters``, the form the reference's DeepSeek cookbook uses.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-deepseek')
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--seq-len', type=int, default=128)
    ap.add_argument('--seqs-per-rank', type=int, default=4)
    ap.add_argument('--out', default=None, help='directory for the PEFT-format adapter')
    a = ap.parse_args(argv)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        dist.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ep_size=world) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    model = TransformersModel(model_id=a.model, device_mesh=mesh, seed=0, max_loras=1, max_r=16)
    model.add_adapter_to_model('sft', LoraConfig(r=16, lora_alpha=32, target_modules='all-linear', exclude_modules=['kv_a_proj_with_mqa'],
                                                 target_parameters=['mlp.experts.gate_up_proj', 'mlp.experts.down_proj']))
    model.set_optimizer('AdamW', lr=1e-3, adapter_name='sft')
    g = torch.Generator().manual_seed(7 + (mesh.data_rank or 0))
    vocab = min(model.config.vocab_size, 4096)
    batch = []
    for _ in range(a.seqs_per_rank):
        ids = torch.randint(0, vocab, (a.seq_len + 1, ), generator=g)
        batch.append({'input_ids': ids[:-1], 'labels': ids[1:]})
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=batch, adapter_name='sft')
        model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='sft')
        losses.append(float(out['loss']))
        if int(os.environ.get('RANK', '0')) == 0:
            print(f'step {step} loss {losses[-1]:.4f}')
    if a.out:
        model.save('adapter', a.out, adapter_name='sft')
    return losses


if __name__ == '__main__':
    main()
