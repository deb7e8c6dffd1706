"""Vision-language SFT (Qwen2-VL family): images in the chat messages, LoRA on the language model or full training with the
vision tower.  python cookbook/mm_sft.py --model tiny-vl --steps 10   (multi-GPU: launch with torch.distributed.run, --fsdp N)"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def synthetic_samples(n: int, seed: int = 0):
    """Images whose brightest quadrant is the answer — learnable from pixels only."""
    g = torch.Generator().manual_seed(seed)
    names = ['top left', 'top right', 'bottom left', 'bottom right']
    out = []
    for _ in range(n):
        k = int(torch.randint(0, 4, (1, ), generator=g))
        img = torch.rand(3, 56, 56, generator=g) * 40
        r, c = divmod(k, 2)
        img[:, r * 28:(r + 1) * 28, c * 28:(c + 1) * 28] += 200
        out.append({'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': img}, {'type': 'text', 'text': 'Which quadrant is bright?'}]},
                                 {'role': 'assistant', 'content': names[k]}]})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-vl', help='preset name or a directory with a Qwen2-VL checkpoint')
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--batch', type=int, default=8)
    ap.add_argument('--lr', type=float, default=3e-3)
    ap.add_argument('--lora-rank', type=int, default=0, help='0 = train everything (tower included); > 0 = LoRA on the language model')
    ap.add_argument('--fsdp', type=int, default=1)
    ap.add_argument('--freeze-vision', action='store_true', help='full run with the tower kept fixed')
    ap.add_argument('--out', default=None)
    a = ap.parse_args(argv)
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    mesh = DeviceMesh.from_sizes(fsdp_size=a.fsdp, dp_size=None) if a.fsdp > 1 else DeviceMesh.from_sizes(dp_size=1)
    model = TransformersModel(model_id=a.model, device_mesh=mesh, seed=0, freeze_vision=a.freeze_vision)
    name = None
    if a.lora_rank > 0:
        name = 'mm'
        model.add_adapter_to_model(name, LoraConfig(r=a.lora_rank, lora_alpha=2 * a.lora_rank, target_modules='all-linear'))
    kw = {'adapter_name': name} if name else {}
    model.set_template('Qwen2VLTemplate', vision_config=model.config.vision, max_length=8192, **kw)
    model.set_optimizer('AdamW', lr=a.lr, **kw)
    rank = int(os.environ.get('RANK', 0))
    data = synthetic_samples(a.batch * max(a.fsdp, 1), seed=1)
    mine = data[mesh.get_slice(len(data), mesh.get_data_rank_from_global_rank(rank))]
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=mine, **kw)
        model.clip_grad_and_step(max_grad_norm=1.0, **kw)
        losses.append(float(out['loss']))
        if rank == 0 and (step % 5 == 0 or step == a.steps - 1):
            print(f'step {step:3d} loss {losses[-1]:.4f}')
    if a.out:
        print('saved', model.save('final', a.out, **kw))
    return losses


if __name__ == '__main__':
    main()
