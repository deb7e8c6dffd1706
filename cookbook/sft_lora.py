"""LoRA SFT.  python cookbook/sft_lora.py --model tiny-dense --steps 20"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--rank', type=int, default=8)
    ap.add_argument('--lr', type=float, default=1e-3)
    ap.add_argument('--out', default=None)
    a = ap.parse_args(argv)
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.metric import LossMetric
    model = TransformersModel(model_id=a.model, seed=0)
    model.add_adapter_to_model('sft', LoraConfig(r=a.rank, lora_alpha=2 * a.rank, target_modules='all-linear'))
    model.set_optimizer('AdamW', lr=a.lr, adapter_name='sft')
    model.set_lr_scheduler('CosineWarmupScheduler', num_warmup_steps=2, num_training_steps=a.steps, adapter_name='sft')
    vocab = model.config.vocab_size
    g = torch.Generator().manual_seed(0)
    batch = []
    for _ in range(4):  # a fixed synthetic batch: the loss must fall as the adapter memorises it
        ids = torch.randint(0, min(vocab, 1024), (65, ), generator=g)
        batch.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    metric, losses = LossMetric(), []
    for step in range(a.steps):
        out = model.forward_backward(inputs=batch, adapter_name='sft')
        norm = model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='sft')
        losses.append(float(out['loss']))
        metric.accumulate(None, {'loss': out['loss'], 'num_tokens': out['num_tokens']}, grad_norm=norm)
        if step % 5 == 0 or step == a.steps - 1:
            print(f'step {step:3d} loss {losses[-1]:.4f} grad_norm {float(norm or 0):.3f}')
    if a.out:
        print('saved', model.save('adapter', a.out, adapter_name='sft'))
    return losses


if __name__ == '__main__':
    main()
