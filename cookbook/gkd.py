"""Knowledge distillation with the generalised Jensen-Shannon loss: a frozen teacher scores the sequences, the student
(LoRA on its own base) is trained towards the teacher's token distributions.

    python cookbook/gkd.py --mode off --steps 6        # off-policy: distil on a fixed set of sequences
    python cookbook/gkd.py --mode on  --steps 3        # on-policy: the student's own samples are what gets distilled
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--mode', default='off', choices=['off', 'on'])
    ap.add_argument('--steps', type=int, default=6)
    ap.add_argument('--beta', type=float, default=0.5)
    ap.add_argument('--topk', type=int, default=0, help='>0: distil on the teacher\'s top-k tokens only')
    ap.add_argument('--max-tokens', type=int, default=12)
    a = ap.parse_args(argv)
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel, TransformersModel
    from twinkle_b200.sampler import TorchSampler

    teacher = TransformersModel(model_id=a.model, seed=1)                     # different weights than the student's base
    student = MultiLoraTransformersModel(model_id=a.model, max_loras=1, max_r=8, seed=0)
    cfg = LoraConfig(r=8, lora_alpha=16, target_modules='all-linear')
    student.add_adapter_to_model('student', cfg)
    student.set_optimizer('AdamW', lr=3e-3, adapter_name='student')
    student.set_loss('GKDLoss', beta=a.beta, topk=a.topk or None, adapter_name='student')
    vocab = min(student.config.vocab_size, 1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, vocab, (10, ), generator=g).tolist() for _ in range(4)]

    def fixed_batch():
        feats = []
        for p in prompts:
            comp = torch.randint(3, vocab, (a.max_tokens, ), generator=g).tolist()
            ids = p + comp
            feats.append({'input_ids': ids[:-1], 'labels': [-100] * (len(p) - 1) + ids[len(p):]})
        return feats

    sampler = None
    if a.mode == 'on':
        sampler = TorchSampler(model_id=a.model, max_loras=1, max_r=8, weight_seed=0)
        sampler.add_adapter_to_sampler('student', cfg)
    feats = fixed_batch()
    losses = []
    for step in range(a.steps):
        if sampler is not None:
            sp = SamplingParams(max_tokens=a.max_tokens, temperature=1.0, num_samples=1)
            resps = sampler.sample([{'input_ids': p} for p in prompts], sp, adapter_name='student')
            feats = [r.sequences[0].new_input_feature for r in resps]
        # the teacher's logits over the same packed rows (one micro-batch on both sides keeps the row order equal)
        t_out = teacher.forward_only(inputs=feats, return_logits=True)
        out = student.forward_backward(inputs=feats, adapter_name='student', teacher_logits=t_out['logits'])
        student.clip_grad_and_step(max_grad_norm=1.0, adapter_name='student')
        losses.append(float(out['loss']))
        print(f'step {step} gkd loss {losses[-1]:.5f}')
        if sampler is not None:
            sampler.update_weights(student.get_state_dict(adapter_name='student'), peft_config=cfg.to_peft_dict(), adapter_name='student')
    return losses


if __name__ == '__main__':
    main()
