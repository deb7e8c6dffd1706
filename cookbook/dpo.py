"""DPO on preference pairs; the reference log-probs come from the same base with the adapter switched off.

    python cookbook/dpo.py --model tiny-dense --steps 5
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--beta', type=float, default=0.1)
    a = ap.parse_args(argv)
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    model = MultiLoraTransformersModel(model_id=a.model, max_loras=1, max_r=8, seed=0)
    model.add_adapter_to_model('dpo', LoraConfig(r=8, lora_alpha=16, target_modules='all-linear'))
    model.set_optimizer('AdamW', lr=2e-3, adapter_name='dpo')
    model.set_loss('DPOLoss', beta=a.beta, adapter_name='dpo')
    vocab = min(model.config.vocab_size, 1024)
    g = torch.Generator().manual_seed(0)
    pairs = []
    for _ in range(4):  # rows alternate chosen, rejected (same prompt, different completion)
        prompt = torch.randint(0, vocab, (12, ), generator=g).tolist()
        for _ in range(2):
            comp = torch.randint(0, vocab, (10, ), generator=g).tolist()
            ids = prompt + comp
            pairs.append({'input_ids': ids[:-1], 'labels': [-100] * (len(prompt) - 1) + ids[len(prompt):]})
    with model.adapter('dpo', disable_lora=True):
        ref = model.forward_only(inputs=pairs, adapter_name='dpo')
    ref_logps = [lp.tolist() if hasattr(lp, 'tolist') else lp for lp in ref['logps']]
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=pairs, adapter_name='dpo', ref_logps=ref_logps)
        model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='dpo')
        losses.append(float(out['loss']))
        print(f'step {step} dpo loss {losses[-1]:.4f}')
    return losses


if __name__ == '__main__':
    main()
