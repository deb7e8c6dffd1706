"""Multi-tenant GRPO: T LoRA tenants share one base model; every step each tenant samples G completions per prompt from
the sampler (which holds the tenant's current adapter), scores them, forms group-normalised advantages, takes one
clipped policy-gradient step and pushes its new adapter to the sampler.

    python cookbook/grpo_multi_lora.py --model tiny-dense --tenants 2 --steps 3
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--tenants', type=int, default=2)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--prompts', type=int, default=4)
    ap.add_argument('--group', type=int, default=4)
    ap.add_argument('--prompt-len', type=int, default=16)
    ap.add_argument('--max-tokens', type=int, default=16)
    ap.add_argument('--rank', type=int, default=8)
    a = ap.parse_args(argv)
    from twinkle_b200.advantage import GRPOAdvantage
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    from twinkle_b200.sampler import TorchSampler

    model = MultiLoraTransformersModel(model_id=a.model, max_loras=a.tenants, max_r=a.rank, seed=0)
    sampler = TorchSampler(model_id=a.model, max_loras=a.tenants, max_r=a.rank, weight_seed=0)
    names = [f'tenant{i}' for i in range(a.tenants)]
    cfg = LoraConfig(r=a.rank, lora_alpha=2 * a.rank, target_modules='all-linear')
    for n in names:
        model.add_adapter_to_model(n, cfg)
        model.set_optimizer('AdamW', lr=1e-3, adapter_name=n)
        model.set_loss('GRPOLoss', epsilon=0.2, beta=0.0, adapter_name=n)
        sampler.add_adapter_to_sampler(n, cfg)
    adv_fn = GRPOAdvantage()
    vocab = min(model.config.vocab_size, 1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, vocab, (a.prompt_len, ), generator=g).tolist() for _ in range(a.prompts)]
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=1.0, top_p=1.0, num_samples=a.group, logprobs=1)
    history = []
    for step in range(a.steps):
        for ti, n in enumerate(names):
            t0 = time.time()
            resps = sampler.sample([{'input_ids': p} for p in prompts], sp, adapter_name=n)
            feats, old_logps, rewards = [], [], []
            for r in resps:
                for s in r.sequences:
                    feats.append(s.new_input_feature)
                    old_logps.append(list(s.logprobs or []))
                    # toy reward: fraction of even token ids in the completion (learnable by the adapter)
                    rewards.append(sum(1 for t in s.tokens if t % 2 == 0) / max(len(s.tokens), 1))
            t_sample = time.time() - t0
            adv = adv_fn(rewards, num_generations=a.group, scale='group')
            out = model.forward_backward(inputs=feats, adapter_name=n, old_logps=old_logps, advantages=adv.tolist())
            model.clip_grad_and_step(max_grad_norm=1.0, adapter_name=n)
            t1 = time.time()
            sampler.update_weights(model.get_state_dict(adapter_name=n), peft_config=cfg.to_peft_dict(), adapter_name=n)
            t_sync = time.time() - t1
            history.append({'step': step, 'tenant': n, 'reward': sum(rewards) / len(rewards), 'loss': float(out['loss']),
                            'sample_s': t_sample, 'sync_s': t_sync})
            print(history[-1])
    return history


if __name__ == '__main__':
    main()
