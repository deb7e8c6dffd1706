"""Multimodal GRPO (Qwen2-VL family): the policy looks at an image, answers, is rewarded for the right answer; LoRA adapter on the
language model, synced into the sampler after every step.  python cookbook/mm_grpo.py --steps 3"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-vl')
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--prompts', type=int, default=4)
    ap.add_argument('--group', type=int, default=4)
    ap.add_argument('--max-tokens', type=int, default=8)
    ap.add_argument('--rank', type=int, default=8)
    a = ap.parse_args(argv)
    from cookbook.mm_sft import synthetic_samples
    from twinkle_b200.advantage import GRPOAdvantage
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.metric import CompletionRewardMetric
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    from twinkle_b200.sampler import TorchSampler

    model = MultiLoraTransformersModel(model_id=a.model, max_loras=1, max_r=a.rank, seed=0)
    sampler = TorchSampler(model_id=a.model, max_loras=1, max_r=a.rank, weight_seed=0)
    cfg = LoraConfig(r=a.rank, lora_alpha=2 * a.rank, target_modules='all-linear')
    model.add_adapter_to_model('policy', cfg)
    model.set_optimizer('AdamW', lr=2e-3, adapter_name='policy')
    model.set_loss('GRPOLoss', epsilon=0.2, beta=0.0, adapter_name='policy')
    for obj in (model, sampler):
        kw = {'adapter_name': 'policy'} if obj is model else {}
        obj.set_template('Qwen2VLTemplate', vision_config=model.config.vision, max_length=4096, **kw)
    sampler.add_adapter_to_sampler('policy', cfg)
    samples = synthetic_samples(a.prompts, seed=3)
    prompts = [{'messages': s['messages'][:1]} for s in samples]          # the question with its image; the answer is the ground truth
    truths = [s['messages'][1]['content'] for s in samples]
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=1.0, num_samples=a.group, logprobs=1)
    adv_fn, history = GRPOAdvantage(), []
    for step in range(a.steps):
        resps = sampler.sample(prompts, sp, adapter_name='policy')
        feats, old_logps, rewards = [], [], []
        for r, truth in zip(resps, truths):
            for q in r.sequences:
                feats.append(q.new_input_feature)                          # keeps the image patches and positions
                old_logps.append(list(q.logprobs or []))
                text = (q.decoded or '').lower()
                # graded so that a random policy sees a signal: 1 for the phrase, 0.5 for one of its two words, small bonus for letters
                words = truth.split()
                rewards.append(1.0 if truth in text else 0.5 * sum(w in text for w in words) / len(words) + 0.1 * sum(c.isalpha() for c in text) / max(len(text), 1))
        adv = adv_fn(rewards, num_generations=a.group, scale='group')
        out = model.forward_backward(inputs=feats, adapter_name='policy', old_logps=old_logps, advantages=adv.tolist())
        model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='policy')
        sampler.update_weights(model.get_state_dict(adapter_name='policy'), peft_config=cfg.to_peft_dict(), adapter_name='policy')
        history.append({'step': step, 'reward': sum(rewards) / len(rewards), 'loss': float(out['loss']), 'sequences': len(feats)})
        print(history[-1])
    return history


if __name__ == '__main__':
    main()
