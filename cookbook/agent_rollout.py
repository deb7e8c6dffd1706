"""Multi-turn tool-use rollouts from the native sampler feeding GRPO (the agentic loop in miniature).

    python cookbook/agent_rollout.py --model tiny-dense --steps 2
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=2)
    ap.add_argument('--group', type=int, default=4)
    a = ap.parse_args(argv)
    from twinkle_b200.advantage import GRPOAdvantage
    from twinkle_b200.agentic import F1Reward, FunctionTool, MultiTurnRollout, ToolManager
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    from twinkle_b200.sampler import TorchSampler

    def lookup(key: str) -> str:
        """Look a fact up."""
        return {'capital of France': 'Paris'}.get(key, 'unknown')

    cfg = LoraConfig(r=8, lora_alpha=16, target_modules='all-linear')
    model = MultiLoraTransformersModel(model_id=a.model, max_loras=1, max_r=8, seed=0)
    model.add_adapter_to_model('agent', cfg)
    model.set_optimizer('AdamW', lr=1e-3, adapter_name='agent')
    model.set_loss('GRPOLoss', epsilon=0.2, adapter_name='agent')
    model.set_template('Template', adapter_name='agent')
    sampler = TorchSampler(model_id=a.model, max_loras=1, max_r=8, weight_seed=0)
    sampler.set_template('Template')
    sampler.add_adapter_to_sampler('agent', cfg)
    rollout = MultiTurnRollout(sampler, ToolManager([FunctionTool(lookup)]), max_turns=2, adapter_name='agent',
                               sampling_params=SamplingParams(max_tokens=24, temperature=1.0))
    reward, adv_fn = F1Reward(), GRPOAdvantage()
    history = []
    for step in range(a.steps):
        prompts = [{'messages': [{'role': 'user', 'content': 'What is the capital of France?'}], 'user_data': {'ground_truth': 'Paris'}}
                   for _ in range(a.group)]
        trajs = rollout(prompts)
        rewards = reward(trajs)
        adv = adv_fn(rewards, num_generations=a.group, scale='group')
        out = model.forward_backward(inputs=trajs, adapter_name='agent', advantages=adv.tolist())
        model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='agent')
        sampler.update_weights(model.get_state_dict(adapter_name='agent'), peft_config=cfg.to_peft_dict(), adapter_name='agent')
        history.append({'step': step, 'mean_reward': sum(rewards) / len(rewards), 'loss': float(out['loss']),
                        'turns': [t['user_data']['rollout']['turns'] for t in trajs]})
        print(history[-1])
    return history


if __name__ == '__main__':
    main()
