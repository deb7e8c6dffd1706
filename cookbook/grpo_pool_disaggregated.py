"""Disaggregated GRPO in pool mode: the driver holds no weights.  A model group (FSDP over its ranks) trains a LoRA
policy, a sampler group generates; after every step the new adapter travels from the trainer's workers to the sampler's
workers through the checkpoint engine (CUDA-IPC peer copies between GPUs, a host-memory store on CPU-only hosts).

    python cookbook/grpo_pool_disaggregated.py --model tiny-dense --steps 3                 # 2 trainer + 1 sampler worker
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--trainers', type=int, default=2)
    ap.add_argument('--samplers', type=int, default=1)
    ap.add_argument('--prompts', type=int, default=4)
    ap.add_argument('--group', type=int, default=4)
    ap.add_argument('--max-tokens', type=int, default=8)
    ap.add_argument('--device', default='auto', choices=['auto', 'cpu', 'cuda'])
    a = ap.parse_args(argv)
    import torch
    import twinkle_b200
    from twinkle_b200 import DeviceGroup, DeviceMesh
    from twinkle_b200.advantage import GRPOAdvantage
    from twinkle_b200.checkpoint_engine import CheckpointEngineManager
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import LoraConfig, TransformersModel
    from twinkle_b200.sampler import TorchSampler
    dev = a.device
    if dev == 'auto':
        dev = 'cuda' if torch.cuda.is_available() and torch.cuda.device_count() >= a.trainers + a.samplers else 'cpu'
    twinkle_b200.initialize(mode='pool', groups=[DeviceGroup(name='model', ranks=a.trainers, device_type=dev),
                                                 DeviceGroup(name='sampler', ranks=a.samplers, device_type=dev)])
    try:
        model = TransformersModel(model_id=a.model, device_mesh=DeviceMesh.from_sizes(fsdp_size=a.trainers, dp_size=None), seed=0,
                                  max_loras=1, max_r=8, remote_group='model')
        cfg = LoraConfig(r=8, lora_alpha=16, target_modules='all-linear')
        model.add_adapter_to_model('policy', cfg)
        model.set_optimizer('AdamW', lr=2e-3, adapter_name='policy')
        model.set_loss('GRPOLoss', epsilon=0.2, beta=0.0, adapter_name='policy')
        sampler = TorchSampler(model_id=a.model, device_mesh=DeviceMesh.from_sizes(dp_size=a.samplers), weight_seed=1, max_loras=1, max_r=8,
                               remote_group='sampler')             # different initial weights: the first sync must overwrite them
        sync = CheckpointEngineManager(model, sampler)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(3, 512, (10, ), generator=g).tolist() for _ in range(a.prompts)]
        sp = SamplingParams(max_tokens=a.max_tokens, temperature=1.0, num_samples=a.group, logprobs=1)
        adv_fn, history = GRPOAdvantage(), []
        for step in range(a.steps):
            t0 = time.time()
            stats = sync.sync_weights(adapter_name='policy')        # first call: base weights, then the adapter; later: adapter only
            t_sync = time.time() - t0
            resps = sampler.sample([{'input_ids': p} for p in prompts], sp)
            feats, old_logps, rewards = [], [], []
            for r in resps:
                for s in r.sequences:
                    feats.append(s.new_input_feature)
                    old_logps.append(list(s.logprobs or []))
                    rewards.append(sum(1 for t in s.tokens if t % 2 == 0) / max(len(s.tokens), 1))
            # the sampler's log-probs must be the trainer's: both sides hold the same weights after the sync
            check = model.forward_only(inputs=feats[:a.group], adapter_name='policy')
            drift = 0.0
            for f, lp, old in zip(feats, check['logps'], old_logps):
                keep = torch.tensor(f['labels']) != -100
                mine = torch.as_tensor(lp).float().reshape(-1)[:len(keep)][keep]
                drift = max(drift, float((mine - torch.tensor(old)).abs().max()))
            adv = adv_fn(rewards, num_generations=a.group, scale='group')
            out = model.forward_backward(inputs=feats, adapter_name='policy', old_logps=old_logps, advantages=adv.tolist())
            model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='policy')
            history.append({'step': step, 'reward': sum(rewards) / len(rewards), 'loss': float(out['loss']), 'sync_bytes': stats['bytes'],
                            'sync_s': round(t_sync, 3), 'samples': len(feats), 'logp_drift': drift})
            print(history[-1])
        sync.finalize()
        return history
    finally:
        twinkle_b200.infra.shutdown()


if __name__ == '__main__':
    main()
