"""Preference optimisation and stop/resume through the Tinker-style client.

DPO needs reference log-probs: the client asks the server for a forward pass with the adapter switched off
(`loss_fn_config={'disable_lora': True}`), attaches the returned log-probs to each datum as `ref_logps` and trains with
`loss_fn='importance_sampling'`; the server recognises the pairs (rows alternate chosen, rejected) and reports the DPO
metrics with the step.  Then the state is saved, the server is rebuilt from scratch, and a new training client created
from the saved state continues with the optimizer state intact.

    python cookbook/server_tinker_dpo_resume.py --model tiny-dense --steps 3
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def build_server(name: str, state_file: str):
    from twinkle_b200.server import ServerLauncher
    return ServerLauncher({
        'persistence': {'mode': 'file', 'file_path': state_file},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': [name]}},
            {'name': 'model', 'route_prefix': f'/model/{name}', 'import_path': 'model', 'args': {'model_id': name, 'backend': 'transformers', 'max_loras': 2}},
            {'name': 'sampler', 'route_prefix': f'/sampler/{name}', 'import_path': 'sampler', 'args': {'model_id': name, 'sampler_type': 'torch'}},
        ],
    })


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--beta', type=float, default=0.1)
    a = ap.parse_args(argv)
    work = tempfile.mkdtemp(prefix='tk_dpo_')
    os.environ['TWINKLE_DEFAULT_SAVE_DIR'] = os.path.join(work, 'ckpt')
    os.environ.setdefault('TWINKLE_POLL_INTERVAL', '0.02')
    from twinkle_b200.client import TinkerClient
    state_file = os.path.join(work, 'state.json')
    client = TinkerClient(app=build_server(a.model, state_file).root, token='demo')
    trainer = client.create_lora_training_client(a.model, rank=8)
    g = torch.Generator().manual_seed(0)
    datums = []
    for _ in range(3):                                           # rows alternate chosen, rejected
        prompt = torch.randint(3, 512, (8, ), generator=g).tolist()
        for _ in range(2):
            ids = prompt + torch.randint(3, 512, (7, ), generator=g).tolist()
            datums.append({'model_input': {'tokens': ids[:-1]},
                           'loss_fn_inputs': {'target_tokens': {'data': ids[1:]}, 'weights': {'data': [0.0] * (len(prompt) - 1) + [1.0] * 7}}})
    ref = trainer.forward(datums, 'cross_entropy', loss_fn_config={'disable_lora': True}).result()
    for d, r in zip(datums, ref['loss_fn_outputs']):
        d['loss_fn_inputs']['ref_logps'] = {'data': r['logprobs']['data']}
    cfg = {'dpo_beta': a.beta, 'dpo_loss_type': 'sigmoid'}
    losses, metrics = [], {}
    for step in range(a.steps):
        out = trainer.forward_backward(datums, 'importance_sampling', loss_fn_config=cfg).result()
        metrics = trainer.optim_step({'learning_rate': 2e-3}).result()['metrics']
        losses.append(out['metrics'].get('loss', out['metrics'].get('loss:sum')))
        print(f'step {step} dpo loss {losses[-1]:.4f}')
    saved = trainer.save_state('dpo-final').result()['path']

    def two_more(tc):
        """Loss now, and loss after one more optimizer step: the second needs the saved Adam moments and step count."""
        first = tc.forward_backward(datums, 'importance_sampling', loss_fn_config=cfg).result()['metrics']
        tc.optim_step({'learning_rate': 2e-3}).result()
        second = tc.forward_backward(datums, 'importance_sampling', loss_fn_config=cfg).result()['metrics']
        k = 'loss' if 'loss' in first else 'loss:sum'
        return first[k], second[k]

    nxt = two_more(trainer)                                       # what an uninterrupted run sees next
    rest = client.create_rest_client()
    runs = rest.list_training_runs()
    info = rest.get_weights_info(saved)
    # a fresh server (same persistence file and checkpoint directory), a fresh client
    client2 = TinkerClient(app=build_server(a.model, state_file).root, token='demo')
    resumed = client2.create_training_client_from_state_with_optimizer(saved)
    again = two_more(resumed)
    sampler = resumed.save_weights_and_get_sampling_client('after-resume')
    toks = sampler.sample(datums[0]['model_input']['tokens'][:8], num_samples=1, sampling_params={'max_tokens': 4}).result()['sequences'][0]['tokens']
    print(f'next two losses uninterrupted {nxt[0]:.5f} {nxt[1]:.5f}, after restart {again[0]:.5f} {again[1]:.5f}; sampled {toks}; metrics {sorted(metrics)}')
    return dict(losses=losses, metrics=metrics, saved=saved, runs=runs, info=info, next_uninterrupted=nxt, next_resumed=again, tokens=toks)


if __name__ == '__main__':
    main()
