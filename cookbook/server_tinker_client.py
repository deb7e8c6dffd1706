"""One-process server (gateway + model + sampler apps) driven through the Tinker-style client: create a LoRA training
client, run forward_backward / optim_step futures, save weights for the sampler and sample from them.

    python cookbook/server_tinker_client.py --backend native --model tiny-dense    # real engine (CPU or GPU)
    python cookbook/server_tinker_client.py --backend mock                         # protocol only
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--backend', default='mock', choices=['mock', 'native'])
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=3)
    a = ap.parse_args(argv)
    os.environ.setdefault('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_ckpt_'))
    os.environ.setdefault('TWINKLE_POLL_INTERVAL', '0.02')
    from twinkle_b200.client import TinkerClient
    from twinkle_b200.server import ServerLauncher
    name = a.model if a.backend == 'native' else 'mock-base'
    cfg = {
        'persistence': {'mode': 'memory'},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': [name]}},
            {'name': 'model', 'route_prefix': f'/model/{name}', 'import_path': 'model',
             'args': {'model_id': name, 'backend': 'mock' if a.backend == 'mock' else 'transformers', 'max_loras': 2}},
            {'name': 'sampler', 'route_prefix': f'/sampler/{name}', 'import_path': 'sampler',
             'args': {'model_id': name, 'sampler_type': 'mock' if a.backend == 'mock' else 'torch'}},
        ],
    }
    server = ServerLauncher(cfg)
    # in-process transport (no socket); ServerLauncher(cfg).launch() serves the same app over HTTP with uvicorn
    client = TinkerClient(app=server.root, token='demo')
    trainer = client.create_lora_training_client(name, rank=8)
    datum = {'model_input': {'tokens': [5, 6, 7, 8, 9, 10]},
             'loss_fn_inputs': {'target_tokens': {'data': [6, 7, 8, 9, 10, 11]}, 'weights': {'data': [0, 1, 1, 1, 1, 1]}}}
    losses = []
    for step in range(a.steps):
        out = trainer.forward_backward([datum, datum]).result()
        trainer.optim_step({'learning_rate': 1e-3}).result()
        lp = [x for d in out['loss_fn_outputs'] for x in d['logprobs']['data'][1:]]
        losses.append(-sum(lp) / max(len(lp), 1))
        print(f'step {step} mean nll {losses[-1]:.4f}')
    saved = trainer.save_weights_for_sampler('demo').result()
    sampler = client.create_sampling_client(name, saved['path'])
    res = sampler.sample([5, 6, 7], num_samples=2, sampling_params={'max_tokens': 4}).result()
    print('sampled', [s['tokens'] for s in res['sequences']])
    return losses


if __name__ == '__main__':
    main()
