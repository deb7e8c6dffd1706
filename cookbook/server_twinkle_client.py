"""The native client twins against a one-process server: a server-side dataset and dataloader feed a LoRA run on the
remote model, the remote sampler generates with the freshly saved adapter.

    python cookbook/server_twinkle_client.py --backend native --model tiny-dense
    python cookbook/server_twinkle_client.py --backend mock                         # protocol only
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
    ap.add_argument('--epochs', type=int, default=2)
    a = ap.parse_args(argv)
    os.environ.setdefault('TWINKLE_DEFAULT_SAVE_DIR', tempfile.mkdtemp(prefix='tk_ckpt_'))
    from twinkle_b200.client import DataLoader, Dataset, MultiLoraTransformersModel, TorchSampler, TwinkleClient
    from twinkle_b200.server import ServerLauncher
    name = a.model if a.backend == 'native' else 'mock-base'
    server = ServerLauncher({
        'persistence': {'mode': 'memory'},
        'applications': [
            {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': [name]}},
            {'name': 'model', 'route_prefix': f'/model/{name}', 'import_path': 'model',
             'args': {'model_id': name, 'backend': 'mock' if a.backend == 'mock' else 'transformers', 'max_loras': 2}},
            {'name': 'sampler', 'route_prefix': f'/sampler/{name}', 'import_path': 'sampler',
             'args': {'model_id': name, 'sampler_type': 'mock' if a.backend == 'mock' else 'torch'}},
            {'name': 'processor', 'route_prefix': '/processor', 'import_path': 'processor', 'args': {}},
        ],
    })
    client = TwinkleClient(app=server.root, token='demo', heartbeat_interval=1.0)      # in-process transport; base_url=… for a real server
    rows = [{'messages': [{'role': 'user', 'content': f'say {i}'}, {'role': 'assistant', 'content': f'{i} ' * 4}]} for i in range(8)]
    ds = Dataset({'__class__': 'DatasetMeta', 'kwargs': {'data': rows}}, client=client)              # lives in the processor application
    dl = DataLoader(ds, batch_size=4, shuffle=False, client=client)
    model = MultiLoraTransformersModel(name, client=client)
    model.add_adapter_to_model('run', {'r': 8, 'lora_alpha': 16, 'target_modules': 'all-linear'})
    model.set_template('Template', adapter_name='run')
    model.set_optimizer('AdamW', lr=2e-3, adapter_name='run')
    losses = []
    for epoch in range(a.epochs):
        for batch in dl:
            out = model.forward_backward(inputs=batch, adapter_name='run')
            model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='run')
            losses.append(float(out['loss']))
    print('losses', [round(x, 4) for x in losses])
    path = model.save('final', adapter_name='run')
    sampler = TorchSampler(name, client=client)
    sampler.set_template('Template')
    res = sampler.sample([{'messages': [{'role': 'user', 'content': 'say 3'}]}], {'max_tokens': 4}, adapter_path=path if a.backend == 'native' else None)
    print('sampled', res[0]['sequences'][0]['tokens'], 'from', path)
    runs = client.list_training_runs()
    client.close()
    return dict(losses=losses, path=path, tokens=res[0]['sequences'][0]['tokens'], runs=runs)


if __name__ == '__main__':
    main()
