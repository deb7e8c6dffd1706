"""Router replay for MoE policy-gradient training: the sampler records which experts every token used, and the trainer
forces the same routing when it recomputes log-probs, so old and new log-probs differ only through the weights.

    python cookbook/moe_routing_replay.py
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-moe')
    ap.add_argument('--max-tokens', type=int, default=8)
    a = ap.parse_args(argv)
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.sampler import TorchSampler
    model = TransformersModel(model_id=a.model, seed=0)
    sampler = TorchSampler(model_id=a.model, weight_seed=0, enable_return_routed_experts=True)
    vocab = min(model.config.vocab_size, 1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, vocab, (9, ), generator=g).tolist() for _ in range(3)]
    resps = sampler.sample([{'input_ids': p} for p in prompts], SamplingParams(max_tokens=a.max_tokens, temperature=1.0, logprobs=1))
    feats = [r.sequences[0].new_input_feature for r in resps]
    assert all(f.get('routed_experts') is not None for f in feats), 'the sampler did not return its routing'
    lens = [len(f['input_ids']) for f in feats]
    recorded = [f['routed_experts'][0].shape[0] for f in feats]           # one row per token the sampler fed: length - 1
    keep = torch.cat([torch.arange(n) < r for n, r in zip(lens, recorded)])   # rows of the packed batch that are replayed

    def routing(inputs):
        model.model.set_record_routing(True)
        return [torch.as_tensor(x).cpu() for x in model.forward_only(inputs=inputs)['routed_experts']]

    # 1) with replay the trainer uses exactly the experts the sampler used
    sampled = [torch.cat([f['routed_experts'][l] for f in feats], 0) for l in range(len(feats[0]['routed_experts']))]
    replayed = routing(feats)
    matches_sampler = all(torch.equal(a[keep[:a.shape[0]]][:, :], b) for a, b in zip(replayed, sampled))
    # 2) after the router's weights change, free routing picks other experts; replay does not
    with torch.no_grad():
        for n, p in model.model.named_parameters():
            if n.endswith('gate.weight'):
                p.add_(0.5 * torch.randn(p.shape, generator=g).to(p))
    replay2 = routing(feats)
    free2 = routing([{k: v for k, v in f.items() if k != 'routed_experts'} for f in feats])
    same_replay = all(torch.equal(x[keep], y[keep]) for x, y in zip(replayed, replay2))
    same_free = all(torch.equal(x[keep], y[keep]) for x, y in zip(replayed, free2))
    print(f'replay reproduces the sampler\'s routing: {matches_sampler}; kept after the router changed: {same_replay}; without replay: {same_free}')
    return dict(matches_sampler=matches_sampler, replay_kept=same_replay, free_kept=same_free, layers=len(replayed), recorded=recorded, lens=lens)


if __name__ == '__main__':
    main()
