"""Embedding model training: last-token pooled embeddings, in-batch contrastive (InfoNCE) loss over (query, positive)
pairs, retrieval accuracy before and after.

    python cookbook/embedding_infonce.py --steps 20
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.nn.functional as F


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='tiny-dense')
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--pairs', type=int, default=8)
    a = ap.parse_args(argv)
    from twinkle_b200.model import TransformersModel
    model = TransformersModel(model_id=a.model, task='embedding', seed=0)
    model.set_optimizer('AdamW', lr=1e-3)
    model.set_loss('InfonceLoss', temperature=0.1, group_size=2, cross_rank=False)
    vocab = min(model.config.vocab_size, 1024)
    g = torch.Generator().manual_seed(0)
    rows = []
    for _ in range(a.pairs):  # a positive shares its topic tokens with the query, in another order and with noise around
        topic = torch.randint(3, vocab, (6, ), generator=g)
        q = torch.cat([topic, torch.randint(3, vocab, (3, ), generator=g)])
        d = torch.cat([torch.randint(3, vocab, (4, ), generator=g), topic[torch.randperm(6, generator=g)]])
        rows += [{'input_ids': q.tolist()}, {'input_ids': d.tolist()}]          # rows alternate query, positive

    def accuracy():
        emb = F.normalize(model.forward_only(inputs=rows)['embeddings'].float(), dim=-1)
        sim = emb[0::2] @ emb[1::2].t()
        return float((sim.argmax(-1) == torch.arange(sim.shape[0], device=sim.device)).float().mean())

    acc0 = accuracy()
    losses = []
    for step in range(a.steps):
        out = model.forward_backward(inputs=rows)
        model.clip_grad_and_step(max_grad_norm=1.0)
        losses.append(float(out['loss']))
    acc1 = accuracy()
    print(f'infonce loss {losses[0]:.4f} -> {losses[-1]:.4f}; retrieval accuracy {acc0:.2f} -> {acc1:.2f}')
    return dict(losses=losses, acc_before=acc0, acc_after=acc1)


if __name__ == '__main__':
    main()
