"""LoRA pools are replicated over data-parallel ranks and trained with summed gradients: they must start equal on every
rank even when the ranks' random streams differ, and a released slot must be reset to the same values everywhere."""
import torch

from tests.dist_utils import run_ranks


def _adapter_spread(rank, world):
    import torch.distributed as dist
    from twinkle_b200.model import LoraConfig, MultiLoraTransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    torch.manual_seed(1000 + rank)                       # what happens when the launcher seeds ranks differently
    m = MultiLoraTransformersModel(model_id='tiny-dense', device_mesh=DeviceMesh.from_sizes(fsdp_size=world, dp_size=None), seed=0,
                                   max_loras=2, max_r=4)
    cfg = LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')
    m.add_adapter_to_model('a', cfg)
    m.set_optimizer('AdamW', lr=1e-2, adapter_name='a')
    g = torch.Generator().manual_seed(3 + rank)          # every rank trains on different rows
    ids = torch.randint(0, 512, (33, ), generator=g)
    feats = [{'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()}]

    def spread(name):
        worst = 0.0
        for k, v in sorted(m.get_state_dict(adapter_name=name).items()):
            parts = [torch.zeros_like(v) for _ in range(world)]
            dist.all_gather(parts, v.contiguous())
            worst = max(worst, max(float((p - parts[0]).abs().max()) for p in parts))
        return worst

    out = []
    for _ in range(2):
        m.forward_backward(inputs=feats, adapter_name='a')
        m.clip_grad_and_step(max_grad_norm=1.0, adapter_name='a')
        out.append(spread('a'))
    trained = float(sum(v.abs().sum() for k, v in m.get_state_dict(adapter_name='a').items() if 'lora_B' in k))
    m.remove_adapter('a')
    m.add_adapter_to_model('b', cfg)                     # takes the released slot
    m.set_optimizer('AdamW', lr=1e-2, adapter_name='b')
    out.append(spread('b'))
    fresh_b = float(sum(v.abs().sum() for k, v in m.get_state_dict(adapter_name='b').items() if 'lora_B' in k))
    return out, trained, fresh_b


def test_lora_pool_equal_across_ranks_despite_different_seeds():
    for spreads, trained, fresh_b in run_ranks(_adapter_spread, 2):
        assert spreads == [0.0, 0.0, 0.0], spreads
        assert trained > 0.0 and fresh_b == 0.0
