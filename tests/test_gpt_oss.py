"""GPT-OSS family (attention sinks, alternating sliding-window layers, biases on projections / router / experts, softmax over
the top-k router logits, clamped gated expert unit) through training, expert parallelism, the sampler and the MXFP4 form of
the released expert tensors.  Parity with the Hugging Face implementation is in ``test_hf_parity.py``."""
import torch

from tests.dist_utils import run_ranks


def _batch(n=2, length=40, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 1024, (length + 1, ), generator=g)
        out.append({'input_ids': ids[:-1].tolist(), 'labels': ids[1:].tolist()})
    return out


def test_config_round_trip_and_training():
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models import preset
    from twinkle_b200.models.config import DecoderConfig
    cfg = preset('tiny-gpt-oss')
    back = DecoderConfig.from_hf(cfg.to_hf())
    for f in ('attn_sinks', 'o_proj_bias', 'router_linear_bias', 'expert_bias', 'expert_act', 'router_scoring', 'num_experts', 'moe_intermediate_size',
              'sliding_window', 'layer_types', 'attention_bias'):
        assert getattr(back, f) == getattr(cfg, f), f
    m = TransformersModel(model_id='tiny-gpt-oss', seed=0, device='cpu')
    names = {n for n, _ in m.model.named_parameters()}
    assert {'layers.0.self_attn.sinks', 'layers.0.self_attn.o_proj.bias', 'layers.0.mlp.gate.bias', 'layers.0.mlp.experts.gate_up_bias',
            'layers.0.mlp.experts.down_bias'} <= names
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    losses = []
    for _ in range(4):
        losses.append(m.forward_backward(inputs=_batch())['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < losses[0] - 0.2, losses
    sinks = dict(m.model.named_parameters())['layers.0.self_attn.sinks']
    assert float(sinks.detach().abs().sum()) > 0                       # the sink logits train


def _ep_worker(rank, world):
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    m = TransformersModel(model_id='tiny-gpt-oss', seed=0, device='cpu', device_mesh=DeviceMesh.from_sizes(dp_size=world, ep_size=world))
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    feats = _batch(n=2 * world)
    out = []
    for _ in range(3):
        out.append(m.forward_backward(inputs=feats[rank * 2:(rank + 1) * 2])['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    return out, tuple(m.model.layers[0].mlp.experts.gate_up_bias.shape)


def test_expert_parallel_keeps_the_expert_biases_with_their_experts():
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-gpt-oss', seed=0, device='cpu')
    m.set_optimizer('AdamW', lr=2e-3, weight_decay=0.0)
    ref = []
    for _ in range(3):
        ref.append(m.forward_backward(inputs=_batch(n=4))['loss'])
        m.clip_grad_and_step(max_grad_norm=1.0)
    res = run_ranks(_ep_worker, 2)
    assert all(shape == (4, 256) for _, shape in res)
    mean = [sum(r[0][i] for r in res) / 2 for i in range(3)]
    for a, b in zip(ref, mean):
        assert abs(a - b) < 2e-4, (ref, res)


def test_sampler_decodes_with_sinks_and_windows():
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.models.decoder import PackedBatch
    from twinkle_b200.sampler import TorchSampler
    s = TorchSampler(model_id='tiny-gpt-oss', weight_seed=0, enable_lora=False, device='cpu')
    with torch.no_grad():
        for n, p in s.model.named_parameters():
            if n.endswith('sinks'):
                p.copy_(torch.linspace(-1.0, 1.0, p.numel()))          # sinks that matter
    prompts = [{'input_ids': list(range(5, 27))}, {'input_ids': [11, 12]}]      # the first prompt is longer than the window
    resps = s.sample(prompts, SamplingParams(max_tokens=5, temperature=1.0, seed=4, logprobs=1))
    for p, r in zip(prompts, resps):
        seq = r.sequences[0]
        ids = torch.tensor(p['input_ids'] + seq.tokens)
        n = len(ids)
        with torch.no_grad():
            hidden = s.model(PackedBatch(ids, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))
            lp, _ = s.model.token_logprobs(hidden[:-1], ids[1:])
        assert torch.allclose(torch.tensor(seq.logprobs), lp[len(p['input_ids']) - 1:].float(), atol=2e-4)


def test_mxfp4_expert_tensors_load_like_their_bf16_form():
    """The released checkpoints store ``gate_up_proj`` / ``down_proj`` of the experts as 4-bit blocks with one shared exponent per
    32 values, laid out ``[E, out, in/32, 16]``; the bridge expands them and reorders gate / up rows."""
    from twinkle_b200.models import preset
    from twinkle_b200.models.bridge import hf_to_internal
    from twinkle_b200.utils.dequantizer import dequant_mxfp4
    cfg = preset('tiny-gpt-oss', hidden_size=64, moe_intermediate_size=32, num_experts=2)
    g = torch.Generator().manual_seed(0)
    blocks = torch.randint(0, 256, (2, 64, 2, 16), generator=g, dtype=torch.uint8)           # gate_up: out = 2·32, in = 64 = 2 blocks of 32
    scales = torch.randint(124, 130, (2, 64, 2), generator=g, dtype=torch.uint8)
    store = {'model.layers.0.mlp.experts.gate_up_proj_blocks': blocks, 'model.layers.0.mlp.experts.gate_up_proj_scales': scales}

    def get(name):
        if name not in store:
            raise KeyError(name)
        return store[name]

    got = hf_to_internal('layers.0.mlp.experts.gate_up_proj', cfg, get)
    full = dequant_mxfp4(blocks, scales).float()                   # [E, out, in] with gate / up rows alternating
    want = torch.cat([full[:, ::2], full[:, 1::2]], 1)
    assert got.shape == (2, 64, 64) and torch.equal(got.float(), want)
