"""Qwen2-VL family: the vision tower, the (time, height, width) rotary positions, preprocessing, the chat template's image
placeholders, packed batches with images, training through the public model API, and checkpoints in both directions —
with ``transformers``' implementation as the oracle where it is installed."""
import json

import numpy as np
import pytest
import torch

from twinkle_b200.models.vision import VisionConfig, VisionTower, mrope_tables, patchify, preprocess_image, rope_index, smart_resize

VC = dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2, in_channels=3)


VC25 = dict(depth=3, hidden_size=64, out_hidden_size=128, intermediate_size=96, num_heads=4, patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
            in_channels=3, window_size=56, fullatt_block_indexes=[1])     # 2 × 2 merge groups per window; block 1 attends over the whole frame


VC3 = dict(depth=3, hidden_size=64, out_hidden_size=128, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
           in_channels=3, num_position_embeddings=64, deepstack_visual_indexes=[0, 1])    # position table 8 × 8; two deep-stack taps


VC35 = dict(depth=3, hidden_size=64, out_hidden_size=128, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
            in_channels=3, num_position_embeddings=64)      # the Qwen3-VL tower without deep-stack taps


def _hf(family='qwen2_vl'):
    T = pytest.importorskip('transformers')
    try:
        if family == 'qwen3_5':     # hybrid decoder (Gated DeltaNet + gated attention, rotary on a quarter of the head) behind the tower
            text = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=64, max_position_embeddings=512, tie_word_embeddings=False, linear_num_key_heads=2, linear_num_value_heads=4,
                        linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
                        layer_types=['linear_attention', 'full_attention', 'linear_attention', 'full_attention'],
                        rope_parameters={'rope_type': 'default', 'rope_theta': 10000.0, 'partial_rotary_factor': 0.25, 'mrope_section': [2, 3, 3],
                                         'mrope_interleaved': True})
            cfg = T.Qwen3_5Config(text_config=text, vision_config=VC35, image_token_id=500, video_token_id=501, vision_start_token_id=502,
                                  vision_end_token_id=503)
            torch.manual_seed(0)
            hf = T.Qwen3_5ForConditionalGeneration(cfg).float().eval()
            for n, p in hf.named_parameters():
                if p.dim() == 1 and 'A_log' not in n and 'dt_bias' not in n:
                    torch.nn.init.normal_(p, 0.0 if ('bias' in n or ('norm' in n and 'visual' not in n and 'linear_attn.norm' not in n)) else 1.0, 0.1)
            return T, cfg, hf
        conf, cls, vc = {'qwen2_vl': (T.Qwen2VLConfig, T.Qwen2VLForConditionalGeneration, VC),
                         'qwen2_5_vl': (T.Qwen2_5_VLConfig, T.Qwen2_5_VLForConditionalGeneration, VC25),
                         'qwen3_vl': (T.Qwen3VLConfig, T.Qwen3VLForConditionalGeneration, VC3)}[family]
        text = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3 if family == 'qwen3_vl' else 2, num_attention_heads=4,
                    num_key_value_heads=2, max_position_embeddings=512, rope_theta=10000.0, tie_word_embeddings=False,
                    rope_scaling={'type': 'mrope', 'mrope_section': [4, 6, 6]})
        if family == 'qwen3_vl':
            text.update(head_dim=32, rope_scaling={'rope_type': 'default', 'mrope_section': [4, 6, 6], 'mrope_interleaved': True})
        cfg = conf(text_config=text, vision_config=vc, image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
        torch.manual_seed(0)
        hf = cls(cfg).float().eval()
        for n, p in hf.named_parameters():   # non-trivial norms and biases so that a dropped or swapped tensor shows
            if p.dim() == 1:
                torch.nn.init.normal_(p, 1.0 if ('norm' in n or 'ln_q' in n) and 'bias' not in n else 0.0, 0.1)
        return T, cfg, hf
    except Exception as e:
        pytest.skip(f'this transformers build cannot make a tiny {family}: {type(e).__name__}: {e}')


def _sample(grid=((1, 4, 6), (1, 2, 2)), patch=14):
    grid = torch.tensor(grid)
    n1, n2 = (int(g[0] * g[1] * g[2]) // 4 for g in grid)
    ids = [5, 6, 502] + [500] * n1 + [503, 7, 8, 502] + [500] * n2 + [503, 9, 10, 11]
    pix = torch.randn(int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * patch * patch, generator=torch.Generator().manual_seed(1))
    return ids, grid, pix


def test_positions_and_tables_by_hand():
    ids = [1, 2, 9, 9, 9, 9, 9, 9, 3, 4]                       # one image with a merged 2 × 3 grid
    pos = rope_index(ids, [(1, 4, 6)], image_token_id=9)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6 and pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8:].tolist() == [[5, 6]] * 3                  # text resumes after the largest position used (2 + 3)
    with pytest.raises(ValueError):
        rope_index(ids[:5], [(1, 4, 6)], 9)
    with pytest.raises(ValueError):
        rope_index([1, 2, 3], [(1, 4, 6)], 9)
    same = torch.arange(7).expand(3, -1)
    cos, sin = mrope_tables(same, 16, 1e4, [2, 3, 3])
    inv = 1.0 / (1e4**(torch.arange(0, 16, 2).float() / 16))
    assert torch.allclose(cos, (torch.arange(7).float()[:, None] * inv).cos())      # equal components = ordinary RoPE
    mixed = torch.tensor([[1], [10], [100]])
    cos, _ = mrope_tables(mixed, 16, 1e4, [2, 3, 3])
    want = torch.cat([1 * inv[:2], 10 * inv[2:5], 100 * inv[5:]]).cos()
    assert torch.allclose(cos[0], want)
    assert smart_resize(100, 150) == (112, 140) and smart_resize(10, 10)[0] % 28 == 0 and smart_resize(5000, 5000)[0] * smart_resize(5000, 5000)[1] <= 14 * 14 * 4 * 1280
    frames = torch.arange(3 * 28 * 56, dtype=torch.float32).view(1, 3, 28, 56)
    flat, g = patchify(frames, VisionConfig(**VC))
    assert g == (1, 2, 4) and flat.shape == (8, 1176)
    # patches come merge-group by merge-group: rows 0-3 are the left 2 × 2 block, and the single frame fills both temporal slots
    first = flat[1].view(3, 2, 14, 14)
    assert torch.equal(first[:, 0], frames[0, :, 0:14, 14:28]) and torch.equal(first[:, 0], first[:, 1])
    assert torch.equal(flat[2].view(3, 2, 14, 14)[:, 0], frames[0, :, 14:28, 0:14])


@pytest.mark.parametrize('family', ['qwen2_vl', 'qwen2_5_vl', 'qwen3_vl', 'qwen3_5'])
def test_tower_positions_and_full_model_match_transformers(family, tmp_path):
    T, cfg, hf = _hf(family)
    from twinkle_b200.models.bridge import hf_to_internal
    from twinkle_b200.models.config import DecoderConfig
    from twinkle_b200.models.decoder import PackedBatch, build_model
    ids, grid, pix = (_sample() if family == 'qwen2_vl' else _sample(((1, 6, 10), (1, 8, 6))) if family == 'qwen2_5_vl' else   # several windows, ragged edges
                      _sample(((1, 4, 6), (1, 6, 4)), patch=16))       # Qwen3-VL and Qwen3.5: 16-pixel patches
    tower = VisionTower(VisionConfig.from_hf(cfg.vision_config.to_dict())).float().eval()
    tower.load_state_dict({k[len('model.visual.'):]: v for k, v in hf.state_dict().items() if k.startswith('model.visual.')})
    ids_t = torch.tensor([ids])
    mm = (ids_t == 500).int()
    with torch.no_grad():
        try:
            want_feats = hf.model.visual(pix, grid_thw=grid)
            want_pos = hf.model.get_rope_index(ids_t, mm_token_type_ids=mm, image_grid_thw=grid)[0][:, 0]
            mine = rope_index(ids, grid.tolist(), 500)
            want = hf(input_ids=ids_t, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=mm, position_ids=mine[:, None, :]).logits[0]
        except TypeError as e:
            pytest.skip(f'different call signature in this transformers build: {e}')
        deep_want = list(getattr(want_feats, 'deepstack_features', None) or [])
        want_feats = getattr(want_feats, 'pooler_output', want_feats[0] if isinstance(want_feats, tuple) else want_feats)
        got_feats, deep_got = tower(pix, grid, return_deepstack=True)
        assert torch.allclose(got_feats, want_feats, atol=1e-5) and len(deep_got) == len(deep_want) == (2 if family == 'qwen3_vl' else 0)
        assert all(torch.allclose(a, b, atol=1e-5) for a, b in zip(deep_got, deep_want))
    # height and width rows always agree. The time row of an image is its start position, as in the model's original
    # implementation; this transformers build multiplies it by tokens_per_second for Qwen2.5-VL images, so it is compared
    # for Qwen2-VL only (the logits above were computed from the same positions on both sides)
    assert torch.equal(mine[1:], want_pos[1:]) and (family == 'qwen2_5_vl' or torch.equal(mine, want_pos))
    dc = DecoderConfig.from_hf(cfg.to_dict())
    assert dc.mrope_section == ([2, 3, 3] if family == 'qwen3_5' else [4, 6, 6]) and dc.image_token_id == 500 and dc.rope_scaling is None
    assert (dc.attention_bias, dc.qk_norm, dc.mrope_interleaved) == ((False, True, True) if family in ('qwen3_vl', 'qwen3_5') else (True, False, False))
    m = build_model(dc)
    sd = hf.state_dict()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(hf_to_internal(n, dc, lambda k: sd[k]))
        n = len(ids)
        got = m.logits(m(PackedBatch(torch.tensor(ids), rope_index(ids, grid.tolist(), 500), torch.tensor([0, n], dtype=torch.int32), n,
                                     pixel_values=pix, image_grid_thw=grid)))
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # the config goes out in the family's own layout and comes back unchanged
    dc.save_pretrained(str(tmp_path))
    written = json.load(open(str(tmp_path / 'config.json')))
    assert written['model_type'] == family and written['architectures'][0].endswith('ForConditionalGeneration')
    assert DecoderConfig.from_pretrained(str(tmp_path)).vision == dc.vision


def test_preprocessing_matches_the_hf_image_processor():
    T = pytest.importorskip('transformers')
    Image = pytest.importorskip('PIL.Image')
    try:
        ip = T.Qwen2VLImageProcessor(min_pixels=56 * 56, max_pixels=14 * 14 * 4 * 1280)
    except Exception as e:
        pytest.skip(str(e))
    vc = VisionConfig(**VC)
    for shape, tol in (((84, 112, 3), 1e-5), ((100, 150, 3), 0.02), ((30, 500, 3), 0.02)):   # no resize: exact; resized: one 8-bit level
        arr = (np.random.RandomState(0).rand(*shape) * 255).astype('uint8')
        out = ip(images=[Image.fromarray(arr)], return_tensors='pt')
        pv, g = preprocess_image(arr, vc)
        assert out['image_grid_thw'].tolist() == [list(g)] and float((out['pixel_values'] - pv).abs().max()) <= tol


def test_template_processor_training_and_checkpoints(tmp_path):
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import DecoderConfig
    from twinkle_b200.processor import InputProcessor
    m = TransformersModel(model_id='tiny-vl', seed=0)
    m.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    g = torch.Generator().manual_seed(0)
    img1, img2 = torch.rand(3, 60, 90, generator=g) * 255, (torch.rand(40, 40, 3, generator=g) * 255).numpy()
    trajs = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': img1}, {'type': 'text', 'text': 'what is this?'}]},
                           {'role': 'assistant', 'content': 'a cat'}]},
             {'messages': [{'role': 'user', 'content': 'hello'}, {'role': 'assistant', 'content': 'hi there'}]},
             {'messages': [{'role': 'user', 'content': 'compare <image> with text'}, {'role': 'assistant', 'content': 'ok'}], 'images': [img2]}]
    tpl = m._group(None).template
    f = tpl.encode(trajs[0])
    t, h, w = f['image_grid_thw'][0]
    assert (t, h, w) == (1, 4, 6) and f['input_ids'].count(tpl.image_token_id) == t * h * w // 4 and f['pixel_values'].shape == (24, 1176)
    assert f['mrope_position_ids'].shape == (3, len(f['input_ids'])) and f['position_ids'] == list(range(len(f['input_ids'])))
    assert all(l == -100 for i, l in zip(f['input_ids'], f['labels']) if i == tpl.image_token_id)   # no loss on placeholders
    assert 'pixel_values' not in tpl.encode(trajs[1])
    with pytest.raises(ValueError):
        tpl.encode({'messages': [{'role': 'user', 'content': '<image>'}], 'images': []})
    mb, = InputProcessor()(tpl.batch_encode(trajs))
    T_ = mb.input_ids.numel()
    assert mb.extras['mrope_position_ids'].shape == (3, T_) and mb.extras['image_grid_thw'].tolist() == [[1, 4, 6], [1, 4, 4]]
    assert mb.extras['pixel_values'].shape[0] == 24 + 16 and mb.cu_seqlens.numel() == 4   # 40 × 40 is scaled up to the minimum pixel count
    a, b = int(mb.cu_seqlens[1]), int(mb.cu_seqlens[2])
    assert mb.extras['mrope_position_ids'][:, a:b].tolist() == [list(range(b - a))] * 3            # the text-only sequence in the middle

    m.set_optimizer('AdamW', lr=1e-2)
    w0 = m.model.visual.patch_embed.proj.weight.detach().clone()
    losses = []
    for _ in range(4):
        losses.append(float(m.forward_backward(inputs=trajs)['loss']))
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < 0.6 * losses[0] and not torch.equal(w0, m.model.visual.patch_embed.proj.weight)   # the tower trains too
    out = m.save('ck', str(tmp_path))
    cfg = json.load(open(out + '/config.json'))
    assert cfg['model_type'] == 'qwen2_vl' and cfg['vision_config']['embed_dim'] == 64 and cfg['text_config']['rope_scaling']['mrope_section'] == [8, 12, 12]
    assert DecoderConfig.from_pretrained(out).vision == m.config.vision
    m2 = TransformersModel(model_id=out, seed=3)
    m2.set_template('Qwen2VLTemplate', vision_config=m2.config.vision, max_length=4096)
    la, lb = m.forward_only(inputs=trajs), m2.forward_only(inputs=trajs)
    assert torch.allclose(torch.as_tensor(la['logps']).float(), torch.as_tensor(lb['logps']).float(), atol=1e-5)
    T = pytest.importorskip('transformers')
    try:
        back = T.Qwen2VLForConditionalGeneration.from_pretrained(out).float().eval()
    except Exception as e:
        pytest.skip(f'transformers could not load the export: {type(e).__name__}: {e}')
    ids = torch.tensor([f['input_ids']])
    with torch.no_grad():
        try:
            theirs = back(input_ids=ids, pixel_values=f['pixel_values'], image_grid_thw=torch.tensor(f['image_grid_thw']),
                          mm_token_type_ids=(ids == tpl.image_token_id).int()).logits[0]
        except TypeError as e:
            pytest.skip(str(e))
        ours = torch.as_tensor(m.forward_only(inputs=[trajs[0]], return_logits=True)['logits']).float().reshape(-1, theirs.shape[-1])[:theirs.shape[0]]
    assert torch.allclose(ours, theirs, atol=5e-5), float((ours - theirs).abs().max())


def _vl_trajs():
    g = torch.Generator().manual_seed(5)
    mk = lambda h, w: torch.rand(3, h, w, generator=g) * 255  # noqa: E731
    return [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': mk(60, 90)}, {'type': 'text', 'text': 'what is this?'}]},
                          {'role': 'assistant', 'content': 'a cat on a mat'}]},
            {'messages': [{'role': 'user', 'content': [{'type': 'text', 'text': 'and this one'}, {'type': 'image', 'image': mk(56, 56)}]},
                          {'role': 'assistant', 'content': 'a dog'}]}]


def _vl_curve(rank, world, steps, sp=1, preset='tiny-vl', cp=False):
    import torch.distributed as dist
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.utils.device_mesh import DeviceMesh
    if cp:
        mesh = DeviceMesh.from_sizes(dp_size=1, cp_size=world)
    else:
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=None, ulysses_size=sp if sp > 1 else None) if world > 1 else DeviceMesh.from_sizes(dp_size=1)
    m = TransformersModel(model_id=preset, device_mesh=mesh, seed=0)
    m.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    m.set_optimizer('AdamW', lr=3e-3, weight_decay=0.0)
    trajs = _vl_trajs()
    sl = mesh.get_slice(len(trajs), mesh.get_data_rank_from_global_rank(rank))
    curve = []
    for _ in range(steps):
        out = m.forward_backward(inputs=trajs[sl])
        m.clip_grad_and_step(max_grad_norm=1.0)
        t = torch.tensor([out['loss'] * out['num_tokens'], out['num_tokens']], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
            t = t / sp  # sequence-parallel peers report the same data group's numbers
        curve.append(float(t[0] / t[1]))
    return curve


def test_sharded_training_with_images_matches_one_process():
    """Two gloo ranks, parameters (vision tower included, in the root unit) sharded over both, one image sample each:
    the global loss curve equals the single-process run on both samples."""
    from tests.dist_utils import run_ranks
    single = _vl_curve(0, 1, 3)
    multi = run_ranks(_vl_curve, 2, 3)
    assert single[-1] < single[0]
    for c in multi:
        for a, b in zip(single, c):
            assert abs(a - b) < 3e-4, (single, c)


def test_clevr_rows_flow_through_template_and_reward():
    from twinkle_b200.preprocessor import CLEVRProcessor
    from twinkle_b200.reward import MultiModalAccuracyReward
    from twinkle_b200.template import template_mapping
    img = torch.rand(3, 56, 56) * 255
    row, = CLEVRProcessor()([{'problem': 'How many cubes?', 'solution': '<answer> 3 </answer>', 'image': img}])
    assert row['images'][0] is img and row['user_data']['ground_truth'] == '3'
    tpl = template_mapping['Qwen2VLTemplate'](model_id=None, vision_config=VC, max_length=4096)
    f = tpl.encode(row)
    assert f['image_grid_thw'] == [[1, 4, 4]] and f['input_ids'].count(tpl.image_token_id) == 4
    text = tpl.decode(f['input_ids'], skip_special_tokens=False)
    assert text.index('<|vision_start|>') < text.index('How many cubes?')          # an unmarked image precedes the question
    done = dict(row, messages=row['messages'][:1] + [{'role': 'assistant', 'content': 'I count. <answer>3</answer>'}])
    assert MultiModalAccuracyReward()([done]) == [1.0]


def test_sampler_takes_images_and_continues_positions():
    """Sampled log-probs after a prompt with an image equal one teacher-forced forward over prompt ⊕ tokens with the
    (time, height, width) positions continued; the returned feature is ready for training."""
    from twinkle_b200.data_format import SamplingParams
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.sampler import TorchSampler
    s = TorchSampler(model_id='tiny-vl', weight_seed=0, enable_lora=False)
    s.set_template('Qwen2VLTemplate', vision_config=s.config.vision, max_length=4096)
    img = torch.rand(3, 56, 84, generator=torch.Generator().manual_seed(4)) * 255
    trajs = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': img}, {'type': 'text', 'text': 'describe'}]}]},
             {'messages': [{'role': 'user', 'content': 'no image here'}]}]
    resps = s.sample(trajs, SamplingParams(max_tokens=5, temperature=1.0, seed=2, logprobs=1))
    f = resps[0].sequences[0].new_input_feature
    n_new = len(resps[0].sequences[0].tokens)
    assert f['mrope_position_ids'].shape[1] == len(f['input_ids']) and f['pixel_values'].shape[0] == 4 * 6
    tail = f['mrope_position_ids'][:, -n_new:]
    assert torch.equal(tail[0], tail[1]) and torch.equal(tail[0], tail[2]) and int(tail[0, 0]) < len(f['input_ids']) - n_new   # compressed by the image
    assert 'pixel_values' not in resps[1].sequences[0].new_input_feature
    m = TransformersModel(model_id='tiny-vl', seed=0)                        # same preset and seed = same weights as the sampler
    for r in resps:
        q = r.sequences[0]
        out = m.forward_only(inputs=[q.new_input_feature])
        lp = torch.as_tensor(out['logps']).float().reshape(-1)
        labels = torch.tensor(q.new_input_feature['labels'])
        got = lp[:labels.numel()][labels != -100]
        assert torch.allclose(got, torch.tensor(q.logprobs), atol=2e-4), (got, q.logprobs)


def test_video_frames_match_transformers_qwen2_vl():
    """A video part (list of frames): two frames share a temporal patch, positions advance along time per patch-pair, and the
    whole model's logits equal ``transformers``' when it is given the same patches as ``pixel_values_videos``."""
    T, cfg, hf = _hf('qwen2_vl')
    from twinkle_b200.models.bridge import hf_to_internal
    from twinkle_b200.models.config import DecoderConfig
    from twinkle_b200.models.decoder import PackedBatch, build_model
    from twinkle_b200.models.vision import preprocess_video
    g = torch.Generator().manual_seed(7)
    frames = [torch.rand(3, 56, 84, generator=g) * 255 for _ in range(3)]            # odd count: the last frame is repeated
    pix, grid = preprocess_video(frames, VisionConfig(**VC), min_pixels=56 * 56)
    assert grid == (2, 4, 6) and pix.shape == (48, 1176)
    n_vid = 2 * 4 * 6 // 4
    ids = [5, 502] + [501] * n_vid + [503, 7, 8]
    pos = rope_index(ids, [grid], 500, video_token_id=501)
    assert pos[0, 2:2 + n_vid].tolist() == [2] * 6 + [3] * 6 and pos[:, -2:].tolist() == [[6, 7]] * 3      # max(t, h/2, w/2) = 3 → text resumes at 2 + 3 + 1
    ids_t, grid_t = torch.tensor([ids]), torch.tensor([grid])
    with torch.no_grad():
        try:
            want = hf(input_ids=ids_t, pixel_values_videos=pix, video_grid_thw=grid_t, mm_token_type_ids=(ids_t == 501).int() * 2,
                      position_ids=pos[:, None, :]).logits[0]
        except TypeError as e:
            pytest.skip(str(e))
    dc = DecoderConfig.from_hf(cfg.to_dict())
    m = build_model(dc)
    sd = hf.state_dict()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(hf_to_internal(n, dc, lambda k: sd[k]))
        got = m.logits(m(PackedBatch(torch.tensor(ids), pos, torch.tensor([0, len(ids)], dtype=torch.int32), len(ids), pixel_values=pix, image_grid_thw=grid_t)))
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    from twinkle_b200.template import template_mapping
    tpl = template_mapping['Qwen2VLTemplate'](model_id=None, vision_config=VC, max_length=4096)
    f = tpl.encode({'messages': [{'role': 'user', 'content': [{'type': 'video', 'video': frames}, {'type': 'text', 'text': 'what happens?'}]},
                                 {'role': 'assistant', 'content': 'it moves'}]})
    assert f['input_ids'].count(tpl.video_token_id) == f['pixel_values'].shape[0] // 4 and f['mrope_position_ids'].shape[1] == len(f['input_ids'])


def test_images_travel_as_data_urls_over_http():
    from twinkle_b200.client import _wire
    from twinkle_b200.models.vision import preprocess_image
    from twinkle_b200.utils.misc import image_to_data_url
    img = (torch.rand(3, 56, 84, generator=torch.Generator().manual_seed(1)) * 255).round()
    url = image_to_data_url(img)
    assert url.startswith('data:image/png;base64,') and image_to_data_url('file.png') == 'file.png'
    a, ga = preprocess_image(img, VisionConfig(**VC))
    b, gb = preprocess_image(url, VisionConfig(**VC))                 # what the server does with the wire form
    assert ga == gb and torch.equal(a, b)                             # PNG is lossless for 8-bit pixels
    body = _wire({'inputs': [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': img}, {'type': 'text', 'text': 'hi'}]}]},
                             {'messages': [{'role': 'user', 'content': '<image> hi'}], 'images': [img.permute(1, 2, 0).numpy()]}]})
    part = body['inputs'][0]['messages'][0]['content'][0]
    assert part['image'] == url and body['inputs'][1]['images'][0] == url and body['inputs'][0]['messages'][0]['content'][1] == {'type': 'text', 'text': 'hi'}


def test_qwen3_vl_trains_through_the_public_api_and_exports(tmp_path):
    """Deep-stack features pass through the engine's layer loop (and their mergers train); the saved checkpoint reloads here
    and in ``transformers`` with the same outputs."""
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-vl3', seed=0)
    m.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    g = torch.Generator().manual_seed(0)
    trajs = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': torch.rand(3, 64, 96, generator=g) * 255}, {'type': 'text', 'text': 'what?'}]},
                           {'role': 'assistant', 'content': 'a red ball'}]},
             {'messages': [{'role': 'user', 'content': 'plain text'}, {'role': 'assistant', 'content': 'yes'}]}]
    tpl = m._group(None).template
    f = tpl.encode(trajs[0])
    assert f['image_grid_thw'] == [[1, 4, 6]] and f['pixel_values'].shape == (24, 3 * 2 * 16 * 16)
    m.set_optimizer('AdamW', lr=1e-2)
    w0 = m.model.visual.deepstack_merger_list[1].linear_fc2.weight.detach().clone()
    losses = []
    for _ in range(4):
        losses.append(float(m.forward_backward(inputs=trajs)['loss']))
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < 0.7 * losses[0] and not torch.equal(w0, m.model.visual.deepstack_merger_list[1].linear_fc2.weight)
    out = m.save('ck', str(tmp_path))
    cfg = json.load(open(out + '/config.json'))
    assert cfg['model_type'] == 'qwen3_vl' and cfg['text_config']['rope_scaling']['mrope_interleaved'] is True
    m2 = TransformersModel(model_id=out, seed=1)
    m2.set_template('Qwen2VLTemplate', vision_config=m2.config.vision, max_length=4096)
    la, lb = m.forward_only(inputs=trajs), m2.forward_only(inputs=trajs)
    assert torch.allclose(torch.as_tensor(la['logps']).float(), torch.as_tensor(lb['logps']).float(), atol=1e-5)
    T = pytest.importorskip('transformers')
    try:
        back = T.Qwen3VLForConditionalGeneration.from_pretrained(out).float().eval()
        ids = torch.tensor([f['input_ids']])
        with torch.no_grad():
            theirs = back(input_ids=ids, pixel_values=f['pixel_values'], image_grid_thw=torch.tensor(f['image_grid_thw']),
                          mm_token_type_ids=(ids == tpl.image_token_id).int()).logits[0]
    except (TypeError, AttributeError, OSError, ValueError) as e:
        pytest.skip(f'transformers could not run the export: {type(e).__name__}: {e}')
    ours = torch.as_tensor(m.forward_only(inputs=[trajs[0]], return_logits=True)['logits']).float().reshape(-1, theirs.shape[-1])[:theirs.shape[0]]
    assert torch.allclose(ours, theirs, atol=5e-5), float((ours - theirs).abs().max())


def test_sequence_parallel_split_of_image_batches_matches_one_process():
    """Two gloo ranks that split every sequence (Ulysses): each runs the tower on all images and keeps the features of the
    placeholder tokens in its half of the row; deep-stack features (Qwen3-VL preset) follow the same rows."""
    from tests.dist_utils import run_ranks
    from twinkle_b200.processor import InputProcessor
    from twinkle_b200.template import template_mapping
    tpl = template_mapping['Qwen2VLTemplate'](model_id=None, vision_config=VC, max_length=4096)
    feats = tpl.batch_encode(_vl_trajs())
    full, = InputProcessor()(feats)
    halves = [InputProcessor(sp_size=2, sp_rank=r)(feats)[0] for r in (0, 1)]
    n_ph = int((full.input_ids == tpl.image_token_id).sum())
    assert torch.equal(torch.cat([h.extras['vision_rows'] for h in halves]), torch.arange(n_ph))
    assert torch.equal(torch.cat([h.extras['mrope_position_ids'] for h in halves], 1)[:, :full.input_ids.numel()], full.extras['mrope_position_ids'])
    for preset in ('tiny-vl', 'tiny-vl3'):
        single = _vl_curve(0, 1, 2, 1, preset)
        for c in run_ranks(_vl_curve, 2, 2, 2, preset):
            for a, b in zip(single, c):
                assert abs(a - b) < 3e-4, (preset, single, c)


def test_qwen3_vl_moe_checkpoint_with_fused_experts(tmp_path):
    """Mixture-of-experts language model under the Qwen3-VL tower; the checkpoint keeps the experts as fused 3-D tensors."""
    T = pytest.importorskip('transformers')
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.decoder import PackedBatch
    try:
        cfg = T.Qwen3VLMoeConfig(
            text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=32, max_position_embeddings=512, rope_theta=10000.0, tie_word_embeddings=False, num_experts=4, num_experts_per_tok=2,
                             moe_intermediate_size=48, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
                             rope_scaling={'rope_type': 'default', 'mrope_section': [4, 6, 6], 'mrope_interleaved': True}),
            vision_config=dict(VC3, depth=2, deepstack_visual_indexes=[0]), image_token_id=500, video_token_id=501, vision_start_token_id=502,
            vision_end_token_id=503)
        torch.manual_seed(0)
        hf = T.Qwen3VLMoeForConditionalGeneration(cfg).float().eval()
        hf.save_pretrained(str(tmp_path / 'hf'), safe_serialization=True)
        grid, pix = torch.tensor([[1, 4, 6]]), torch.randn(24, 3 * 2 * 16 * 16, generator=torch.Generator().manual_seed(2))
        ids = [5, 6, 502] + [500] * 6 + [503, 7, 8]
        ids_t = torch.tensor([ids])
        with torch.no_grad():
            want = hf(input_ids=ids_t, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids_t == 500).int()).logits[0]
    except (AttributeError, TypeError) as e:
        pytest.skip(f'{type(e).__name__}: {e}')
    m = TransformersModel(model_id=str(tmp_path / 'hf'))
    assert m.config.is_moe and m.config.mrope_interleaved and m.config.to_hf()['model_type'] == 'qwen3_vl_moe'
    with torch.no_grad():
        got = m.model.logits(m.model(PackedBatch(torch.tensor(ids), rope_index(ids, grid.tolist(), 500), torch.tensor([0, len(ids)], dtype=torch.int32),
                                                 len(ids), pixel_values=pix, image_grid_thw=grid)))
    assert torch.allclose(got.float(), want, atol=2e-5), float((got - want).abs().max())


def test_context_parallel_split_of_image_batches_matches_one_process():
    """Zig-zag context parallelism over 2 gloo ranks: each rank holds two chunks of every sequence; placeholder features and
    position columns follow the same index."""
    from tests.dist_utils import run_ranks
    single = _vl_curve(0, 1, 2, 1, 'tiny-vl')
    for c in run_ranks(_vl_curve, 2, 2, 2, 'tiny-vl', True):     # sp argument 2: both ranks report the same data group's numbers
        for a, b in zip(single, c):
            assert abs(a - b) < 3e-4, (single, c)


def test_images_through_the_http_server_native_backend(tmp_path, monkeypatch):
    """Train-as-a-service with pictures: the client twin sends chat messages whose image parts travel as PNG data URLs, the
    server's model app (native backend, vision-language preset) encodes them and trains a LoRA adapter; the sampler app
    answers an image prompt."""
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', str(tmp_path / 'ckpt'))
    from twinkle_b200.client import MultiLoraTransformersModel, TorchSampler, TwinkleClient
    from twinkle_b200.server import ServerLauncher
    name = 'tiny-vl'
    server = ServerLauncher({'persistence': {'mode': 'memory'}, 'applications': [
        {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': [name]}},
        {'name': 'model', 'route_prefix': f'/model/{name}', 'import_path': 'model', 'args': {'model_id': name, 'backend': 'transformers', 'max_loras': 2}},
        {'name': 'sampler', 'route_prefix': f'/sampler/{name}', 'import_path': 'sampler', 'args': {'model_id': name, 'sampler_type': 'torch'}}]})
    client = TwinkleClient(app=server.root, token='demo', heartbeat_interval=5.0)
    try:
        g = torch.Generator().manual_seed(0)
        batch = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': (torch.rand(3, 56, 84, generator=g) * 255).round()},
                                                            {'type': 'text', 'text': 'what is it?'}]}, {'role': 'assistant', 'content': 'a boat'}]},
                 {'messages': [{'role': 'user', 'content': 'and in words?'}, {'role': 'assistant', 'content': 'a small boat'}]}]
        model = MultiLoraTransformersModel(name, client=client)
        model.add_adapter_to_model('run', {'r': 4, 'lora_alpha': 8, 'target_modules': 'all-linear'})
        model.set_template('Qwen2VLTemplate', adapter_name='run', vision_config=VC | {'hidden_size': 256}, max_length=4096)
        model.set_optimizer('AdamW', lr=1e-2, adapter_name='run')
        losses = []
        for _ in range(3):
            losses.append(float(model.forward_backward(inputs=batch, adapter_name='run')['loss']))
            model.clip_grad_and_step(max_grad_norm=1.0, adapter_name='run')
        assert losses[-1] < losses[0]
        sampler = TorchSampler(name, client=client)
        sampler.set_template('Qwen2VLTemplate', vision_config=VC | {'hidden_size': 256}, max_length=4096)
        res = sampler.sample([{'messages': batch[0]['messages'][:1]}], {'max_tokens': 3})
        seq = res[0]['sequences'][0]
        assert len(seq['tokens']) <= 3 and len(seq['new_input_feature']['input_ids']) > 24 // 4
    finally:
        client.close()


def test_video_time_positions_follow_real_time_for_qwen2_5_vl():
    ids = [1] + [8] * 12 + [2]                                   # a video of 3 temporal patches on a merged 2 × 2 grid
    plain = rope_index(ids, [(3, 4, 4)], 9, video_token_id=8)
    assert plain[0, 1:13].tolist() == [1] * 4 + [2] * 4 + [3] * 4 and plain[:, -1].tolist() == [4, 4, 4]
    timed = rope_index(ids, [(3, 4, 4)], 9, video_token_id=8, time_steps=[2.0])      # e.g. 2 frames per patch at 2 fps × 2 tokens per second
    assert timed[0, 1:13].tolist() == [1] * 4 + [3] * 4 + [5] * 4 and timed[1:, 1:13].tolist() == plain[1:, 1:13].tolist()
    assert timed[:, -1].tolist() == [6, 6, 6]                     # text resumes after the last time position
    from twinkle_b200.template import template_mapping
    frames = [torch.rand(3, 56, 56) * 255 for _ in range(4)]
    msg = lambda **kw: {'messages': [{'role': 'user', 'content': [dict(type='video', video=frames, **kw), {'type': 'text', 'text': 'go'}]}]}  # noqa: E731
    t25 = template_mapping['Qwen2VLTemplate'](model_id=None, vision_config=VC25, max_length=8192)
    a, b = t25.encode(msg()), t25.encode(msg(fps=1.0))
    ta, tb = a['mrope_position_ids'][0], b['mrope_position_ids'][0]
    vid = torch.tensor(a['input_ids']) == t25.video_token_id
    ua, ub = ta[vid].unique().tolist(), tb[vid].unique().tolist()
    assert len(ua) == len(ub) == 2 and ua[1] - ua[0] == 1 and ub[1] - ub[0] == 4      # 2 frames per patch ÷ 1 fps × 2 tokens per second
    t2 = template_mapping['Qwen2VLTemplate'](model_id=None, vision_config=VC, max_length=8192)
    assert torch.equal(t2.encode(msg(fps=1.0))['mrope_position_ids'], t2.encode(msg())['mrope_position_ids'])   # Qwen2-VL counts patches


def test_dataset_encode_and_dataloader_carry_images():
    """The data-layer route of the multimodal cookbook: rows with image parts → ``Dataset.set_template`` + ``encode`` →
    ``DataLoader`` batches of features (with patches) → ``forward_backward``."""
    from twinkle_b200.dataloader import DataLoader
    from twinkle_b200.dataset import Dataset, DatasetMeta
    from twinkle_b200.model import TransformersModel
    g = torch.Generator().manual_seed(0)
    rows = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': torch.rand(3, 56, 56, generator=g) * 255}, {'type': 'text', 'text': f'q{i}'}]},
                          {'role': 'assistant', 'content': f'answer {i}'}]} for i in range(4)]
    m = TransformersModel(model_id='tiny-vl', seed=0)
    ds = Dataset(DatasetMeta(data=rows))
    ds.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    ds.encode()
    assert {'pixel_values', 'image_grid_thw', 'mrope_position_ids', 'input_ids', 'labels'} <= set(ds[0]) and ds[0]['pixel_values'].shape == (16, 1176)
    m.set_optimizer('AdamW', lr=1e-2)
    losses = []
    for _ in range(2):
        for batch in DataLoader(ds, batch_size=2, shuffle=False):
            losses.append(float(m.forward_backward(inputs=batch)['loss']))
            m.clip_grad_and_step(max_grad_norm=1.0)
    assert len(losses) == 4 and losses[2] < losses[0] and losses[3] < losses[1]       # second pass over the same batches is cheaper


def test_packed_documents_with_images_train_like_separate_ones():
    from twinkle_b200.dataset.packing import concat_features
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-vl', seed=0)
    m.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    tpl = m._group(None).template
    feats = tpl.batch_encode(_vl_trajs() + [{'messages': [{'role': 'user', 'content': 'text only'}, {'role': 'assistant', 'content': 'fine'}]}])
    packed = concat_features(feats)
    assert packed['pixel_values'].shape[0] == sum(f['pixel_values'].shape[0] for f in feats[:2]) and len(packed['image_grid_thw']) == 2
    assert packed['mrope_position_ids'].shape == (3, len(packed['input_ids'])) and packed['position_ids'].count(0) == 3
    a, b = m.forward_only(inputs=feats), m.forward_only(inputs=[packed])
    la = torch.cat([torch.as_tensor(x).float().reshape(-1)[:len(f['input_ids'])] for x, f in zip(a['logps'], feats)])
    lb = torch.as_tensor(b['logps']).float().reshape(-1)[:la.numel()]
    assert torch.allclose(la, lb, atol=1e-5)                 # same log-probs token for token: no attention across documents, same positions


def test_tinker_datums_with_image_tensors(tmp_path, monkeypatch):
    """The Tinker-style route for pictures: the client preprocesses, puts one placeholder per merged patch in the tokens and
    sends ``pixel_values`` / ``image_grid_thw`` in ``loss_fn_inputs``; the server rebuilds the positions and trains."""
    monkeypatch.setenv('TWINKLE_DEFAULT_SAVE_DIR', str(tmp_path / 'ckpt'))
    monkeypatch.setenv('TWINKLE_POLL_INTERVAL', '0.02')
    from twinkle_b200.client import TinkerClient
    from twinkle_b200.models.config import preset
    from twinkle_b200.server import ServerLauncher
    from twinkle_b200.server.backends import datum_to_input_feature
    cfg = preset('tiny-vl')
    pix, grid = preprocess_image(torch.rand(3, 56, 84, generator=torch.Generator().manual_seed(0)) * 255, VisionConfig.from_hf(cfg.vision))
    n_pad = grid[0] * grid[1] * grid[2] // 4
    tokens = [40, 41, cfg.vision_start_token_id] + [cfg.image_token_id] * n_pad + [cfg.vision_end_token_id, 42, 43, 44, 45]
    datum = {'model_input': {'chunks': [{'type': 'encoded_text', 'tokens': tokens}]},
             'loss_fn_inputs': {'target_tokens': {'data': tokens[1:] + [0], 'dtype': 'int64', 'shape': [len(tokens)]},
                                'weights': {'data': [0.0] * (len(tokens) - 4) + [1.0, 1.0, 1.0, 0.0], 'dtype': 'float32', 'shape': [len(tokens)]},
                                'pixel_values': {'data': pix.flatten().tolist(), 'dtype': 'float32', 'shape': list(pix.shape)},
                                'image_grid_thw': {'data': list(grid), 'dtype': 'int64', 'shape': [1, 3]}}}
    f = datum_to_input_feature(datum, cfg)
    assert f['pixel_values'].shape == pix.shape and f['image_grid_thw'] == [list(grid)] and f['mrope_position_ids'].shape == (3, len(tokens))
    with pytest.raises(ValueError):
        datum_to_input_feature(datum, preset('tiny-dense'))
    server = ServerLauncher({'persistence': {'mode': 'memory'}, 'applications': [
        {'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': ['tiny-vl']}},
        {'name': 'model', 'route_prefix': '/model/tiny-vl', 'import_path': 'model', 'args': {'model_id': 'tiny-vl', 'backend': 'transformers', 'max_loras': 2}}]})
    trainer = TinkerClient(app=server.root, token='demo').create_lora_training_client('tiny-vl', rank=4)
    nll = []
    for _ in range(3):
        out = trainer.forward_backward([datum]).result()
        trainer.optim_step({'learning_rate': 1e-2}).result()
        lp = out['loss_fn_outputs'][0]['logprobs']['data']
        nll.append(-sum(lp[-4:-1]))
    assert nll[-1] < nll[0]


@pytest.mark.parametrize('which', ['freeze_vision', 'freeze_llm'])
def test_freezing_one_side_of_a_vision_language_model(which):
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-vl', seed=0, **{which: True})
    m.set_template('Qwen2VLTemplate', vision_config=m.config.vision, max_length=4096)
    m.set_optimizer('AdamW', lr=1e-2)
    tower0 = m.model.visual.merger.mlp[2].weight.detach().clone()
    llm0 = m.model.layers[0].mlp.down_proj.weight.detach().clone()
    trajs = _vl_trajs()
    losses = []
    for _ in range(3):
        losses.append(float(m.forward_backward(inputs=trajs)['loss']))
        m.clip_grad_and_step(max_grad_norm=1.0)
    tower_moved = not torch.equal(tower0, m.model.visual.merger.mlp[2].weight)
    llm_moved = not torch.equal(llm0, m.model.layers[0].mlp.down_proj.weight)
    assert (tower_moved, llm_moved) == ((False, True) if which == 'freeze_vision' else (True, False)) and losses[-1] < losses[0]


def test_qwen3_5_vision_language_trains_through_the_public_api_and_exports(tmp_path):
    """Qwen3.5 with its tower: image parts through ``Qwen3_5Template`` (which takes the model's vision config by itself), training
    of tower + hybrid decoder, and an export that reloads here and in ``transformers`` with the same outputs."""
    from twinkle_b200.model import TransformersModel
    m = TransformersModel(model_id='tiny-qwen3.5-vl', seed=0, device='cpu')
    m.set_template('Qwen3_5Template', max_length=4096)
    g = torch.Generator().manual_seed(0)
    trajs = [{'messages': [{'role': 'user', 'content': [{'type': 'image', 'image': torch.rand(3, 64, 96, generator=g) * 255}, {'type': 'text', 'text': 'what?'}]},
                           {'role': 'assistant', 'content': 'a red ball'}]},
             {'messages': [{'role': 'user', 'content': 'plain text'}, {'role': 'assistant', 'content': 'yes'}]}]
    tpl = m._group(None).template
    f = tpl.encode(trajs[0])
    assert f['image_grid_thw'] == [[1, 4, 6]] and f['pixel_values'].shape == (24, 3 * 2 * 16 * 16) and f['mrope_position_ids'].shape[0] == 3
    m.set_optimizer('AdamW', lr=1e-2)
    w0 = m.model.visual.merger.linear_fc2.weight.detach().clone()
    losses = []
    for _ in range(4):
        losses.append(float(m.forward_backward(inputs=trajs)['loss']))
        m.clip_grad_and_step(max_grad_norm=1.0)
    assert losses[-1] < 0.8 * losses[0] and not torch.equal(w0, m.model.visual.merger.linear_fc2.weight)
    out = m.save('ck', str(tmp_path))
    cfg = json.load(open(out + '/config.json'))
    assert cfg['model_type'] == 'qwen3_5' and cfg['text_config']['rope_parameters']['mrope_section'] == [2, 3, 3] and cfg['vision_config']['model_type'] == 'qwen3_5'
    m2 = TransformersModel(model_id=out, seed=1, device='cpu')
    m2.set_template('Qwen3_5Template', max_length=4096)
    la, lb = m.forward_only(inputs=trajs), m2.forward_only(inputs=trajs)
    assert torch.allclose(torch.as_tensor(la['logps']).float(), torch.as_tensor(lb['logps']).float(), atol=1e-5)
    T = pytest.importorskip('transformers')
    try:
        back = T.Qwen3_5ForConditionalGeneration.from_pretrained(out).float().eval()
        ids = torch.tensor([f['input_ids']])
        with torch.no_grad():
            theirs = back(input_ids=ids, pixel_values=f['pixel_values'], image_grid_thw=torch.tensor(f['image_grid_thw']),
                          mm_token_type_ids=(ids == tpl.image_token_id).int()).logits[0]
    except (TypeError, AttributeError, OSError, ValueError) as e:
        pytest.skip(f'transformers could not run the export: {type(e).__name__}: {e}')
    ours = torch.as_tensor(m.forward_only(inputs=[trajs[0]], return_logits=True)['logits']).float().reshape(-1, theirs.shape[-1])[:theirs.shape[0]]
    assert torch.allclose(ours, theirs, atol=5e-5), float((ours - theirs).abs().max())
