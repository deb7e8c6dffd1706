"""Vision side of the Qwen2-VL family: the patch encoder that turns images into embeddings at the language model's
width, the three-component ("multimodal") rotary position tables, the position index that lays images out on a
(time, height, width) grid inside the token stream, and the image → patch preprocessing.

Parameter names and shapes follow the Hugging Face checkpoint (``visual.patch_embed.proj``, ``visual.blocks.N.{norm1,
attn.qkv, attn.proj, norm2, mlp.fc1, mlp.fc2}``, ``visual.merger.{ln_q, mlp.0, mlp.2}``), so weights load by name.

The reference trains such models through ``transformers`` (``cookbook/mm/fsdp2.py``; ``template/base.py:611-667``
``pre_forward_hook``); here the tower is part of the owned model, its output is scattered into the embedding stream of
the packed batch, and the language model's RoPE kernels take the multimodal tables unchanged (they are per-token tables).
Attention inside the tower is dense per image (no causal mask, head width ≠ 128) and runs on PyTorch's SDPA."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584          # output width = the language model's hidden size
    num_heads: int = 16
    mlp_ratio: float = 4.0
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    in_channels: int = 3
    # Qwen2.5-VL: RMSNorm + gated SiLU MLP (``intermediate_size``), attention inside ``window_size``-pixel windows except in
    # the blocks listed in ``fullatt_block_indexes``; ``tokens_per_second`` scales video time positions
    tokens_per_second: float = 2.0
    arch: str = 'qwen2_vl'
    intermediate_size: int = 0
    window_size: int = 112
    fullatt_block_indexes: Tuple[int, ...] = ()
    # Qwen3-VL: learned position table (a square grid, interpolated to the image's patch grid), tanh-GELU MLP, and extra
    # mergers after the listed blocks whose outputs are added to the language model's first layers ("deep stack")
    num_position_embeddings: int = 0
    deepstack_visual_indexes: Tuple[int, ...] = ()

    @classmethod
    def from_hf(cls, d: Dict[str, Any]) -> 'VisionConfig':
        d = dict(d)
        if 'num_position_embeddings' in d and d.get('num_position_embeddings'):
            d.update(arch='qwen3_vl', embed_dim=d['hidden_size'], hidden_size=d['out_hidden_size'],
                     deepstack_visual_indexes=tuple(d.get('deepstack_visual_indexes') or ()))
        elif 'out_hidden_size' in d:  # Qwen2.5-VL spelling: hidden_size = tower width, out_hidden_size = language model width
            d.update(arch='qwen2_5_vl', embed_dim=d['hidden_size'], hidden_size=d['out_hidden_size'],
                     fullatt_block_indexes=tuple(d.get('fullatt_block_indexes') or ()))
        elif 'fullatt_block_indexes' in d:
            d['fullatt_block_indexes'] = tuple(d['fullatt_block_indexes'] or ())
        keys = ('depth', 'embed_dim', 'hidden_size', 'num_heads', 'mlp_ratio', 'patch_size', 'spatial_merge_size', 'temporal_patch_size', 'in_channels',
                'arch', 'intermediate_size', 'window_size', 'fullatt_block_indexes', 'num_position_embeddings', 'deepstack_visual_indexes',
                'tokens_per_second')
        return cls(**{k: d[k] for k in keys if k in d})

    def to_hf(self) -> Dict[str, Any]:
        base = dict(depth=self.depth, num_heads=self.num_heads, patch_size=self.patch_size, spatial_merge_size=self.spatial_merge_size,
                    temporal_patch_size=self.temporal_patch_size, in_channels=self.in_channels)
        if self.arch == 'qwen3_vl':
            return {'model_type': 'qwen3_vl', **base, 'hidden_size': self.embed_dim, 'out_hidden_size': self.hidden_size,
                    'intermediate_size': self.intermediate_size, 'num_position_embeddings': self.num_position_embeddings,
                    'deepstack_visual_indexes': list(self.deepstack_visual_indexes), 'hidden_act': 'gelu_pytorch_tanh'}
        if self.arch == 'qwen2_5_vl':
            return {'model_type': 'qwen2_5_vl', **base, 'hidden_size': self.embed_dim, 'out_hidden_size': self.hidden_size,
                    'intermediate_size': self.intermediate_size, 'window_size': self.window_size,
                    'fullatt_block_indexes': list(self.fullatt_block_indexes), 'hidden_act': 'silu', 'tokens_per_second': self.tokens_per_second}
        return {'model_type': 'qwen2_vl', **base, 'embed_dim': self.embed_dim, 'hidden_size': self.hidden_size, 'mlp_ratio': self.mlp_ratio,
                'hidden_act': 'quick_gelu'}

    @property
    def image_mean_std(self) -> Tuple[Tuple[float, ...], Tuple[float, ...]]:
        return ((0.5, 0.5, 0.5), (0.5, 0.5, 0.5)) if self.arch == 'qwen3_vl' else (IMAGE_MEAN, IMAGE_STD)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


class _PatchEmbed(nn.Module):

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        # kept in Conv3d layout [E, C, T, P, P] so the checkpoint tensor loads as is; applied as one GEMM over flat patches
        self.proj = nn.Conv3d(cfg.in_channels, cfg.embed_dim, (cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size),
                              stride=(cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size), bias=cfg.arch == 'qwen3_vl')

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.proj.weight
        return F.linear(x.to(w.dtype), w.view(w.shape[0], -1), self.proj.bias)


class _Attn(nn.Module):

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, 3 * dim, bias=True)
        self.proj = nn.Linear(dim, dim, bias=True)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, bounds: Sequence[int]) -> torch.Tensor:
        n, dim = x.shape
        q, k, v = self.qkv(x).view(n, 3, self.heads, dim // self.heads).unbind(1)
        q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        outs = []
        for a, b in zip(bounds[:-1], bounds[1:]):           # one frame (or image) attends within itself
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1), k[a:b].transpose(0, 1), v[a:b].transpose(0, 1))
            outs.append(o.transpose(0, 1))
        return self.proj(torch.cat(outs, 0).reshape(n, dim))


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE with half-width tables ``[N, D/2]`` on ``x [N, H, D]`` (pairs ``(i, i + D/2)``), in fp32."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


class _Mlp(nn.Module):

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        h = self.fc1(x)
        return self.fc2(h * torch.sigmoid(1.702 * h))      # "quick" GELU


class _GatedMlp(nn.Module):

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = nn.Linear(dim, hidden), nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _TanhGeluMlp(nn.Module):

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.linear_fc1, self.linear_fc2 = nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        return self.linear_fc2(F.gelu(self.linear_fc1(x), approximate='tanh'))


class _Merger3(nn.Module):
    """Qwen3-VL merger; ``postshuffle`` normalises the joined ``merge²`` group instead of every patch."""

    def __init__(self, cfg: VisionConfig, postshuffle: bool = False):
        super().__init__()
        self.group, self.postshuffle = cfg.embed_dim * cfg.spatial_merge_size**2, postshuffle
        self.norm = nn.LayerNorm(self.group if postshuffle else cfg.embed_dim, eps=1e-6)
        self.linear_fc1, self.linear_fc2 = nn.Linear(self.group, self.group), nn.Linear(self.group, cfg.hidden_size)

    def forward(self, x):
        x = self.norm(x.view(-1, self.group) if self.postshuffle else x).view(-1, self.group)
        return self.linear_fc2(F.gelu(self.linear_fc1(x)))


def _norm(cfg: VisionConfig) -> nn.Module:
    return nn.RMSNorm(cfg.embed_dim, eps=1e-6) if cfg.arch == 'qwen2_5_vl' else nn.LayerNorm(cfg.embed_dim, eps=1e-6)


class _Block(nn.Module):

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.norm1, self.norm2 = _norm(cfg), _norm(cfg)
        self.attn = _Attn(cfg.embed_dim, cfg.num_heads)
        self.mlp = (_GatedMlp(cfg.embed_dim, cfg.intermediate_size) if cfg.arch == 'qwen2_5_vl' else
                    _TanhGeluMlp(cfg.embed_dim, cfg.intermediate_size) if cfg.arch == 'qwen3_vl' else _Mlp(cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio)))

    def forward(self, x, cos, sin, bounds):
        x = x + self.attn(self.norm1(x), cos, sin, bounds)
        return x + self.mlp(self.norm2(x))


class _Merger(nn.Module):
    """Joins every ``merge × merge`` neighbourhood (consecutive in patch order) into one token of the language model's width."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.group = cfg.embed_dim * cfg.spatial_merge_size**2
        self.ln_q = _norm(cfg)
        self.mlp = nn.Sequential(nn.Linear(self.group, self.group), nn.GELU(), nn.Linear(self.group, cfg.hidden_size))

    def forward(self, x):
        return self.mlp(self.ln_q(x).view(-1, self.group))


class VisionTower(nn.Module):

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = _PatchEmbed(cfg)
        self.blocks = nn.ModuleList([_Block(cfg) for _ in range(cfg.depth)])
        if cfg.arch == 'qwen3_vl':
            self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.embed_dim)
            self.merger = _Merger3(cfg)
            self.deepstack_merger_list = nn.ModuleList([_Merger3(cfg, postshuffle=True) for _ in cfg.deepstack_visual_indexes])
        else:
            self.merger = _Merger(cfg)

    def position_embeddings(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """Qwen3-VL: the learned ``side × side`` position table sampled bilinearly at every patch of an ``h × w`` grid
        (corners aligned), repeated per frame, in merge-group order ``[N, embed_dim]``."""
        side = int(self.cfg.num_position_embeddings**0.5)
        m, table, out = self.cfg.spatial_merge_size, self.pos_embed.weight, []
        for t, h, w in grid_thw.tolist():
            hi, wi = torch.linspace(0, side - 1, h, device=table.device), torch.linspace(0, side - 1, w, device=table.device)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            corner = lambda a, b: table[(a[:, None] * side + b[None, :]).long().flatten()].view(h, w, -1)  # noqa: E731
            e = (corner(h0, w0) * ((1 - dh) * (1 - dw))[..., None] + corner(h0, w1) * ((1 - dh) * dw)[..., None] +
                 corner(h1, w0) * (dh * (1 - dw))[..., None] + corner(h1, w1) * (dh * dw)[..., None])
            e = e.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out, 0)

    def rotary_tables(self, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos/sin ``[N, head_dim/2]``: the first quarter of the head rotates with the patch's row, the second with its
        column (patches are ordered merge-group by merge-group, as the preprocessing emits them)."""
        m, dev = self.cfg.spatial_merge_size, grid_thw.device
        quarter = self.cfg.embed_dim // self.cfg.num_heads // 4
        inv = 1.0 / (10000.0**(torch.arange(0, 2 * quarter, 2, dtype=torch.float32, device=dev) / (2 * quarter)))
        pos = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=dev)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w, device=dev)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            pos.append(torch.stack([hp, wp], -1).repeat(t, 1))
        pos = torch.cat(pos, 0).float()
        ang = torch.cat([pos[:, 0:1] * inv[None, :], pos[:, 1:2] * inv[None, :]], -1)
        return ang.cos(), ang.sin()

    def window_order(self, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, List[int]]:
        """Qwen2.5-VL: a permutation of the merge groups that makes every ``window_size``-pixel window contiguous, and the
        patch boundaries of the windows in that order (edge windows are smaller)."""
        m = self.cfg.spatial_merge_size
        vw = self.cfg.window_size // m // self.cfg.patch_size          # window side in merge groups
        order, bounds, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).view(t, gh, gw)
            ph, pw = vw - gh % vw, vw - gw % vw
            pad = F.pad(idx, (0, pw, 0, ph), value=-100)
            nh, nw = (gh + ph) // vw, (gw + pw) // vw
            win = pad.view(t, nh, vw, nw, vw).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, vw, vw)
            counts = (win != -100).sum((2, 3)).reshape(-1)
            flat = win.reshape(-1)
            order.append(flat[flat != -100] + base)
            for c in counts.tolist():
                if c:
                    bounds.append(bounds[-1] + c * m * m)
            base += t * gh * gw
        return torch.cat(order).to(grid_thw.device), bounds

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, return_deepstack: bool = False):
        """``pixel_values [N, C·T·P·P]`` (flat patches of all images, in order), ``grid_thw [n_images, 3]`` →
        ``[N / merge², hidden_size]``; with ``return_deepstack`` also the list of deep-stack features (same shape each;
        empty for towers without them)."""
        x = self.patch_embed(pixel_values)
        cos, sin = self.rotary_tables(grid_thw)
        frames = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        bounds = [0] + frames.cumsum(0).tolist()
        if self.cfg.arch == 'qwen3_vl':
            x = x + self.position_embeddings(grid_thw).to(x.dtype)
            deep = []
            for i, blk in enumerate(self.blocks):
                x = blk(x, cos, sin, bounds)
                if i in self.cfg.deepstack_visual_indexes:
                    deep.append(self.deepstack_merger_list[self.cfg.deepstack_visual_indexes.index(i)](x))
            return (self.merger(x), deep) if return_deepstack else self.merger(x)
        if return_deepstack:
            return self.forward(pixel_values, grid_thw), []
        if self.cfg.arch != 'qwen2_5_vl':
            for blk in self.blocks:
                x = blk(x, cos, sin, bounds)
            return self.merger(x)
        unit = self.cfg.spatial_merge_size**2
        order, win_bounds = self.window_order(grid_thw)
        regroup = lambda t: t.view(t.shape[0] // unit, unit, -1)[order].reshape(t.shape[0], -1)  # noqa: E731
        x, cos, sin = regroup(x), regroup(cos), regroup(sin)
        # a frame's patches stay contiguous under the window order, so the per-frame boundaries are unchanged
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, bounds if i in self.cfg.fullatt_block_indexes else win_bounds)
        return self.merger(x)[torch.argsort(order)]


# ------------------------------------------------------------------------------------------ positions in the LLM
def mrope_tables(position_ids: torch.Tensor, head_dim: int, theta: float, section: Sequence[int], interleaved: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[T, head_dim/2]`` from ``position_ids [3, T]`` (time, height, width): frequency ``j`` uses the component
    whose section (``section`` sums to ``head_dim/2``) contains ``j``. Text tokens carry the same value in all three
    components, which reduces to ordinary RoPE."""
    half = head_dim // 2
    assert sum(section) == half, f'mrope sections {list(section)} must sum to head_dim/2 = {half}'
    inv = 1.0 / (theta**(torch.arange(0, head_dim, 2, dtype=torch.float32, device=position_ids.device) / head_dim))
    if interleaved:  # Qwen3-VL: t h w t h w … over the low frequencies (height on j ≡ 1, width on j ≡ 2 mod 3, while their sections last), time elsewhere
        j = torch.arange(half, device=position_ids.device)
        comp = torch.where((j % 3 == 1) & (j < 3 * section[1]), 1, torch.where((j % 3 == 2) & (j < 3 * section[2]), 2, 0))
    else:
        comp = torch.repeat_interleave(torch.arange(3, device=position_ids.device), torch.tensor(list(section), device=position_ids.device))
    pos = position_ids.float()[comp, :].t()                  # [T, half]: the component each frequency follows
    ang = pos * inv[None, :]
    return ang.cos(), ang.sin()


def rope_index(input_ids: Sequence[int], grids: Sequence[Sequence[int]], image_token_id: int, merge: int = 2,
               video_token_id: Optional[int] = None, time_steps: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Positions ``[3, L]`` of one sequence whose images appear as runs of ``image_token_id`` (``t·h·w / merge²`` tokens
    per image, in the order of ``grids``). Text advances all three components together; an image keeps time fixed and
    spreads height and width over its merged grid; the text after it continues from the largest position used + 1.
    ``time_steps[g]`` (Qwen2.5-VL videos: seconds per temporal patch × the tower's ``tokens_per_second``) stretches the
    time axis of entry ``g`` so that positions follow real time; 1 (the default, and always for images) counts patches."""
    ids = list(int(t) for t in input_ids)
    out = torch.zeros(3, len(ids), dtype=torch.long)
    nxt, i, g = 0, 0, 0
    special = {image_token_id} | ({video_token_id} if video_token_id is not None else set())
    while i < len(ids):
        if ids[i] in special:
            t, h, w = grids[g]
            g += 1
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            if ids[i:i + n] != [ids[i]] * n:
                raise ValueError(f'image {g - 1}: expected a run of {n} placeholder tokens at position {i}')
            step = float(time_steps[g - 1]) if time_steps is not None and time_steps[g - 1] is not None else 1.0
            tt = (torch.arange(t) * step).long().view(-1, 1, 1).expand(t, gh, gw).flatten()
            hh = torch.arange(gh).view(1, -1, 1).expand(t, gh, gw).flatten()
            ww = torch.arange(gw).view(1, 1, -1).expand(t, gh, gw).flatten()
            out[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt += max(int(tt.max()) + 1, gh, gw)
            i += n
        else:
            out[:, i] = nxt
            nxt += 1
            i += 1
    if g != len(grids):
        raise ValueError(f'{len(grids)} images given but {g} placeholder runs found')
    return out


# ---------------------------------------------------------------------------------------------- preprocessing
IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Nearest size whose sides are multiples of ``factor`` with the pixel count inside ``[min_pixels, max_pixels]`` and
    the aspect ratio kept as far as possible."""
    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError(f'aspect ratio of {height}x{width} exceeds 200')
    h, w = max(factor, round(height / factor) * factor), max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h, w = math.floor(height / beta / factor) * factor, math.floor(width / beta / factor) * factor
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h, w = math.ceil(height * beta / factor) * factor, math.ceil(width * beta / factor) * factor
    return max(h, factor), max(w, factor)


def patchify(frames: torch.Tensor, cfg: VisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """``frames [T, C, H, W]`` (already resized so that H, W are multiples of ``patch·merge``, normalised) →
    (``[t·h·w, C·Tp·P·P]`` flat patches ordered merge-group by merge-group, ``(t, h, w)``). A single image is repeated
    to fill the temporal patch."""
    tp, p, m = cfg.temporal_patch_size, cfg.patch_size, cfg.spatial_merge_size
    if frames.shape[0] % tp:
        frames = torch.cat([frames, frames[-1:].expand(tp - frames.shape[0] % tp, -1, -1, -1)], 0)
    T, C, H, W = frames.shape
    t, h, w = T // tp, H // p, W // p
    x = frames.reshape(t, tp, C, h // m, m, p, w // m, m, p)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                # t, h/m, w/m, m, m, C, tp, p, p
    return x.reshape(t * h * w, C * tp * p * p), (t, h, w)


def preprocess_image(image: Any, cfg: VisionConfig, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """A PIL image, a path / URL / bytes (see ``utils.misc.load_image``) or a ``[C, H, W]`` / ``[H, W, C]`` array in 0…255 →
    normalised flat patches and the patch grid."""
    if not torch.is_tensor(image):
        import numpy as np
        if not hasattr(image, 'shape'):
            from ..utils.misc import load_image
            image = np.asarray(load_image(image))
        image = torch.as_tensor(np.asarray(image))
    x = image.float()
    if x.dim() == 3 and x.shape[-1] in (1, 3) and x.shape[0] not in (1, 3):
        x = x.permute(2, 0, 1)
    if x.shape[0] == 1:
        x = x.expand(3, -1, -1)
    factor = cfg.patch_size * cfg.spatial_merge_size
    h, w = smart_resize(x.shape[1], x.shape[2], factor, min_pixels, max_pixels)
    if (h, w) != tuple(x.shape[1:]):
        try:  # the same resampling as the Hugging Face processor (PIL bicubic on 8-bit pixels), so features match its output
            import numpy as np
            from PIL import Image
            pil = Image.fromarray(x.clamp(0, 255).round().byte().permute(1, 2, 0).numpy()).resize((w, h), resample=Image.BICUBIC)
            x = torch.as_tensor(np.array(pil)).permute(2, 0, 1).float()
        except ImportError:
            x = F.interpolate(x[None], size=(h, w), mode='bicubic', align_corners=False, antialias=True)[0].clamp(0, 255)
    mean, std = (torch.tensor(v).view(3, 1, 1) for v in cfg.image_mean_std)
    x = (x / 255.0 - mean) / std
    return patchify(x[None], cfg)


def preprocess_video(frames: Sequence[Any], cfg: VisionConfig, min_pixels: int = 128 * 28 * 28, max_pixels: int = 768 * 28 * 28) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """A list of frames (anything :func:`preprocess_image` takes, all of one size) → flat patches and the ``(t, h, w)`` grid;
    ``temporal_patch_size`` consecutive frames share a patch, an odd tail frame is repeated."""
    if not len(frames):
        raise ValueError('a video needs at least one frame')
    import numpy as np
    tensors = []
    for fr in frames:
        if not torch.is_tensor(fr):
            if not hasattr(fr, 'shape'):
                from ..utils.misc import load_image
                fr = np.asarray(load_image(fr))
            fr = torch.as_tensor(np.array(fr))
        x = fr.float()
        if x.dim() == 3 and x.shape[-1] in (1, 3) and x.shape[0] not in (1, 3):
            x = x.permute(2, 0, 1)
        tensors.append(x.expand(3, -1, -1) if x.shape[0] == 1 else x)
    x = torch.stack(tensors)
    factor = cfg.patch_size * cfg.spatial_merge_size
    h, w = smart_resize(x.shape[2], x.shape[3], factor, min_pixels, max_pixels)
    if (h, w) != tuple(x.shape[2:]):
        x = F.interpolate(x, size=(h, w), mode='bicubic', align_corners=False, antialias=True).clamp(0, 255)
    mean, std = (torch.tensor(v).view(1, 3, 1, 1) for v in cfg.image_mean_std)
    return patchify((x / 255.0 - mean) / std, cfg)
