"""Checkpoint de-quantisers used at load time only.

Parity: reference ``src/twinkle/utils/dequantizer.py:7-46`` — block-(128,128)
fp8 weights with an inverse-scale grid are expanded to fp32/bf16; MXFP4 blocks
(32 e2m1 values sharing one e8m0 scale) likewise.  Training never runs in fp8.
"""
from __future__ import annotations

import torch

_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def dequant_fp8_block(weight: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128), dtype=torch.bfloat16) -> torch.Tensor:
    rows, cols = weight.shape[-2:]
    br, bc = block
    s = scale_inv.float().repeat_interleave(br, dim=-2)[..., :rows, :].repeat_interleave(bc, dim=-1)[..., :cols]
    return (weight.float() * s).to(dtype)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """``blocks`` uint8 [..., G, 16] (two nibbles per byte, low first), ``scales``
    uint8 e8m0 [..., G] → [..., G*32]."""
    lut = _E2M1.to(blocks.device)
    lo = lut[(blocks & 0xF).long()]
    hi = lut[(blocks >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).flatten(-2)
    scale = torch.exp2(scales.float() - 127.0).unsqueeze(-1)
    return (vals * scale).flatten(-2).to(dtype)


class Dequantizer:

    @staticmethod
    def maybe_dequantize(name: str, tensor: torch.Tensor, lookup) -> torch.Tensor:
        """``lookup(name)`` returns a companion tensor or None."""
        if tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            s = lookup(name + '_scale_inv')
            if s is not None:
                return dequant_fp8_block(tensor, s)
            return tensor.to(torch.bfloat16)
        return tensor
