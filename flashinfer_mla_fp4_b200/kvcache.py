"""The custom FP4 MLA cache format: layout constants and a torch writer.

Format (reference README.md:28-42 and tests/test_cute_dsl_mla_fp4.py:56-93):
one 320-byte row per token = 256 bytes of packed E2M1 latent (512 values, low
nibble = even element, nibble bit 3 = sign) followed by 64 bytes of E4M3 RoPE,
plus one FP32 scale per token held in a separate [pages, page_size, 1] tensor.
The reference leaves cache writes to the caller (README.md:81-83); this module
is the torch writer used to build caches (any device).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

LATENT_DIM = 512
ROPE_DIM = 64
HEAD_DIM_QK = LATENT_DIM + ROPE_DIM  # 576
LATENT_BYTES = LATENT_DIM // 2  # 256
ROW_BYTES = LATENT_BYTES + ROPE_DIM  # 320
BYTES_PER_TOKEN = ROW_BYTES + 4  # cache row + FP32 scale = 324

_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


@torch.no_grad()
def quantize_tokens(
    latent: torch.Tensor,
    rope: torch.Tensor,
    token_scale: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise tokens to cache rows.

    latent [..., 512] and rope [..., 64] (any float dtype) -> (rows uint8 [..., 320],
    scale f32 [..., 1]).  ``token_scale`` defaults to amax/6 per token (1 for an
    all-zero token).  Rounding is to the nearest E2M1 magnitude with a tie going
    to the smaller one, as the reference fixture builder does.
    """
    lat = latent.float()
    if token_scale is None:
        s = lat.abs().amax(dim=-1, keepdim=True) / 6.0
        token_scale = torch.where(s > 0, s, torch.ones_like(s))
    token_scale = token_scale.float()
    x = lat / token_scale
    thr = torch.tensor(_THRESHOLDS, dtype=torch.float32, device=lat.device)
    code = torch.bucketize(x.abs(), thr).to(torch.uint8)
    code |= (x < 0).to(torch.uint8) << 3
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    rope_u8 = rope.to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.cat((packed, rope_u8), dim=-1).contiguous(), token_scale.contiguous()
