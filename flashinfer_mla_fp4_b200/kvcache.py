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

from .api_log import api_logged

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


@api_logged
@torch.no_grad()
def write_tokens(
    latent: torch.Tensor,
    rope: torch.Tensor,
    slot_mapping: Optional[torch.Tensor],
    kv_cache: torch.Tensor,
    kv_cache_sf: torch.Tensor,
    token_scale: Optional[torch.Tensor] = None,
) -> None:
    """Quantise tokens and scatter them into the paged cache with the CUDA writer kernel.

    latent [T, 512] and rope [T, 64] (bf16, f16 or f32, CUDA, unit inner stride) are written to
    slot ``slot_mapping[t] = page * page_size + offset`` of ``kv_cache`` ([pages, page_size, 320]
    uint8, contiguous) and ``kv_cache_sf`` ([pages, page_size, 1] f32, contiguous); a negative slot
    skips the token, ``slot_mapping=None`` writes token t to slot t.  ``token_scale`` ([T] f32)
    replaces the default amax/6.  Produces the bytes ``quantize_tokens`` produces (the reference's
    fixture builder, tests/test_cute_dsl_mla_fp4.py:56-93; cache writes are the caller's job there,
    README.md:81-83).  Asynchronous on the current stream; there is no CPU path.
    """
    from . import _cabi

    if not (latent.is_cuda and rope.is_cuda and kv_cache.is_cuda and kv_cache_sf.is_cuda):
        raise ValueError("write_tokens needs CUDA tensors (use quantize_tokens to build a cache on the host)")
    if latent.ndim != 2 or latent.shape[1] != LATENT_DIM or rope.ndim != 2 or rope.shape[1] != ROPE_DIM or rope.shape[0] != latent.shape[0]:
        raise ValueError("latent must be [T, 512] and rope [T, 64]")
    if latent.dtype != rope.dtype or latent.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError("latent and rope must share a dtype among bfloat16, float16, float32")
    if latent.stride(1) != 1 or rope.stride(1) != 1:
        raise ValueError("latent and rope must have unit inner stride")
    if kv_cache.dtype != torch.uint8 or kv_cache.shape[-1] != ROW_BYTES or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be a contiguous uint8 tensor [..., 320]")
    if kv_cache_sf.dtype != torch.float32 or not kv_cache_sf.is_contiguous():
        raise ValueError("kv_cache_sf must be a contiguous float32 tensor")
    num_slots = kv_cache.numel() // ROW_BYTES
    if kv_cache_sf.numel() != num_slots:
        raise ValueError("kv_cache_sf must hold one scale per cache row")
    tokens = latent.shape[0]
    for name, t in (("rope", rope), ("kv_cache", kv_cache), ("kv_cache_sf", kv_cache_sf), ("slot_mapping", slot_mapping),
                    ("token_scale", token_scale)):
        if t is not None and (not t.is_cuda or t.device != latent.device):
            raise ValueError(f"{name} must be a CUDA tensor on the device of latent ({latent.device}), got {t.device}")
    if slot_mapping is not None:
        if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != tokens or not slot_mapping.is_contiguous():
            raise ValueError("slot_mapping must be a contiguous int64 tensor [T]")
    if token_scale is not None:
        token_scale = token_scale.reshape(-1)
        if token_scale.dtype != torch.float32 or token_scale.numel() != tokens or not token_scale.is_contiguous():
            raise ValueError("token_scale must be a contiguous float32 tensor [T]")
    dt = {torch.bfloat16: _cabi.IN_BF16, torch.float16: _cabi.IN_F16, torch.float32: _cabi.IN_F32}[latent.dtype]
    with torch.cuda.device(latent.device):
        _cabi.check(_cabi.lib.mla_fp4_cache_write(
            latent.data_ptr(), latent.stride(0), rope.data_ptr(), rope.stride(0), dt,
            token_scale.data_ptr() if token_scale is not None else None,
            slot_mapping.data_ptr() if slot_mapping is not None else None,
            tokens, kv_cache.data_ptr(), kv_cache_sf.data_ptr(), num_slots,
            torch.cuda.current_stream(latent.device).cuda_stream))
