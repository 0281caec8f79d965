"""CPU oracle for per-token-scaled FP4 MLA decode.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, the smoke entry and the benchmark's CPU-baseline leg may
import this module; the product path never does.

What is restated here, and from where in the reference project:

* cache format, quantiser and dequantiser: ``tests/test_cute_dsl_mla_fp4.py:56-93``
  (``_make_w512_cache``): thresholds ``[.25,.75,1.25,1.75,2.5,3.5,5]``, sign in
  nibble bit 3, low nibble = even element, magnitude table
  ``[0,.5,1,1.5,2,3,4,6]``, latent = table * sign * per-token scale, RoPE kept
  as E4M3 bytes 256..319 of every 320-byte row.
* paging and byte split 256|64: ``flashinfer_mla_fp4/wrappers/batch_mla_fp4.py:381-388``.
* score = scale_t * <q_lat, c_t> + <q_rope, r_t>:
  ``flashinfer_mla_fp4/roles/mla_compute_fp4.py:208-223``.
* masking of tokens >= seq_len: ``flashinfer_mla_fp4/roles/mla_compute_fp4.py:225-229``.
* V = scale_t * c_t (latent only), softmax over raw scores times softmax_scale,
  final multiply by output_scale: ``flashinfer_mla_fp4/roles/mla_compute_fp4.py:345-379``
  and the inherited epilogue of the pinned dependency flashinfer-python==0.6.17
  (``cute_dsl/attention/roles/mla_correction.py``; un-vendored, read at 0.6.11.post2).
* LSE is base-2: log2(sum exp(softmax_scale * score)).

Pinning status.  The format/quantiser/dequantiser half is pinned by golden
vectors produced by executing the reference's own ``_make_w512_cache`` (see
``tests/golden/make_golden.py``).  The attention half has no CPU
implementation, golden vector or stored expectation in the reference (its only
check is GPU kernel against GPU kernel), so for that half: PARITY UNPINNED by
the reference; it is cross-checked against the dependency's own torch
reference ``flashinfer/trace/templates/attention.py::_cute_dsl_batch_mla_run_reference``
(golden vectors generated from it are committed too) and judged by the
tolerance the task states: per-head cosine >= 0.9999 and
max-abs <= 2e-2 * RMS(out).

Everything is computed in FP32 (accumulations in FP32 via torch CPU matmul).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

LATENT_DIM = 512
ROPE_DIM = 64
ROW_BYTES = LATENT_DIM // 2 + ROPE_DIM  # 320
LOG2_E = 1.4426950408889634

#: E2M1 magnitudes for codes 0..7 (reference tests/test_cute_dsl_mla_fp4.py:80-84)
E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
#: round-to-nearest thresholds between them (reference tests/...:70-75)
E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
#: E4M3 byte of each E2M1 code 0..7; codes 8..15 are the same bytes | 0x80
E2M1_TO_E4M3_BYTES = (0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C)


def e4m3_decode_table() -> np.ndarray:
    """All 256 E4M3 (fn) byte values as float32, computed from the bit fields."""
    tab = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if (b >> 7) else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** -6
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        tab[b] = v
    return tab


def e2m1_decode_table() -> np.ndarray:
    """The 16 E2M1 nibble values as float32 (sign = bit 3)."""
    mags = np.asarray(E2M1_MAGNITUDES, dtype=np.float32)
    return np.concatenate([mags, -mags]).astype(np.float32)


def e2m1_to_e4m3_byte_table() -> np.ndarray:
    """16-entry nibble -> E4M3 byte table (the table the kernel must match bit for bit)."""
    pos = np.asarray(E2M1_TO_E4M3_BYTES, dtype=np.uint8)
    return np.concatenate([pos, pos | 0x80]).astype(np.uint8)


# --------------------------------------------------------------------------- quantiser


@torch.no_grad()
def quantize_latent(latent: torch.Tensor, token_scale: torch.Tensor) -> torch.Tensor:
    """FP32 latent [..., 512] + per-token scale [..., 1] -> packed E2M1 bytes [..., 256].

    Follows reference tests/test_cute_dsl_mla_fp4.py:70-78: bucketize |x/scale|
    against the thresholds (a tie goes to the lower code), sign bit 3 when the
    normalised value is negative, low nibble = even element.
    """
    normalized = latent.float() / token_scale.float()
    thr = torch.tensor(E2M1_THRESHOLDS, dtype=torch.float32, device=latent.device)
    mag = torch.bucketize(normalized.abs(), thr)
    nib = mag | ((normalized < 0).to(torch.int64) << 3)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).to(torch.uint8)


@torch.no_grad()
def pack_cache(latent: torch.Tensor, rope: torch.Tensor, token_scale: torch.Tensor) -> torch.Tensor:
    """Build the [pages, page_size, 320] uint8 cache from FP32 latent, rope and scale."""
    packed = quantize_latent(latent, token_scale)
    rope_u8 = rope.to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.cat((packed, rope_u8), dim=-1).contiguous()


@torch.no_grad()
def make_reference_style_cache(source: torch.Tensor):
    """Restatement of the reference fixture builder (tests/...:56-93).

    ``source`` is [pages, page_size, 576] (any float dtype).  The scale alternates
    0.5 / 1.0 by global token parity.  Returns (fp4_cache u8 [P,ps,320],
    token_scale f32 [P,ps,1], fp8_cache e4m3 [P,ps,576]).
    """
    num_pages, page_size, _ = source.shape
    ids = torch.arange(num_pages * page_size, dtype=torch.int64, device=source.device)
    token_scale = torch.where(ids.view(num_pages, page_size) % 2 == 0, 0.5, 1.0)[..., None].float()
    latent = source[..., :LATENT_DIM].float()
    rope = source[..., LATENT_DIM:]
    fp4_cache = pack_cache(latent, rope, token_scale)
    deq_lat, deq_rope = dequantize_cache(fp4_cache, token_scale)
    fp8_cache = torch.cat((deq_lat, deq_rope), dim=-1).to(torch.float8_e4m3fn)
    return fp4_cache, token_scale, fp8_cache


@torch.no_grad()
def amax_scale(latent: torch.Tensor) -> torch.Tensor:
    """Per-token scale = amax / 6 (FP32); an all-zero token gets scale 1."""
    amax = latent.float().abs().amax(dim=-1, keepdim=True)
    s = amax / 6.0
    return torch.where(s > 0, s, torch.ones_like(s))


# --------------------------------------------------------------------------- dequantiser


@torch.no_grad()
def unpack_e2m1_codes(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 256] -> int64 nibble codes [..., 512] (low nibble first)."""
    lo = (packed & 0xF).to(torch.int64)
    hi = (packed >> 4).to(torch.int64)
    return torch.stack((lo, hi), dim=-1).flatten(-2)


@torch.no_grad()
def dequantize_cache(cache_u8: torch.Tensor, token_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[..., 320] uint8 + [..., 1] f32 -> (latent f32 [..., 512] already scaled, rope f32 [..., 64])."""
    assert cache_u8.dtype == torch.uint8 and cache_u8.shape[-1] == ROW_BYTES
    codes = unpack_e2m1_codes(cache_u8[..., : LATENT_DIM // 2])
    lut = torch.from_numpy(e2m1_decode_table()).to(cache_u8.device)
    latent = lut[codes] * token_scale.float()
    e4 = torch.from_numpy(e4m3_decode_table()).to(cache_u8.device)
    rope = e4[cache_u8[..., LATENT_DIM // 2 :].to(torch.int64)]
    return latent, rope


@torch.no_grad()
def decode_e4m3(x: torch.Tensor) -> torch.Tensor:
    """E4M3 tensor (float8_e4m3fn or its uint8 view) -> float32 through the 256-entry table."""
    u8 = x.view(torch.uint8) if x.dtype != torch.uint8 else x
    e4 = torch.from_numpy(e4m3_decode_table()).to(u8.device)
    return e4[u8.to(torch.int64)]


# --------------------------------------------------------------------------- attention


@torch.no_grad()
def mla_decode(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    kv_cache_sf: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    softmax_scale: float,
    output_scale: float = 1.0,
    logits_soft_cap: float = 0.0,
    sink: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense FP32 MLA decode over the dequantised cache.

    Attention variants (the hooks of flashinfer's ``cute_dsl/attention/fusion/variant.py`` that the reference
    wrapper forwards, wrappers/batch_mla_fp4.py:237-253, restated as plain arithmetic):
    ``logits_soft_cap`` > 0 turns every raw score s = q.k into cap * tanh(s / cap) before ``softmax_scale``
    (the soft-capping ``score_mod``); ``sink`` f32 [H] adds one virtual token per head with logit sink[h]
    (compared with the scaled scores) and a zero value row, i.e. exp(sink[h]) in the denominator only
    (``AttentionWithSink.update_statistics``).

    q: E4M3 (or float) [B, q_len, H, 576]; kv_cache uint8 [P, ps, 320] (or 4-D with a
    singleton dim 1); kv_cache_sf f32 [P, ps, 1]; block_tables int [B, max_pages];
    seq_lens int [B].  Every query position attends to all seq_len tokens.
    Returns (out f32 [B, q_len, H, 512], lse2 f32 [B, q_len, H]); a request with
    seq_len == 0 gives zeros and lse2 = -inf (with a sink: zeros and the sink's logit in base 2).
    """
    if kv_cache.dim() == 4:
        kv_cache = kv_cache.squeeze(1)
    if kv_cache_sf.dim() == 4:
        kv_cache_sf = kv_cache_sf.squeeze(1)
    q = q.detach().cpu()
    kv_cache = kv_cache.detach().cpu()
    kv_cache_sf = kv_cache_sf.detach().cpu()
    block_tables = block_tables.detach().cpu()
    seq_lens = seq_lens.detach().cpu()
    B, q_len, H, D = q.shape
    assert D == LATENT_DIM + ROPE_DIM
    page_size = kv_cache.shape[1]
    qf = decode_e4m3(q) if q.dtype in (torch.float8_e4m3fn, torch.uint8) else q.float()
    out = torch.zeros(B, q_len, H, LATENT_DIM, dtype=torch.float32)
    lse2 = torch.full((B, q_len, H), float("-inf"), dtype=torch.float32)
    for b in range(B):
        n = int(seq_lens[b])
        if n <= 0:
            if sink is not None:  # the softmax is over the sink alone: zero output, LSE = the sink's logit
                lse2[b] = (sink.detach().cpu().float().reshape(1, H) * LOG2_E).expand(q_len, H)
            continue
        n_pages = (n + page_size - 1) // page_size
        pages = block_tables[b, :n_pages].to(torch.long)
        lat, rope = dequantize_cache(kv_cache[pages], kv_cache_sf[pages])
        lat = lat.reshape(-1, LATENT_DIM)[:n]
        rope = rope.reshape(-1, ROPE_DIM)[:n]
        qb = qf[b].reshape(q_len * H, D)
        score = qb[:, :LATENT_DIM] @ lat.T + qb[:, LATENT_DIM:] @ rope.T
        if logits_soft_cap > 0:
            score = float(logits_soft_cap) * torch.tanh(score / float(logits_soft_cap))
        x = score * float(softmax_scale)
        m = x.max(dim=-1, keepdim=True).values
        if sink is not None:
            sk = sink.detach().cpu().float().reshape(1, H).expand(q_len, H).reshape(q_len * H, 1)
            m = torch.maximum(m, sk)
        p = torch.exp(x - m)
        l = p.sum(dim=-1, keepdim=True)
        if sink is not None:
            l = l + torch.exp(sk - m)
        o = (p @ lat) / l * float(output_scale)
        out[b] = o.reshape(q_len, H, LATENT_DIM)
        lse2[b] = ((m + torch.log(l)) * LOG2_E).reshape(q_len, H)
    return out, lse2


@torch.no_grad()
def merge_partials(outs: Sequence[torch.Tensor], lse2s: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge normalised partial outputs [..., 512] with base-2 LSEs [...] (split-KV / context-parallel).

    Same arithmetic as the reference's split-KV reduction
    (flashinfer 0.6.17 ``cute_dsl/attention/mla_decode.py`` reduction_kernel, read at 0.6.11.post2:644-707):
    w_i = exp2(lse_i - lse_max) / sum_j exp2(lse_j - lse_max).  A partial with lse = -inf contributes nothing.
    """
    o = torch.stack([t.float() for t in outs], dim=0)
    l = torch.stack([t.float() for t in lse2s], dim=0)
    lmax = l.max(dim=0).values
    safe = torch.where(torch.isfinite(lmax), lmax, torch.zeros_like(lmax))
    w = torch.exp2(l - safe)
    w = torch.where(torch.isfinite(l), w, torch.zeros_like(w))
    den = w.sum(dim=0)
    merged = (w[..., None] * torch.where(torch.isfinite(o), o, torch.zeros_like(o))).sum(dim=0)
    merged = merged / torch.where(den > 0, den, torch.ones_like(den))[..., None]
    lse = torch.where(den > 0, torch.log2(torch.where(den > 0, den, torch.ones_like(den))) + safe,
                      torch.full_like(den, float("-inf")))
    return merged, lse


# --------------------------------------------------------------------------- parity metrics


def parity_metrics(out: torch.Tensor, ref: torch.Tensor) -> dict:
    """Per-head parity: cosine, and max-abs error relative to that head's output RMS.

    ``out``/``ref``: [B, q_len, H, 512]; every (request, query position, head) row is judged on
    its own and the worst row is reported.  Rows whose reference is all zero (seq_len == 0)
    must be all zero in ``out`` and are left out of both figures.
    """
    o = out.detach().float().cpu().reshape(-1, out.shape[-1])
    r = ref.detach().float().cpu().reshape(-1, ref.shape[-1])
    rn = r.norm(dim=-1)
    on = o.norm(dim=-1)
    live = rn > 0
    cos = torch.ones_like(rn)
    cos[live] = (o[live] * r[live]).sum(-1) / (on[live] * rn[live]).clamp_min(1e-30)
    dead_ok = bool((on[~live] == 0).all()) if (~live).any() else True
    row_rms = r.pow(2).mean(dim=-1).sqrt()
    row_err = (o - r).abs().amax(dim=-1)
    rel = torch.zeros_like(row_rms)
    rel[live] = row_err[live] / row_rms[live]
    return {
        "min_cos": float(cos.min()) if cos.numel() else 1.0,
        "max_abs": float(row_err.max()) if row_err.numel() else 0.0,
        "rms": float(r[live].pow(2).mean().sqrt()) if live.any() else 0.0,
        "max_abs_over_rms": float(rel.max()) if rel.numel() else 0.0,
        "finite": bool(torch.isfinite(o).all()),
        "dead_rows_zero": dead_ok,
    }


COS_BAR = 0.9999
MAXABS_OVER_RMS_BAR = 2e-2


def assert_parity(out: torch.Tensor, ref: torch.Tensor, what: str = "") -> dict:
    m = parity_metrics(out, ref)
    assert m["finite"], f"{what}: non-finite output"
    assert m["dead_rows_zero"], f"{what}: rows with seq_len 0 are not zero"
    assert m["min_cos"] >= COS_BAR, f"{what}: min per-head cosine {m['min_cos']:.6f} < {COS_BAR}"
    assert m["max_abs_over_rms"] <= MAXABS_OVER_RMS_BAR, (
        f"{what}: max-abs/RMS {m['max_abs_over_rms']:.4e} > {MAXABS_OVER_RMS_BAR}"
    )
    return m
