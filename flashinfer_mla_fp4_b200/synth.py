"""Seeded synthetic decode workloads with the shapes and value distributions of
the benchmark configurations (they stand in for model activations, which are
not available offline).

Every generator draws from one ``torch.Generator`` seeded by the caller, on the
requested device, so a case can be rebuilt bit for bit from (name, seed).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .kvcache import HEAD_DIM_QK, LATENT_DIM, ROPE_DIM, quantize_tokens


@dataclass
class DecodeCase:
    name: str
    q: torch.Tensor  # e4m3 [B, q_len, H, 576]
    kv_cache: torch.Tensor  # u8 [P, page_size, 320]
    kv_cache_sf: torch.Tensor  # f32 [P, page_size, 1]
    block_tables: torch.Tensor  # i32 [B, max_pages]
    seq_lens: torch.Tensor  # i32 [B]
    page_size: int
    num_heads: int
    q_len: int
    softmax_scale: float
    seed: int
    seq_lens_host: List[int] = field(default_factory=list)

    @property
    def batch(self) -> int:
        return self.q.shape[0]

    @property
    def max_seq_len(self) -> int:
        return max(1, max(self.seq_lens_host) if self.seq_lens_host else 1)

    @property
    def kv_tokens(self) -> int:
        return int(sum(self.seq_lens_host))

    def kv_bytes(self) -> int:
        """Algorithmic KV bytes of one decode step: 324 per attended token."""
        return 324 * self.kv_tokens

    def step_bytes(self) -> int:
        """KV bytes + query + BF16 output + page ids + seq_lens actually needed by one step."""
        B, ql, H = self.batch, self.q_len, self.num_heads
        pages = sum((n + self.page_size - 1) // self.page_size for n in self.seq_lens_host)
        return self.kv_bytes() + B * ql * H * HEAD_DIM_QK + B * ql * H * LATENT_DIM * 2 + 4 * pages + 4 * B

    def flops(self) -> int:
        return 2176 * self.kv_tokens * self.num_heads * self.q_len


def _randn(shape, gen, device):
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32)


def _student_t3(shape, gen, device):
    """Student-t with 3 degrees of freedom: z / sqrt(chi2_3 / 3)."""
    z = _randn(shape, gen, device)
    chi = _randn((*shape[:-1], 3), gen, device).pow(2).sum(-1, keepdim=True)
    return z / torch.sqrt(chi / 3.0)


@torch.no_grad()
def build_case(
    name: str,
    seq_lens: List[int],
    num_heads: int,
    page_size: int = 64,
    q_len: int = 1,
    seed: int = 0,
    device="cpu",
    pool_factor: float = 2.0,
    latent_dist: str = "normal",
    q_std: float = 1.0,
    chunk_pages: int = 4096,
) -> DecodeCase:
    """Build one decode case.

    Pages of all requests are scattered over a pool of ``pool_factor`` x the pages
    needed by a seeded permutation; the unused pool pages hold random bytes (their
    rows may decode to NaN RoPE, which a correct kernel never reads into a result).
    """
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    B = len(seq_lens)
    pages_per_req = [(n + page_size - 1) // page_size for n in seq_lens]
    need = sum(pages_per_req)
    pool = max(need + 1, int(math.ceil(need * pool_factor)))
    perm = torch.randperm(pool, generator=gen, device=device)[:need].to(torch.int32)
    max_pages = max(1, max(pages_per_req) if pages_per_req else 1)
    block_tables = torch.zeros(B, max_pages, dtype=torch.int32, device=device)
    off = 0
    for b, n in enumerate(pages_per_req):
        block_tables[b, :n] = perm[off : off + n]
        off += n

    # pool filled with random bytes, then the used pages are written properly
    kv_cache = torch.randint(0, 256, (pool, page_size, 320), generator=gen, device=device, dtype=torch.uint8)
    kv_cache_sf = torch.empty(pool, page_size, 1, dtype=torch.float32, device=device)
    kv_cache_sf.copy_(_randn((pool, page_size, 1), gen, device).abs() + 0.1)
    for start in range(0, need, chunk_pages):
        idx = perm[start : start + chunk_pages].to(torch.long)
        n = idx.numel()
        if latent_dist == "normal":
            lat = _randn((n, page_size, LATENT_DIM), gen, device)
        elif latent_dist == "student_t3":
            lat = _student_t3((n, page_size, LATENT_DIM), gen, device)
        else:
            raise ValueError(latent_dist)
        rope = _randn((n, page_size, ROPE_DIM), gen, device)
        rows, sf = quantize_tokens(lat, rope)
        kv_cache[idx] = rows
        kv_cache_sf[idx] = sf
    q = (_randn((B, q_len, num_heads, HEAD_DIM_QK), gen, device) * q_std).to(torch.float8_e4m3fn)
    return DecodeCase(
        name=name,
        q=q,
        kv_cache=kv_cache,
        kv_cache_sf=kv_cache_sf,
        block_tables=block_tables,
        seq_lens=torch.tensor(seq_lens, dtype=torch.int32, device=device),
        page_size=page_size,
        num_heads=num_heads,
        q_len=q_len,
        softmax_scale=1.0 / math.sqrt(LATENT_DIM),
        seed=seed,
        seq_lens_host=list(seq_lens),
    )


def _log_uniform_lens(n: int, lo: int, hi: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=g, dtype=torch.float64)
    v = torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo))).round().clamp(lo, hi)
    return [int(x) for x in v]


def _uniform_lens(n: int, lo: int, hi: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return [int(x) for x in torch.randint(lo, hi + 1, (n,), generator=g)]


def config_case(config: str, device="cpu", seed: Optional[int] = None, scale: float = 1.0) -> DecodeCase:
    """The named benchmark configurations.

    ``small``      B=2  H=16  S=256            page 64 (8 pages, permuted)
    ``uniform``    B=4  H=64  S=4096           page 64, pool 2x
    ``northstar``  B=8  H=64  S=32768          page 64, pool 2x
    ``varlen``     B=128 H=64 S~logU[128,32768], Student-t(3) latents
    ``spec``       B=2  H=128 q_len=2 S=131072
    ``scale`` < 1 shrinks sequence lengths (for tests); shapes otherwise unchanged.
    """
    base_seed = {"small": 1000, "uniform": 1001, "northstar": 1005, "varlen": 1002, "spec": 1003}

    def sl(n):
        return max(1, int(round(n * scale)))

    sd = base_seed[config] if seed is None else seed
    if config == "small":
        return build_case("small", [sl(256)] * 2, 16, 64, 1, sd, device, pool_factor=1.0)
    if config == "uniform":
        return build_case("uniform", [sl(4096)] * 4, 64, 64, 1, sd, device)
    if config == "northstar":
        return build_case("northstar", [sl(32768)] * 8, 64, 64, 1, sd, device)
    if config == "varlen":
        lens = [sl(n) for n in _log_uniform_lens(128, 128, 32768, sd)]
        return build_case("varlen", lens, 64, 64, 1, sd, device, latent_dist="student_t3")
    if config == "spec":
        return build_case("spec", [sl(131072)] * 2, 128, 64, 2, sd, device)
    raise ValueError(f"unknown config {config!r}")


def dp_lens(batch: int = 512, lo: int = 1024, hi: int = 16384, seed: int = 1004) -> List[int]:
    """Sequence lengths of the data-parallel configuration (uniform in [lo, hi])."""
    return _uniform_lens(batch, lo, hi, seed)
