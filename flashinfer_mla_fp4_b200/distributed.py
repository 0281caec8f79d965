"""Multi-GPU decode: data-parallel attention and decode context parallel.

The reference has no multi-GPU code (its README only mentions DPA=8 / DCP=8 runs in a private
serving fork, README.md:122-126).  Two ways the path shards across the GPUs of one box:

* data-parallel attention: requests are split across ranks, every rank decodes its own requests
  against its own pages; there is no data-path collective (``shard_requests``).
* decode context parallel: the KV pages of every request are cut into contiguous, page-aligned
  shards, one per rank; every rank decodes its shard into a normalised FP32 partial output plus a
  base-2 LSE per (request, head); one NCCL all-gather brings all partials into local memory and
  the merge kernel (``mla_fp4_merge_partials``) combines them: w_r = exp2(lse_r - max) / sum.

One process per GPU; collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs,
gloo in the CPU tests of the sharding logic).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _cabi
from .api_log import api_logged
from .kvcache import LATENT_DIM


def shard_requests(seq_lens: Sequence[int], world: int, balance: bool = True) -> List[List[int]]:
    """Request indices per rank for data-parallel attention.

    ``balance=True`` assigns the longest remaining request to the least loaded rank (LPT), which
    keeps the max-over-ranks KV volume close to the mean; ``False`` cuts contiguous blocks.
    """
    n = len(seq_lens)
    if not balance:
        per = (n + world - 1) // world
        return [list(range(r * per, min(n, (r + 1) * per))) for r in range(world)]
    order = sorted(range(n), key=lambda i: -int(seq_lens[i]))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(seq_lens[i])
    return [sorted(x) for x in out]


def shard_context(block_tables: torch.Tensor, seq_lens: torch.Tensor, page_size: int, rank: int, world: int
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rank-local (block_tables, seq_lens) of a context-parallel decode.

    Request b with n_b pages gives rank r the logical pages [r*n_b//world, (r+1)*n_b//world);
    the ragged last page stays with the rank that owns it.  Ranks whose shard is empty get
    seq_len 0 (their partial has lse = -inf and does not contribute).
    """
    B, max_pages = block_tables.shape
    sl = seq_lens.to(torch.int64)
    n_pages = (sl + page_size - 1) // page_size
    lo = (n_pages * rank) // world
    hi = (n_pages * (rank + 1)) // world
    width = max(1, int((hi - lo).max().item())) if B > 0 else 1
    cols = torch.arange(width, device=block_tables.device).unsqueeze(0) + lo.unsqueeze(1)
    valid = cols < hi.unsqueeze(1)
    local_bt = torch.where(valid, block_tables.gather(1, cols.clamp_(0, max_pages - 1)), torch.zeros_like(cols, dtype=block_tables.dtype))
    local_sl = (torch.minimum(sl, hi * page_size) - lo * page_size).clamp_(min=0)
    local_sl = torch.where(hi > lo, local_sl, torch.zeros_like(local_sl))
    return local_bt.to(torch.int32).contiguous(), local_sl.to(torch.int32)


class ContextParallelDecoder:
    """Decode over a KV cache whose tokens are sharded across the ranks of ``group``.

    Every rank calls ``run`` with ITS shard (rank-local cache pages, block tables and seq_lens, for
    instance from ``shard_context``) and the full, replicated query; every rank gets the full output.
    """

    def __init__(self, wrapper, group=None) -> None:
        from .wrapper import BatchMLADecodeCuteDSLFP4Wrapper

        self._group = group if group is not None else dist.group.WORLD
        self._world = dist.get_world_size(self._group)
        self._rank = dist.get_rank(self._group)
        self._final_dtype = wrapper._o_dtype
        # the local pass writes FP32 partials; it shares the caller's workspace
        self._local = BatchMLADecodeCuteDSLFP4Wrapper(wrapper._workspace_buffer)
        self._local.plan(num_heads=wrapper._num_heads, page_size=wrapper._page_size, out_dtype=torch.float32,
                         is_var_seq=wrapper._is_var_seq, enable_pdl=wrapper._enable_pdl)
        self._buf: Optional[torch.Tensor] = None
        self._gathered: Optional[torch.Tensor] = None

    def _buffers(self, rows: int, device) -> None:
        n = rows * LATENT_DIM + ((rows + 3) // 4) * 4  # partial outputs, then LSEs (padded to 16 bytes)
        if self._buf is None or self._buf.numel() != n:
            self._buf = torch.empty(n, dtype=torch.float32, device=device)
            self._gathered = torch.empty(self._world * n, dtype=torch.float32, device=device)

    @api_logged
    def run(self, q, kv_cache, block_tables, seq_lens, max_seq_len, softmax_scale, output_scale: float = 1.0,
            out: Optional[torch.Tensor] = None, kv_cache_sf: Optional[torch.Tensor] = None, return_lse: bool = False):
        B, ql, H, _ = q.shape
        rows = B * ql * H
        self._buffers(rows, q.device)
        part_o = self._buf[: rows * LATENT_DIM].view(B, ql, H, LATENT_DIM)
        # 1. local shard -> normalised FP32 partial + base-2 LSE, packed [rows*512 | rows]
        _, lse = self._local.run(q, kv_cache, block_tables, seq_lens, max(1, max_seq_len), softmax_scale,
                                 output_scale=output_scale, out=part_o, kv_cache_sf=kv_cache_sf, return_lse=True)
        self._buf[rows * LATENT_DIM: rows * LATENT_DIM + rows].copy_(lse.view(-1))
        # 2. one all-gather into local memory
        dist.all_gather_into_tensor(self._gathered, self._buf, group=self._group)
        # 3. merge kernel over the gathered partials
        if out is None:
            out = torch.empty(B, ql, H, LATENT_DIM, dtype=self._final_dtype, device=q.device)
        lse_out = torch.empty(B, ql, H, dtype=torch.float32, device=q.device) if return_lse else None
        stride = self._buf.numel()
        base = self._gathered.data_ptr()
        _cabi.check(_cabi.lib.mla_fp4_merge_partials(
            C.c_void_p(base), C.c_void_p(base + 4 * rows * LATENT_DIM), self._world, rows, stride, stride,
            C.c_void_p(out.data_ptr()), {torch.bfloat16: _cabi.OUT_BF16, torch.float32: _cabi.OUT_F32, torch.float8_e4m3fn: _cabi.OUT_E4M3}[out.dtype],
            C.c_void_p(lse_out.data_ptr()) if lse_out is not None else None,
            C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)))
        return (out, lse_out) if return_lse else out
