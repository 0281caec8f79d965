"""Multi-GPU decode: data-parallel attention and decode context parallel.

The reference has no multi-GPU code (its README only mentions DPA=8 / DCP=8 runs in a private
serving fork, README.md:122-126).  Two ways the path shards across the GPUs of one box:

* data-parallel attention: requests are split across ranks, every rank decodes its own requests
  against its own pages; there is no data-path collective (``shard_requests``).
* decode context parallel: the KV pages of every request are cut into contiguous, page-aligned
  shards, one per rank; every rank decodes its shard into a normalised FP32 partial output plus a
  base-2 LSE per (request, head), and the partials are merged: w_r = exp2(lse_r - max) / sum.
  Two exchanges: ``"peer"`` (the default on GPUs) is one kernel per rank that pushes the partial into
  every peer's memory with plain stores over NVLink, flags it, waits (bounded) for the peers' flags and
  merges (``mla_fp4_cp_exchange_merge``); ``"nccl"`` is one NCCL all-gather into local memory followed by
  the merge kernel (``mla_fp4_merge_partials``), the form that also runs over gloo on CPUs.

One process per GPU; set-up and the ``"nccl"`` exchange go through ``torch.distributed``.
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
    All ranks must make the same sequence of ``run`` calls.

    ``exchange="peer"`` needs all ranks on GPUs of one NVLink domain (one box) and at most 8 ranks; its
    exchange block (``max_rows`` rows of partials, double buffered, ``world`` sources) is allocated here,
    once, and mapped into every peer through CUDA IPC.  ``exchange="nccl"`` has no such limits.
    """

    def __init__(self, wrapper, group=None, exchange: str = "peer", max_rows: int = 1024, algo: str = "auto") -> None:
        from .wrapper import BatchMLADecodeCuteDSLFP4Wrapper

        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self._group = group if group is not None else dist.group.WORLD
        self._world = dist.get_world_size(self._group)
        self._rank = dist.get_rank(self._group)
        self._final_dtype = wrapper._o_dtype
        self._device = wrapper._device
        # the local pass writes FP32 partials; it shares the caller's workspace
        self._local = BatchMLADecodeCuteDSLFP4Wrapper(wrapper._workspace_buffer)
        self._local.plan(num_heads=wrapper._num_heads, page_size=wrapper._page_size, out_dtype=torch.float32,
                         is_var_seq=wrapper._is_var_seq, enable_pdl=wrapper._enable_pdl)
        # the attention variant of the caller's plan; a sink joins the denominator once per request: on rank 0 only
        self._local._soft_cap = wrapper._soft_cap
        self._local._sink = wrapper._sink if self._rank == 0 else None
        self._local._num_ctas = wrapper._num_ctas
        self._buf: Optional[torch.Tensor] = None
        self._gathered: Optional[torch.Tensor] = None
        self._exchange = exchange
        self._max_rows = max_rows
        self._blocks = None
        self._own_block = None
        self._wait_polls = 0
        # form of the peer exchange: "all_gather" (one hop, world-1 partials per rank), "reduce_scatter" (every row merged by
        # one owner rank, two hops, under two partials per rank) or "auto" (all-gather below four ranks)
        self._algo = {"auto": _cabi.CP_AUTO, "all_gather": _cabi.CP_ALL_GATHER, "reduce_scatter": _cabi.CP_REDUCE_SCATTER}[algo]
        if exchange == "peer":
            self._setup_peer_blocks()

    # ------------------------------------------------------------------ peer exchange set-up
    def _setup_peer_blocks(self) -> None:
        if self._world > _cabi.CP_MAX_RANKS:
            raise ValueError(f"exchange='peer' supports at most {_cabi.CP_MAX_RANKS} ranks, got {self._world}")
        nbytes = C.c_size_t(0)
        _cabi.check(_cabi.lib.mla_fp4_cp_exchange_bytes(self._world, self._max_rows, C.byref(nbytes)))
        own = C.c_void_p()
        handle = C.create_string_buffer(_cabi.CP_HANDLE_BYTES)
        with torch.cuda.device(self._device):
            _cabi.check(_cabi.lib.mla_fp4_cp_alloc(nbytes.value, C.byref(own), handle))
        self._own_block = own.value
        handles: List[Optional[bytes]] = [None] * self._world
        dist.all_gather_object(handles, handle.raw, group=self._group)
        blocks = (C.c_void_p * _cabi.CP_MAX_RANKS)()
        for r in range(self._world):
            if r == self._rank:
                blocks[r] = self._own_block
            else:
                peer = C.c_void_p()
                with torch.cuda.device(self._device):
                    _cabi.check(_cabi.lib.mla_fp4_cp_open(handles[r], C.byref(peer)))
                blocks[r] = peer.value
        self._blocks = blocks
        dist.barrier(group=self._group)  # every rank has mapped every block before the first step

    def close(self) -> None:
        """Unmap the peers' exchange blocks and free the own one (after a barrier: nobody is still using them)."""
        if self._blocks is None:
            return
        torch.cuda.synchronize(self._device)
        dist.barrier(group=self._group)
        with torch.cuda.device(self._device):
            for r in range(self._world):
                if r != self._rank and self._blocks[r]:
                    _cabi.lib.mla_fp4_cp_close(self._blocks[r])
            dist.barrier(group=self._group)
            _cabi.lib.mla_fp4_cp_free(self._own_block)
        self._blocks = None
        self._own_block = None

    def _buffers(self, rows: int, device) -> None:
        n = rows * LATENT_DIM + ((rows + 3) // 4) * 4  # partial outputs, then LSEs (padded to 16 bytes)
        if self._buf is None or self._buf.numel() != n:
            self._buf = torch.empty(n, dtype=torch.float32, device=device)
            if self._exchange == "nccl":
                self._gathered = torch.empty(self._world * n, dtype=torch.float32, device=device)

    @api_logged
    def run(self, q, kv_cache, block_tables, seq_lens, max_seq_len, softmax_scale, output_scale: float = 1.0,
            out: Optional[torch.Tensor] = None, kv_cache_sf: Optional[torch.Tensor] = None, return_lse: bool = False,
            lse_out: Optional[torch.Tensor] = None):
        B, ql, H, _ = q.shape
        rows = B * ql * H
        if self._exchange == "peer" and rows > self._max_rows:
            raise ValueError(f"batch*q_len*num_heads = {rows} exceeds max_rows = {self._max_rows} of the exchange block")
        self._buffers(rows, q.device)
        part_o = self._buf[: rows * LATENT_DIM].view(B, ql, H, LATENT_DIM)
        part_lse = self._buf[rows * LATENT_DIM: rows * LATENT_DIM + rows].view(B, ql, H)
        # 1. local shard -> normalised FP32 partial + base-2 LSE, written straight into the packed buffer [rows*512 | rows]
        local_max = max(1, min(int(max_seq_len), block_tables.shape[1] * self._local._page_size))  # the shard's own bound
        self._local.run(q, kv_cache, block_tables, seq_lens, local_max, softmax_scale,
                        output_scale=output_scale, out=part_o, kv_cache_sf=kv_cache_sf, return_lse=True, lse_out=part_lse)
        if out is None:
            out = torch.empty(B, ql, H, LATENT_DIM, dtype=self._final_dtype, device=q.device)
        if return_lse and lse_out is None:
            lse_out = torch.empty(B, ql, H, dtype=torch.float32, device=q.device)
        if not return_lse:
            lse_out = None
        odt = {torch.bfloat16: _cabi.OUT_BF16, torch.float32: _cabi.OUT_F32, torch.float8_e4m3fn: _cabi.OUT_E4M3}[out.dtype]
        lse_ptr = C.c_void_p(lse_out.data_ptr()) if lse_out is not None else None
        with torch.cuda.device(q.device):
            stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
            if self._exchange == "peer":
                # 2+3. one kernel: push to the peers, flag, wait for their flags, merge
                _cabi.check(_cabi.lib.mla_fp4_cp_exchange_merge(
                    self._blocks, self._world, self._rank, C.c_void_p(self._buf.data_ptr()), rows, self._max_rows,
                    C.c_void_p(out.data_ptr()), odt, lse_ptr, C.c_void_p(self._local._status.data_ptr()), self._wait_polls,
                    1 if self._local._enable_pdl else 0, self._algo, stream))
            else:
                # 2. one all-gather into local memory  3. merge kernel over the gathered partials
                dist.all_gather_into_tensor(self._gathered, self._buf, group=self._group)
                stride = self._buf.numel()
                base = self._gathered.data_ptr()
                _cabi.check(_cabi.lib.mla_fp4_merge_partials(
                    C.c_void_p(base), C.c_void_p(base + 4 * rows * LATENT_DIM), self._world, rows, stride, stride,
                    C.c_void_p(out.data_ptr()), odt, lse_ptr, stream))
        return (out, lse_out) if return_lse else out

    def check_device_status(self) -> None:
        self._local.check_device_status()
