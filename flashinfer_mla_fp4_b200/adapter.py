"""Serving-engine side of the FP4 MLA decode path: a paged-attention backend shim.

The reference ships the kernel wrapper only; "KV cache quantization, cache writes, prefill
handling, and SGLang backend routing remain the caller's responsibility" (reference
README.md:81-83) and its serving integration is private (README.md:124-126).  This module is
that caller for the decode step, in the shape paged-attention backends have:

* ``FP4MLAPagedCache``        the two cache tensors of the format (rows + per-token scales);
* ``decode_slot_mapping``     flat cache slots of the tokens a decode step appends;
* ``FP4MLADecodeBackend``     persistent (CUDA-graph-safe) step metadata, ``prepare()`` to
  refresh it from the scheduler's tensors, ``forward()`` = append the step's tokens to the cache
  with the CUDA writer, then attend with ``BatchMLADecodeCuteDSLFP4Wrapper.run`` (or, with a
  context-parallel group, ``ContextParallelDecoder.run``); ``capture()`` records ``forward`` in a
  CUDA graph that ``prepare()`` + ``replay()`` drive afterwards.

Data-parallel attention needs no wiring: every rank owns a backend and its own requests.
"""
from __future__ import annotations

from typing import Optional

import torch

from .api_log import api_logged
from .kvcache import HEAD_DIM_QK, LATENT_DIM, ROPE_DIM, ROW_BYTES, write_tokens
from .wrapper import BatchMLADecodeCuteDSLFP4Wrapper


class FP4MLAPagedCache:
    """The paged cache of one layer: ``kv_cache`` u8 [pages, page_size, 320] and ``kv_cache_sf`` f32 [pages, page_size, 1]."""

    def __init__(self, num_pages: int, page_size: int, device) -> None:
        self.page_size = page_size
        self.kv_cache = torch.zeros(num_pages, page_size, ROW_BYTES, dtype=torch.uint8, device=device)
        self.kv_cache_sf = torch.zeros(num_pages, page_size, 1, dtype=torch.float32, device=device)

    @property
    def num_pages(self) -> int:
        return self.kv_cache.shape[0]

    def bytes(self) -> int:
        return self.kv_cache.numel() + 4 * self.kv_cache_sf.numel()


def decode_slot_mapping(block_tables: torch.Tensor, seq_lens: torch.Tensor, page_size: int, q_len: int = 1) -> torch.Tensor:
    """Cache slots of the ``q_len`` newest tokens of every request (int64 [batch * q_len]).

    ``seq_lens`` counts the tokens the step appends (the convention of paged-attention backends:
    the new token attends to itself), so request b writes positions ``seq_len - q_len .. seq_len - 1``
    at ``block_tables[b, pos // page_size] * page_size + pos % page_size``.  Positions below zero
    (a padded request with ``seq_len`` 0, or fewer than ``q_len`` tokens) give -1, which the writer skips.
    """
    sl = seq_lens.to(torch.int64).unsqueeze(1)
    pos = sl - q_len + torch.arange(q_len, device=seq_lens.device, dtype=torch.int64).unsqueeze(0)
    valid = pos >= 0
    posc = pos.clamp(min=0)
    page = block_tables.to(torch.int64).gather(1, (posc // page_size).clamp(max=block_tables.shape[1] - 1))
    slot = page * page_size + posc % page_size
    return torch.where(valid, slot, torch.full_like(slot, -1)).reshape(-1).contiguous()


class FP4MLADecodeBackend:
    """Decode-step backend over persistent metadata buffers (one instance per layer group and device).

    The scheduler's per-step tensors (block tables, sequence lengths counting the new tokens, and
    optionally the slot mapping) are copied by ``prepare()`` into buffers whose addresses never
    change, sized for ``max_batch`` requests of ``max_seq_len`` tokens; rows past the step's batch
    are padding (``seq_len`` 0 -> zero output, slot -1 -> no cache write).  ``forward()`` reads only
    those buffers and its tensor arguments, launches on the current stream and never synchronises,
    so it can be recorded in a CUDA graph once and replayed for every later step.
    """

    def __init__(self, num_heads: int, page_size: int, max_batch: int, max_seq_len: int, softmax_scale: float, device,
                 *, q_len: int = 1, out_dtype: Optional[torch.dtype] = None, output_scale: float = 1.0,
                 workspace_buffer: Optional[torch.Tensor] = None, cp_group=None) -> None:
        from . import _cabi

        self.device = torch.device(device)
        self.num_heads, self.page_size, self.q_len = num_heads, page_size, q_len
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.softmax_scale, self.output_scale = float(softmax_scale), float(output_scale)
        if workspace_buffer is None:
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            workspace_buffer = torch.empty(_cabi.workspace_bytes(max_batch, q_len, num_heads, sms), dtype=torch.int8, device=self.device)
        self.wrapper = BatchMLADecodeCuteDSLFP4Wrapper(workspace_buffer)
        self.wrapper.plan(num_heads=num_heads, page_size=page_size, out_dtype=out_dtype)
        self._runner = self.wrapper
        if cp_group is not None:
            from .distributed import ContextParallelDecoder

            self._runner = ContextParallelDecoder(self.wrapper, cp_group, max_rows=max_batch * q_len * num_heads)
        self.max_pages = (max_seq_len + page_size - 1) // page_size
        self.block_tables = torch.zeros(max_batch, self.max_pages, dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.slot_mapping = torch.full((max_batch * q_len,), -1, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ metadata
    def clear(self) -> None:
        """Make every row padding (what the buffers hold before the first ``prepare``)."""
        self.seq_lens.zero_()
        self.slot_mapping.fill_(-1)

    @api_logged
    def prepare(self, block_tables: torch.Tensor, seq_lens: torch.Tensor, slot_mapping: Optional[torch.Tensor] = None) -> int:
        """Refresh the persistent metadata for one step; returns the step's batch size.

        ``block_tables`` int32 [batch, <= max_pages] (physical page ids), ``seq_lens`` [batch] counting
        the tokens this step appends, ``slot_mapping`` int64 [batch * q_len] or None to derive it
        (``decode_slot_mapping``).  Host or device tensors; the copies are asynchronous on the current
        stream (pin host tensors to keep them so).  With a context-parallel group all three are the
        rank's LOCAL view (its pages, its share of every request's tokens, -1 for tokens it does not own).
        """
        batch = int(seq_lens.shape[0])
        if batch > self.max_batch:
            raise ValueError(f"batch {batch} exceeds max_batch {self.max_batch}")
        if block_tables.dim() != 2 or block_tables.shape[0] != batch or block_tables.shape[1] > self.max_pages:
            raise ValueError(f"block_tables must be [batch, <= {self.max_pages}], got {tuple(block_tables.shape)}")
        if slot_mapping is None:
            slot_mapping = decode_slot_mapping(block_tables, seq_lens, self.page_size, self.q_len)
        elif slot_mapping.numel() != batch * self.q_len:
            raise ValueError(f"slot_mapping must hold batch * q_len = {batch * self.q_len} slots")
        self.block_tables[:batch, : block_tables.shape[1]].copy_(block_tables, non_blocking=True)
        self.seq_lens[:batch].copy_(seq_lens, non_blocking=True)
        self.seq_lens[batch:].zero_()
        self.slot_mapping[: batch * self.q_len].copy_(slot_mapping.reshape(-1), non_blocking=True)
        self.slot_mapping[batch * self.q_len:].fill_(-1)
        return batch

    # ------------------------------------------------------------------ the step
    @api_logged
    def forward(self, q: torch.Tensor, latent: torch.Tensor, rope: torch.Tensor, cache: FP4MLAPagedCache,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Append this step's tokens to ``cache`` and attend over it.

        ``q`` e4m3 [batch, q_len, H, 576]; ``latent`` [batch * q_len, 512] and ``rope`` [batch * q_len, 64]
        (bf16, f16 or f32) are the new tokens' compressed KV and RoPE key, in request order; ``batch`` may
        be anything up to ``max_batch`` (rows the last ``prepare`` did not fill are padding).  Returns
        ``out`` [batch, q_len, H, 512].

        With ``q_len`` > 1 all ``q_len`` new tokens are appended first and EVERY query position then attends to
        all ``seq_len`` tokens, the later draft tokens included: there is no causal mask among the query
        positions (the reference itself accepts only ``q_len`` = 1, wrappers/batch_mla_fp4.py:297-298).  That is
        the attention of a batched multi-token step whose positions may see one another; a verification step of
        speculative decoding that needs position i blind to positions > i must issue its positions as separate
        requests (``q_len`` = 1, ``seq_len`` reduced accordingly).
        """
        batch = q.shape[0]
        if batch > self.max_batch or q.shape[1] != self.q_len:
            raise ValueError(f"q must be [<= {self.max_batch}, {self.q_len}, H, {HEAD_DIM_QK}], got {tuple(q.shape)}")
        n = batch * self.q_len
        if latent.shape != (n, LATENT_DIM) or rope.shape != (n, ROPE_DIM):
            raise ValueError(f"latent must be [{n}, {LATENT_DIM}] and rope [{n}, {ROPE_DIM}]")
        if cache.page_size != self.page_size:
            raise ValueError(f"cache page size {cache.page_size} does not match the backend's {self.page_size}")
        write_tokens(latent, rope, self.slot_mapping[:n], cache.kv_cache, cache.kv_cache_sf)
        return self._runner.run(q, cache.kv_cache, self.block_tables[:batch], self.seq_lens[:batch], self.max_seq_len,
                                self.softmax_scale, output_scale=self.output_scale, out=out, kv_cache_sf=cache.kv_cache_sf)

    def capture(self, cache: FP4MLAPagedCache, batch: Optional[int] = None, in_dtype: torch.dtype = torch.bfloat16,
                warmup: int = 2) -> "CapturedDecodeStep":
        """Record ``forward`` for ``batch`` (default ``max_batch``) requests in a CUDA graph.

        The warm-up runs and the capture see padding metadata only, so they touch neither the cache nor
        any request; afterwards fill ``step.q / step.latent / step.rope``, call ``prepare()`` and
        ``step.replay()`` each step and read ``step.out``.
        """
        batch = self.max_batch if batch is None else batch
        n = batch * self.q_len
        step = CapturedDecodeStep()
        step.q = torch.zeros(batch, self.q_len, self.num_heads, HEAD_DIM_QK, dtype=torch.float8_e4m3fn, device=self.device)
        step.latent = torch.zeros(n, LATENT_DIM, dtype=in_dtype, device=self.device)
        step.rope = torch.zeros(n, ROPE_DIM, dtype=in_dtype, device=self.device)
        step.out = torch.empty(batch, self.q_len, self.num_heads, LATENT_DIM, dtype=self.wrapper._o_dtype, device=self.device)
        self.clear()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.forward(step.q, step.latent, step.rope, cache, out=step.out)
        torch.cuda.current_stream(self.device).wait_stream(side)
        step.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step.graph):
            self.forward(step.q, step.latent, step.rope, cache, out=step.out)
        return step


class CapturedDecodeStep:
    """A recorded ``FP4MLADecodeBackend.forward``: static input/output tensors and the graph."""

    q: torch.Tensor
    latent: torch.Tensor
    rope: torch.Tensor
    out: torch.Tensor
    graph: "torch.cuda.CUDAGraph"

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out


__all__ = ["FP4MLAPagedCache", "FP4MLADecodeBackend", "CapturedDecodeStep", "decode_slot_mapping"]
