"""Host side of the drop-in: ``BatchMLADecodeCuteDSLFP4Wrapper.plan()/run()``.

Mirrors reference ``flashinfer_mla_fp4/wrappers/batch_mla_fp4.py:182-458`` (and the
constructor it inherits from flashinfer ``cute_dsl/attention/wrappers/batch_mla.py:368-375``):
same names, argument meaning, defaults and exceptions.  Where the reference JIT-compiles a
CuTe-DSL kernel in ``plan()`` and calls it in ``run()``, this class only validates, sizes the
split-KV scratch and calls the C ABI (``include/mla_fp4_b200.h``) with raw pointers on torch's
current stream.  There is no CPU or library fallback.

Additions over the reference (all opt-in, defaults keep the reference behaviour):
``run(..., return_lse=True)`` returns the base-2 log-sum-exp the reference computes but drops;
``q_len`` > 1 is accepted (every query position attends to all ``seq_len`` tokens);
``out_dtype`` may be ``torch.bfloat16`` (default), ``torch.float8_e4m3fn`` (both as in the reference) or ``torch.float32``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple, Union

import torch

from . import _cabi
from .api_log import api_logged
from .kvcache import LATENT_DIM, ROPE_DIM, ROW_BYTES
from .variants import resolve as resolve_variant

_OUT_DTYPES = {torch.bfloat16: _cabi.OUT_BF16, torch.float32: _cabi.OUT_F32, torch.float8_e4m3fn: _cabi.OUT_E4M3}


def _require_sm100(device: torch.device) -> None:
    """The kernels are sm_100a only (reference wrappers/batch_mla_fp4.py:205 requires a tcgen05 part)."""
    if device.type != "cuda":
        raise RuntimeError("Per-token-scaled FP4 MLA requires a CUDA device (sm_100a)")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"Per-token-scaled FP4 MLA requires sm_100a, got sm_{major}{minor}")


class BatchMLADecodeCuteDSLFP4Wrapper:
    """Stateful per-token-scaled FP4 MLA decode wrapper (plan once, run per step).

    The query and the RoPE part of the cache are E4M3; the 512-value latent is packed E2M1 with
    one FP32 scale per token.  The workspace buffer is borrowed, never copied or freed.
    """

    def __init__(self, workspace_buffer: torch.Tensor) -> None:
        assert workspace_buffer.dtype == torch.int8, "workspace_buffer must be torch.int8"
        self._workspace_buffer = workspace_buffer
        self._device = workspace_buffer.device
        self._planned = False
        self._kernel = _cabi.KERNEL_TCGEN05
        self._status: Optional[torch.Tensor] = None
        self._num_ctas = 0
        self._phase_mask = 0  # profiling aid of the two-kernel mode: 1 = decode kernel only, 2 = combine kernel only
        self._wait_polls = 0  # 0 = the library's default poll budget of a bounded device wait

    # ------------------------------------------------------------------ plan
    @api_logged
    def plan(
        self,
        kv_lora_rank: int = 512,
        qk_rope_head_dim: int = 64,
        num_heads: int = 128,
        page_size: int = 1,
        q_dtype: torch.dtype = torch.float8_e4m3fn,
        out_dtype: Optional[torch.dtype] = None,
        is_var_seq: bool = True,
        enable_pdl: Optional[bool] = None,
        variant=None,
        kv_dtype: torch.dtype = torch.uint8,
        max_ctas: Optional[int] = None,
    ) -> None:
        """Validate the configuration and bind it (nothing is compiled: the kernels are built ahead of time).

        ``variant``: None / ``StandardAttention``, ``AttentionWithSink`` or ``SoftCappingAttention`` (``variants.py``).
        ``max_ctas`` (not in the reference, whose per-request split counts ``block_split_kvs`` are plumbed but switched
        off, wrappers/batch_mla_fp4.py:231, :453): caps the persistent grid, and with it into how many partials the
        requests are split (the tiles of all requests are dealt to the CTAs in order); None = one CTA per SM.
        """
        if kv_lora_rank != 512:
            raise ValueError(f"Per-token-scaled FP4 MLA requires kv_lora_rank=512, got {kv_lora_rank}")
        if qk_rope_head_dim != 64:
            raise ValueError(f"Per-token-scaled FP4 MLA requires qk_rope_head_dim=64, got {qk_rope_head_dim}")
        if q_dtype != torch.float8_e4m3fn:
            raise ValueError("Per-token-scaled FP4 MLA requires an E4M3 query")
        if kv_dtype != torch.uint8:
            raise ValueError("Per-token-scaled FP4 MLA requires a byte-packed uint8 KV cache")
        if not (1 <= num_heads <= 128):
            raise ValueError(f"Unsupported num_heads={num_heads}: must be in [1, 128]")
        soft_cap, sink = resolve_variant(variant, num_heads, self._device)
        o_dtype = torch.bfloat16 if out_dtype is None else out_dtype
        # the reference accepts page sizes that divide 128 except 1, at most 128 heads, bf16/e4m3 output
        # (flashinfer cute_dsl/attention/mla_config.py:186-229); this build: pages of 8..128 tokens, bf16/f32 output
        if page_size not in (8, 16, 32, 64, 128):
            raise ValueError(f"Unsupported page_size={page_size}: must be one of 8, 16, 32, 64, 128")
        if o_dtype not in _OUT_DTYPES:
            raise ValueError(f"Unsupported out_dtype={o_dtype}: must be torch.bfloat16, torch.float8_e4m3fn or torch.float32")
        _require_sm100(self._device)

        self._kv_lora_rank = kv_lora_rank
        self._qk_rope_head_dim = qk_rope_head_dim
        self._num_heads = num_heads
        self._page_size = page_size
        self._q_dtype = q_dtype
        self._o_dtype = o_dtype
        self._is_var_seq = is_var_seq
        self._enable_pdl = True if enable_pdl is None else bool(enable_pdl)
        self._num_ctas = torch.cuda.get_device_properties(self._device).multi_processor_count
        if max_ctas is not None:
            if max_ctas < 1:
                raise ValueError(f"max_ctas must be at least 1, got {max_ctas}")
            self._num_ctas = min(self._num_ctas, int(max_ctas))
        self._soft_cap = soft_cap
        self._sink = sink
        if self._status is None:
            self._status = torch.zeros(8, dtype=torch.int32, device=self._device)
        self._init_workspace()
        self._planned = True

    def _init_workspace(self) -> None:
        """Zero the workspace's header (generation and slot flags of the split-KV merge)."""
        if self._workspace_buffer.is_cuda and self._workspace_buffer.numel() >= _cabi.WORKSPACE_HEADER_BYTES:
            with torch.cuda.device(self._device):
                _cabi.workspace_init(self._workspace_buffer.data_ptr(), self._workspace_buffer.numel(),
                                     torch.cuda.current_stream(self._device).cuda_stream)

    # ------------------------------------------------------------------ run
    def _validate_run_inputs(self, q, kv_cache, kv_cache_sf, out) -> None:
        if q.ndim != 4:
            raise ValueError("q must have shape [batch, q_len, num_heads, head_dim]")
        expected_dim = self._kv_lora_rank + self._qk_rope_head_dim
        if q.shape[-1] != expected_dim or q.shape[2] != self._num_heads:
            raise ValueError(f"q must end in [{self._num_heads}, {expected_dim}], got shape {tuple(q.shape)}")
        if q.dtype != self._q_dtype:
            raise ValueError(f"q.dtype={q.dtype} does not match planned {self._q_dtype}")
        if kv_cache.dtype != torch.uint8:
            raise ValueError("FP4 kv_cache must have dtype torch.uint8")
        if kv_cache_sf is None:
            raise ValueError("FP4 MLA requires kv_cache_sf")
        if kv_cache_sf.dtype != torch.float32:
            raise ValueError("kv_cache_sf must contain FP32 per-token scales")
        if out is not None and out.dtype != self._o_dtype:
            raise ValueError(f"out.dtype={out.dtype} does not match planned {self._o_dtype}")

    @api_logged
    def run(
        self,
        q: torch.Tensor,
        kv_cache: torch.Tensor,
        block_tables: torch.Tensor,
        seq_lens: torch.Tensor,
        max_seq_len: int,
        softmax_scale: float,
        output_scale: float = 1.0,
        out: Optional[torch.Tensor] = None,
        kv_cache_sf: Optional[torch.Tensor] = None,
        return_lse: bool = False,
        lse_out: Optional[torch.Tensor] = None,
    ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        """One decode step on torch's current stream; asynchronous, CUDA-graph capturable.

        ``lse_out`` (f32, contiguous [batch, q_len, num_heads], on q's device) receives the base-2 LSE in
        place when ``return_lse`` is set, instead of a freshly allocated tensor."""
        if not self._planned:
            raise RuntimeError("Call plan() before run().")
        self._validate_run_inputs(q, kv_cache, kv_cache_sf, out)

        if kv_cache.dim() == 4:
            if kv_cache.shape[1] != 1:
                raise ValueError("4D kv_cache must have shape [pages, 1, page_size, dim]")
            kv_cache = kv_cache.squeeze(1)
        elif kv_cache.dim() != 3:
            raise ValueError("kv_cache must be 3D or 4D")
        if kv_cache.shape[1] != self._page_size:
            raise ValueError(f"kv_cache page size {kv_cache.shape[1]} does not match planned {self._page_size}")
        if kv_cache_sf.dim() == 4:
            if kv_cache_sf.shape[1] != 1:
                raise ValueError("4D kv_cache_sf must have shape [pages, 1, page_size, 1]")
            kv_cache_sf = kv_cache_sf.squeeze(1)
        elif kv_cache_sf.dim() != 3:
            raise ValueError("kv_cache_sf must be 3D or 4D")
        if kv_cache.shape[-1] != ROW_BYTES:
            raise ValueError(f"kv_cache.shape[-1]={kv_cache.shape[-1]}, expected {ROW_BYTES}")
        expected_sf_shape = (*kv_cache.shape[:2], 1)
        if tuple(kv_cache_sf.shape) != expected_sf_shape:
            raise ValueError(f"kv_cache_sf must have shape {expected_sf_shape}, got {tuple(kv_cache_sf.shape)}")
        if q.device != kv_cache.device or q.device != kv_cache_sf.device:
            raise ValueError("q, kv_cache, and kv_cache_sf must share a device")
        if not kv_cache.is_contiguous() or not kv_cache_sf.is_contiguous():
            raise ValueError("kv_cache and kv_cache_sf must be contiguous")
        if max_seq_len <= 0:
            raise ValueError(f"max_seq_len must be positive, got {max_seq_len}")
        if q.stride(-1) != 1:
            raise ValueError("q must have unit stride in its last dimension")
        if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.stride(-1) != 1:
            raise ValueError("block_tables must be an int32 [batch, max_pages] tensor with unit inner stride")
        if q.device != self._device:
            raise ValueError("q must live on the device of the workspace buffer")

        batch_size, q_len, num_heads, _ = q.shape
        if block_tables.shape[0] != batch_size or seq_lens.shape[0] != batch_size:
            raise ValueError("block_tables and seq_lens must have one row per request")
        if max_seq_len > block_tables.shape[1] * self._page_size:
            raise ValueError(f"max_seq_len={max_seq_len} exceeds what block_tables can address "
                             f"({block_tables.shape[1]} pages of {self._page_size} tokens)")
        if os.environ.get("MLA_FP4_VALIDATE", "0") not in ("", "0"):
            validate_page_ids(block_tables, seq_lens, self._page_size, kv_cache.shape[0])
        need = _cabi.workspace_bytes(batch_size, q_len, num_heads, self._num_ctas)
        if self._workspace_buffer.numel() < need:
            raise ValueError(f"workspace_buffer has {self._workspace_buffer.numel()} bytes, but {need} are required")

        # every pointer handed to the kernels must be a device pointer of q's device
        for name, t in (("block_tables", block_tables), ("seq_lens", seq_lens), ("out", out)):
            if t is not None and (not t.is_cuda or t.device != q.device):
                raise ValueError(f"{name} must be a CUDA tensor on the device of q ({q.device}), got {t.device}")
        if out is None:
            out = torch.empty((batch_size, q_len, num_heads, self._kv_lora_rank), dtype=self._o_dtype, device=q.device)
        elif tuple(out.shape) != (batch_size, q_len, num_heads, self._kv_lora_rank) or not out.is_contiguous():
            raise ValueError("out must be a contiguous [batch, q_len, num_heads, 512] tensor")
        lse = None
        if return_lse:
            if lse_out is not None:
                if (lse_out.dtype != torch.float32 or tuple(lse_out.shape) != (batch_size, q_len, num_heads)
                        or not lse_out.is_contiguous() or lse_out.device != q.device):
                    raise ValueError("lse_out must be a contiguous float32 [batch, q_len, num_heads] tensor on the device of q")
                lse = lse_out
            else:
                lse = torch.empty((batch_size, q_len, num_heads), dtype=torch.float32, device=q.device)
        cache_seqs = seq_lens if seq_lens.dtype == torch.int32 else seq_lens.to(torch.int32)
        if not cache_seqs.is_contiguous():
            cache_seqs = cache_seqs.contiguous()

        a = _cabi.DecodeArgs()
        a.q = q.data_ptr()
        a.q_stride_batch, a.q_stride_qpos, a.q_stride_head = q.stride(0), q.stride(1), q.stride(2)
        a.kv_cache = kv_cache.data_ptr()
        a.kv_cache_sf = kv_cache_sf.data_ptr()
        a.block_tables = block_tables.data_ptr()
        a.block_table_stride = block_tables.stride(0)
        a.seq_lens = cache_seqs.data_ptr()
        a.out = out.data_ptr()
        a.lse = lse.data_ptr() if lse is not None else None
        a.workspace = self._workspace_buffer.data_ptr()
        a.workspace_bytes = self._workspace_buffer.numel()
        a.status = self._status.data_ptr()
        a.batch, a.q_len, a.num_heads, a.page_size = batch_size, q_len, num_heads, self._page_size
        a.num_pages = kv_cache.shape[0]
        a.softmax_scale, a.output_scale = float(softmax_scale), float(output_scale)
        a.out_dtype = _OUT_DTYPES[self._o_dtype]
        a.kernel = self._kernel
        a.num_ctas = self._num_ctas
        a.enable_pdl = 1 if self._enable_pdl else 0
        a.phase_mask = self._phase_mask
        a.max_pages_per_request = block_tables.shape[1]
        a.logits_soft_cap = self._soft_cap
        a.sink = self._sink.data_ptr() if self._sink is not None else None
        a.wait_polls = self._wait_polls
        with torch.cuda.device(q.device):
            a.stream = torch.cuda.current_stream(q.device).cuda_stream
            _cabi.check(_cabi.lib.mla_fp4_decode(C.byref(a)))
        if return_lse:
            return out, lse
        return out

    # ------------------------------------------------------------------ diagnostics
    def device_status(self) -> Tuple[int, ...]:
        """Read the device status words (synchronises). Word 0 != 0 means a bounded device wait expired."""
        if self._status is None:
            return (0,) * 8
        return tuple(int(x) for x in self._status.cpu())

    def check_device_status(self) -> None:
        st = self.device_status()
        if st[0] != 0:
            self._status.zero_()
            self._init_workspace()  # start from a clean header after a step that gave up on a wait
            raise RuntimeError(
                f"mla_fp4 device error {st[0]} (barrier {st[1]}, CTA {st[2]}, thread {st[3]}, parity {st[4]})"
            )


def validate_page_ids(block_tables: torch.Tensor, seq_lens: torch.Tensor, page_size: int, num_pages: int) -> None:
    """Debug check (``MLA_FP4_VALIDATE=1``; synchronises): every block-table entry a step will read is a page of the pool.

    The kernels read entries ``[0, ceil(seq_len / page_size))`` of each row and nothing beyond
    (the reference reads the ids unchecked: flashinfer ``roles/mla_loader_fp8.py:185-210``).
    Raises ``ValueError`` naming the first offending request.
    """
    lens = seq_lens.detach().to("cpu", torch.int64)
    bt = block_tables.detach().to("cpu")
    width = bt.shape[1]
    for b in range(bt.shape[0]):
        n = int(lens[b])
        if n <= 0:
            continue
        used = -(-n // page_size)
        if used > width:
            raise ValueError(f"request {b}: seq_len {n} needs {used} pages but block_tables has {width} per request")
        row = bt[b, :used]
        bad = (row < 0) | (row >= num_pages)
        if bool(bad.any()):
            i = int(bad.nonzero()[0])
            raise ValueError(f"request {b}: block_tables[{b}, {i}] = {int(row[i])} is outside the pool of {num_pages} pages")


__all__ = ["BatchMLADecodeCuteDSLFP4Wrapper", "validate_page_ids"]
