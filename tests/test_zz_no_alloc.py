"""The allocation-free entry point (mla_fp4_decode_static) against the regular one.

Some callers cannot allocate device memory or lend a workspace: a plugin inside an engine whose memory
pool owns the device, worker threads on which cudaMalloc is forbidden, a step that must still run when
the allocator is exhausted.  For them the library carries its own scratch array.  This test calls the
entry point through the C ABI, twice in a row on the same stream (the second call finds the first call's
partials still in the scratch), and compares with mla_fp4_decode on the same inputs and with the CPU
oracle; between two further steps it zeroes the scratch header with mla_fp4_static_reset, the way back
after a kernel that did not run to its end.  It lives in its own file, collected last, and does not
depend on what ran before it.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(case, out, lse, status, workspace=None):
    from flashinfer_mla_fp4_b200 import _cabi

    a = _cabi.DecodeArgs()
    q = case.q
    a.q = q.data_ptr()
    a.q_stride_batch, a.q_stride_qpos, a.q_stride_head = q.stride(0), q.stride(1), q.stride(2)
    a.kv_cache = case.kv_cache.data_ptr()
    a.kv_cache_sf = case.kv_cache_sf.data_ptr()
    a.block_tables = case.block_tables.data_ptr()
    a.block_table_stride = case.block_tables.stride(0)
    a.seq_lens = case.seq_lens.data_ptr()
    a.out = out.data_ptr()
    a.lse = lse.data_ptr()
    a.workspace = workspace.data_ptr() if workspace is not None else None
    a.workspace_bytes = workspace.numel() if workspace is not None else 0
    a.status = status.data_ptr()
    a.batch, a.q_len, a.num_heads, a.page_size = case.batch, case.q_len, case.num_heads, case.page_size
    a.num_pages = case.kv_cache.shape[0]
    a.softmax_scale, a.output_scale = case.softmax_scale, 1.0
    a.out_dtype, a.kernel, a.num_ctas, a.enable_pdl, a.phase_mask = _cabi.OUT_BF16, _cabi.KERNEL_TCGEN05, 0, 1, 0
    a.stream = torch.cuda.current_stream(q.device).cuda_stream
    return a


def test_static_scratch_entry_point_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    from flashinfer_mla_fp4_b200 import _cabi, synth

    dev = torch.device("cuda:0")
    # two different ragged batches, both split across CTAs, so the second call overwrites live partials
    cases = [synth.build_case("na0", [5000, 130, 64, 1, 9000, 777], 64, 64, seed=41, device=dev),
             synth.build_case("na1", [3000, 4097, 12000], 128, 32, seed=42, device=dev)]
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    ws = torch.empty(64 << 20, dtype=torch.int8, device=dev)
    _cabi.workspace_init(ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)  # counter header
    for case in cases:  # two static calls in a row, each checked against the regular entry point
        shape = (case.batch, case.q_len, case.num_heads, 512)
        ref_out = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        ref_lse = torch.zeros(shape[:3], dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib.mla_fp4_decode(C.byref(_args(case, ref_out, ref_lse, status, ws))))
        out = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        lse = torch.zeros(shape[:3], dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib.mla_fp4_decode_static(C.byref(_args(case, out, lse, status))))
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        # same kernels, same partition, deterministic reduction: the tolerance of the parity tests
        # (2e-2 of the output RMS) is met with room to spare; in practice the results are identical
        rms = ref_out.float().pow(2).mean().sqrt()
        assert (out.float() - ref_out.float()).abs().max() <= 2e-2 * rms
        torch.testing.assert_close(lse, ref_lse, atol=2e-3, rtol=1e-4)
        assert torch.isfinite(out).all()
        # and against the CPU oracle, with the tolerance of the parity tests
        from oracle import mla_fp4_oracle as O

        want, want_lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, case.block_tables, case.seq_lens,
                                      case.softmax_scale)
        O.assert_parity(out, want, f"static/{case.name}")
        torch.testing.assert_close(lse.cpu(), want_lse, atol=2e-3, rtol=1e-4)

    # the reset entry point: header back to zero (generation restarts), the next static step is still right
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    first = out.clone()
    _cabi.check(_cabi.lib.mla_fp4_static_reset(stream))
    out.zero_()
    _cabi.check(_cabi.lib.mla_fp4_decode_static(C.byref(_args(cases[-1], out, lse, status))))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(out, first)

    # sizes beyond the built-in scratch are refused with a clear message, nothing is launched
    a = _args(cases[0], out, lse, status)
    a.num_ctas = 149
    assert _cabi.lib.mla_fp4_decode_static(C.byref(a)) == _cabi.ERR_UNSUPPORTED
    assert "at most 148" in _cabi.last_error()
