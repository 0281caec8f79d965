"""Host logic without a GPU: the library loads and exports its ABI, the work partition is a
partition, the package quantiser equals the oracle's, and the wrapper validates like the reference."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from oracle import mla_fp4_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from flashinfer_mla_fp4_b200 import _cabi

    header = (ROOT / "include" / "mla_fp4_b200.h").read_text()
    declared = set(re.findall(r"^\s*(?:const\s+)?(?:int|char\s*\*|const char\*)\s+(mla_fp4_\w+)\s*\(", header, re.M))
    assert declared, "no declarations parsed"
    lib = ctypes.CDLL(str(_cabi.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(_cabi.EXPORTS) == declared
    assert lib.mla_fp4_abi_version() == _cabi.ABI_VERSION == 5


def test_abi_rejects_bad_arguments_without_a_gpu():
    from flashinfer_mla_fp4_b200 import _cabi

    assert _cabi.lib.mla_fp4_decode(None) == _cabi.ERR_BAD_ARG
    assert "null" in _cabi.last_error()
    n = ctypes.c_size_t(0)
    assert _cabi.lib.mla_fp4_workspace_bytes(8, 1, 64, 148, ctypes.byref(n)) == 0
    assert n.value == 2048 + 2 * 148 * (512 * 64 * 2 + 64 * 4 + 16)  # header (generation, slot flags) + two slots per CTA
    assert _cabi.lib.mla_fp4_workspace_init(None, 4096, None) == _cabi.ERR_BAD_ARG
    assert _cabi.lib.mla_fp4_cache_write(None, 512, None, 64, 0, None, None, 4, None, None, 16, None) == _cabi.ERR_BAD_ARG
    assert _cabi.lib.mla_fp4_cache_write(None, 512, None, 64, 0, None, None, 0, None, None, 16, None) == 0  # nothing to write
    assert _cabi.lib.mla_fp4_workspace_bytes(8, 0, 64, 148, ctypes.byref(n)) == _cabi.ERR_BAD_ARG
    with pytest.raises(ValueError):
        _cabi.check(_cabi.ERR_WORKSPACE_TOO_SMALL)


@pytest.mark.parametrize(
    "seq_lens,q_len,heads,ctas",
    [
        ([32768] * 8, 1, 64, 148),
        ([4096] * 4, 1, 64, 148),
        ([256, 256], 1, 16, 148),
        ([131072, 131072], 2, 128, 148),
        ([1, 0, 129, 128, 127, 5000, 0, 3], 1, 128, 7),
        ([0, 0], 1, 64, 4),
        ([77], 1, 64, 1),
        ([512, 1, 0, 300, 129], 2, 128, 148),
        ([512, 513], 1, 64, 148),
        (list(range(1, 400, 7)), 1, 64, 148),
    ],
)
def test_partition_is_a_partition(seq_lens, q_len, heads, ctas):
    from flashinfer_mla_fp4_b200 import planner

    segs = planner.plan_partition(seq_lens, q_len, heads, ctas)
    groups = planner.num_groups(q_len, heads)
    covered = {}
    per_cta = {}
    for s in segs:
        assert 0 <= s.tile_begin < s.tile_end <= planner.tiles_of(seq_lens[s.request])
        for t in range(s.tile_begin, s.tile_end):
            key = (s.group, s.request, t)
            assert key not in covered, "tile covered twice"
            covered[key] = s.cta
        per_cta.setdefault(s.cta, []).append(s)
        whole = s.tile_begin == 0 and s.tile_end == planner.tiles_of(seq_lens[s.request])
        assert (s.slot == -1) == whole
    total = groups * sum(planner.tiles_of(n) for n in seq_lens)
    assert len(covered) == total
    # balance: the flat space that is cut evenly counts P extra (phantom) tiles in front of every non-empty
    # request, so a CTA's tiles plus P per request start it holds stay close to the even share
    from flashinfer_mla_fp4_b200 import _cabi

    P = _cabi.PHANTOM_TILES
    flat = groups * sum(planner.tiles_of(n) + P for n in seq_lens if n > 0)
    # short requests are not split: when none has more than four tiles and there are no more (request, group) pairs
    # than CTAs, pair v is decoded whole by CTA v
    if max((planner.tiles_of(n) for n in seq_lens), default=0) <= 4 and groups * len(seq_lens) <= ctas:
        assert all(s.slot == -1 for s in segs)
        assert all(s.cta == s.group * len(seq_lens) + s.request for s in segs)
        return
    for i in range(ctas):
        ss = per_cta.get(i, [])
        real = sum(s.tile_end - s.tile_begin for s in ss)
        starts = sum(1 for s in ss if s.tile_begin == 0)  # the phantom of one of them may lie in the CTA before
        assert real <= -(-flat // ctas), (i, real, flat, ctas)
        assert flat // ctas - P <= real + P * starts <= -(-flat // ctas) + P, (i, real, starts, flat, ctas)
    # partial slots: unique, at most two per CTA, only at the ends of a CTA's walk
    slots = [s.slot for s in segs if s.slot >= 0]
    assert len(slots) == len(set(slots))
    for i, ss in per_cta.items():
        partial = [k for k, s in enumerate(ss) if s.slot >= 0]
        assert all(k in (0, len(ss) - 1) for k in partial)
        for k in partial:
            assert ss[k].slot == 2 * i + (0 if k == 0 else 1)
    assert planner.workspace_bytes(len(seq_lens), q_len, heads, ctas) >= (max(slots) + 1 if slots else 0) * 65808


def test_package_quantiser_is_bit_identical_to_the_oracle():
    from flashinfer_mla_fp4_b200.kvcache import quantize_tokens

    g = torch.Generator().manual_seed(3)
    lat = torch.randn(5, 16, 512, generator=g) * 3
    rope = torch.randn(5, 16, 64, generator=g)
    lat[0, 0] = 0
    rows, sf = quantize_tokens(lat, rope)
    ref_sf = O.amax_scale(lat)
    assert torch.equal(sf, ref_sf)
    assert torch.equal(rows, O.pack_cache(lat, rope, ref_sf))
    # round trip: dequantised values are within half a quantisation step of the input
    deq, _ = O.dequantize_cache(rows, sf)
    assert ((deq - lat).abs() <= sf * 1.0 + 1e-6).all()


def _planned_cpu_wrapper(monkeypatch, **kw):
    import flashinfer_mla_fp4_b200.wrapper as W

    monkeypatch.setattr(W, "_require_sm100", lambda device: None)

    class _Props:
        multi_processor_count = 148

    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda d: _Props())
    w = W.BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(64 << 20, dtype=torch.int8))
    args = dict(num_heads=16, page_size=64)
    args.update(kw)
    w.plan(**args)
    return w


def test_wrapper_plan_validation(monkeypatch):
    import flashinfer_mla_fp4_b200 as pkg

    with pytest.raises(AssertionError):
        pkg.BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(16, dtype=torch.uint8))
    w = pkg.BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(16, dtype=torch.int8))
    with pytest.raises(RuntimeError, match="plan"):
        w.run(None, None, None, None, 1, 1.0)
    for bad in (dict(kv_lora_rank=256), dict(qk_rope_head_dim=32), dict(q_dtype=torch.bfloat16),
                dict(kv_dtype=torch.float8_e4m3fn), dict(page_size=1), dict(num_heads=129, page_size=64),
                dict(out_dtype=torch.float16, page_size=64), dict(variant=object(), page_size=64)):
        with pytest.raises(ValueError):
            w.plan(**bad)
    # a CPU workspace cannot be planned: the kernels are sm_100a only
    with pytest.raises(RuntimeError, match="CUDA"):
        w.plan(num_heads=16, page_size=64)
    _planned_cpu_wrapper(monkeypatch)


def test_wrapper_run_validation(monkeypatch):
    w = _planned_cpu_wrapper(monkeypatch)
    from flashinfer_mla_fp4_b200 import synth

    c = synth.config_case("small")
    ok = dict(q=c.q, kv_cache=c.kv_cache, block_tables=c.block_tables, seq_lens=c.seq_lens, max_seq_len=256,
              softmax_scale=c.softmax_scale, kv_cache_sf=c.kv_cache_sf)

    def bad(**kw):
        a = dict(ok)
        a.update(kw)
        with pytest.raises(ValueError):
            w.run(**a)

    bad(q=c.q[0])
    bad(q=c.q[..., :512])
    bad(q=c.q.float())
    bad(kv_cache=c.kv_cache.to(torch.int8))
    bad(kv_cache_sf=None)
    bad(kv_cache_sf=c.kv_cache_sf.double())
    bad(kv_cache=c.kv_cache[:, :32])
    bad(kv_cache=c.kv_cache[..., :256])
    bad(kv_cache=c.kv_cache.unsqueeze(1).expand(-1, 2, -1, -1))
    bad(kv_cache_sf=c.kv_cache_sf[:, :32])
    bad(kv_cache=c.kv_cache.transpose(0, 1).contiguous().transpose(0, 1))
    bad(max_seq_len=0)
    bad(out=torch.empty(2, 1, 16, 512, dtype=torch.float16))
    bad(block_tables=c.block_tables.long())
    # the workspace bound is checked with the reference's message
    import flashinfer_mla_fp4_b200.wrapper as W
    small = W.BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(1024, dtype=torch.int8))
    small.__dict__.update({k: v for k, v in w.__dict__.items() if k != "_workspace_buffer"})
    with pytest.raises(ValueError, match="are required"):
        small.run(**ok)


def test_wrapper_rejects_host_tensors_before_any_launch(monkeypatch):
    """Every pointer the kernels dereference must be a device pointer of q's device: a host (or other-device)
    block table, seq_lens or out would be read as a device address.  The checks run before the C call."""
    import flashinfer_mla_fp4_b200.wrapper as W
    from flashinfer_mla_fp4_b200 import _cabi, synth

    w = _planned_cpu_wrapper(monkeypatch)
    c = synth.config_case("small")
    called = []
    monkeypatch.setattr(_cabi.lib, "mla_fp4_decode", lambda *a: called.append(a) or 0, raising=False)
    # on this GPU-less host every tensor is a host tensor: the first one the kernels would dereference is refused
    with pytest.raises(ValueError, match="block_tables must be a CUDA tensor"):
        w.run(c.q, c.kv_cache, c.block_tables, c.seq_lens, 256, c.softmax_scale, kv_cache_sf=c.kv_cache_sf)
    assert not called
    # a sequence longer than the block table can address is refused on the host
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    with pytest.raises(ValueError, match="exceeds what block_tables can address"):
        w.run(c.q, c.kv_cache, c.block_tables, c.seq_lens, 64 * c.block_tables.shape[1] + 1, c.softmax_scale,
              kv_cache_sf=c.kv_cache_sf)
    assert not called


def test_write_tokens_rejects_host_tensors():
    from flashinfer_mla_fp4_b200.kvcache import write_tokens

    lat, rope = torch.zeros(4, 512, dtype=torch.bfloat16), torch.zeros(4, 64, dtype=torch.bfloat16)
    cache, sf = torch.zeros(1, 64, 320, dtype=torch.uint8), torch.zeros(1, 64, 1)
    with pytest.raises(ValueError, match="CUDA"):
        write_tokens(lat, rope, torch.arange(4), cache, sf)


def test_page_id_validator():
    """MLA_FP4_VALIDATE=1 makes run() check, on the host, every block-table entry a step will read."""
    from flashinfer_mla_fp4_b200.wrapper import validate_page_ids

    bt = torch.tensor([[0, 1, 2, 99], [3, 4, -7, 5]], dtype=torch.int32)
    validate_page_ids(bt, torch.tensor([192, 128]), 64, 6)          # entries beyond ceil(seq_len / page) are never read
    validate_page_ids(bt, torch.tensor([0, 1]), 64, 6)
    with pytest.raises(ValueError, match=r"block_tables\[0, 3\] = 99"):
        validate_page_ids(bt, torch.tensor([193, 128]), 64, 100 - 1)
    with pytest.raises(ValueError, match=r"block_tables\[1, 2\] = -7"):
        validate_page_ids(bt, torch.tensor([10, 129]), 64, 6)
    with pytest.raises(ValueError, match="needs 5 pages"):
        validate_page_ids(bt, torch.tensor([257, 1]), 64, 200)


def test_partition_charges_phantom_tiles_for_a_request_start():
    """One request of 10 tiles on 10 + P CTAs: the first P CTAs get the phantom tiles and no segment."""
    from flashinfer_mla_fp4_b200 import _cabi, planner

    P = _cabi.PHANTOM_TILES
    segs = planner.plan_partition([1280], 1, 64, 10 + P)
    assert [s.cta for s in segs] == list(range(P, 10 + P))
    assert [(s.tile_begin, s.tile_end) for s in segs] == [(t, t + 1) for t in range(10)]
    assert segs[0].slot == 2 * P and all(s.slot == 2 * s.cta for s in segs)


def test_partition_beyond_32_bits_is_refused():
    """Flat tile positions are 32-bit: a tile space x CTA count that does not fit is refused, not wrapped round."""
    from flashinfer_mla_fp4_b200 import planner

    with pytest.raises(ValueError, match="32 bits"):
        planner.plan_partition([2**31 - 1] * 64, 1, 64, 148)
    assert planner.plan_partition([2**20] * 64, 1, 64, 148)  # 64 M tokens: fits
