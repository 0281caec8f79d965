"""The oracle against the reference-generated golden vectors (CPU)."""
from pathlib import Path

import numpy as np
import torch

from oracle import mla_fp4_oracle as O

GOLD = Path(__file__).resolve().parent / "golden"


def test_e2m1_to_e4m3_table_is_the_known_answer():
    tab = O.e2m1_to_e4m3_byte_table()
    assert tab.tolist() == [0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C,
                            0x80, 0xB0, 0xB8, 0xBC, 0xC0, 0xC4, 0xC8, 0xCC]
    # and it agrees with torch's own E4M3 encoder applied to the E2M1 values
    vals = torch.from_numpy(O.e2m1_decode_table()).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(tab, vals)


def test_e4m3_decode_table_matches_torch():
    ours = O.e4m3_decode_table()
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    assert np.array_equal(ours[~np.isnan(ours)], ref[~np.isnan(ref)])


def test_cache_format_matches_reference_builder():
    g = np.load(GOLD / "cache_format.npz")
    source = torch.from_numpy(g["source_f16_bits"]).view(torch.float16)
    fp4, scale, fp8 = O.make_reference_style_cache(source)
    assert np.array_equal(fp4.numpy(), g["fp4_cache"])
    assert np.array_equal(scale.numpy(), g["token_scale"])
    assert np.array_equal(fp8.view(torch.uint8).numpy(), g["fp8_cache_bits"])
    # size identity of the reference test (tests/test_cute_dsl_mla_fp4.py:128-130)
    tokens = fp4.shape[0] * fp4.shape[1]
    assert fp4.numel() + scale.numel() * 4 == tokens * 324
    assert tokens * 324 / (tokens * 576) < 0.565


def test_dequantised_cache_equals_reference_materialisation():
    g = np.load(GOLD / "cache_format.npz")
    fp4 = torch.from_numpy(g["fp4_cache"])
    scale = torch.from_numpy(g["token_scale"])
    lat, rope = O.dequantize_cache(fp4, scale)
    ref = O.decode_e4m3(torch.from_numpy(g["fp8_cache_bits"]))
    # power-of-two scales make the reference's E4M3 materialisation exact
    assert torch.equal(torch.cat((lat, rope), -1), ref)


def test_attention_matches_dependency_reference():
    g = np.load(GOLD / "attention_fi_reference.npz")
    q = torch.from_numpy(g["q_bits"]).view(torch.float8_e4m3fn)
    out, lse = O.mla_decode(q, torch.from_numpy(g["fp4_cache"]), torch.from_numpy(g["token_scale"]),
                            torch.from_numpy(g["block_tables"]), torch.from_numpy(g["seq_lens"]),
                            float(g["softmax_scale"]), float(g["output_scale"]))
    torch.testing.assert_close(out, torch.from_numpy(g["out"]), atol=2e-6, rtol=1e-5)
    assert torch.isfinite(lse).all()


def test_merge_partials_equals_unsplit():
    from flashinfer_mla_fp4_b200 import synth

    c = synth.build_case("t", [300, 77], 8, page_size=16, seed=5)
    full, lse = O.mla_decode(c.q, c.kv_cache, c.kv_cache_sf, c.block_tables, c.seq_lens, c.softmax_scale)
    # split every request's pages into two shards and merge
    ps = c.page_size
    outs, lses = [], []
    for lo_frac, hi_frac in ((0.0, 0.5), (0.5, 1.0)):
        bt = torch.zeros_like(c.block_tables)
        sl = torch.zeros_like(c.seq_lens)
        for b, n in enumerate(c.seq_lens_host):
            pages = (n + ps - 1) // ps
            lo, hi = int(pages * lo_frac), int(pages * hi_frac)
            bt[b, : hi - lo] = c.block_tables[b, lo:hi]
            sl[b] = max(0, min(n, hi * ps) - lo * ps)
        o, l = O.mla_decode(c.q, c.kv_cache, c.kv_cache_sf, bt, sl, c.softmax_scale)
        outs.append(o)
        lses.append(l)
    merged, mlse = O.merge_partials(outs, lses)
    torch.testing.assert_close(merged, full, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(mlse, lse, atol=1e-4, rtol=1e-5)


def test_empty_request_gives_zero_and_minus_inf():
    from flashinfer_mla_fp4_b200 import synth

    c = synth.build_case("t", [40, 1], 4, page_size=16, seed=6)
    sl = torch.tensor([40, 0], dtype=torch.int32)
    out, lse = O.mla_decode(c.q, c.kv_cache, c.kv_cache_sf, c.block_tables, sl, c.softmax_scale)
    assert (out[1] == 0).all() and torch.isinf(lse[1]).all() and (lse[1] < 0).all()
    assert torch.isfinite(out[0]).all()


def test_sink_equals_merging_a_zero_partial_and_huge_cap_changes_nothing():
    """The two attention variants, pinned by identities: a sink is one more partial with a zero value row and
    LSE = sink * log2(e); a soft cap far above every score is the identity, one far below gives uniform weights."""
    from flashinfer_mla_fp4_b200 import synth

    c = synth.build_case("t", [300, 77], 8, page_size=16, seed=7)
    args = (c.q, c.kv_cache, c.kv_cache_sf, c.block_tables, c.seq_lens, c.softmax_scale)
    plain, lse = O.mla_decode(*args)
    sink = torch.linspace(-3.0, 6.0, 8)
    with_sink, lse_sink = O.mla_decode(*args, sink=sink)
    zero = torch.zeros_like(plain)
    sink_lse = (sink * O.LOG2_E).view(1, 1, 8).expand_as(lse).contiguous()
    merged, mlse = O.merge_partials([plain, zero], [lse, sink_lse])
    torch.testing.assert_close(with_sink, merged, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(lse_sink, mlse, atol=1e-4, rtol=1e-5)
    same, _ = O.mla_decode(*args, logits_soft_cap=1e6)
    torch.testing.assert_close(same, plain, atol=1e-5, rtol=1e-4)
    flat, _ = O.mla_decode(*args, logits_soft_cap=1e-4)
    lat, _ = O.dequantize_cache(c.kv_cache, c.kv_cache_sf)
    mean0 = lat[c.block_tables[0, : (300 + 15) // 16].long()].reshape(-1, 512)[:300].mean(dim=0)
    torch.testing.assert_close(flat[0, 0, 0], mean0, atol=1e-4, rtol=1e-3)
