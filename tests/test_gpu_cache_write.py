"""The CUDA cache writer against the oracle's quantiser (a restatement of the reference fixture
builder, tests/test_cute_dsl_mla_fp4.py:56-93, itself pinned by tests/golden/cache_format.npz):
the bytes and the scales must be identical, whatever the input dtype, slot order or value range."""
import pytest
import torch

from oracle import mla_fp4_oracle as O

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def _expected(latent, rope, scale=None):
    lat = latent.float().cpu()
    s = O.amax_scale(lat) if scale is None else scale.float().cpu().view(-1, 1)
    return O.pack_cache(lat, rope.cpu(), s), s


def _write(latent, rope, slots, pages, page_size, scale=None, poison=0xAB):
    from flashinfer_mla_fp4_b200.kvcache import write_tokens

    dev = latent.device
    cache = torch.full((pages, page_size, 320), poison, dtype=torch.uint8, device=dev)
    sf = torch.full((pages, page_size, 1), -7.0, dtype=torch.float32, device=dev)
    write_tokens(latent, rope, slots, cache, sf, token_scale=scale)
    torch.cuda.synchronize()
    return cache.cpu(), sf.cpu()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("page_size", [16, 64])
def test_writer_is_byte_identical_to_the_oracle(dtype, page_size):
    dev = _dev()
    g = torch.Generator().manual_seed(7 + page_size)
    T, pages = 1000, 80
    latent = (torch.randn(T, 512, generator=g) * torch.rand(T, 1, generator=g) * 8).to(dtype)
    rope = (torch.randn(T, 64, generator=g) * 3).to(dtype)
    latent[5] = 0  # an all-zero token gets scale 1
    slots = torch.randperm(pages * page_size, generator=g)[:T]
    slots[17] = -1  # padding token: skipped
    cache, sf = _write(latent.to(dev), rope.to(dev), slots.to(dev), pages, page_size)
    rows, s = _expected(latent, rope)
    flat, sff = cache.view(-1, 320), sf.view(-1)
    keep = slots >= 0
    assert torch.equal(flat[slots[keep]], rows[keep])
    assert torch.equal(sff[slots[keep]], s.view(-1)[keep])
    assert float(sff[slots[5]]) == 1.0
    untouched = torch.ones(pages * page_size, dtype=torch.bool)
    untouched[slots[keep]] = False
    assert (flat[untouched] == 0xAB).all() and (sff[untouched] == -7.0).all()


def test_ties_signed_zero_given_scales_and_rope_range():
    dev = _dev()
    # values exactly on the rounding thresholds of every magnitude, both signs, power-of-two scales:
    # a tie stays on the smaller magnitude; -0.0 carries no sign bit; rope beyond 464 becomes NaN
    thr = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    grid = torch.cat([thr, -thr, thr * (1 + 2 ** -20), -thr * (1 + 2 ** -20), torch.tensor([0.0, -0.0, 6.0, -6.0, 7.5])])
    latent = torch.zeros(4, 512)
    latent[:, : grid.numel()] = grid
    scale = torch.tensor([1.0, 0.5, 2.0, 0.125])
    latent = latent * scale[:, None]
    rope = torch.zeros(4, 64)
    rope[0, :8] = torch.tensor([448.0, 463.9, 464.0, 465.0, -500.0, 2.0 ** -10, 2.0 ** -9 * 0.5, 1e-4])
    cache, sf = _write(latent.to(dev), rope.to(dev), None, 1, 4, scale=scale.to(dev))
    rows, s = _expected(latent, rope, scale)
    assert torch.equal(cache.view(-1, 320), rows)
    assert torch.equal(sf.view(-1), scale)


def test_written_cache_decodes_like_the_torch_built_one():
    """Writer -> decode kernel end to end: the same attention output as with the host-built cache."""
    dev = _dev()
    from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper, synth
    from flashinfer_mla_fp4_b200.kvcache import write_tokens

    case = synth.build_case("writer", [700, 129, 2500], 64, 64, seed=99, device=dev)
    g = torch.Generator().manual_seed(99)
    pages, ps = case.kv_cache.shape[0], case.page_size
    lat = torch.randn(pages * ps, 512, generator=g).bfloat16().to(dev)
    rope = torch.randn(pages * ps, 64, generator=g).bfloat16().to(dev)
    cache = torch.zeros_like(case.kv_cache)
    sf = torch.zeros_like(case.kv_cache_sf)
    write_tokens(lat, rope, None, cache, sf)
    w = BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(32 << 20, dtype=torch.int8, device=dev))
    w.plan(num_heads=case.num_heads, page_size=ps)
    out = w.run(case.q, cache, case.block_tables, case.seq_lens, case.max_seq_len, case.softmax_scale, kv_cache_sf=sf)
    torch.cuda.synchronize()
    w.check_device_status()
    ref, _ = O.mla_decode(case.q.cpu(), cache.cpu(), sf.cpu(), case.block_tables.cpu(), case.seq_lens.cpu(), case.softmax_scale)
    O.assert_parity(out.float().cpu(), ref, "writer->decode")
