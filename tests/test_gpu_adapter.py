"""The serving-side adapter end to end on the GPU: requests grow token by token through the CUDA
cache writer and the decode kernel (one CUDA graph replayed every step, metadata refreshed in
place), and both the cache bytes and the attention output are checked against the oracle."""
import pytest
import torch

from oracle import mla_fp4_oracle as O

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


class _Requests:
    """A toy scheduler: page allocation from a shuffled free list and the raw tokens written so far."""

    def __init__(self, num_pages, page_size, batch, seed):
        g = torch.Generator().manual_seed(seed)
        self.g, self.ps = g, page_size
        self.free = torch.randperm(num_pages, generator=g).tolist()
        self.tables = [[] for _ in range(batch)]
        self.lens = [0] * batch
        self.lat = [[] for _ in range(batch)]
        self.rope = [[] for _ in range(batch)]

    def append(self, b, n=1):
        lat = torch.randn(n, 512, generator=self.g).bfloat16() * (0.25 + 3 * torch.rand(n, 1, generator=self.g)).bfloat16()
        rope = torch.randn(n, 64, generator=self.g).bfloat16()
        self.lens[b] += n
        while len(self.tables[b]) * self.ps < self.lens[b]:
            self.tables[b].append(self.free.pop())
        self.lat[b].append(lat)
        self.rope[b].append(rope)
        return lat, rope

    def metadata(self):
        width = max(1, max(len(t) for t in self.tables))
        bt = torch.zeros(len(self.tables), width, dtype=torch.int32)
        for b, t in enumerate(self.tables):
            bt[b, : len(t)] = torch.tensor(t, dtype=torch.int32)
        return bt, torch.tensor(self.lens, dtype=torch.int32)

    def expected_cache_rows(self, b):
        lat = torch.cat(self.lat[b]).float()
        s = O.amax_scale(lat)
        return O.pack_cache(lat, torch.cat(self.rope[b]), s), s


def _check_cache(cache, reqs):
    kv, sf = cache.kv_cache.cpu(), cache.kv_cache_sf.cpu()
    for b, table in enumerate(reqs.tables):
        rows, s = reqs.expected_cache_rows(b)
        pages = torch.tensor(table, dtype=torch.int64)
        got = kv[pages].reshape(-1, 320)[: reqs.lens[b]]
        assert torch.equal(got, rows), f"cache rows of request {b}"
        assert torch.equal(sf[pages].reshape(-1)[: reqs.lens[b]], s.view(-1)), f"scales of request {b}"


def test_growing_requests_through_one_captured_graph():
    dev = _dev()
    from flashinfer_mla_fp4_b200 import FP4MLADecodeBackend, FP4MLAPagedCache
    from flashinfer_mla_fp4_b200.adapter import decode_slot_mapping
    from flashinfer_mla_fp4_b200.kvcache import write_tokens

    H, ps, batch, max_batch = 16, 16, 3, 4
    scale = 576 ** -0.5
    backend = FP4MLADecodeBackend(H, ps, max_batch, 512, scale, dev)
    cache = FP4MLAPagedCache(96, ps, dev)
    reqs = _Requests(96, ps, batch, seed=21)
    step = backend.capture(cache)
    assert int(cache.kv_cache.sum()) == 0  # warm-up and capture ran on padding only

    # prefill stand-in: the prompt tokens go through the same writer, slot by slot
    for b, n in enumerate((30, 0, 200)):
        if n == 0:
            continue
        lat, rope = reqs.append(b, n)
        pos = torch.arange(n)
        slots = torch.tensor(reqs.tables[b], dtype=torch.int64)[pos // ps] * ps + pos % ps
        write_tokens(lat.to(dev), rope.to(dev), slots.to(dev), cache.kv_cache, cache.kv_cache_sf)

    g = torch.Generator().manual_seed(22)
    for i in range(40):  # requests 0 and 2 cross page boundaries; request 1 starts empty
        new = [reqs.append(b) for b in range(batch)]
        bt, sl = reqs.metadata()
        assert backend.prepare(bt.pin_memory(), sl.pin_memory()) == batch
        q = (torch.randn(batch, 1, H, 576, generator=g) * 0.5).to(torch.float8_e4m3fn)
        step.q[:batch].copy_(q)
        step.latent[:batch].copy_(torch.cat([x[0] for x in new]))
        step.rope[:batch].copy_(torch.cat([x[1] for x in new]))
        out = step.replay()
        if i in (0, 15, 39):
            torch.cuda.synchronize()
            backend.wrapper.check_device_status()
            assert torch.equal(backend.slot_mapping[:batch].cpu(), decode_slot_mapping(bt, sl, ps))
            _check_cache(cache, reqs)
            ref, _ = O.mla_decode(q, cache.kv_cache, cache.kv_cache_sf, bt, sl, scale)
            O.assert_parity(out[:batch].float().cpu(), ref, f"adapter step {i}")
            assert not out[batch:].float().any(), "a padding row must come out as zeros"


def test_forward_without_a_graph_q_len_2_and_a_smaller_batch():
    dev = _dev()
    from flashinfer_mla_fp4_b200 import FP4MLADecodeBackend, FP4MLAPagedCache

    H, ps, q_len = 64, 64, 2
    scale = 576 ** -0.5
    backend = FP4MLADecodeBackend(H, ps, 8, 4096, scale, dev, q_len=q_len, out_dtype=torch.float32, output_scale=0.5)
    cache = FP4MLAPagedCache(40, ps, dev)
    reqs = _Requests(40, ps, 2, seed=31)
    g = torch.Generator().manual_seed(32)
    for i in range(3):  # the first step writes a 700-token and a 63-token draft-sized chunk; then two tokens per step
        new = [reqs.append(b, n) for b, n in enumerate(((700, 63) if i == 0 else (q_len, q_len)))]
        if i == 0:  # chunks longer than q_len: written directly, as a prefill would
            from flashinfer_mla_fp4_b200.kvcache import write_tokens
            for b, (lat, rope) in enumerate(new):
                pos = torch.arange(lat.shape[0])
                slots = torch.tensor(reqs.tables[b], dtype=torch.int64)[pos // ps] * ps + pos % ps
                write_tokens(lat.to(dev), rope.to(dev), slots.to(dev), cache.kv_cache, cache.kv_cache_sf)
            continue
        bt, sl = reqs.metadata()
        backend.prepare(bt.to(dev), sl.to(dev))  # device tensors work as well
        q = (torch.randn(2, q_len, H, 576, generator=g) * 0.5).to(torch.float8_e4m3fn)
        out = backend.forward(q.to(dev), torch.cat([x[0] for x in new]).to(dev), torch.cat([x[1] for x in new]).to(dev), cache)
        torch.cuda.synchronize()
        backend.wrapper.check_device_status()
        assert out.shape == (2, q_len, H, 512) and out.dtype == torch.float32
        _check_cache(cache, reqs)
        ref, _ = O.mla_decode(q, cache.kv_cache, cache.kv_cache_sf, bt, sl, scale, output_scale=0.5)
        O.assert_parity(out.cpu(), ref, f"adapter q_len 2 step {i}")


def test_adapter_rejects_what_it_cannot_hold():
    dev = _dev()
    from flashinfer_mla_fp4_b200 import FP4MLADecodeBackend, FP4MLAPagedCache

    backend = FP4MLADecodeBackend(16, 16, 2, 64, 0.1, dev)
    with pytest.raises(ValueError, match="exceeds max_batch"):
        backend.prepare(torch.zeros(3, 1, dtype=torch.int32), torch.ones(3, dtype=torch.int32))
    with pytest.raises(ValueError, match="block_tables"):
        backend.prepare(torch.zeros(2, 5, dtype=torch.int32), torch.ones(2, dtype=torch.int32))
    q = torch.zeros(2, 1, 16, 576, device=dev).to(torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="page size"):
        backend.forward(q, torch.zeros(2, 512, device=dev), torch.zeros(2, 64, device=dev), FP4MLAPagedCache(4, 32, dev))
