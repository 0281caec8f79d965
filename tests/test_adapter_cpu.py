"""Host logic of the serving-side adapter and of the call logging (no GPU)."""
import torch

from flashinfer_mla_fp4_b200 import api_log
from flashinfer_mla_fp4_b200.adapter import decode_slot_mapping


def _slots_by_loop(block_tables, seq_lens, page_size, q_len):
    out = []
    for b, s in enumerate(seq_lens.tolist()):
        for j in range(q_len):
            pos = s - q_len + j
            out.append(-1 if pos < 0 else int(block_tables[b, pos // page_size]) * page_size + pos % page_size)
    return torch.tensor(out, dtype=torch.int64)


def test_decode_slot_mapping_matches_a_plain_loop():
    g = torch.Generator().manual_seed(5)
    for page_size in (8, 64):
        for q_len in (1, 2, 4):
            batch, width = 9, 7
            bt = torch.randperm(batch * width, generator=g).view(batch, width).to(torch.int32)
            sl = torch.randint(0, width * page_size + 1, (batch,), generator=g, dtype=torch.int32)
            sl[0], sl[1], sl[2] = 0, 1, width * page_size  # padding, shorter than q_len (for q_len > 1), a full table
            got = decode_slot_mapping(bt, sl, page_size, q_len)
            assert got.dtype == torch.int64 and got.is_contiguous()
            assert torch.equal(got, _slots_by_loop(bt, sl, page_size, q_len))


def test_slots_of_a_growing_request_never_repeat():
    page_size, pages = 16, 5
    bt = torch.tensor([[3, 0, 4, 1, 2]], dtype=torch.int32)
    seen = set()
    for s in range(1, pages * page_size + 1):
        slot = int(decode_slot_mapping(bt, torch.tensor([s]), page_size)[0])
        assert slot not in seen and 0 <= slot < pages * page_size
        seen.add(slot)
    assert len(seen) == pages * page_size


def test_api_log_levels(tmp_path):
    calls = []

    @api_log.api_logged
    def step(x, scale=1.0, *, tag=None):
        calls.append(tag)
        return x * scale

    x = torch.tensor([1.0, float("nan"), 3.0])
    try:
        api_log.configure(level=0, nvtx=False)
        step(x, tag="off")
        dest = tmp_path / "log_%i.txt"
        api_log.configure(level=1, dest=str(dest))
        step(x, tag="names")
        api_log.configure(level=5)
        step(x, 2.0, tag="stats")
    finally:
        api_log.configure(level=0, dest="stdout", nvtx=False)
    files = list(tmp_path.iterdir())
    assert len(files) == 1 and "%i" not in files[0].name
    text = files[0].read_text()
    assert calls == ["off", "names", "stats"]
    assert text.count("mla_fp4 API call: ") == 2 and "step" in text
    assert "x = Tensor(shape=(3,), dtype=torch.float32" in text and "nan=1" in text and "scale = 2.0" in text
    assert "tag = 'stats'" in text and "-> Tensor(shape=(3,)" in text and "max=6" in text


def test_api_log_level_10_dumps_tensors(tmp_path):
    """Level 10: every tensor argument and the result are written to a directory per call, with a description;
    a tensor above the size limit is described but not written."""
    import json

    @api_log.api_logged
    def step(x, pair, scale=1.0):
        return x * scale, pair[0] + 1

    x = torch.arange(6, dtype=torch.float32).view(2, 3)
    big = torch.zeros(1 << 20)
    try:
        api_log.configure(level=10, dest=str(tmp_path / "log.txt"), dump_dir=str(tmp_path / "dumps"), dump_max_mb=1.0)
        step(x, (big, 3), scale=0.5)
    finally:
        api_log.configure(level=0, dest="stdout", dump_dir="mla_fp4_dumps", dump_max_mb=256)
    dirs = sorted((tmp_path / "dumps").iterdir())
    assert len(dirs) == 1 and dirs[0].name.endswith("step")
    ins = torch.load(dirs[0] / "inputs.pt")
    outs = torch.load(dirs[0] / "outputs.pt")
    meta = json.loads((dirs[0] / "meta.json").read_text())
    assert torch.equal(ins["x"], x) and "pair.0" not in ins            # 4 MiB > the 1 MiB limit
    assert meta["inputs"]["pair.0"]["skipped"] and meta["inputs"]["x"]["shape"] == [2, 3]
    assert torch.equal(outs["result.0"], x * 0.5) and meta["scalars"]["scale"] == "0.5"
    assert "inputs dumped to" in (tmp_path / "log.txt").read_text()


def test_public_entry_points_are_logged():
    from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper, FP4MLADecodeBackend
    from flashinfer_mla_fp4_b200.kvcache import write_tokens

    for fn in (BatchMLADecodeCuteDSLFP4Wrapper.plan, BatchMLADecodeCuteDSLFP4Wrapper.run, FP4MLADecodeBackend.forward,
               FP4MLADecodeBackend.prepare, write_tokens):
        assert hasattr(fn, "__wrapped__"), fn
