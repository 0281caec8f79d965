"""Multi-rank host logic on CPU (gloo, world_size 2): request sharding for data-parallel attention and
KV sharding + all-gather + merge for decode context parallel.  The per-rank decode and the merge are
done by the oracle here (there is no GPU); what is under test is the package's sharding arithmetic and
the packed all-gather layout that the CUDA merge kernel reads."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cp_worker(rank: int, world: int, port: int, tmp: str) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashinfer_mla_fp4_b200 import synth
        from flashinfer_mla_fp4_b200.distributed import shard_context
        from oracle import mla_fp4_oracle as O

        case = synth.build_case("cp", [700, 65, 64, 1, 2500], 8, page_size=16, seed=21)
        bt, sl = shard_context(case.block_tables, case.seq_lens, case.page_size, rank, world)
        out, lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, bt, sl, case.softmax_scale)
        rows = out.numel() // 512
        pad = ((rows + 3) // 4) * 4
        buf = torch.zeros(rows * 512 + pad)  # the packed per-rank layout: partial outputs, then LSEs
        buf[: rows * 512] = out.reshape(-1)
        buf[rows * 512: rows * 512 + rows] = lse.reshape(-1)
        gathered = torch.empty(world * buf.numel())
        dist.all_gather_into_tensor(gathered, buf)
        g = gathered.view(world, -1)
        outs = [g[r, : rows * 512].view_as(out) for r in range(world)]
        lses = [g[r, rows * 512: rows * 512 + rows].view_as(lse) for r in range(world)]
        merged, mlse = O.merge_partials(outs, lses)
        full, full_lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, case.block_tables, case.seq_lens,
                                      case.softmax_scale)
        torch.testing.assert_close(merged, full, atol=2e-5, rtol=1e-5)
        torch.testing.assert_close(mlse, full_lse, atol=1e-4, rtol=1e-5)
        # every token is owned by exactly one rank
        tot = sl.clone()
        dist.all_reduce(tot)
        assert torch.equal(tot, case.seq_lens)
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_context_parallel_sharding_and_merge_gloo(tmp_path):
    world = 2
    mp.spawn(_cp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_context_is_page_aligned_and_complete():
    from flashinfer_mla_fp4_b200.distributed import shard_context

    bt = torch.arange(40, dtype=torch.int32).view(4, 10)
    sl = torch.tensor([160, 1, 0, 145], dtype=torch.int32)
    for world in (1, 2, 3, 8):
        total = torch.zeros(4, dtype=torch.int64)
        seen = [[] for _ in range(4)]
        for r in range(world):
            lbt, lsl = shard_context(bt, sl, 16, r, world)
            total += lsl.long()
            for b in range(4):
                n = (int(lsl[b]) + 15) // 16
                seen[b] += lbt[b, :n].tolist()
                # all but the owner of the last page hold whole pages
                if int(lsl[b]) % 16:
                    assert seen[b][-1] == int(bt[b, (int(sl[b]) + 15) // 16 - 1])
        assert torch.equal(total, sl.long())
        for b in range(4):
            assert seen[b] == bt[b, : (int(sl[b]) + 15) // 16].tolist()


def test_shard_requests_balances_kv_volume():
    from flashinfer_mla_fp4_b200 import synth
    from flashinfer_mla_fp4_b200.distributed import shard_requests

    lens = synth.dp_lens()
    for world in (2, 4, 8):
        parts = shard_requests(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(len(lens)))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) <= 1.02 * (sum(lens) / world)
        naive = shard_requests(lens, world, balance=False)
        assert sorted(i for p in naive for i in p) == list(range(len(lens)))
