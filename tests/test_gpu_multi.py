"""Two-rank GPU tests (NCCL): context-parallel decode equals the unsharded decode and the oracle;
data-parallel attention needs no collective.  Run as child processes, one per GPU."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cp_worker(rank: int, world: int, port: int, tmp: str) -> None:
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper, synth
        from flashinfer_mla_fp4_b200.distributed import ContextParallelDecoder, shard_context
        from oracle import mla_fp4_oracle as O

        # every rank builds the same global case (same seed), then keeps only its shard's page lists:
        # a ragged batch with shards that are empty on one rank, and the shape of the context-parallel
        # benchmark configuration (B=8, H=64) at 4096 tokens per rank
        w = BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(64 << 20, dtype=torch.int8, device=dev))
        cp = ContextParallelDecoder(w, dist.group.WORLD)
        for name, lens, seed in (("cp_ragged", [5000, 130, 64, 1, 9000, 777], 31), ("cp_b8", [4096 * world] * 8, 32)):
            case = synth.build_case(name, lens, 64, 64, seed=seed, device=dev)
            bt, sl = shard_context(case.block_tables, case.seq_lens, case.page_size, rank, world)
            w.plan(num_heads=case.num_heads, page_size=case.page_size)
            out, lse = cp.run(case.q, case.kv_cache, bt, sl, case.max_seq_len, case.softmax_scale,
                              kv_cache_sf=case.kv_cache_sf, return_lse=True)
            torch.cuda.synchronize()
            ref, ref_lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, case.block_tables, case.seq_lens,
                                        case.softmax_scale)
            O.assert_parity(out, ref, f"{name} rank {rank}")
            torch.testing.assert_close(lse.cpu(), ref_lse, atol=2e-3, rtol=1e-4)
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_context_parallel_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_cp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
