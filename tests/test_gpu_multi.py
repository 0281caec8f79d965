"""Two-rank GPU tests: context-parallel decode equals the oracle, with the one-kernel peer exchange (plain stores
into the peers' memory over NVLink, flags, bounded waits) and with the NCCL all-gather + merge kernel; a peer that
does not show up makes the bounded wait run out and is reported.  Run as child processes, one per GPU."""
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
        w.plan(num_heads=64, page_size=64)
        outs = {}
        for exchange, algo in (("peer", "all_gather"), ("peer", "reduce_scatter"), ("nccl", "auto")):
            cp = ContextParallelDecoder(w, dist.group.WORLD, exchange=exchange, algo=algo)
            for name, lens, seed in (("cp_ragged", [5000, 130, 64, 1, 9000, 777], 31), ("cp_b8", [4096 * world] * 8, 32)):
                case = synth.build_case(name, lens, 64, 64, seed=seed, device=dev)
                bt, sl = shard_context(case.block_tables, case.seq_lens, case.page_size, rank, world)
                for rep in range(3):  # the peer exchange alternates between two buffers: go round more than once
                    out, lse = cp.run(case.q, case.kv_cache, bt, sl, case.max_seq_len, case.softmax_scale,
                                      kv_cache_sf=case.kv_cache_sf, return_lse=True)
                torch.cuda.synchronize()
                cp.check_device_status()
                ref, ref_lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, case.block_tables, case.seq_lens,
                                            case.softmax_scale)
                O.assert_parity(out, ref, f"{name} rank {rank} {exchange} {algo}")
                torch.testing.assert_close(lse.cpu(), ref_lse, atol=2e-3, rtol=1e-4)
                outs[(exchange, algo, name)] = out.clone()
                if exchange == "peer":  # the other output types travel as one or two words per thread in the reduce-scatter form
                    for dt in (torch.float32, torch.float8_e4m3fn):
                        o2 = torch.empty(out.shape, dtype=dt, device=dev)
                        cp.run(case.q, case.kv_cache, bt, sl, case.max_seq_len, case.softmax_scale, kv_cache_sf=case.kv_cache_sf, out=o2)
                        torch.cuda.synchronize()
                        cp.check_device_status()
                        tol = 2e-2 if dt == torch.float32 else 0.3
                        assert (o2.float() - out.float()).abs().max().item() <= tol * max(1.0, out.float().abs().max().item()), (name, algo, dt)
            if exchange == "peer" and algo == "all_gather":
                # Failure made on the host: rank 1 skips a step, so its flag never reaches rank 0, whose bounded wait
                # runs out (a small poll budget here); the kernel returns and the status says so.  Nothing faults.
                dist.barrier()
                if rank == 0:
                    cp._wait_polls = 2000
                    cp.run(case.q, case.kv_cache, bt, sl, case.max_seq_len, case.softmax_scale, kv_cache_sf=case.kv_cache_sf)
                    torch.cuda.synchronize()
                    try:
                        cp.check_device_status()
                        raise AssertionError("the missing peer went unnoticed")
                    except RuntimeError as e:
                        assert "device error 5" in str(e)
                dist.barrier()
            cp.close()
        for name in ("cp_ragged", "cp_b8"):  # same merge arithmetic every way
            torch.testing.assert_close(outs[("peer", "all_gather", name)].float(), outs[("nccl", "auto", name)].float(), atol=1e-2, rtol=0)
            assert torch.equal(outs[("peer", "all_gather", name)], outs[("peer", "reduce_scatter", name)]), name
        # an attention sink joins the denominator once per request, whichever rank holds the request's first tokens
        from flashinfer_mla_fp4_b200 import AttentionWithSink

        sink = torch.linspace(-3.0, 8.0, 64, device=dev)
        w2 = BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(64 << 20, dtype=torch.int8, device=dev))
        w2.plan(num_heads=64, page_size=64, variant=AttentionWithSink(sink))
        cp = ContextParallelDecoder(w2, dist.group.WORLD, exchange="peer")
        case = synth.build_case("cp_sink", [5000, 130, 64, 1, 9000, 777], 64, 64, seed=33, device=dev)
        bt, sl = shard_context(case.block_tables, case.seq_lens, case.page_size, rank, world)
        out, lse = cp.run(case.q, case.kv_cache, bt, sl, case.max_seq_len, case.softmax_scale, kv_cache_sf=case.kv_cache_sf, return_lse=True)
        torch.cuda.synchronize()
        cp.check_device_status()
        ref, ref_lse = O.mla_decode(case.q, case.kv_cache, case.kv_cache_sf, case.block_tables, case.seq_lens, case.softmax_scale, sink=sink)
        O.assert_parity(out, ref, f"cp_sink rank {rank}")
        torch.testing.assert_close(lse.cpu(), ref_lse, atol=2e-3, rtol=1e-4)
        cp.close()
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
