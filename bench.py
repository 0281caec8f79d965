#!/usr/bin/env python
"""Benchmark of the FP4 MLA decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--mode dp|cp] [--impl reference]

One "step" = one decode step (decode kernel + split-KV combine) over one batch of synthetic
requests.  At N=1 the workload is the configuration the headline metric is quoted on:
B=8, H=64, KV=32768, page 64 (``northstar``).  At N>1 every rank runs that workload on its own
requests (data-parallel attention: no data-path collective, weak scaling) unless ``--mode cp``
asks for the context-parallel case (KV sharded over ranks, partial outputs + LSE all-gathered
over NCCL and merged by the merge kernel).

Prints ONE JSON line (rank 0).  ``value`` is device time per step in microseconds with all
inputs resident in HBM, cold L2 (the timed CUDA graph rotates through cache copies whose
combined size exceeds L2); ``e2e`` is the same step through the public wrapper with the step's
inputs (q, block tables, seq_lens) copied from pinned host memory and the BF16 output read back,
inside the timed region.  The KV cache itself is persistent device state and is not a step input.

``--impl reference`` times the reference's dequantise-then-attend arithmetic on the host cores
(the CPU restatement under oracle/; the reference ships no CPU path and its GPU kernel needs
flashinfer-python==0.6.17, which is not installable offline).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fp4_mla_decode_us_per_step"
UNIT = "us"
L2_BYTES = 126 * 1024 * 1024
PUBLISHED_US = {"northstar": 37.726, "uniform": 13.461}  # reference README, one B300, cold L2


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode kernel, from the ncu capture summarised in
# profiles/decode_sm100_northstar_ncu_full.md (87.26 MB read + 15.18 MB written); None where no capture exists.
NCU_TRAFFIC_BYTES = {("northstar", "fused"): 100.8e6}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def wait_first_sample(self, timeout_s: float = 10.0) -> None:
        """Block until nvidia-smi has printed its first line, so that later samples fall inside the timed region."""
        if self.proc is None or self.proc.stdout is None:
            return
        import select

        ready, _, _ = select.select([self.proc.stdout], [], [], timeout_s)
        if ready:
            self.first = self.proc.stdout.readline()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], None, set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_workload(name: str, device, rank: int, world: int, mode: str):
    from flashinfer_mla_fp4_b200 import synth

    if mode == "cp":
        # context parallel: B=8, H=64, KV=262144 sharded contiguously over the ranks (page aligned)
        total = 262144
        per = (total // world // 64) * 64
        lens = [per if rank < world - 1 else total - per * (world - 1)] * 8
        return synth.build_case(f"cp{world}", lens, 64, 64, 1, 1100 + rank, device)
    if name == "dp512":
        lens = synth.dp_lens()
        per = (len(lens) + world - 1) // world
        mine = lens[rank * per:(rank + 1) * per]
        return synth.build_case(f"dp512/{world}", mine, 64, 64, 1, 1200 + rank, device)
    return synth.config_case(name, device=device, seed=None if world == 1 else 1300 + rank)


def cpu_oracle_us_per_step(case, sample_requests: int, threads: int, repeats: int = 1):
    """Oracle (CPU dequantise-then-attend, torch) timed on `sample_requests` requests, scaled to the batch by tokens."""
    from oracle import mla_fp4_oracle as O

    torch.set_num_threads(threads)
    n = min(sample_requests, case.batch)
    idx = sorted(range(case.batch), key=lambda i: -case.seq_lens_host[i])[:n]
    q = case.q[idx].cpu()
    bt = case.block_tables[idx].cpu()
    sl = case.seq_lens[idx].cpu()
    cache = case.kv_cache.cpu()
    sf = case.kv_cache_sf.cpu()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.mla_decode(q, cache, sf, bt, sl, case.softmax_scale)
        best = min(best, time.perf_counter() - t0)
    tok = sum(case.seq_lens_host[i] for i in idx)
    scale = case.kv_tokens / max(tok, 1)
    return best * 1e6 * scale, f"{n} of {case.batch} requests ({tok} of {case.kv_tokens} KV tokens), best of {repeats}, scaled by tokens"


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    case = build_workload(args.workload, "cpu", 0, 1, "dp")
    threads = os.cpu_count() or 1
    # warm-up + K steps, each a bounded sample (one request)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_oracle_us_per_step(case, 1, threads)
    t0 = time.perf_counter()
    vals = []
    for _ in range(args.steps):
        v, sample = cpu_oracle_us_per_step(case, 1, threads)
        vals.append(v)
    us = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": case.name, "batch": case.batch, "heads": case.num_heads, "kv_len": case.max_seq_len,
                   "page_size": case.page_size, "note": "reference arithmetic (dequantise, dense FP32 attention) on host cores"},
        "cpu_baseline": {"value": us, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="northstar", choices=["small", "uniform", "northstar", "varlen", "spec", "dp512"])
    ap.add_argument("--mode", default="dp", choices=["dp", "cp"])
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--copies", type=int, default=0, help="cache copies rotated for cold L2 (0 = enough to exceed L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--repeats", type=int, default=5, help="timed graph replays; the median is reported")
    ap.add_argument("--kernel", default="fused", choices=["fused", "2pass"],
                    help="fused: one kernel that also merges the split-KV partials (the product path); "
                         "2pass: the same decode kernel followed by a separate combine kernel")
    ap.add_argument("--profile-steps", type=int, default=0,
                    help="run this many plain (no graph) steps after the warm-up and exit: the command line for ncu captures")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    warmup = max(args.warmup, 3)

    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper
    from flashinfer_mla_fp4_b200.distributed import ContextParallelDecoder

    case = build_workload(args.workload, device, rank, world, args.mode)
    B, H, ql = case.batch, case.num_heads, case.q_len
    cache_bytes = case.kv_cache.numel() + case.kv_cache_sf.numel() * 4
    copies = args.copies or max(2, -(-int(1.5 * L2_BYTES) // max(case.kv_bytes(), 1)))
    copies = min(copies, 16)
    caches = [(case.kv_cache, case.kv_cache_sf)] + [(case.kv_cache.clone(), case.kv_cache_sf.clone()) for _ in range(copies - 1)]

    ws = torch.empty(64 << 20, dtype=torch.int8, device=device)
    wrapper = BatchMLADecodeCuteDSLFP4Wrapper(ws)
    wrapper.plan(num_heads=H, page_size=case.page_size, out_dtype=torch.bfloat16, is_var_seq=True)
    from flashinfer_mla_fp4_b200 import _cabi
    wrapper._kernel = _cabi.KERNEL_TCGEN05 if args.kernel == "fused" else _cabi.KERNEL_TCGEN05_2PASS
    launches_per_step = 1 if args.kernel == "fused" else 2
    out = torch.empty(B, ql, H, 512, dtype=torch.bfloat16, device=device)
    cp = ContextParallelDecoder(wrapper, dist.group.WORLD) if (args.mode == "cp" and world > 1) else None

    def step(i: int):
        kc, sf = caches[i % copies]
        if cp is not None:
            return cp.run(case.q, kc, case.block_tables, case.seq_lens, case.max_seq_len, case.softmax_scale,
                          out=out, kv_cache_sf=sf)
        return wrapper.run(case.q, kc, case.block_tables, case.seq_lens, case.max_seq_len, case.softmax_scale,
                           out=out, kv_cache_sf=sf)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (also the parity spot-check input)
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    wrapper.check_device_status()
    if args.profile_steps > 0:
        for i in range(args.profile_steps):
            step(i)
        torch.cuda.synchronize()
        wrapper.check_device_status()
        print(json.dumps({"profile_steps": args.profile_steps, "workload": case.name, "kernel": args.kernel}), flush=True)
        return

    # ---- device-timed K steps: one CUDA graph holding the K steps, replayed `repeats` times
    K = args.steps
    stream = torch.cuda.Stream(device)
    use_graph = cp is None
    graph = None
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for i in range(K):
                    step(i)
    sampler = ClockSampler(local_rank)
    times = []
    sampler.start()
    sampler.wait_first_sample()

    def timed_replay():
        barrier()
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            if graph is not None:
                graph.replay()
            else:
                for i in range(K):
                    step(i)
            e1.record(stream)
        barrier()
        times.append(e0.elapsed_time(e1) * 1e3 / K)  # us per step

    for _ in range(max(1, args.repeats)):
        timed_replay()
    # The K steps of one replay last a millisecond or two; nvidia-smi samples every 100 ms.  Keep taking timed
    # replays (all of them count toward the median) until the device has been under load for about 0.7 s, the
    # same number on every rank.
    extra = torch.tensor([min(3000, int(0.7e6 / max(K * statistics.median(times), 1.0)))], dtype=torch.int64, device=device)
    if world > 1:
        dist.all_reduce(extra, op=dist.ReduceOp.MAX)
    for _ in range(int(extra.item())):
        timed_replay()
    clocks = sampler.stop()
    us_local = statistics.median(times)

    # ---- decode kernel alone (roofline of the dominant kernel), same rotation, events on the launching stream
    # (in the fused mode the decode kernel is the whole step; in the two-kernel mode the combine kernel is left out)
    wrapper._phase_mask = 1
    kgraph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for i in range(3):
            step(i)
        with torch.cuda.graph(kgraph, stream=stream):
            for i in range(K):
                wrapper.run(case.q, caches[i % copies][0], case.block_tables, case.seq_lens, case.max_seq_len,
                            case.softmax_scale, out=out, kv_cache_sf=caches[i % copies][1])
    ktimes = []
    for _ in range(max(1, args.repeats)):
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            kgraph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        ktimes.append(e0.elapsed_time(e1) * 1e3 / K)
    wrapper._phase_mask = 0
    kernel_us = statistics.median(ktimes)

    # ---- end to end through the wrapper: step inputs from pinned host memory, output read back
    q_h = case.q.cpu().pin_memory()
    bt_h = case.block_tables.cpu().pin_memory()
    sl_h = case.seq_lens.cpu().pin_memory()
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    q_d, bt_d, sl_d = torch.empty_like(case.q), torch.empty_like(case.block_tables), torch.empty_like(case.seq_lens)
    h2d = q_h.numel() * q_h.element_size() + bt_h.numel() * 4 + sl_h.numel() * 4
    d2h = out_h.numel() * out_h.element_size()

    def e2e_step(i: int):
        q_d.copy_(q_h, non_blocking=True)
        bt_d.copy_(bt_h, non_blocking=True)
        sl_d.copy_(sl_h, non_blocking=True)
        kc, sf = caches[i % copies]
        if cp is not None:
            cp.run(q_d, kc, bt_d, sl_d, case.max_seq_len, case.softmax_scale, out=out, kv_cache_sf=sf)
        else:
            wrapper.run(q_d, kc, bt_d, sl_d, case.max_seq_len, case.softmax_scale, out=out, kv_cache_sf=sf)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller consumes the result of every step

    for i in range(warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        e2e_step(i)
    barrier()
    e2e_us_local = (time.perf_counter() - t0) * 1e6 / K
    wrapper.check_device_status()

    # ---- reduce over ranks (max), aggregate
    vals = torch.tensor([us_local, kernel_us, e2e_us_local], dtype=torch.float64, device=device)
    tot = torch.tensor([float(case.kv_bytes()), float(case.step_bytes()), float(case.flops())], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    us, kernel_us_max, e2e_us = (float(x) for x in vals.cpu())
    kv_bytes_all, step_bytes_all, flops_all = (float(x) for x in tot.cpu())

    if rank == 0:
        hbm_peak, bf16_peak, peak_kind = peaks()
        # roofline of the decode kernel on THIS rank's launch: algorithmic bytes of one launch / its mean duration
        achieved = case.step_bytes() / (kernel_us * 1e-6) / 1e9
        fp8_peak = 2.0 * bf16_peak  # no measured FP8 figure: 2 x measured BF16
        t_hbm = case.step_bytes() / (hbm_peak * 1e9) * 1e6
        t_fp8 = case.flops() / (fp8_peak * 1e12) * 1e6
        line = {
            "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup,
            "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": "strong" if args.mode == "cp" and world > 1 else "weak",
            "vs_baseline": (us / PUBLISHED_US[args.workload]) if (world == 1 and args.workload in PUBLISHED_US) else None,
            "dtype": "fp4(e2m1)xfp8(e4m3)->f32", "data": "synthetic",
            "config": {"workload": case.name, "batch_per_gpu": B, "heads": H, "q_len": ql, "kv_len_max": case.max_seq_len,
                       "kv_tokens_per_gpu": case.kv_tokens, "page_size": case.page_size, "parallelism": f"{args.mode}{world}",
                       "l2": f"cold: {copies} cache copies rotated ({copies * case.kv_bytes() / 2**20:.0f} MiB > L2)",
                       "timing": f"CUDA graph of {K} steps, events on the launching stream, median of {len(times)} timed replays, max over ranks"
                                 if use_graph else f"{K} eager steps between events, max over ranks",
                       "published_baseline": "reference README, one B300 (not a B200)"},
            "tb_per_s": kv_bytes_all / (us * 1e-6) / 1e12,
            "tflops": flops_all / (us * 1e-6) / 1e12,
            "roofline": {"bound": "hbm" if t_hbm >= t_fp8 else "tensor", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, args.kernel)), "peak_kind": peak_kind,
                         "kernel": "mla_fp4_decode_sm100_kernel", "kernel_mode": args.kernel, "kernel_us": kernel_us, "algorithmic_bytes": case.step_bytes(),
                         "roofline_us": max(t_hbm, t_fp8), "step_frac_of_roofline": max(t_hbm, t_fp8) / us,
                         "fp8_peak_tflops_assumed": fp8_peak},
            "e2e": {"value": e2e_us, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * K + (1 if cp is not None else 0) * K,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, sample = cpu_oracle_us_per_step(case, 2, threads, repeats=2)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
