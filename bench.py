#!/usr/bin/env python
"""Benchmark of the FP4 MLA decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--mode auto|dp|cp]
                    [--impl native|reference|reference_gpu] [--exchange peer|nccl]

One "step" = one decode step over one batch of synthetic requests (one launch of the decode kernel,
which also merges the split-KV partials).

* N = 1: the workload is the configuration the headline metric is quoted on: B=8, H=64, KV=32768,
  page 64 (``northstar``).  The line also carries ``extra``: the other single-GPU configurations
  (uniform, small, varlen, spec), measured in the same run after the headline.
* N > 1 (``--mode auto`` = ``cp``): decode context parallel.  B=8, H=64, KV = 32768 x N tokens per request,
  every request's pages sharded contiguously over the N ranks, so that each rank does exactly the
  north-star work and N=8 is the KV=262144 configuration; the step is decode + exchange of the
  partials over NVLink + merge, all inside the timed CUDA graph.  ``value`` is the max over ranks.
  ``--mode dp`` measures data-parallel attention instead (every rank its own north-star batch, no
  data-path collective).  ``extra`` holds the other mode's figure.

Prints ONE JSON line (rank 0).  ``value`` is device time per step in microseconds with all inputs
resident in HBM, cold L2 (the timed CUDA graph rotates through cache copies whose combined size exceeds
L2); ``e2e`` is the same step through the public wrapper with the step's inputs (q, block tables,
seq_lens) copied from pinned host memory and the BF16 output read back, inside the timed region.  The
KV cache itself is persistent device state and is not a step input.

``--impl reference`` times the reference's dequantise-then-attend arithmetic on the host cores (the CPU
restatement under oracle/: the reference ships no CPU path).  ``--impl reference_gpu`` (not run by default)
times, on the same GPU and with the same harness, FlashInfer's installed FP8 MLA decode kernel on the same
cache materialised as E4M3 and the reference's own CuTe-DSL FP4 kernel from ``baseline/_ref`` under a shim
for its version gate; whatever cannot be imported, compiled or launched is reported as unavailable with the
error text.
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
TRAFFIC_SUMMARY = ROOT / "profiles" / "decode_sm100_northstar_ncu_full.md"


def ncu_traffic_bytes():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode kernel on the north-star workload, read
    from the tracked ncu summary (a line ``dram_bytes_per_launch: <number>``); None when the summary has none."""
    try:
        for line in TRAFFIC_SUMMARY.read_text().splitlines():
            if line.strip().startswith("dram_bytes_per_launch:"):
                return float(line.split(":", 1)[1].strip().split()[0])
    except OSError:
        pass
    return None


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
    from flashinfer_mla_fp4_b200 import synth  # helper module: does not load the product library

    if mode == "cp":
        # context parallel: B=8, H=64, KV = 32768 tokens per request and rank (N=8: KV 262144), the rank's shard of
        # every request's pages (contiguous, page aligned), as ContextParallelDecoder expects them
        return synth.build_case(f"cp{world}", [32768] * 8, 64, 64, 1, 1100 + rank, device)
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
    """The reference arithmetic on the host cores.  Nothing of the product (package library, kernels) is loaded here."""
    if rank != 0:
        return
    case = build_workload(args.workload, "cpu", 0, 1, "dp")
    threads = os.cpu_count() or 1
    sample = min(case.batch, 8)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_oracle_us_per_step(case, sample, threads)
    t0 = time.perf_counter()
    vals = []
    what = ""
    for _ in range(args.steps):
        v, what = cpu_oracle_us_per_step(case, sample, threads)
        vals.append(v)
        if time.perf_counter() - t0 > 150.0:  # keep the whole run within a few minutes
            break
    us = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": world, "steps": len(vals),
        "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": case.name, "batch": case.batch, "heads": case.num_heads, "kv_len": case.max_seq_len,
                   "page_size": case.page_size, "note": "reference arithmetic (dequantise, dense FP32 attention) on host cores"},
        "cpu_baseline": {"value": us, "unit": UNIT, "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------------
# timing helpers (device time with CUDA events on the launching stream, steps inside one CUDA graph)
# ----------------------------------------------------------------------------------------------------------------
def cache_copies(case, copies: int = 0):
    n = copies or max(2, -(-int(1.5 * L2_BYTES) // max(case.kv_bytes(), 1)))
    n = min(n, 16)
    return [(case.kv_cache, case.kv_cache_sf)] + [(case.kv_cache.clone(), case.kv_cache_sf.clone()) for _ in range(n - 1)]


def time_graph(step, K: int, stream, repeats: int, barrier=None, warm: int = 3):
    """Median device time per step (us) of a CUDA graph holding K calls of step(i), replayed `repeats` times."""
    with torch.cuda.stream(stream):
        for i in range(warm):
            step(i)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(K):
                step(i)
    times = []

    def replay():
        if barrier is not None:
            barrier()
        else:
            torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        if barrier is not None:
            barrier()
        else:
            torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / K)

    for _ in range(max(1, repeats)):
        replay()
    return times, replay


def measure_single(name: str, device, K: int, repeats: int):
    """One single-GPU configuration: us per step (cold L2, graph of K steps) and its roofline fraction."""
    from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper

    case = build_workload(name, device, 0, 1, "dp")
    caches = cache_copies(case)
    w = BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(64 << 20, dtype=torch.int8, device=device))
    w.plan(num_heads=case.num_heads, page_size=case.page_size, out_dtype=torch.bfloat16, is_var_seq=True)
    out = torch.empty(case.batch, case.q_len, case.num_heads, 512, dtype=torch.bfloat16, device=device)

    def step(i):
        kc, sf = caches[i % len(caches)]
        w.run(case.q, kc, case.block_tables, case.seq_lens, case.max_seq_len, case.softmax_scale, out=out, kv_cache_sf=sf)

    times, _ = time_graph(step, K, torch.cuda.Stream(device), repeats)
    torch.cuda.synchronize()
    w.check_device_status()
    us = statistics.median(times)
    hbm_peak, bf16_peak, kind = peaks()
    t_hbm = case.step_bytes() / (hbm_peak * 1e9) * 1e6
    t_fp8 = case.flops() / (2.0 * bf16_peak * 1e12) * 1e6
    return {"us_per_step": us, "tb_per_s": case.kv_bytes() / (us * 1e-6) / 1e12, "kv_tokens": case.kv_tokens,
            "batch": case.batch, "heads": case.num_heads, "q_len": case.q_len,
            "roofline_us": max(t_hbm, t_fp8), "bound": "hbm" if t_hbm >= t_fp8 else "tensor (FP8 peak taken as 2 x measured BF16)",
            "frac_of_roofline": max(t_hbm, t_fp8) / us, "cache_copies": len(caches)}


def bench_cache_write(device, tokens: int = 1 << 20, reps: int = 10):
    """The CUDA cache writer on `tokens` bf16 tokens (inputs and cache larger than L2): tokens/s and roofline fraction."""
    from flashinfer_mla_fp4_b200.kvcache import BYTES_PER_TOKEN, HEAD_DIM_QK, LATENT_DIM, ROPE_DIM, ROW_BYTES, write_tokens

    page_size = 64
    pages = (tokens + page_size - 1) // page_size
    g = torch.Generator(device=device).manual_seed(1234)
    latent = torch.randn(tokens, LATENT_DIM, generator=g, device=device, dtype=torch.float32).bfloat16()
    rope = torch.randn(tokens, ROPE_DIM, generator=g, device=device, dtype=torch.float32).bfloat16()
    slots = torch.randperm(pages * page_size, generator=g, device=device)[:tokens].contiguous()
    cache = torch.empty(pages, page_size, ROW_BYTES, dtype=torch.uint8, device=device)
    sf = torch.empty(pages, page_size, 1, dtype=torch.float32, device=device)
    for _ in range(3):
        write_tokens(latent, rope, slots, cache, sf)
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        write_tokens(latent, rope, slots, cache, sf)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e-3)
    t = statistics.median(times)
    bytes_per_token = HEAD_DIM_QK * 2 + BYTES_PER_TOKEN + 8  # bf16 inputs, cache row + scale, slot id
    peak, _, kind = peaks()
    achieved = tokens * bytes_per_token / t / 1e9
    return {"metric": "fp4_cache_write_tokens_per_s", "value": tokens / t, "unit": "tokens/s", "tokens": tokens, "us": t * 1e6,
            "dtype": "bf16->e2m1/e4m3", "higher_is_better": True, "data": "synthetic", "n_gpus": 1,
            "config": {"workload": "cache_write", "tokens": tokens, "l2": f"cold by size: {tokens * bytes_per_token / 2**20:.0f} MiB touched per call"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": kind, "algorithmic_bytes_per_token": bytes_per_token, "kernel": "cache_write_kernel"}}


def bench_merge_partials(device, parts: int = 8, rows: int = 512, reps: int = 10):
    """The merge kernel of the NCCL form of context parallel on `parts` gathered partials of `rows` rows (the north-star
    shape at 8 ranks), L2 flushed before every launch: microseconds and roofline fraction."""
    import ctypes as C

    from flashinfer_mla_fp4_b200 import _cabi

    g = torch.Generator(device=device).manual_seed(77)
    n = rows * 512 + rows
    gathered = torch.randn(parts * n, generator=g, device=device, dtype=torch.float32)
    out = torch.empty(rows, 512, dtype=torch.bfloat16, device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    times = []
    for i in range(3 + reps):
        flush.fill_(i & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _cabi.check(_cabi.lib.mla_fp4_merge_partials(C.c_void_p(gathered.data_ptr()), C.c_void_p(gathered.data_ptr() + 4 * rows * 512), parts, rows,
                                                    n, n, C.c_void_p(out.data_ptr()), _cabi.OUT_BF16, None, stream))
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1) * 1e-3)
    t = statistics.median(times)
    nbytes = parts * n * 4 + rows * 512 * 2
    peak, _, kind = peaks()
    return {"metric": "cp_merge_partials_us", "value": t * 1e6, "unit": "us", "higher_is_better": False, "data": "synthetic", "n_gpus": 1,
            "dtype": "f32", "config": {"workload": "merge_partials", "parts": parts, "rows": rows, "l2": "flushed before every launch (256 MiB written)"},
            "roofline": {"bound": "hbm", "achieved": nbytes / t / 1e9, "peak": peak, "unit": "GB/s", "frac": nbytes / t / 1e9 / peak,
                         "peak_kind": kind, "algorithmic_bytes": nbytes, "kernel": "merge_partials_kernel"}}


# ----------------------------------------------------------------------------------------------------------------
# the reference's kernels on this GPU (not the default arm)
# ----------------------------------------------------------------------------------------------------------------
def run_reference_gpu_arm(args, rank: int, world: int):
    if rank != 0:
        return
    import importlib
    import traceback

    device = torch.device("cuda", 0)
    from oracle import mla_fp4_oracle as O  # the reference's fixture builder restated: the E4M3 materialisation of the cache

    case = build_workload(args.workload, device, 0, 1, "dp")
    res = {"impl": "reference_gpu", "metric": METRIC, "unit": UNIT, "n_gpus": 1, "higher_is_better": False, "data": "synthetic",
           "config": {"workload": case.name, "batch": case.batch, "heads": case.num_heads, "kv_len": case.max_seq_len,
                      "page_size": case.page_size, "l2": "cold: cache copies rotated", "harness": "same CUDA-graph harness as the native arm"}}
    import flashinfer

    res["flashinfer_version"] = getattr(flashinfer, "__version__", "?")
    # the same cache as E4M3 [pages, page, 576]: dequantised latent (exact when the scales are powers of two, else rounded
    # to E4M3: the FP8 kernel then sees slightly different data; only its time is used here) + the RoPE bytes
    with torch.no_grad():
        lat, _ = O.dequantize_cache(case.kv_cache.cpu(), case.kv_cache_sf.cpu())
        fp8 = torch.cat((lat.to(torch.float8_e4m3fn).view(torch.uint8), case.kv_cache.cpu()[..., 256:]), dim=-1).to(device)
    K = args.steps
    out = torch.empty(case.batch, 1, case.num_heads, 512, dtype=torch.bfloat16, device=device)
    ws = torch.empty(256 << 20, dtype=torch.int8, device=device)
    common = dict(kv_lora_rank=512, qk_rope_head_dim=64, num_heads=case.num_heads, page_size=case.page_size,
                  q_dtype=case.q.dtype, out_dtype=torch.bfloat16, is_var_seq=True, enable_pdl=False)

    def timed(make_step, copies):
        times, _ = time_graph(make_step, K, torch.cuda.Stream(device), args.repeats)
        torch.cuda.synchronize()
        return statistics.median(times)

    # (a) FlashInfer's installed FP8 kernel
    try:
        from flashinfer.cute_dsl.attention.wrappers.batch_mla import BatchMLADecodeCuteDSLWrapper

        w8 = BatchMLADecodeCuteDSLWrapper(ws)
        w8.plan(**common)
        n = min(16, max(2, -(-int(1.5 * L2_BYTES) // max(fp8.numel(), 1))))
        fp8s = [fp8.view(torch.float8_e4m3fn)] + [fp8.clone().view(torch.float8_e4m3fn) for _ in range(n - 1)]

        def step8(i):
            w8.run(q=case.q, kv_cache=fp8s[i % n], block_tables=case.block_tables, seq_lens=case.seq_lens,
                   max_seq_len=case.max_seq_len, softmax_scale=case.softmax_scale, out=out)

        res["flashinfer_fp8_us"] = timed(step8, n)
        res["flashinfer_fp8_label"] = f"flashinfer {res['flashinfer_version']} BatchMLADecodeCuteDSLWrapper, E4M3 cache of the same tokens"
        del fp8s
    except Exception as e:  # noqa: BLE001
        res["flashinfer_fp8_unavailable"] = f"unavailable on this box: {type(e).__name__}: {e}"[:600]
        res["flashinfer_fp8_trace"] = traceback.format_exc()[-800:]
        # The installed release splits the KV only with 128 heads.  The nearest shape it accepts: the same requests with
        # H = 128; the native kernel is timed on that very case beside it, so the pair is a same-box, same-shape comparison.
        try:
            from flashinfer.cute_dsl.attention.wrappers.batch_mla import BatchMLADecodeCuteDSLWrapper
            from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper, synth

            c128 = synth.build_case(case.name + "_h128", case.seq_lens_host, 128, case.page_size, 1, 1400, device)
            lat, _ = O.dequantize_cache(c128.kv_cache.cpu(), c128.kv_cache_sf.cpu())
            f8 = torch.cat((lat.to(torch.float8_e4m3fn).view(torch.uint8), c128.kv_cache.cpu()[..., 256:]), dim=-1).to(device)
            n = min(16, max(2, -(-int(1.5 * L2_BYTES) // max(f8.numel(), 1))))
            f8s = [f8.view(torch.float8_e4m3fn)] + [f8.clone().view(torch.float8_e4m3fn) for _ in range(n - 1)]
            o128 = torch.empty(c128.batch, 1, 128, 512, dtype=torch.bfloat16, device=device)
            w8 = BatchMLADecodeCuteDSLWrapper(ws)
            w8.plan(**{**common, "num_heads": 128})

            def step8h(i):
                w8.run(q=c128.q, kv_cache=f8s[i % n], block_tables=c128.block_tables, seq_lens=c128.seq_lens,
                       max_seq_len=c128.max_seq_len, softmax_scale=c128.softmax_scale, out=o128)

            res["flashinfer_fp8_h128_us"] = timed(step8h, n)
            del f8s
            cs = cache_copies(c128)
            wn = BatchMLADecodeCuteDSLFP4Wrapper(torch.empty(64 << 20, dtype=torch.int8, device=device))
            wn.plan(num_heads=128, page_size=c128.page_size)

            def stepn(i):
                wn.run(c128.q, cs[i % len(cs)][0], c128.block_tables, c128.seq_lens, c128.max_seq_len, c128.softmax_scale,
                       out=o128, kv_cache_sf=cs[i % len(cs)][1])

            res["native_h128_us"] = timed(stepn, len(cs))
            res["h128_label"] = (f"same requests with 128 heads: flashinfer {res['flashinfer_version']} FP8 kernel on the E4M3 cache "
                                 "vs this library's FP4 kernel on the FP4 cache, same harness, same box")
        except Exception as e2:  # noqa: BLE001
            res["flashinfer_fp8_h128_unavailable"] = f"unavailable on this box: {type(e2).__name__}: {e2}"[:600]
    # (b) the reference's own FP4 kernel, unmodified sources from baseline/_ref, under a shim for its version gate
    try:
        ref_dir = ROOT / "baseline" / "_ref"
        if not (ref_dir / "flashinfer_mla_fp4").exists():
            raise ImportError("baseline/_ref/flashinfer_mla_fp4 is missing (install the reference there)")
        import importlib.metadata as md

        real_version = md.version

        def shim_version(name):  # the reference refuses anything but flashinfer-python 0.6.17
            return "0.6.17" if name.replace("_", "-").lower() == "flashinfer-python" else real_version(name)

        md.version = shim_version
        import flashinfer.cute_dsl.utils as fu

        if not hasattr(fu, "require_cute_dsl_arch"):  # the one symbol the installed release lacks
            fu.require_cute_dsl_arch = lambda *a, **k: None
        sys.path.insert(0, str(ref_dir))
        try:
            ref = importlib.import_module("flashinfer_mla_fp4")
        finally:
            md.version = real_version
        w4 = ref.BatchMLADecodeCuteDSLFP4Wrapper(ws)
        w4.plan(**common, kv_dtype=torch.uint8)
        caches = cache_copies(case)

        def step4(i):
            kc, sf = caches[i % len(caches)]
            w4.run(q=case.q, kv_cache=kc, block_tables=case.block_tables, seq_lens=case.seq_lens,
                   max_seq_len=case.max_seq_len, softmax_scale=case.softmax_scale, out=out, kv_cache_sf=sf)

        res["reference_fp4_us"] = timed(step4, len(caches))
        res["reference_fp4_label"] = f"reference sources unmodified, shimmed onto flashinfer {res['flashinfer_version']} (pinned: 0.6.17)"
    except Exception as e:  # noqa: BLE001
        res["reference_fp4_unavailable"] = f"unavailable on this box: {type(e).__name__}: {e}"[:600]
        res["reference_fp4_trace"] = traceback.format_exc()[-800:]
    res["value"] = res.get("reference_fp4_us", res.get("flashinfer_fp8_us"))
    print(json.dumps(res), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="northstar", choices=["small", "uniform", "northstar", "varlen", "spec", "dp512", "cache_write", "merge_partials"])
    ap.add_argument("--mode", default="auto", choices=["auto", "dp", "cp"], help="N > 1: context parallel (auto, cp) or data parallel")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="context parallel: how the partials travel")
    ap.add_argument("--algo", default="auto", choices=["auto", "all_gather", "reduce_scatter"],
                    help="context parallel, peer exchange: every rank merges every row, or every row has an owner rank (auto: from 4 ranks on)")
    ap.add_argument("--impl", default="native", choices=["native", "reference", "reference_gpu"])
    ap.add_argument("--copies", type=int, default=0, help="cache copies rotated for cold L2 (0 = enough to exceed L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations / the other multi-GPU mode")
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
    if args.impl == "reference_gpu":
        run_reference_gpu_arm(args, rank, world)
        return
    warmup = max(args.warmup, 3)

    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.workload in ("cache_write", "merge_partials"):  # the two side kernels; --profile-steps N: a short run for an ncu capture
        if rank == 0:
            if args.workload == "cache_write":
                res = bench_cache_write(device, 262144, args.profile_steps) if args.profile_steps else bench_cache_write(device)
            else:
                res = bench_merge_partials(device, reps=args.profile_steps or 10)
            print(json.dumps(res), flush=True)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    mode = args.mode
    if mode == "auto":
        mode = "cp" if world > 1 else "dp"
    if world == 1:
        mode = "dp"

    from flashinfer_mla_fp4_b200 import BatchMLADecodeCuteDSLFP4Wrapper, _cabi
    from flashinfer_mla_fp4_b200.distributed import ContextParallelDecoder

    def barrier():
        # The device is drained before the ranks meet: an NCCL barrier kernel launched beside a still running graph
        # would share the GPU with kernels that need every SM (the decode kernel is a cooperative launch) or, in the
        # "nccl" exchange, with another collective of the same communicator.
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    K = args.steps
    stream = torch.cuda.Stream(device)

    def measure_mode(m: str, with_clocks: bool):
        """us per step (max over ranks), kernel-only us, the case and the step function of one multi-GPU mode (or the 1-GPU run)."""
        case = build_workload(args.workload, device, rank, world, m)
        caches = cache_copies(case, args.copies)
        copies = len(caches)
        ws = torch.empty(64 << 20, dtype=torch.int8, device=device)
        wrapper = BatchMLADecodeCuteDSLFP4Wrapper(ws)
        wrapper.plan(num_heads=case.num_heads, page_size=case.page_size, out_dtype=torch.bfloat16, is_var_seq=True)
        wrapper._kernel = _cabi.KERNEL_TCGEN05 if args.kernel == "fused" else _cabi.KERNEL_TCGEN05_2PASS
        out = torch.empty(case.batch, case.q_len, case.num_heads, 512, dtype=torch.bfloat16, device=device)
        cp = ContextParallelDecoder(wrapper, dist.group.WORLD, exchange=args.exchange, algo=args.algo) if (m == "cp" and world > 1) else None
        runner = cp if cp is not None else wrapper

        def step(i: int, q=None, bt=None, sl=None):
            kc, sf = caches[i % copies]
            return runner.run(case.q if q is None else q, kc, case.block_tables if bt is None else bt,
                              case.seq_lens if sl is None else sl, case.max_seq_len, case.softmax_scale, out=out, kv_cache_sf=sf)

        for i in range(warmup):
            step(i)
        barrier()
        runner.check_device_status()
        if args.profile_steps > 0:
            for i in range(args.profile_steps):
                step(i)
            torch.cuda.synchronize()
            runner.check_device_status()
            return None
        sampler = ClockSampler(local_rank) if with_clocks else None
        if sampler:
            sampler.start()
            sampler.wait_first_sample()
        times, replay = time_graph(step, K, stream, args.repeats, barrier=barrier, warm=0)
        clocks = None
        if sampler:
            # The K steps of one replay last a millisecond or two; nvidia-smi samples every 100 ms.  Keep taking timed
            # replays (all of them count toward the median) until the device has been under load for about 0.7 s, the
            # same number on every rank.
            extra = torch.tensor([min(3000, int(0.7e6 / max(K * statistics.median(times), 1.0)))], dtype=torch.int64, device=device)
            if world > 1:
                dist.all_reduce(extra, op=dist.ReduceOp.MAX)
            for _ in range(int(extra.item())):
                replay()
            clocks = sampler.stop()
        barrier()
        runner.check_device_status()
        us_local = statistics.median(times)
        # the decode kernel alone (roofline of the dominant kernel): same rotation, no exchange
        ktimes, _ = time_graph(lambda i: wrapper.run(case.q, caches[i % copies][0], case.block_tables, case.seq_lens, case.max_seq_len,
                                                     case.softmax_scale, out=out, kv_cache_sf=caches[i % copies][1]),
                               K, stream, args.repeats)
        kernel_us = statistics.median(ktimes)
        return {"case": case, "us_local": us_local, "kernel_us": kernel_us, "clocks": clocks, "copies": copies, "n_times": len(times),
                "step": step, "runner": runner, "out": out, "cp": cp}

    main_run = measure_mode(mode, with_clocks=True)
    if main_run is None:
        if rank == 0:
            print(json.dumps({"profile_steps": args.profile_steps, "workload": args.workload, "kernel": args.kernel}), flush=True)
        return
    case, out, step, runner = main_run["case"], main_run["out"], main_run["step"], main_run["runner"]
    B, H, ql = case.batch, case.num_heads, case.q_len

    # ---- end to end through the public API: the step's inputs come from pinned host memory into persistent device
    # buffers, the step itself is a captured CUDA graph (what a serving engine replays), the output is read back
    # The three inputs travel as ONE staging buffer (q | block tables | seq_lens, 256-byte aligned parts): one copy
    # node per step instead of three, each of which costs several microseconds whatever its size.
    parts = [case.q.contiguous().view(torch.uint8).reshape(-1), case.block_tables.contiguous().view(torch.uint8).reshape(-1),
             case.seq_lens.contiguous().view(torch.uint8).reshape(-1)]
    offs, total = [], 0
    for t in parts:
        offs.append(total)
        total += (t.numel() + 255) // 256 * 256
    in_h = torch.zeros(total, dtype=torch.uint8).pin_memory()
    in_d = torch.zeros(total, dtype=torch.uint8, device=device)
    for t, o in zip(parts, offs):
        in_h[o:o + t.numel()].copy_(t.cpu())
    in_d.copy_(in_h)
    q_d = in_d[offs[0]:offs[0] + parts[0].numel()].view(case.q.dtype).view(case.q.shape)
    bt_d = in_d[offs[1]:offs[1] + parts[1].numel()].view(torch.int32).view(case.block_tables.shape)
    sl_d = in_d[offs[2]:offs[2] + parts[2].numel()].view(torch.int32).view(case.seq_lens.shape)
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(t.numel() for t in parts)
    d2h = out_h.numel() * out_h.element_size()
    copies = main_run["copies"]
    e2e_graphs = []
    with torch.cuda.stream(stream):
        for j in range(copies):  # one captured step per cache copy, so the rotation (cold L2) stays
            step(j, q_d, bt_d, sl_d)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):  # H2D of the step's inputs, the step, D2H of its output: one graph launch per step
                in_d.copy_(in_h, non_blocking=True)
                step(j, q_d, bt_d, sl_d)
                out_h.copy_(out, non_blocking=True)
            e2e_graphs.append(g)
    torch.cuda.synchronize()

    def e2e_step(i: int):
        with torch.cuda.stream(stream):
            e2e_graphs[i % copies].replay()
        stream.synchronize()  # the caller consumes the result of every step

    for i in range(warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        e2e_step(i)
    barrier()
    e2e_us_local = (time.perf_counter() - t0) * 1e6 / K
    runner.check_device_status()

    # ---- reduce over ranks (max), aggregate
    vals = torch.tensor([main_run["us_local"], main_run["kernel_us"], e2e_us_local], dtype=torch.float64, device=device)
    tot = torch.tensor([float(case.kv_bytes()), float(case.step_bytes()), float(case.flops())], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    us, kernel_us_max, e2e_us = (float(x) for x in vals.cpu())
    kv_bytes_all, step_bytes_all, flops_all = (float(x) for x in tot.cpu())
    kernel_us = main_run["kernel_us"]

    # ---- the other configurations / the other multi-GPU mode, in the same run
    extra = {}
    if not args.no_extra and args.workload == "northstar":
        if world == 1:
            for name in ("uniform", "small", "varlen", "spec"):
                try:
                    extra[name] = measure_single(name, device, K, args.repeats)
                except Exception as e:  # noqa: BLE001
                    extra[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        else:
            other = "dp" if mode == "cp" else "cp"
            del step, runner
            if main_run["cp"] is not None:
                main_run["cp"].close()
            o = measure_mode(other, with_clocks=False)
            ov = torch.tensor([o["us_local"]], dtype=torch.float64, device=device)
            dist.all_reduce(ov, op=dist.ReduceOp.MAX)
            extra[f"{other}{world}"] = {"us_per_step": float(ov.item()), "kernel_us_rank0": o["kernel_us"],
                                        "what": "every rank its own north-star batch, no data-path collective (weak scaling)" if other == "dp"
                                        else "context parallel, KV = 32768 x N per request sharded over the ranks"}
            if o["cp"] is not None:
                o["cp"].close()

    if rank == 0:
        hbm_peak, bf16_peak, peak_kind = peaks()
        # roofline of the decode kernel on THIS rank's launch: algorithmic bytes of one launch / its mean duration
        achieved = case.step_bytes() / (kernel_us * 1e-6) / 1e9
        fp8_peak = 2.0 * bf16_peak  # no measured FP8 figure: 2 x measured BF16
        t_hbm = case.step_bytes() / (hbm_peak * 1e9) * 1e6
        t_fp8 = case.flops() / (fp8_peak * 1e12) * 1e6
        traffic = ncu_traffic_bytes() if (args.workload == "northstar" and args.kernel == "fused") else None
        launches_per_step = (1 if args.kernel == "fused" else 2) + (0 if mode != "cp" or world == 1 else (1 if args.exchange == "peer" else 2))
        line = {
            "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup,
            "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": "weak",
            "vs_baseline": (us / PUBLISHED_US[args.workload]) if (world == 1 and args.workload in PUBLISHED_US) else None,
            "dtype": "fp4(e2m1)xfp8(e4m3)->f32", "data": "synthetic",
            "config": {"workload": case.name, "batch_per_gpu": B, "heads": H, "q_len": ql, "kv_len_max": case.max_seq_len,
                       "kv_tokens_per_gpu": case.kv_tokens, "page_size": case.page_size, "parallelism": f"{mode}{world}",
                       "what": ("context parallel: every request holds 32768 x N tokens, sharded over the N ranks (per-GPU work fixed as N grows); "
                                f"step = decode + exchange ({args.exchange}) + merge" if mode == "cp" and world > 1 else
                                "every GPU decodes its own batch; no data-path collective"),
                       "l2": f"cold: {copies} cache copies rotated ({copies * case.kv_bytes() / 2**20:.0f} MiB > L2)",
                       "timing": f"CUDA graph of {K} steps, events on the launching stream, median of {main_run['n_times']} timed replays, max over ranks",
                       "published_baseline": "reference README, one B300 (not a B200)"},
            "tb_per_s": kv_bytes_all / (us * 1e-6) / 1e12,
            "tflops": flops_all / (us * 1e-6) / 1e12,
            "roofline": {"bound": "hbm" if t_hbm >= t_fp8 else "tensor", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": traffic,
                         "traffic_source": f"{TRAFFIC_SUMMARY.relative_to(ROOT)} (ncu capture, not this run)" if traffic else None,
                         "peak_kind": peak_kind,
                         "kernel": "mla_fp4_decode_sm100_kernel", "kernel_mode": args.kernel, "kernel_us": kernel_us, "algorithmic_bytes": case.step_bytes(),
                         "roofline_us": max(t_hbm, t_fp8), "step_frac_of_roofline": max(t_hbm, t_fp8) / us,
                         "fp8_peak_tflops_assumed": fp8_peak},
            "e2e": {"value": e2e_us, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "one captured graph per step: one pinned host -> device copy of the packed inputs (q, block tables, seq_lens); the decode step; output -> pinned host; then stream synchronize"},
            "gpu_launches": launches_per_step * K,
            "clocks": main_run["clocks"],
            "extra": extra,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, sample = cpu_oracle_us_per_step(case, 8, threads, repeats=2)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the process group down: the captured graphs still hold NCCL work, and destroying the
        # communicator under them has hung at exit.  Everything is measured and printed by now.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
