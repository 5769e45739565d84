#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Headline workload (N=1): FP8 E4M3 GEMM M=N=K=4096, per-tensor scales, fp32 accumulate, bf16 out — the
configuration the metric "quantized GEMM TFLOPS ... % roofline" is quoted on.  With N>1 ranks every rank
owns a 4096-row column-parallel shard of the weight (out_features = 4096*N, activations replicated), so
per-GPU work is fixed ("weak") and the path needs no collective.

One "step" = one pass of the GEMM over one batch of activations.  Prints ONE JSON line (rank 0).
`--impl reference` times the CPU restatement of the reference's own arithmetic (oracle/) instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 4096
FLOP_PER_STEP = 2.0 * M * N * K


_JSON_FD = None


def emit(line: dict):
    """Writes the result line to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nm, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(threads: int | None = None, rows: int = 2048, k: int = K):
    """Times the oracle's FP8 GEMM (Fp8Codec decode + k-ascending fp32 FMA, the reference's arithmetic) on a
    rows x rows x k slice of the workload (full K, a block of the output); returns (TFLOP/s, cores, description)."""
    import numpy as np
    from oracle import api
    # all host cores this process may use (a launcher may have exported OMP_NUM_THREADS=1 for its workers)
    api.set_threads(threads or len(os.sched_getaffinity(0)))
    cores = api.num_threads()
    rng = np.random.default_rng(1)
    a = rng.integers(0, 0x7E, (rows, k)).astype(np.uint8)
    w = rng.integers(0, 0x7E, (rows, k)).astype(np.uint8)
    one = np.ones(1, np.float32)
    api.gemm_fp8(a[:64], w[:64], one, one, 0, 0, "bf16")          # page in, spin up the thread pool
    t0 = time.perf_counter()
    api.gemm_fp8(a, w, one, one, 0, 0, "bf16")
    dt = time.perf_counter() - t0
    return 2.0 * rows * rows * k / dt / 1e12, cores, f"{rows}x{rows} output block x K={k} of the 4096^3 GEMM ({rows * rows * 100 // (M * N)} % of the step), {dt:.2f} s"


def run_reference(args, rank: int):
    """CPU arm: the reference's own arithmetic for this path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    vals = []
    desc = ""
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_sample(rows=512)
    t_start = time.perf_counter()
    steps = 0
    for _ in range(args.steps):
        v, cores, desc = cpu_sample(rows=2048)
        vals.append(v)
        steps += 1
        if time.perf_counter() - t_start > 150:            # keep the whole arm within a few minutes
            break
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": FLOP_PER_STEP / (value * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": "fp8_e4m3_gemm_m4096_n4096_k4096_bf16out", "m": M, "n": N, "k": K,
                   "note": "CPU restatement of the reference's arithmetic (Fp8Codec decode + k-ascending fp32 FMA); "
                           "ms_per_step is the full 4096^3 step extrapolated from the timed sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b2q", choices=["b2q", "reference"])
    ap.add_argument("--rounding", default="rne", choices=["rne", "ref"], help="E4M3 encoder used to make the operands")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMV / INT8 side measurements")
    ap.add_argument("--case", default=None,
                    help="run ONE kernel case a few times and exit (for ncu captures): gemm_fp8:M:N:K | gemv_fp4:K:N:tokens | gemv_int4:K:N:tokens:group | kv_quant:tokens:head_dim:axis:bf16 | rms_quant:rows:cols:residual")
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        run_case(args.case, args.iters)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; keep it for the one JSON line.
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from oxicuda_b200 import _build
    if rank == 0:
        _build.build()
    if world > 1:
        dist.barrier()
    from oxicuda_b200.blas import gemm_fp8, select_tile
    from oxicuda_b200.quant import Fp8Codec

    peaks = load_peaks()
    warmup = max(args.warmup, 3)
    codec = Fp8Codec.e4m3(args.rounding)

    # ---- operands: SETS rotating (A, W shard, C) triples so that successive steps do not hit in L2 ----
    SETS = 4                                              # 4 x 64 MiB = 256 MiB > 126 MB L2
    g = torch.Generator(device=dev).manual_seed(0xB2000001 + rank)
    sets = []
    for _ in range(SETS):
        a = torch.randn(M, K, device=dev, generator=g)
        w = torch.randn(N, K, device=dev, generator=g) * 0.02      # this rank's 4096 output rows of W[4096*world x 4096]
        ac, sa = codec.quantize_rows(a, 1, M * K)
        wc, sw = codec.quantize_rows(w, 1, N * K)
        sets.append((ac.view(M, K), wc.view(N, K), sa, sw, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
        del a, w
    torch.cuda.synchronize()

    def step(i):
        ac, wc, sa, sw, out = sets[i % SETS]
        gemm_fp8(ac, wc, sa, sw, out=out)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    ms_per_step = ms / args.steps
    value = FLOP_PER_STEP * world / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public call with HOST buffers: H2D activations, GEMM, D2H result ----
    ac, wc, sa, sw, out = sets[0]
    h_a = torch.empty(M, K, dtype=torch.uint8).pin_memory()
    h_a.copy_(ac.cpu())
    h_sa = sa.cpu().pin_memory()
    h_out = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    d_a = torch.empty_like(ac)
    d_sa = torch.empty_like(sa)
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        d_a.copy_(h_a, non_blocking=True)
        d_sa.copy_(h_sa, non_blocking=True)
        gemm_fp8(d_a, wc, d_sa, sw, out=out)
        h_out.copy_(out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = FLOP_PER_STEP * world / (e2e_ms / e2e_steps * 1e-3) / 1e12
    clocks = sampler.stop() if rank == 0 else None

    extras = {}
    if not args.no_extras:
        for s_ in sets:                                # free the GEMM operands before the side measurements
            del s_
        sets.clear()
        torch.cuda.empty_cache()
        try:
            tp = tp_mlp_measurements(dev, rank, world)     # every rank takes part (all-reduce)
        except Exception as exc:
            tp = {"error": repr(exc)}
        if rank == 0:
            try:
                extras = side_measurements(dev, peaks)
                try:
                    extras["quantizers"] = quantizer_measurements(dev, peaks)
                except Exception as exc:  # noqa: BLE001 - side numbers must never kill the headline line
                    extras["quantizers"] = {"error": repr(exc)}
            except Exception as exc:                   # side numbers never block the headline line
                extras = {"error": repr(exc)}
            extras["tp_fp8_mlp_8192_28672"] = tp

    if rank == 0:
        tile, kid = select_tile("fp8", M, N, K)
        kernel_tflops = FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        cpu = None
        if world == 1:
            v, cores, desc = cpu_sample(rows=2048)
            cpu = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}
        traffic = None                                  # dram read + write bytes of one launch, from the committed ncu summary
        prof = ROOT / "profiles" / "gemm_tc2_fp8_4096.md"
        if prof.exists():
            import re
            mt = re.search(r"dram_bytes_per_launch:\s*(\d+)", prof.read_text())
            traffic = int(mt.group(1)) if mt else None
        line = {
            "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": "fp8_e4m3_gemm_m4096_n4096_k4096_bf16out", "m": M, "n": N, "k": K,
                       "scales": "per-tensor absmax/448", "encoder": args.rounding, "accumulate": "fp32 (TMEM)",
                       "sharding": f"column-parallel, {N} output rows per rank, out_features={N * world}, no collective",
                       "l2": f"rotating {SETS} operand sets ({SETS * 64} MiB) so inputs exceed the 126 MB L2",
                       "tile": f"{tile.tile_m}x{tile.tile_n}x{tile.tile_k}", "kernel_id": kid},
            "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": kernel_tflops / fp8_peak, "traffic": traffic,
                         "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}): dense FP8 issues at twice the bf16 rate",
                         "frac_of_nominal_4500": kernel_tflops / 4500.0,
                         "frac_of_measured_bf16": kernel_tflops / peaks["bf16_tflops"]},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K + 4, "d2h_bytes_per_step": M * N * 2,
                    "steps": e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "extras": extras,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_case(case: str, iters: int):
    """One kernel on synthetic operands, `iters` launches, CUDA-event time of the last ones printed."""
    import torch
    from oxicuda_b200.blas import MicroScalingConfig, MicroScalingQuantizer, ScalingFormat, gemm_fp8, gemv_fp4_wo
    from oxicuda_b200.quant import Fp8Codec
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    kind, *dims = case.split(":")
    if kind == "quantizers":        # the quantizer table of the extras, alone
        print(json.dumps(quantizer_measurements(dev, load_peaks()), indent=1))
        return
    d = [int(v) for v in dims]
    if kind == "gemm_fp8":
        m, n, k = d
        codec = Fp8Codec.e4m3("rne")
        ac, sa = codec.quantize_rows(torch.randn(m, k, device=dev), 1, m * k)
        wc, sw = codec.quantize_rows(torch.randn(n, k, device=dev) * 0.02, 1, n * k)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: gemm_fp8(ac.view(m, k), wc.view(n, k), sa, sw, out=out)
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"
    elif kind == "gemv_fp4":
        k, n, tokens = d
        codes, scales = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0)).quantize_fp4(torch.randn(n * k, device=dev) * 0.02)
        x = torch.randn(tokens, k, device=dev).to(torch.bfloat16)
        out = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: gemv_fp4_wo(codes, scales, x, n, k, out=out)
        work, unit = (n * k // 2 + n * k // 32 + 2 * tokens * k + 2 * tokens * n) / 1e9, "GB/s"
    elif kind == "gemv_int4":       # gemv_int4:K:N:tokens:group
        from oxicuda_b200.blas import gemv_int4_wo
        k, n, tokens, group = d
        packed = torch.randint(-2**31, 2**31 - 1, (n * k // 8,), dtype=torch.int32, device=dev)
        scales = (torch.rand(n * k // group, device=dev) * 0.01).to(torch.float16)
        x = torch.randn(tokens, k, device=dev).to(torch.bfloat16)
        out = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: gemv_int4_wo(packed, scales, group, x, n, k, out=out)
        work, unit = (n * k // 2 + 2 * n * k // group + 2 * tokens * k + 2 * tokens * n) / 1e9, "GB/s"
    elif kind == "kv_quant":        # kv_quant:n_tokens:head_dim:axis:bf16  (KvCacheQuantizer, 8 bits)
        from oxicuda_b200._lib import default_handle, ptr
        tokens, hd, axis, bf16 = d
        x = torch.randn(tokens, hd, device=dev)
        x = x.to(torch.bfloat16) if bf16 else x
        groups = tokens if axis == 0 else hd
        codes = torch.empty(tokens * hd, dtype=torch.uint8, device=dev)
        sc, zp = torch.empty(groups, device=dev), torch.empty(groups, device=dev)
        name = "b2q_kv_cache_quantize_bf16" if bf16 else "b2q_kv_cache_quantize_f32"
        fn = lambda: default_handle().call(name, ptr(x), tokens, hd, 8, axis, ptr(codes), ptr(sc), ptr(zp))
        work, unit = (tokens * hd * (x.element_size() + 1) + 8 * groups) / 1e9, "GB/s"
    elif kind == "rms_quant":       # rms_quant:rows:cols:residual
        from oxicuda_b200.kv_cache import rms_norm_quantize_fp8
        rows, cols, with_res = d
        x = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
        gamma = torch.ones(cols, device=dev, dtype=torch.bfloat16)
        res = torch.zeros(rows, cols, device=dev, dtype=torch.bfloat16) if with_res else None
        fn = lambda: rms_norm_quantize_fp8(x, gamma, 1e-6, residual=res)
        work, unit = (rows * cols * (3 + (4 if with_res else 0)) + 2 * cols + 4 * rows) / 1e9, "GB/s"
    else:
        raise SystemExit(f"unknown case {case}")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = []
    for _ in range(iters):
        flush.zero_()                                  # evict the operands from L2 between launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e-3)
    best = min(times)
    print(json.dumps({"case": case, "iters": iters, "best_us": best * 1e6, "rate": work / best, "unit": unit}))


def _time_calls(fn, iters, warm=5):
    import torch
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def _time_graph(fn, calls_per_graph, replays=20):
    """Seconds per call with the calls captured in a CUDA graph and replayed: removes the host launch cost
    (a decode step launches these kernels back to back from a graph)."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(3):
            fn(i)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls_per_graph):
            fn(i)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * calls_per_graph) * 1e-3


def tp_mlp_measurements(dev, rank, world):
    """Tensor-parallel FP8 SwiGLU MLP of a 70B-shaped layer (hidden 8192, FFN 28672): gate/up column-parallel,
    down row-parallel, NCCL all-reduce after the down projection; tokens in {1, 64, 4096}; tp = number of ranks."""
    import torch
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp
    hidden, ffn = 8192, 28672
    F = ffn // world
    g = torch.Generator(device=dev).manual_seed(0xB2000003 + rank)
    mk = lambda r, c: torch.randn(r, c, device=dev, generator=g) * 0.01
    mlp = TpFp8Mlp.from_shards(mk(F, hidden), mk(F, hidden), mk(hidden, F), DistInferHandle(rank, ParallelismConfig(tp=world)))
    torch.cuda.empty_cache()
    res = {"tp": world, "weights_bytes_per_gpu": 3 * hidden * F}
    for tokens in (1, 64, 4096):
        x = torch.randn(tokens, hidden, device=dev, generator=g).to(torch.bfloat16)
        sec = _time_calls(lambda i: mlp.forward(x), 20 if tokens < 4096 else 10, 3)
        timing = "eager launches"
        if tokens < 4096 and world == 1:
            # decode-sized steps are launch-bound from Python: replay them from a CUDA graph, as a serving loop does
            # (single rank only: a capture that one rank refuses must not leave the others waiting in a collective)
            try:
                sec_graph = _time_graph(lambda i: mlp.forward(x), 4, 10)
                if sec_graph < sec:
                    sec, timing = sec_graph, "CUDA-graph replay"
            except Exception:
                pass
        t = torch.tensor([sec], device=dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
        flops = 6.0 * tokens * hidden * ffn
        res[f"m{tokens}"] = {"us": sec * 1e6, "timing": timing, "tflops_all_gpus": flops / sec / 1e12,
                             "weight_gbs_per_gpu": 3 * hidden * F / sec / 1e9}
    return res


def quantizer_measurements(dev, peaks):
    """HBM-bound quantize / dequantize entry points on inputs far larger than L2: µs per call, algorithmic GB/s (input
    bytes + output bytes + parameters, each counted once) and the fraction of the measured copy peak."""
    import torch
    from oxicuda_b200._lib import default_handle, ptr
    h = default_handle()
    res = {"timing": "CUDA events around 10 back-to-back calls through the C ABI after 3 warm-up calls; operands of 128-512 MiB"}
    g = torch.Generator(device=dev).manual_seed(0xB2000007)
    n = 64 << 20
    x32 = torch.randn(n, device=dev, generator=g)
    x16 = x32.to(torch.bfloat16)
    u8 = torch.empty(n, dtype=torch.uint8, device=dev)
    i32 = torch.empty(n, dtype=torch.int32, device=dev)
    f32o = torch.empty(n, dtype=torch.float32, device=dev)

    def run(name, nbytes, fn):
        try:
            sec = _time_calls(lambda i: fn(), 10, 3)
            h.check()
            res[name] = {"us": sec * 1e6, "gbs": nbytes / sec / 1e9, "frac_of_measured_hbm": nbytes / sec / 1e9 / peaks["hbm_gbs"]}
        except Exception as exc:  # noqa: BLE001 - keep the remaining rows
            res[name] = {"error": repr(exc)}

    rows, cols = 8192, 8192
    sc = torch.empty(1 << 21, device=dev)
    zp = torch.empty(1 << 21, dtype=torch.int32, device=dev)
    zpf = torch.empty(1 << 21, device=dev)
    run("fp8_quantize_rows_bf16_8192x8192", n * 3, lambda: h.call("b2q_fp8_quantize_rows_bf16", ptr(x16), rows, cols, 0, 1, ptr(sc), ptr(u8)))
    run("fp8_quantize_rows_f32_8192x8192", n * 5, lambda: h.call("b2q_fp8_quantize_rows_f32", ptr(x32), rows, cols, 0, 1, ptr(sc), ptr(u8)))
    run("fp8_quantize_per_tensor_f32_64M_ref_rounding", n * 5, lambda: h.call("b2q_fp8_quantize_rows_f32", ptr(x32), 1, n, 0, 0, ptr(sc), ptr(u8)))
    run("fp8_encode_f32_64M", n * 5, lambda: h.call("b2q_fp8_encode_f32", ptr(x32), n, 0, 0, ptr(u8)))
    run("fp8_decode_f32_64M", n * 5, lambda: h.call("b2q_fp8_decode_f32", ptr(u8), n, 0, 0, ptr(f32o)))
    h.call("b2q_minmax_calibrate_f32", ptr(x32), n // 128, 128, 8, 0, ptr(sc), ptr(zp))
    run("minmax_calibrate_f32_group128", n * 4 + n // 16, lambda: h.call("b2q_minmax_calibrate_f32", ptr(x32), n // 128, 128, 8, 0, ptr(sc), ptr(zp)))
    run("minmax_quantize_f32_group128", n * 8 + n // 16, lambda: h.call("b2q_minmax_quantize_f32", ptr(x32), n // 128, 128, ptr(sc), ptr(zp), 8, 0, ptr(i32)))
    run("minmax_dequantize_f32_group128", n * 8 + n // 16, lambda: h.call("b2q_minmax_dequantize_f32", ptr(i32), n // 128, 128, ptr(sc), ptr(zp), ptr(f32o)))
    run("fp4_block_quantize_f32_e8m0", n * 4 + n // 2 + n // 32, lambda: h.call("b2q_fp4_block_quantize_f32", ptr(x32), n, 32, 0, 1, ptr(u8), ptr(sc)))
    run("fp4_block_quantize_f32_f32scales", n * 4 + n // 2 + n // 8, lambda: h.call("b2q_fp4_block_quantize_f32", ptr(x32), n, 32, 0, 0, ptr(u8), ptr(sc)))
    run("fp4_block_dequantize_f32_f32scales", n * 4 + n // 2 + n // 8, lambda: h.call("b2q_fp4_block_dequantize_f32", ptr(u8), n, 32, 0, 0, ptr(sc), ptr(f32o)))
    run("nf4_encode_f32_block64", n * 4 + n // 2 + n // 16, lambda: h.call("b2q_nf4_encode_f32", ptr(x32), n, 64, ptr(u8), ptr(sc)))
    run("nf4_decode_f32_block64", n * 4 + n // 2 + n // 16, lambda: h.call("b2q_nf4_decode_f32", ptr(u8), n // 2, 64, ptr(sc), ptr(f32o)))
    run("int8_quant_f32", n * 5, lambda: h.call("b2q_int8_quant_f32", ptr(x32), n, 0.03, ptr(u8)))
    run("int8_dequant_f32", n * 5, lambda: h.call("b2q_int8_dequant_f32", ptr(u8), n, 0.03, ptr(f32o)))
    run("distfp8_quantize_block_f32_block128", n * 5 + n // 32, lambda: h.call("b2q_distfp8_quantize_block_f32", ptr(x32), n, 128, ptr(u8), ptr(sc)))
    run("fake_quant_inplace_f32", n * 8, lambda: h.call("b2q_fake_quant_inplace_f32", ptr(f32o), n, 0.03, 0.0, -128.0, 127.0))
    tokens, hd = n // 128, 128
    run("kv_cache_quantize_per_token_bf16_d128", n * 3 + tokens * 8, lambda: h.call("b2q_kv_cache_quantize_bf16", ptr(x16), tokens, hd, 8, 0, ptr(u8), ptr(sc), ptr(zpf)))
    run("kv_cache_quantize_per_token_f32_d128", n * 5 + tokens * 8, lambda: h.call("b2q_kv_cache_quantize_f32", ptr(x32), tokens, hd, 8, 0, ptr(u8), ptr(sc), ptr(zpf)))
    run("kv_cache_quantize_per_channel_bf16_d128", n * 3, lambda: h.call("b2q_kv_cache_quantize_bf16", ptr(x16), tokens, hd, 8, 1, ptr(u8), ptr(sc), ptr(zpf)))
    run("kv_cache_dequantize_per_token_bf16_d128", n * 3 + tokens * 8, lambda: h.call("b2q_kv_cache_dequantize_bf16", ptr(u8), tokens, hd, 0, ptr(sc), ptr(zpf), ptr(x16)))
    gamma = torch.ones(cols, dtype=torch.bfloat16, device=dev)
    res16 = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    run("rms_norm_quantize_fp8_bf16_8192x8192", n * 3, lambda: h.call("b2q_rms_norm_quantize_fp8_bf16", ptr(x16), None, ptr(gamma), rows, cols, 1e-6, 0, 1, ptr(sc), ptr(u8), None))
    run("rms_norm_quantize_fp8_bf16_residual_8192x8192", n * 7, lambda: h.call("b2q_rms_norm_quantize_fp8_bf16", ptr(x16), ptr(res16), ptr(gamma), rows, cols, 1e-6, 0, 1, ptr(sc), ptr(u8), None))
    return res


def side_measurements(dev, peaks):
    """Decode GEMV (HBM GB/s) on the four Llama-3-8B-shaped projections and the INT8 W8A8 linear, rank 0 only."""
    import torch
    from oxicuda_b200.blas import MicroScalingConfig, MicroScalingQuantizer, ScalingFormat, gemv_fp4_wo
    from oxicuda_b200.quant import LlmInt8Config, LlmInt8Quantizer
    res = {"gemv_fp4_e8m0": {"timing": "CUDA-graph replay of back-to-back launches over rotating weight copies (> L2); "
                                       "consecutive launches of the tcgen05 kernel overlap their prologue with the previous tail "
                                       "(programmatic dependent launch), as they do in a decode step"}}
    msq = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0))
    # the four Llama-3-8B-shaped projections of the configuration, and the 70B-shaped FFN projection
    for (Kd, Nd) in ((4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (8192, 28672)):
        copies = max(4, int(300e6 // (Nd * Kd // 2)) + 1)         # rotate weight copies: > 126 MB L2 in total
        ws = []
        for c in range(copies):
            w = torch.randn(Nd * Kd, device=dev) * 0.02
            ws.append(msq.quantize_fp4(w))
            del w
        for tokens in (1, 4, 16, 32):
            x = torch.randn(tokens, Kd, device=dev).to(torch.bfloat16)
            out = torch.empty(tokens, Nd, dtype=torch.bfloat16, device=dev)
            call = lambda i: gemv_fp4_wo(ws[i % copies][0], ws[i % copies][1], x, Nd, Kd, out=out)
            key = f"k{Kd}_n{Nd}_m{tokens}"
            try:
                sec = _time_graph(call, 4 * copies)
                sec_eager = _time_calls(call, 100, 10)
            except Exception as exc:
                res["gemv_fp4_e8m0"][key] = {"error": repr(exc)}
                continue
            nbytes = Nd * Kd // 2 + Nd * Kd // 32 + 2 * tokens * Kd + 2 * tokens * Nd
            res["gemv_fp4_e8m0"][key] = {
                "us": sec * 1e6, "us_eager_launch": sec_eager * 1e6, "gbs": nbytes / sec / 1e9,
                "frac_of_measured_hbm": nbytes / sec / 1e9 / peaks["hbm_gbs"]}
        del ws
    # FP8 W8A8 with few tokens (decode / small batch) on the 70B-shaped FFN projection: HBM-bound, GB/s of algorithmic bytes
    from oxicuda_b200.blas import gemm_fp8
    from oxicuda_b200.quant import Fp8Codec
    codec = Fp8Codec.e4m3("rne")
    Kd, Nd = 8192, 28672
    fw = []
    for c in range(3):                                             # 3 x 235 MB > L2
        wc, sw = codec.quantize_rows(torch.randn(Nd, Kd, device=dev) * 0.02, Nd, Kd)
        fw.append((wc.view(Nd, Kd), sw))
    res["gemm_fp8_few_tokens_k8192_n28672"] = {"timing": res["gemv_fp4_e8m0"]["timing"]}
    for tokens in (1, 16, 32, 64):
        ac, sa = codec.quantize_rows(torch.randn(tokens, Kd, device=dev), tokens, Kd)
        ac = ac.view(tokens, Kd)
        out = torch.empty(tokens, Nd, dtype=torch.bfloat16, device=dev)
        call = lambda i: gemm_fp8(ac, fw[i % 3][0], sa, fw[i % 3][1], out=out)
        try:
            sec = _time_graph(call, 12)
        except Exception as exc:
            res["gemm_fp8_few_tokens_k8192_n28672"][f"m{tokens}"] = {"error": repr(exc)}
            continue
        nbytes = Nd * Kd + tokens * Kd + 2 * tokens * Nd
        res["gemm_fp8_few_tokens_k8192_n28672"][f"m{tokens}"] = {
            "us": sec * 1e6, "gbs": nbytes / sec / 1e9, "frac_of_measured_hbm": nbytes / sec / 1e9 / peaks["hbm_gbs"],
            "tflops": 2.0 * tokens * Nd * Kd / sec / 1e12}
    del fw
    x = torch.randn(8, 1024, device=dev)
    w = torch.randn(1024, 1024, device=dev) * 0.02
    q = LlmInt8Quantizer(LlmInt8Config(1e30, True))
    sec = _time_calls(lambda i: q.matmul(x, w, 8, 1024, 1024), 50, 5)
    res["int8_w8a8_linear_8x1024x1024"] = {"us": sec * 1e6, "note": "quantizes W and X on every call, as the reference entry point does"}
    return res


if __name__ == "__main__":
    main()
