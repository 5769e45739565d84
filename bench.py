#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Headline workload, the same at every GPU count (strong scaling): the tensor-parallel FP8 E4M3 SwiGLU MLP of a
70B-shaped layer (hidden 8192, FFN 28672, 4096 tokens, bf16 out) — gate/up column-parallel, down row-parallel, the
partial results summed over the ranks — in TFLOP/s of its three GEMMs.  One "step" = one forward pass of the layer
over one batch of activations through the library's C entry point (b2q_mlp_swiglu_fp8_forward).  At every GPU
count the sharded result is checked on every rank against the un-sharded layer and against the CPU oracle.

`roofline` describes the dominant kernel (the tcgen05 FP8 GEMM) and carries compact tables of the other halves of the
metric: the single 4096^3 FP8 / INT8 GEMM with a library ceiling beside it, the FP4 decode GEMV in HBM GB/s, the
decode-sized MLP steps.  Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference's own arithmetic (oracle/) on a bounded sample of the same workload instead.
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

# Headline workload, the same at every GPU count (strong scaling): the tensor-parallel FP8 SwiGLU MLP of a
# 70B-shaped layer (hidden 8192, FFN 28672, 4096 tokens): gate/up column-parallel, down row-parallel, sum over ranks.
HIDDEN, FFN, TOKENS = 8192, 28672, 4096
NCU_DRAM_BYTES_GATE_UP_TP1 = 668990720 + 225613056      # gate | up GEMM with the SwiGLU epilogue, 4096 x 57344 x 8192
FLOP_PER_STEP = 6.0 * TOKENS * HIDDEN * FFN
WORKLOAD = "tp_fp8_e4m3_swiglu_mlp_hidden8192_ffn28672_tokens4096_bf16out"
M = N = K = 4096                                    # the single-GEMM configuration, reported in roofline.gemm_fp8_4096


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


_CPU_WEIGHTS = None


def cpu_sample(threads: int | None = None, tokens: int = 32):
    """Times the oracle's statement of the MLP (Fp8Codec decode + k-ascending fp32 FMA GEMMs, SwiGLU, per-token
    quantizers: the reference's own arithmetic) on `tokens` tokens of the 4096 against the full-size weights;
    returns (TFLOP/s, cores, description)."""
    import numpy as np
    from oracle import api
    global _CPU_WEIGHTS
    # all host cores this process may use (a launcher may have exported OMP_NUM_THREADS=1 for its workers)
    api.set_threads(threads or len(os.sched_getaffinity(0)))
    cores = api.num_threads()
    rng = np.random.default_rng(1)
    if _CPU_WEIGHTS is None:
        wgu = rng.integers(0, 0x7E, (2 * FFN, HIDDEN), dtype=np.uint8)
        wd = rng.integers(0, 0x7E, (HIDDEN, FFN), dtype=np.uint8)
        _CPU_WEIGHTS = (wgu, np.full(2 * FFN, 1e-4, np.float32), wd, np.full(HIDDEN, 1e-4, np.float32))
    wgu, sgu, wd, sd = _CPU_WEIGHTS
    x = rng.standard_normal((tokens, HIDDEN)).astype(np.float32)
    t0 = time.perf_counter()
    xc, xs, _ = api.fp8_quantize_rows(x, tokens, HIDDEN, 0, 1)
    gu = api.gemm_fp8(xc.reshape(tokens, HIDDEN), wgu, xs, sgu, 0, 1, "bf16")
    h = api.swiglu(gu[:, :FFN], gu[:, FFN:])
    hc, hs, _ = api.fp8_quantize_rows(h, tokens, FFN, 0, 1)
    api.gemm_fp8(hc.reshape(tokens, FFN), wd, hs, sd, 0, 1, "bf16")
    dt = time.perf_counter() - t0
    flops = 6.0 * tokens * HIDDEN * FFN
    return flops / dt / 1e12, cores, f"{tokens} of the {TOKENS} tokens through the full-size layer ({tokens * 100.0 / TOKENS:.2f} % of the step), {dt:.2f} s"


def base_config(world: int) -> dict:
    """The workload description both arms print (same keys, same values)."""
    return {"workload": WORKLOAD, "hidden": HIDDEN, "ffn": FFN, "tokens": TOKENS, "tp": world,
            "scales": "per-token activations, per-output-row weights, absmax/448", "accumulate": "fp32",
            "sharding": "gate/up column-parallel, down row-parallel, sum over ranks after the down projection"}


def run_reference(args, rank: int, world: int):
    """CPU arm: the reference's own arithmetic for this path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    vals = []
    desc = ""
    cpu_sample(tokens=4)                                    # builds the weights, spins up the thread pool
    t_start = time.perf_counter()
    steps = 0
    for _ in range(args.steps):
        v, cores, desc = cpu_sample(tokens=32)
        vals.append(v)
        steps += 1
        if time.perf_counter() - t_start > 150:            # keep the whole arm within a few minutes
            break
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": FLOP_PER_STEP / (value * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": base_config(world),
        "note": "CPU restatement of the reference's arithmetic (Fp8Codec decode + k-ascending fp32 FMA); each step is a "
                "bounded sample and ms_per_step is the full step extrapolated from it",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def _rel_err(got, ref):
    """max |got - ref| / (|ref| + rms(ref)) over torch tensors (the bound of the MLP parity tests)."""
    g, r = got.double(), ref.double()
    rms = float((r * r).mean().sqrt()) + 1e-30
    return float(((g - r).abs() / (r.abs() + rms)).max())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b2q", choices=["b2q", "reference"])
    ap.add_argument("--rounding", default="rne", choices=["rne", "ref"], help="E4M3 encoder used to make the operands")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMV / GEMM / quantizer side measurements")
    ap.add_argument("--chunks", type=int, default=0, help="token chunks of the overlapped all-reduce (0 = automatic)")
    ap.add_argument("--case", default=None,
                    help="run ONE kernel case a few times and exit (for ncu captures): gemm_fp8:M:N:K | gemv_fp4:K:N:tokens | gemv_int4:K:N:tokens:group | kv_quant:tokens:head_dim:axis:bf16 | rms_quant:rows:cols:residual | fp8_quant_rows:rows:cols:bf16 | swiglu_quant:rows:ffn | gemm_fp4_bs:tokens:N:K:mxfp8 | grouped_fp8:experts:rows_each:N:K | wq_gemv:rows:cols:group:bits:split_k | wq_dequant:rows:cols:group:bits:bf16 | tp_breakdown (under torchrun: the headline layer's pieces timed one by one on every rank)")
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    if args.case == "tp_breakdown":
        run_tp_breakdown(args.iters)
        return
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
        run_reference(args, rank, world)
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
    from oxicuda_b200._lib import default_handle
    from oxicuda_b200.blas import gemm_fp8, select_tile
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp, column_shard_rows, tp_group

    peaks = load_peaks()
    warmup = max(args.warmup, 3)

    # ---- the layer: every rank draws the SAME full weights (same seed) and keeps its shard; with several ranks it
    # also keeps the un-sharded layer as the parity reference of the sharded result ----
    handle = DistInferHandle(rank, ParallelismConfig(tp=world))
    g = torch.Generator(device=dev).manual_seed(0xB2000003)
    wg = torch.randn(FFN, HIDDEN, device=dev, generator=g) * 0.01
    wu = torch.randn(FFN, HIDDEN, device=dev, generator=g) * 0.01
    wd = torch.randn(HIDDEN, FFN, device=dev, generator=g) * 0.01
    # every rank's shard, quantized exactly as that rank quantizes it: this rank's own is the layer under test, the
    # others let it rebuild the whole sharded computation locally as the parity reference
    shards = [TpFp8Mlp(wg, wu, wd, DistInferHandle(r, ParallelismConfig(tp=world)), args.rounding) for r in range(world)]
    mlp = shards[rank]
    del wg, wu, wd
    torch.cuda.empty_cache()
    group = tp_group(handle)
    if args.chunks:
        group.set_chunks(args.chunks)
    F = mlp.local_ffn
    SETS = 3                                              # rotating activation / result sets (weights alone exceed the 126 MB L2)
    xs_ = [torch.randn(TOKENS, HIDDEN, device=dev, generator=g).to(torch.bfloat16) for _ in range(SETS)]
    ys_ = [torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(SETS)]
    torch.cuda.synchronize()

    def step(i):
        mlp.forward(xs_[i % SETS], out=ys_[i % SETS])

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    if world > 1:
        dist.barrier()                                     # nobody enters the timed region while rank 0 starts the sampler
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
    value = FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
    default_handle().check()

    # ---- end to end through the public call with HOST buffers: H2D activations, MLP, D2H result, every step ----
    h_x = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16).pin_memory()
    h_x.copy_(xs_[0].cpu())
    h_y = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        xs_[1].copy_(h_x, non_blocking=True)
        mlp.forward(xs_[1], out=ys_[1])
        h_y.copy_(ys_[1], non_blocking=True)

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
    e2e_value = FLOP_PER_STEP / (e2e_ms / e2e_steps * 1e-3) / 1e12
    clocks = sampler.stop() if rank == 0 else None

    # ---- the dominant kernel alone: this rank's gate|up GEMM (tokens x 2*ffn/tp x hidden), CUDA events ----
    xc, xsc = mlp.codec.quantize_rows(xs_[0], TOKENS, HIDDEN)
    gu = torch.empty(TOKENS, 2 * F, dtype=torch.bfloat16, device=dev)
    gemm_sec = _time_calls(lambda i: gemm_fp8(xc.view(TOKENS, HIDDEN), mlp.gate_up.codes, xsc, mlp.gate_up.scales, out=gu), 10, 3)
    gemm_flop = 2.0 * TOKENS * 2 * F * HIDDEN
    gemm_tflops = gemm_flop / gemm_sec / 1e12
    del gu, xc, xsc

    # ---- parity of the sharded result, on every rank: against the same sharded computation redone locally (every
    # rank's partial from that rank's own codes, added in rank order in fp32; 64 and 4096 tokens) and, rank 0, against
    # the CPU oracle's composition over the same codes with the ranks simulated in order (first 8 of the 64 tokens) ----
    tp_summary = {"tp": world, "m4096_us": ms_per_step * 1e3, "timing_m4096": "CUDA events over the timed steps, max over ranks"}
    parity = {}
    x64 = xs_[2][:64].contiguous()
    y64 = mlp.forward(x64)
    y4096 = mlp.forward(xs_[2])
    if world > 1:
        def local_sum(xin):
            tot = None
            for sh in shards:
                part = sh.forward_partial(xin).float()
                tot = part if tot is None else tot + part
            return tot.to(torch.bfloat16)
        parity["m64_vs_local_rank_order_sum"] = _rel_err(y64, local_sum(x64))
        parity["m4096_vs_local_rank_order_sum"] = _rel_err(y4096, local_sum(xs_[2]))
    y64_host = y64.float().cpu()
    default_handle().check()
    # decode-sized steps, timed the same way at every tp: CUDA-graph replay of 4 steps (the peer-memory all-reduce is a
    # plain kernel, so the whole step is capturable on every rank); eager launches as the fallback
    for tokens in (1, 64):
        xt = xs_[2][:tokens].contiguous()
        yt = torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev)
        timing = "CUDA-graph replay"
        try:
            sec = _time_graph(lambda i: mlp.forward(xt, out=yt), 4, 10)
        except Exception:                                  # noqa: BLE001
            timing = "eager launches"
            sec = _time_calls(lambda i: mlp.forward(xt, out=yt), 20, 3)
        t = torch.tensor([sec], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tp_summary[f"m{tokens}_us"] = float(t.item()) * 1e6
        tp_summary[f"timing_m{tokens}"] = timing
        tp_summary[f"m{tokens}_weight_gbs_per_gpu"] = 3 * HIDDEN * F / float(t.item()) / 1e9
    default_handle().check()
    tp_summary["boundary"] = {f"m{tk}": dict(zip(("mode", "chunks"), group.plan(tk, HIDDEN))) for tk in (1, 64, 4096)}
    if rank == 0:
        try:
            parity["m64_first8_vs_oracle"] = oracle_mlp_check(shards, x64[:8], y64_host[:8], args.rounding)
        except Exception as exc:                           # noqa: BLE001
            parity["oracle_error"] = repr(exc)
    worst = max([v for v in parity.values() if isinstance(v, float)] or [0.0])
    ok = torch.tensor([1 if worst <= 1e-2 and "oracle_error" not in parity else 0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        wt = torch.tensor([worst], device=dev)
        dist.all_reduce(wt, op=dist.ReduceOp.MAX)
        worst = float(wt.item())
    tp_summary["parity"] = parity
    tp_summary["parity_max_rel_err_all_ranks"] = worst
    tp_summary["parity_ok"] = bool(int(ok.item()) == 1)

    extras = {}
    roof_extra = {}
    if not args.no_extras and rank == 0:
        shards.clear()
        xs_.clear(); ys_.clear()
        torch.cuda.empty_cache()
        try:
            roof_extra, extras = side_measurements(dev, peaks)
        except Exception as exc:                           # side numbers never block the headline line
            extras = {"error": repr(exc)}
        try:
            extras["quantizers"] = quantizer_measurements(dev, peaks)
        except Exception as exc:  # noqa: BLE001
            extras["quantizers"] = {"error": repr(exc)}
    if world > 1:
        dist.barrier()

    if rank == 0:
        tile, kid = select_tile("fp8", TOKENS, 2 * F, HIDDEN)
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        cpu = None
        if world == 1:
            cpu_sample(tokens=4)
            v, cores, desc = cpu_sample(tokens=64)
            cpu = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}
        cfg = base_config(world)
        cfg.update({"encoder": args.rounding, "l2": "weights alone (705 MB / tp per rank) exceed the 126 MB L2; activations rotate over 3 sets",
                    "tile": f"{tile.tile_m}x{tile.tile_n}x{tile.tile_k}", "kernel_id": kid})
        roofline = {"bound": "tensor", "kernel": f"gemm_tc2_kernel<fp8> on this rank's gate|up GEMM {TOKENS}x{2 * F}x{HIDDEN}",
                    "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                    # dram__bytes_read.sum + dram__bytes_write.sum of this launch at tp = 1 (one-pass ncu capture of this very
                    # command with --steps 2 --warmup 3 --no-extras); not captured for the shards of tp > 1
                    "traffic": NCU_DRAM_BYTES_GATE_UP_TP1 if world == 1 else None,
                    "algorithmic_bytes": TOKENS * HIDDEN + 2 * F * HIDDEN + TOKENS * F * 2,
                    "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}): the step runs for milliseconds under the power cap, "
                                   "and dense FP8 issues at twice the bf16 rate",
                    "frac_of_nominal_4500": gemm_tflops / 4500.0, "us_per_launch": gemm_sec * 1e6,
                    "tp_mlp": tp_summary}
        roofline.update(roof_extra)
        line = {
            "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": cfg,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": TOKENS * HIDDEN * 2, "d2h_bytes_per_step": TOKENS * HIDDEN * 2,
                    "steps": e2e_steps},
            # this library's kernels per timed step and rank: quantize x, gate|up GEMM (SwiGLU in its epilogue), quantize h, then the
            # down GEMM and, on the scatter boundary, the sum-and-gather kernel once per column chunk (NCCL's kernels are not counted)
            "gpu_launches": args.steps * _launches_per_step(tp_summary["boundary"]["m4096"], args.chunks),
            "clocks": clocks,
            "extras": extras,
        }
        emit(line)
    group.close()
    if world > 1:
        dist.destroy_process_group()


def oracle_mlp_check(shards, x_dev, y_host, rounding):
    """rel. error of y (the sharded layer's result for the tokens of x) against the oracle composition over the ranks'
    own codes: per-token E4M3 quantizer, k-ascending fp32 GEMMs, SwiGLU, per-rank re-quantization, rank-ordered sum."""
    import numpy as np
    import torch
    from oracle import api
    api.set_threads(len(os.sched_getaffinity(0)))
    mode = 1 if rounding == "rne" else 0
    tokens, hidden = x_dev.shape
    x = x_dev.float().cpu().numpy()
    xc, xs, _ = api.fp8_quantize_rows(x, tokens, hidden, 0, mode)
    total = None
    for sh in shards:
        F = sh.local_ffn
        inter = sh.gu_codes is not None
        h = api.swiglu_mlp_hidden(xc, xs, (sh.gu_codes if inter else sh.gate_up.codes).cpu().numpy(),
                                  (sh.gu_scales if inter else sh.gate_up.scales).cpu().numpy(), tokens, hidden, F, inter)
        hc, hs, _ = api.fp8_quantize_rows(h, tokens, F, 0, mode)
        part = api.gemm_fp8(hc.reshape(tokens, F), sh.down.codes.cpu().numpy(), hs, sh.down.scales.cpu().numpy(), 0, 1, "f32")
        total = part if total is None else total + part
    ref = torch.from_numpy(np.ascontiguousarray(total, np.float32)).to(torch.bfloat16).float()
    return _rel_err(y_host, ref)


def run_tp_breakdown(iters: int):
    """Under torchrun, one rank per GPU: the headline layer (this rank's shard) as a whole and piece by piece, CUDA events
    around `iters` back-to-back calls after 3 warm-up calls, maximum over ranks.  `boundary` = whole layer minus the same
    layer without its row-parallel boundary; `down_scatter_local` is the scatter GEMM storing into local buffers (the cost
    of the epilogue without NVLink)."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from oxicuda_b200 import _lib as L
    from oxicuda_b200._lib import default_handle, ptr
    from oxicuda_b200.blas import EpilogueOp, gemm_fp8, gemm_fp8_ex
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp, tp_group
    rank, world, lr = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    h = DistInferHandle(rank, ParallelismConfig(tp=world))
    iters = max(iters, 10)

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t.item()) * 1e3, 1)

    F = FFN // world
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    mk = lambda r, c: torch.randn(r, c, device=dev, generator=gen) * 0.01
    mlp = TpFp8Mlp.from_shards(mk(F, HIDDEN), mk(F, HIDDEN), mk(HIDDEN, F), h)
    x = torch.randn(TOKENS, HIDDEN, device=dev).to(torch.bfloat16)
    y = torch.empty_like(x)
    out = {"tp": world, "unit": "us", "layer": timeit(lambda: mlp.forward(x, out=y)), "layer_without_boundary": timeit(lambda: mlp.forward_partial(x))}
    out["boundary"] = round(out["layer"] - out["layer_without_boundary"], 1)
    codec = mlp.codec
    xc, xs = codec.quantize_rows(x, TOKENS, HIDDEN)
    hd = default_handle()
    # the quantizers through the C ABI into preallocated outputs: the host mirror's two allocations per call cost more than
    # these kernels take
    out["quantize_x"] = timeit(lambda: hd.call("b2q_fp8_quantize_rows_bf16", ptr(x), TOKENS, HIDDEN, L.FP8_E4M3, codec.rounding, ptr(xs), ptr(xc)))
    hb = torch.empty(TOKENS, F, dtype=torch.bfloat16, device=dev)
    out["gate_up_gemm_with_swiglu"] = timeit(lambda: gemm_fp8_ex(xc.view(TOKENS, HIDDEN), mlp.gu_codes, xs, mlp.gu_scales, out=hb, epilogue=EpilogueOp.SwiGluPairs))
    hc, hs = codec.quantize_rows(hb, TOKENS, F)
    out["quantize_h"] = timeit(lambda: hd.call("b2q_fp8_quantize_rows_bf16", ptr(hb), TOKENS, F, L.FP8_E4M3, codec.rounding, ptr(hs), ptr(hc)))
    yd = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev)
    out["down_gemm"] = timeit(lambda: gemm_fp8(hc.view(TOKENS, F), mlp.down.codes, hs, mlp.down.scales, out=yd))
    if world > 1:
        rows = TOKENS // world
        local = [torch.empty(world, rows, HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        lp = (C.c_void_p * world)(*[t.data_ptr() for t in local])
        out["down_scatter_local"] = timeit(lambda: hd.call("b2q_gemm_fp8_scatter", ptr(hc), ptr(mlp.down.codes), TOKENS, HIDDEN, F, L.FP8_E4M3, ptr(hs),
                                                           ptr(mlp.down.scales), None, lp, world, rank))
        nvlink_bytes = 2 * (world - 1) / world * TOKENS * HIDDEN * 2        # per rank and direction: scatter + gather
        out["nvlink_bytes_per_rank"] = int(nvlink_bytes)
        out["boundary_floor_us_at_770GBs"] = round(nvlink_bytes / 770e9 * 1e6, 1)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        tp_group(h).close()
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
    if kind in ("gemm_fp8", "gemm_fp8_rows"):      # gemm_fp8: per-tensor scales; gemm_fp8_rows: per-token and per-output-row scales
        m, n, k = d
        codec = Fp8Codec.e4m3("rne")
        rows = kind == "gemm_fp8_rows"
        ac, sa = codec.quantize_rows(torch.randn(m, k, device=dev), m if rows else 1, k if rows else m * k)
        wc, sw = codec.quantize_rows(torch.randn(n, k, device=dev) * 0.02, n if rows else 1, k if rows else n * k)
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
    elif kind == "fp8_quant_rows":  # fp8_quant_rows:rows:cols:bf16  (per-row absmax / 448 scales, RNE)
        rows, cols, bf16 = d
        x = torch.randn(rows, cols, device=dev)
        x = x.to(torch.bfloat16) if bf16 else x
        codec = Fp8Codec.e4m3("rne")
        fn = lambda: codec.quantize_rows(x, rows, cols)
        work, unit = (rows * cols * (x.element_size() + 1) + 4 * rows) / 1e9, "GB/s"
    elif kind == "swiglu_quant":    # swiglu_quant:rows:ffn  (silu(gate) * up over a [rows x 2 ffn] bf16 GEMM result, per-row E4M3)
        from oxicuda_b200._lib import default_handle, ptr
        import oxicuda_b200._lib as L
        rows, ffn = d
        gu = torch.randn(rows, 2 * ffn, device=dev).to(torch.bfloat16)
        hc = torch.empty(rows, ffn, dtype=torch.uint8, device=dev)
        hs = torch.empty(rows, device=dev)
        fn = lambda: default_handle().call("b2q_swiglu_quantize_rows_bf16", ptr(gu), ptr(gu[:, ffn:]), rows, ffn, 2 * ffn, L.FP8_E4M3, L.ROUND_RNE,
                                           ptr(hs), ptr(hc))
        work, unit = (rows * ffn * 5 + 4 * rows) / 1e9, "GB/s"
    elif kind == "gemm_fp4_bs":     # gemm_fp4_bs:tokens:N:K:mxfp8  (block-scaled FP4 prefill GEMM; mxfp8 = 1: W4A8, 0: split activations)
        from oxicuda_b200.blas import gemm_fp4_blockscaled
        tokens, n, k, mx = d
        codes, scales = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0)).quantize_fp4(torch.randn(n * k, device=dev) * 0.02)
        x = torch.randn(tokens, k, device=dev).to(torch.bfloat16)
        out = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: gemm_fp4_blockscaled(codes, scales, x, n, k, mxfp8_activations=bool(mx), out=out)
        work, unit = 2.0 * tokens * n * k / 1e12, "TFLOP/s"
    elif kind == "grouped_fp8":     # grouped_fp8:experts:rows_each:N:K  (one launch over a device table)
        from oxicuda_b200._lib import default_handle, ptr
        import oxicuda_b200._lib as L
        experts, rows_each, n, k = d
        pad = (rows_each + 255) // 256 * 256
        cap = experts * pad
        a = torch.randint(0, 120, (cap, k), dtype=torch.uint8, device=dev)
        w = torch.randint(0, 120, (experts * n, k), dtype=torch.uint8, device=dev)
        sa, sw = torch.ones(cap, device=dev), torch.ones(experts * n, device=dev)
        off = (torch.arange(experts, device=dev, dtype=torch.int32) * pad).contiguous()
        cnt = torch.full((experts,), rows_each, dtype=torch.int32, device=dev)
        out = torch.empty(cap, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: default_handle().call("b2q_grouped_gemm_fp8_rows", ptr(a), ptr(sa), ptr(w), ptr(sw), ptr(off), ptr(cnt), experts, cap, n, k,
                                           L.FP8_E4M3, ptr(out), L.OUT_BF16)
        work, unit = 2.0 * experts * rows_each * n * k / 1e12, "TFLOP/s"
    elif kind in ("wq_gemv", "wq_dequant"):   # wq_gemv:rows:cols:group:bits:split_k | wq_dequant:rows:cols:group:bits:bf16  (GPTQ / AWQ packed weights)
        from oxicuda_b200._lib import default_handle, ptr
        import oxicuda_b200._lib as L
        rows, cols, group, bits, last = d
        words = rows * cols // (32 // bits)
        packed = torch.randint(-2**31, 2**31 - 1, (words,), dtype=torch.int32, device=dev)
        scales = torch.rand(rows * cols // group, device=dev) * 0.01
        if kind == "wq_gemv":
            x, y = torch.randn(cols, device=dev), torch.empty(rows, device=dev)
            fn = lambda: default_handle().call("b2q_fused_dequant_gemv_f32", ptr(packed), ptr(scales), None, ptr(x), rows, cols, group, bits, last, ptr(y))
            work = (4 * words + 4 * rows * cols // group + 4 * cols + 4 * rows) / 1e9
        else:
            out = torch.empty(rows, cols, dtype=torch.bfloat16 if last else torch.float32, device=dev)
            fn = lambda: default_handle().call("b2q_wq_dequantize", ptr(packed), ptr(scales), None, rows, cols, group, bits, ptr(out),
                                               L.OUT_BF16 if last else L.OUT_F32)
            work = (4 * words + 4 * rows * cols // group + rows * cols * out.element_size()) / 1e9
        unit = "GB/s"
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


def _launches_per_step(boundary, chunks_override):
    mode, chunks = boundary["mode"], max(1, chunks_override or boundary["chunks"])
    if mode == 4:
        return 3 + 2 * chunks
    if mode == 3:
        return 1 + 3 * chunks          # token chunks repeat the two GEMMs and the quantizer
    return 4


def side_measurements(dev, peaks):
    """Rank 0 only.  Returns (roofline fields, extras): the decode GEMV in HBM GB/s on the four Llama-3-8B-shaped
    projections (the other half of the metric), the single FP8 / INT8 GEMM of 4096^3 with a library ceiling beside it,
    the few-token FP8 GEMM and the INT8 W8A8 linear."""
    import torch
    from oxicuda_b200.blas import MicroScalingConfig, MicroScalingQuantizer, ScalingFormat, gemm_fp8, gemm_i8, gemv_fp4_wo
    from oxicuda_b200.quant import Fp8Codec, LlmInt8Config, LlmInt8Quantizer
    roof, res = {}, {}
    hbm = peaks["hbm_gbs"]
    # ---- FP4 (E2M1, E8M0 block scales) weight-only decode GEMV ----
    gv = {"timing": "CUDA-graph replay of back-to-back launches over rotating weight copies (> L2); [us, GB/s of algorithmic bytes, fraction of the measured HBM copy peak]"}
    msq = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0))
    for (Kd, Nd) in ((4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (8192, 28672)):
        copies = max(4, int(300e6 // (Nd * Kd // 2)) + 1)         # rotate weight copies: > 126 MB L2 in total
        ws = []
        for c in range(copies):
            w = torch.randn(Nd * Kd, device=dev) * 0.02
            ws.append(msq.quantize_fp4(w))
            del w
        row = {}
        for tokens in (1, 4, 16, 32):
            x = torch.randn(tokens, Kd, device=dev).to(torch.bfloat16)
            out = torch.empty(tokens, Nd, dtype=torch.bfloat16, device=dev)
            call = lambda i: gemv_fp4_wo(ws[i % copies][0], ws[i % copies][1], x, Nd, Kd, out=out)
            try:
                sec = _time_graph(call, 4 * copies)
            except Exception as exc:
                row[f"m{tokens}"] = repr(exc)
                continue
            nbytes = Nd * Kd // 2 + Nd * Kd // 32 + 2 * tokens * Kd + 2 * tokens * Nd
            row[f"m{tokens}"] = [round(sec * 1e6, 2), round(nbytes / sec / 1e9, 1), round(nbytes / sec / 1e9 / hbm, 3)]
        gv[f"k{Kd}_n{Nd}"] = row
        del ws
    roof["gemv_fp4"] = gv

    # ---- single GEMM, 4096^3: FP8 (burst and a >= 1 s sustained loop), INT8, and a library ceiling ----
    codec = Fp8Codec.e4m3("rne")
    M = N = K = 4096
    sets = []
    for _ in range(4):                                             # 4 x 64 MiB operand sets > L2
        ac, sa = codec.quantize_rows(torch.randn(M, K, device=dev), 1, M * K)
        wc, sw = codec.quantize_rows(torch.randn(N, K, device=dev) * 0.02, 1, N * K)
        sets.append((ac.view(M, K), wc.view(N, K), sa, sw, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
    call = lambda i: gemm_fp8(sets[i % 4][0], sets[i % 4][1], sets[i % 4][2], sets[i % 4][3], out=sets[i % 4][4])
    flop = 2.0 * M * N * K
    sec = _time_calls(call, 20, 5)
    iters = max(200, int(1.2 / sec))
    sec_sus = _time_calls(call, iters, 5)
    g48 = {"us_burst20": round(sec * 1e6, 2), "tflops_burst20": round(flop / sec / 1e12, 1),
           "us_sustained": round(sec_sus * 1e6, 2), "tflops_sustained": round(flop / sec_sus / 1e12, 1), "sustained_iters": iters,
           "frac_of_2x_bf16_burst": round(flop / sec / 1e12 / (2 * peaks["bf16_tflops"]), 3),
           "frac_of_2x_bf16_sustained": round(flop / sec_sus / 1e12 / (2 * peaks["bf16_tflops_sustained"]), 3),
           "frac_of_nominal_4500": round(flop / sec / 1e12 / 4500.0, 3)}
    try:                                                           # a library FP8 GEMM on the same box, as a ceiling only
        a8 = [torch.randn(M, K, device=dev).to(torch.float8_e4m3fn) for _ in range(4)]
        b8 = [torch.randn(N, K, device=dev).to(torch.float8_e4m3fn) for _ in range(4)]
        one = torch.ones((), device=dev)
        lib_call = lambda i: torch._scaled_mm(a8[i % 4], b8[i % 4].t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        lsec = _time_calls(lib_call, 20, 5)
        lsec_sus = _time_calls(lib_call, iters, 5)
        g48["library_ceiling"] = {"what": "torch._scaled_mm (cuBLASLt) on the same operands' shapes, never on the product path",
                                  "tflops_burst20": round(flop / lsec / 1e12, 1), "tflops_sustained": round(flop / lsec_sus / 1e12, 1)}
        g48["frac_of_library_burst"] = round(lsec / sec, 3)
        g48["frac_of_library_sustained"] = round(lsec_sus / sec_sus, 3)
        del a8, b8
    except Exception as exc:                                       # noqa: BLE001
        g48["library_ceiling"] = {"error": repr(exc)}
    roof["gemm_fp8_4096"] = g48
    del sets
    ia = [torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev) for _ in range(4)]
    ib = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(4)]
    ic = torch.empty(M, N, dtype=torch.int32, device=dev)
    try:
        from oxicuda_b200._lib import default_handle, ptr
        hnd = default_handle()
        isec = _time_calls(lambda i: hnd.call("b2q_gemm_i8", ptr(ia[i % 4]), ptr(ib[i % 4]), M, N, K, ptr(ic), None, None, None), 20, 5)
        roof["gemm_i8_4096"] = {"us": round(isec * 1e6, 2), "tops": round(flop / isec / 1e12, 1), "out": "s32"}
    except Exception as exc:                                       # noqa: BLE001
        roof["gemm_i8_4096"] = {"error": repr(exc)}
    del ia, ib, ic

    # ---- block-scaled FP4 prefill GEMM (E2M1 weights, E8M0 block scales) on tcgen05 kind::mxf8f6f4.block_scale ----
    try:
        from oxicuda_b200.blas import gemm_fp4_blockscaled
        tk, Nd, Kd = 4096, 8192, 8192
        wsets = [msq.quantize_fp4(torch.randn(Nd * Kd, device=dev) * 0.02) for _ in range(4)]      # 4 x 36 MB of codes and scales
        xs4 = [torch.randn(tk, Kd, device=dev).to(torch.bfloat16) for _ in range(4)]
        o4 = torch.empty(tk, Nd, dtype=torch.bfloat16, device=dev)
        fl4 = 2.0 * tk * Nd * Kd
        row = {"shape": "4096 tokens x N 8192 x K 8192, bf16 activations in, bf16 out; the time includes the activation quantization pre-pass"}
        for name, mx in (("w4a8_mx_e4m3_activations", True), ("weight_only_split_activations", False)):
            sec4 = _time_calls(lambda i: gemm_fp4_blockscaled(wsets[i % 4][0], wsets[i % 4][1], xs4[i % 4], Nd, Kd, mxfp8_activations=mx, out=o4), 20, 5)
            row[name] = {"us": round(sec4 * 1e6, 1), "tflops": round(fl4 / sec4 / 1e12, 1),
                         "frac_of_2x_bf16_burst": round(fl4 / sec4 / 1e12 / (2 * peaks["bf16_tflops"]), 3)}
        roof["gemm_fp4_blockscaled"] = row
        del wsets, xs4, o4
    except Exception as exc:                                       # noqa: BLE001
        roof["gemm_fp4_blockscaled"] = {"error": repr(exc)}

    # ---- grouped FP8 MoE layer, Mixtral-shaped (8 experts 4096 -> 14336 -> 4096, top-2 over 4096 tokens), one GPU ----
    try:
        from oxicuda_b200.dist_infer import DistInferHandle, MoeFp8Layer, ParallelismConfig
        E, hid, ffn_e, tk, topk = 8, 4096, 14336, 4096, 2
        gen = torch.Generator(device=dev).manual_seed(0xB2000005)
        experts = [(torch.randn(ffn_e, hid, device=dev, generator=gen) * 0.02, torch.randn(ffn_e, hid, device=dev, generator=gen) * 0.02,
                    torch.randn(hid, ffn_e, device=dev, generator=gen) * 0.02) for _ in range(E)]
        layer = MoeFp8Layer(experts, E, topk, DistInferHandle(0, ParallelismConfig(ep=1)))
        del experts
        # expert popularity ~ Dirichlet(1): logits = log p + Gumbel noise draws experts in proportion to p
        p = torch.distributions.Dirichlet(torch.ones(E)).sample().to(dev)
        lg = (p.log()[None, :] - torch.log(-torch.log(torch.rand(tk, E, device=dev, generator=gen)))).float().contiguous()
        xm = torch.randn(tk, hid, device=dev, generator=gen).to(torch.bfloat16)
        ym = torch.empty_like(xm)
        secm = _time_calls(lambda i: layer.forward(xm, lg, out=ym), 10, 3)
        flm = 2.0 * tk * topk * 3 * hid * ffn_e
        roof["moe_fp8_mixtral"] = {"experts": E, "top_k": topk, "tokens": tk, "hidden": hid, "ffn": ffn_e, "us": round(secm * 1e6, 1),
                                   "tflops": round(flm / secm / 1e12, 1), "rows_per_expert": [int(v) for v in layer.last_counts.tolist()],
                                   "launches_per_call": "route, slot, scatter, quantize, ONE grouped gate|up GEMM, SwiGLU + quantize, ONE grouped down GEMM, gather",
                                   "frac_of_2x_bf16_sustained": round(flm / secm / 1e12 / (2 * peaks["bf16_tflops_sustained"]), 3)}
        del layer
        # the same layer over block-scaled FP4 experts (E2M1, E8M0 per 32), W4A8 activations
        from oxicuda_b200.dist_infer import MoeFp4Layer
        gen = torch.Generator(device=dev).manual_seed(0xB2000005)
        experts = [(torch.randn(ffn_e, hid, device=dev, generator=gen) * 0.02, torch.randn(ffn_e, hid, device=dev, generator=gen) * 0.02,
                    torch.randn(hid, ffn_e, device=dev, generator=gen) * 0.02) for _ in range(E)]
        layer4 = MoeFp4Layer(experts, E, topk, DistInferHandle(0, ParallelismConfig(ep=1)))
        del experts
        sec4 = _time_calls(lambda i: layer4.forward(xm, lg, out=ym), 10, 3)
        roof["moe_fp4_mixtral"] = {"us": round(sec4 * 1e6, 1), "tflops": round(flm / sec4 / 1e12, 1), "activations": "MX E4M3 per 32 (W4A8)",
                                   "weight_bytes": int(E * 3 * hid * ffn_e * (0.5 + 1 / 32)),
                                   "frac_of_2x_bf16_sustained": round(flm / sec4 / 1e12 / (2 * peaks["bf16_tflops_sustained"]), 3)}
        del layer4, xm, ym, lg
    except Exception as exc:                                       # noqa: BLE001
        roof.setdefault("moe_fp8_mixtral", {"error": repr(exc)})
        roof.setdefault("moe_fp4_mixtral", {"error": repr(exc)})
    torch.cuda.empty_cache()

    # ---- GPTQ / AWQ fused dequant GEMV (4-bit codes, f32 scales per 128) on the same 8192 -> 28672 projection ----
    try:
        from oxicuda_b200._lib import default_handle, ptr
        rows_q, cols_q, grp_q = 28672, 8192, 128
        qsets = [(torch.randint(-2**31, 2**31 - 1, (rows_q * cols_q // 8,), dtype=torch.int32, device=dev),
                  torch.rand(rows_q * cols_q // grp_q, device=dev) * 0.01) for _ in range(3)]      # 3 x 125 MB > L2
        xq, yq = torch.randn(cols_q, device=dev), torch.empty(rows_q, device=dev)
        hq = default_handle()
        qbytes = rows_q * cols_q // 2 + 4 * rows_q * cols_q // grp_q + 4 * cols_q + 4 * rows_q
        ent = {"rows": rows_q, "cols": cols_q, "bits": 4, "group": grp_q, "bytes": qbytes,
               "timing": "CUDA events over back-to-back calls on rotating weight copies; [us, GB/s, fraction of the measured HBM peak]"}
        for name, split in (("reference_order", 1), ("split_columns", 0)):
            secq = _time_calls(lambda i: hq.call("b2q_fused_dequant_gemv_f32", ptr(qsets[i % 3][0]), ptr(qsets[i % 3][1]), None, ptr(xq), rows_q,
                                                 cols_q, grp_q, 4, split, ptr(yq)), 12, 3)
            ent[name] = [round(secq * 1e6, 1), round(qbytes / secq / 1e9, 1), round(qbytes / secq / 1e9 / hbm, 3)]
        roof["gptq_awq_gemv"] = ent
        del qsets, xq, yq
    except Exception as exc:                                       # noqa: BLE001
        roof["gptq_awq_gemv"] = {"error": repr(exc)}

    # ---- FP8 W8A8 with few tokens on the 70B-shaped FFN projection: HBM-bound ----
    Kd, Nd = 8192, 28672
    fw = []
    for c in range(3):                                             # 3 x 235 MB > L2
        wc, sw = codec.quantize_rows(torch.randn(Nd, Kd, device=dev) * 0.02, Nd, Kd)
        fw.append((wc.view(Nd, Kd), sw))
    few = {"timing": "CUDA-graph replay; [us, GB/s, fraction of the measured HBM peak]"}
    for tokens in (1, 16, 32, 48, 64):
        ac, sa = codec.quantize_rows(torch.randn(tokens, Kd, device=dev), tokens, Kd)
        ac = ac.view(tokens, Kd)
        out = torch.empty(tokens, Nd, dtype=torch.bfloat16, device=dev)
        call = lambda i: gemm_fp8(ac, fw[i % 3][0], sa, fw[i % 3][1], out=out)
        try:
            sec = _time_graph(call, 12)
        except Exception as exc:
            few[f"m{tokens}"] = repr(exc)
            continue
        nbytes = Nd * Kd + tokens * Kd + 2 * tokens * Nd
        few[f"m{tokens}"] = [round(sec * 1e6, 2), round(nbytes / sec / 1e9, 1), round(nbytes / sec / 1e9 / hbm, 3)]
    res["gemm_fp8_few_tokens_k8192_n28672"] = few
    del fw
    x = torch.randn(8, 1024, device=dev)
    w = torch.randn(1024, 1024, device=dev) * 0.02
    q = LlmInt8Quantizer(LlmInt8Config(1e30, True))
    sec = _time_calls(lambda i: q.matmul(x, w, 8, 1024, 1024), 50, 5)
    res["int8_w8a8_linear_8x1024x1024"] = {"us": round(sec * 1e6, 2), "note": "quantizes W and X on every call, as the reference entry point does"}
    return roof, res


if __name__ == "__main__":
    main()
