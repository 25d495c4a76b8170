#!/usr/bin/env python
"""Benchmark of the grouped-affine (gaf4_64) decode GEMV path on B200.

    python bench.py --gpus 1 --steps K --warmup W            # this repo's CUDA path
    python bench.py --impl reference --gpus 1 ...             # the CPU path (oracle port) on the host cores
    torchrun ... bench.py --gpus N ...                        # N > 1: one rank per GPU

Workloads (synthetic, seeded; shapes from the reference's model families):
  * N = 1  `llama3_8b_ffn`: a stack of distinct Llama-3-8B FFN layers in gaf4_64
    (gate|up [2 x 14336, 4096] issued as one fused launch, down [4096, 14336]),
    bf16 activations, M = 1 (also timed at M = 4 and 16).  A step is one pass over
    the whole stack; the stack (1.19 GB) is several times the 126 MB L2, so every
    weight byte comes from HBM.
  * N > 1  `llama3_70b_stack`: Llama-3-70B-shaped decoder-layer linears (qkv, o,
    gate|up, down) in gaf4_64, column- / row-sharded over the ranks, NCCL allreduce
    on the row-parallel outputs; strong scaling (total work fixed).

One JSON line on stdout (rank 0).  `value` is GB/s of algorithmic bytes (packed
codes + scales + biases + activations in + out, each once per launch).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gaf4_64 decode GEMV HBM GB/s"
GROUP, BITS = 64, 4
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the step's two launch shapes
# (gate|up 78,993,664 + 2,137,856 B; down 47,757,056 + 12,544 B), from the ncu capture summarised in
# profiles/gemv_dp4a_llama8b_ffn_m1.md.  Each launch's reads include ~10.9 MB of next-weight L2 prefetch
# (2 units x 148 CTAs); ncu flushes the caches between kernels, so under ncu those bytes are read again by
# the next launch, while in a back-to-back run they replace the same bytes of that launch.
NCU_TRAFFIC_PER_LAUNCH = (78_993_664 + 2_137_856 + 47_757_056 + 12_544) // 2


def measured_peak_hbm():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def weight_bytes(N, K, group=GROUP, bits=BITS):
    return N * K * bits // 8 + 2 * N * (K // group) * 2


def launch_bytes(N, K, M):
    return weight_bytes(N, K) + M * K * 2 + M * N * 2


def synth_weight(rng, N, K):
    """Random codes with realistic scale / bias magnitudes.  Timing does not depend on the
    values; parity on converter-made weights is the job of tests/."""
    packed = rng.integers(0, 2 ** 32, size=(N, K * BITS // 32), dtype=np.uint32)
    scales = (np.full((N, K // GROUP), 0.0053, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    biases = (np.full((N, K // GROUP), -0.04, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return packed, scales, biases


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self._nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------- CPU arm
def cpu_path(sample_seconds: float, threads: int, N: int = 14336, K: int = 4096):
    """Times the CPU restatement of the reference's gaf4_64 matmul (oracle port) on one
    matrix [N, K] (default: an 8B gate matrix), M = 1, f32 activations, for about sample_seconds."""
    from oracle import gaf_oracle as oracle
    oracle.build()
    rng = np.random.default_rng(0)
    packed, scales, biases = synth_weight(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    oracle.matmul_f32(x, packed, scales, biases, GROUP, BITS, nthreads=threads)  # warm the pool and the caches
    t0, n = time.perf_counter(), 0
    while True:
        oracle.matmul_f32(x, packed, scales, biases, GROUP, BITS, nthreads=threads)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= sample_seconds or n >= 2000:
            break
    per_call = dt / n
    gbs = launch_bytes(N, K, 1) / per_call / 1e9
    return gbs, per_call, n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import gaf_oracle as oracle
    oracle.build()
    cores = oracle.logical_cpu_count()
    # each step is a bounded sample of the workload of the matching arm: one 8B gate matrix at N = 1, one
    # 70B o-projection matrix when the arm runs the 70B stack (N > 1); M = 1
    multi = args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1
    N, K = (8192, 8192) if multi else (14336, 4096)
    workload = "llama3_70b_stack" if multi else "llama3_8b_ffn"
    per_step = max(0.2, min(2.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_path(per_step, cores, N, K)
    vals, t_per = [], []
    for _ in range(args.steps):
        g, per_call, _ = cpu_path(per_step, cores, N, K)
        vals.append(g)
        t_per.append(per_call)
    value = float(np.mean(vals))
    sample = f"one matrix [{N} x {K}] gaf4_64 of the workload, M=1, f32 activations, repeated; C port of the reference CPU kernels (oracle/), the Zig reference cannot be built here"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(float(np.mean(t_per)) * 1e3, 4),
        "higher_is_better": True, "scaling": "strong" if multi else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "scheme": "gaf4_64", "M": 1},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------- GPU arm
def time_graph(ctx, torch, stream, launch_step, steps, warmup):
    """Captures one step into a CUDA graph on `stream`, replays it, returns ms per step."""
    with torch.cuda.stream(stream):
        launch_step()  # sizes the library's scratch before capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            launch_step()
        for _ in range(max(3, warmup)):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ctx.synchronize()
    return e0.elapsed_time(e1) / steps


def measured_peak_tflops():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return float(j["bf16_tflops"]), float(j["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


def time_prefill(gaf, ctx, torch, stream, rng, iters=20):
    """gaf4_64 prefill dequant-GEMM: x bf16 [2048, 4096], W [14336, 4096] (tcgen05 path).
    TFLOP/s = 2*M*N*K / time; the dequant work is not counted."""
    M, K, N = 2048, 4096, 14336
    ws = [gaf.Weight.from_host(ctx, *synth_weight(rng, N, K), GROUP, BITS) for _ in range(2)]
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    with torch.cuda.stream(stream):
        for _ in range(3):
            for w in ws:
                gaf.linear(ctx, w, x, out=y)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            for w in ws:
                gaf.linear(ctx, w, x, out=y)
        e1.record(stream)
        stream.synchronize()
    ctx.synchronize()
    ms = e0.elapsed_time(e1) / (iters * len(ws))
    tf = 2.0 * M * N * K / ms / 1e9
    burst, sustained, kind = measured_peak_tflops()
    for w in ws:
        w.free()
    return {"workload": "gaf4_64 prefill M=2048 K=4096 N=14336", "tflops": round(tf, 1), "ms": round(ms, 4),
            "frac_of_burst_peak": round(tf / burst, 4), "frac_of_sustained_peak": round(tf / sustained, 4),
            "peak_tflops": {"burst": burst, "sustained": sustained, "kind": f"of {kind}"},
            "bound": "tensor"}


def run_single(args):
    import torch
    import talu_b200 as gaf

    dev = 0
    torch.cuda.set_device(dev)
    stream = torch.cuda.Stream()
    ctx = gaf.Context(dev, stream=stream.cuda_stream)
    rng = np.random.default_rng(0)
    layers = args.layers
    shapes = [("gate_up", 2 * 14336, 4096), ("down", 4096, 14336)]
    weights = []
    for _ in range(layers):
        for name, N, K in shapes:
            p, s, b = synth_weight(rng, N, K)
            weights.append((name, gaf.Weight.from_host(ctx, p, s, b, GROUP, BITS)))
    ring_bytes = sum(weight_bytes(w.N, w.K) for _, w in weights)

    def make_io(M, pinned=False):
        xs = {K: torch.randn((M, K), device="cuda").to(torch.bfloat16) for K in (4096, 14336)}
        ys = [torch.empty((M, w.N), dtype=torch.bfloat16, device="cuda") for _, w in weights]
        return xs, ys

    if args.quick and args.case == "prefill":
        print(json.dumps({"quick": True, "prefill": time_prefill(gaf, ctx, torch, stream, rng, iters=2)}))
        return
    if args.quick and args.case == "stack70b":
        from talu_b200 import tp_bench
        ms, nbytes, *_ = tp_bench.measure(args, existing_ctx=ctx, existing_stream=stream, M=args.m)
        print(json.dumps({"quick": True, "workload": "llama3_70b_stack", "M": args.m, "layers": args.layers,
                          "ms_per_step": ms, "gbs": round(nbytes / ms / 1e6, 2)}))
        return
    results = {}
    clocks = ClockSampler(dev)
    with clocks:
        for M in ((args.m,) if args.quick else (1, 2, 4, 8, 16)):
            xs, ys = make_io(M)

            def step():
                # a decoder knows its layer order: each call names the weight the following call streams
                for i, ((_, w), y) in enumerate(zip(weights, ys)):
                    gaf.hint_next_weight(ctx, weights[(i + 1) % len(weights)][1])
                    gaf.linear(ctx, w, xs[w.K], out=y)

            ms = time_graph(ctx, torch, stream, step, args.steps, args.warmup)
            nbytes = sum(launch_bytes(w.N, w.K, M) for _, w in weights)
            results[M] = {"ms_per_step": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes}

        if args.quick:
            print(json.dumps({"quick": True, "M": args.m, f"M{args.m}_gbs": round(results[args.m]["gbs"], 2),
                              "ms_per_step": results[args.m]["ms_per_step"]}))
            return
        # ---- end to end through the C ABI with host buffers (pinned), M = 1 ----
        M = 1
        hx = {K: torch.randn((M, K)).to(torch.bfloat16).pin_memory() for K in (4096, 14336)}
        hy = [torch.empty((M, w.N), dtype=torch.bfloat16).pin_memory() for _, w in weights]
        hx_np = {K: v.view(torch.int16).numpy().view(np.uint16) for K, v in hx.items()}
        hy_np = [v.view(torch.int16).numpy().view(np.uint16) for v in hy]

        batch = gaf.HostBatch(ctx, [w for _, w in weights], [hx_np[w.K] for _, w in weights], hy_np)
        e2e_mode = "tgaf_host_batch_submit (the list recorded once as a CUDA graph)"
        try:
            batch.record()
        except gaf.GafError as exc:   # the queued form without the graph measures the same path, a little slower
            e2e_mode = f"tgaf_linear_bf16_host_async_batch (recording failed: {exc})"

        def e2e_step():
            # per launch: H2D copy of x from page-locked memory, kernel, D2H copy of y; one submit and one wait per step
            batch.submit()
            ctx.synchronize()

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(e2e_steps):
                e2e_step()
            e1.record(stream)
            stream.synchronize()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d = sum(M * w.K * 2 for _, w in weights)
    d2h = sum(M * w.N * 2 for _, w in weights)
    e2e_gbs = results[1]["bytes"] / e2e_ms / 1e6

    prefill = time_prefill(gaf, ctx, torch, stream, rng)
    # the multi-GPU workload on this one GPU, so that the N > 1 lines have their N = 1 reference
    from talu_b200 import tp_bench
    st_ms, st_bytes, st_launches, st_layers, *_ = tp_bench.measure(args, existing_ctx=ctx, existing_stream=stream)
    stack70b = {"workload": "llama3_70b_stack", "layers": st_layers, "ms_per_step": round(st_ms, 5),
                "gbs": round(st_bytes / st_ms / 1e6, 2), "launches_per_step": st_launches}
    # the skinny case of the same stack (64 activation rows: the tcgen05 GEMM with one 128-row half), HBM-bound
    # by its roofline, limited here by the rate at which the dequant warps produce the bf16 operand
    sk_ms, sk_bytes, *_ = tp_bench.measure(args, existing_ctx=ctx, existing_stream=stream, M=64)
    stack70b["m64"] = {"ms_per_step": round(sk_ms, 5), "gbs": round(sk_bytes / sk_ms / 1e6, 2)}

    peak, peak_kind = measured_peak_hbm()
    launches_per_step = len(weights)
    avg_launch_ms = results[1]["ms_per_step"] / launches_per_step
    achieved = results[1]["bytes"] / launches_per_step / avg_launch_ms / 1e6
    cores = os.cpu_count() or 1
    cpu_gbs, cpu_per_call, cpu_n = cpu_path(args.cpu_seconds, cores)

    out = {
        "metric": METRIC, "value": round(results[1]["gbs"], 2), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(results[1]["ms_per_step"], 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama3_8b_ffn", "scheme": "gaf4_64", "M": 1, "layers": layers,
                   "launches_per_step": launches_per_step, "gate_up_fused": True,
                   "l2": f"distinct weights per launch, ring {ring_bytes / 1e9:.2f} GB > 126 MB L2 (no flush needed)",
                   "timing": "CUDA graph replay, CUDA events on the launching stream"},
        "decode": {f"M{m}": {"gbs": round(r["gbs"], 2), "ms_per_step": round(r["ms_per_step"], 5),
                             "frac_of_measured_hbm": round(r["gbs"] / peak, 4),
                             "frac_of_nominal_8TBs": round(r["gbs"] / NOMINAL_HBM_GBS, 4)} for m, r in results.items()},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                     "traffic": NCU_TRAFFIC_PER_LAUNCH,
                     "traffic_note": "ncu dram bytes per launch, mean of the step's two shapes (algorithmic mean 49.6 MB; 10.9 MB of it is the next launch's head, prefetched to L2 and counted twice under ncu's cache flush)"},
        "cpu_baseline": {"value": round(cpu_gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{cpu_n} calls of one gate-shaped matrix [14336 x 4096], M=1, f32 activations ({cpu_per_call * 1e3:.2f} ms each)"},
        "e2e": {"value": round(e2e_gbs, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms, 4), "note": e2e_mode + " + tgaf_synchronize per step: per launch pinned host x -> device, kernel, y -> pinned host, copies on their own streams"},
        "prefill": prefill,
        "llama3_70b_stack_1gpu": stack70b,
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=12, help="distinct FFN layers in the weight ring")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="length of the CPU-baseline sample")
    ap.add_argument("--case", default="decode", choices=["decode", "prefill", "stack70b"],
                    help="with --quick: which kernel the small case runs")
    ap.add_argument("--m", type=int, default=1, help="activation rows of the --quick decode / stack70b case")
    ap.add_argument("--quick", action="store_true",
                    help="M = 1 only, no end-to-end and no CPU leg (small case for profilers; not a bench value)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        from talu_b200 import tp_bench
        tp_bench.run(args)
        return
    run_single(args)


if __name__ == "__main__":
    main()
