#!/usr/bin/env python
"""Benchmark of the grouped-affine (gaf4_64) decode GEMV path on B200.

    python bench.py --gpus 1 --steps K --warmup W            # this repo's CUDA path
    python bench.py --impl reference --gpus 1 ...             # the CPU path (oracle port) on the host cores
    torchrun ... bench.py --gpus N ...                        # N > 1: one rank per GPU

Workloads (synthetic, seeded; shapes from the reference's model families):
  * N = 1  `llama3_8b_ffn`: a stack of distinct Llama-3-8B FFN layers in gaf4_64
    (gate|up [2 x 14336, 4096] stacked, down [4096, 14336]), bf16 activations ~ N(0, 1),
    each GEMV with its own activations, M = 1 (also M = 2, 4, 8, 16).  A step is one pass
    over the whole stack (24 GEMVs, 1.19 GB of weights: several times the 126 MB L2, so
    every weight byte comes from HBM).  The step is submitted as ONE launch list
    (tgaf_batch_run); the same step as 24 separate launches, and as a list in which every
    GEMV waits for its predecessor, is timed beside it.
  * N > 1  `llama3_70b_stack`: Llama-3-70B-shaped decoder-layer linears (qkv, o,
    gate|up, down) in gaf4_64, column- / row-sharded over the ranks, the sum over ranks on
    the row-parallel outputs; strong scaling (total work fixed).

Timing: the step is captured into a CUDA graph and replayed for at least a second; an
event is recorded after every replay, so each case reports min / p50 / p90 / mean of the
per-step times (the reference's harness reports the same four,
core/bench/compute/cpu/harness.zig:8-35).  `ms_per_step` / `value` are the mean of the LAST
K steps of that run (K = --steps), i.e. with the clocks where a long run leaves them.

One JSON line on stdout (rank 0).  `value` is GB/s of algorithmic bytes (packed codes +
scales + biases + activations in + out, each once per GEMV).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gaf4_64 decode GEMV HBM GB/s"
GROUP, BITS = 64, 4
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch list of the --quick case (2 layers = 4 GEMVs,
# 198,377,472 algorithmic bytes), from the ncu capture summarised in profiles/gemv_list_llama8b_ffn_m1.md,
# divided by the four GEMVs of the launch: (198,450,432 read + 4,838,400 written) / 4
NCU_TRAFFIC_PER_GEMV = 50822208


def measured_peak_hbm():
    from talu_b200.peaks import measured_peak_hbm as f
    return f()


def weight_bytes(N, K, group=GROUP, bits=BITS):
    return N * K * bits // 8 + 2 * N * (K // group) * 2


def launch_bytes(N, K, M, group=GROUP, bits=BITS):
    return weight_bytes(N, K, group, bits) + M * K * 2 + M * N * 2


def synth_weight(rng, N, K, group=GROUP, bits=BITS):
    """Random codes with realistic scale / bias magnitudes.  Timing does not depend on the
    values; parity on converter-made weights is the job of tests/ (and of the output check
    below, which runs the timed configuration against the oracle once)."""
    packed = rng.integers(0, 2 ** 32, size=(N, K * bits // 32), dtype=np.uint32)
    scales = (np.full((N, K // group), 0.0053 if bits == 4 else 0.00031, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    biases = (np.full((N, K // group), -0.04, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return packed, scales, biases


def stats_ms(samples):
    a = np.sort(np.asarray(samples, np.float64))
    return {"min": round(float(a[0]), 5), "p50": round(float(np.percentile(a, 50)), 5),
            "p90": round(float(np.percentile(a, 90)), 5), "mean": round(float(a.mean()), 5), "n": int(a.size)}


# --------------------------------------------------------------------------- CPU arm
def cpu_stack(shapes, rng_seed=0):
    """The weights of one step on the host (the same generator and seed as the GPU arm)."""
    rng = np.random.default_rng(rng_seed)
    return [(N, K, *synth_weight(rng, N, K)) for (N, K) in shapes]


def cpu_time_step(oracle, stack, threads, steps, warmup):
    """One step = one pass of the reference CPU matmul (C port) over every matrix of the stack, M = 1, f32
    activations.  Returns per-step seconds."""
    xs = {K: np.random.default_rng(1).standard_normal((1, K), dtype=np.float32) for K in {k for _, k, *_ in stack}}
    out = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for N, K, p, s, b in stack:
            oracle.matmul_f32(xs[K], p, s, b, GROUP, BITS, nthreads=threads)
        if i >= warmup:
            out.append(time.perf_counter() - t0)
    return out


def ffn_shapes(layers):
    return [s for _ in range(layers) for s in ((2 * 14336, 4096), (4096, 14336))]


def stack70b_shapes(layers):
    return [s for _ in range(layers) for s in ((10240, 8192), (8192, 8192), (2 * 28672, 8192), (8192, 28672))]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import gaf_oracle as oracle
    oracle.build()
    logical = oracle.logical_cpu_count()
    policy = oracle.reference_thread_count()
    multi = args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1
    # the same matrices as the GPU arm of the same N: the whole 8B FFN stack (N = 1), the 70B-shaped stack (N > 1)
    layers = 8 if (multi and args.layers == 12) else args.layers
    shapes = stack70b_shapes(layers) if multi else ffn_shapes(layers)
    workload = "llama3_70b_stack" if multi else "llama3_8b_ffn"
    stack = cpu_stack(shapes)
    nbytes = sum(launch_bytes(N, K, 1) for N, K, *_ in stack)
    # keep the whole run within a couple of minutes whatever --steps says
    probe = cpu_time_step(oracle, stack, logical, 1, 1)[0]
    steps = max(1, min(args.steps, int(60.0 / max(probe, 1e-3))))
    warmup = max(1, min(args.warmup, 3))
    t_all = cpu_time_step(oracle, stack, logical, steps, warmup)
    t_pol = cpu_time_step(oracle, stack, policy, max(1, steps // 2), 1)
    value = nbytes / float(np.mean(t_all)) / 1e9
    sample = (f"every matrix of the arm's own stack ({len(stack)} GEMVs, {nbytes / 1e9:.2f} GB per step), M=1, f32 activations; "
              "C port of the reference CPU kernels (oracle/), the Zig reference cannot be built here")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(float(np.mean(t_all)) * 1e3, 4),
        "higher_is_better": True, "scaling": "strong" if multi else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "scheme": "gaf4_64", "M": 1, "layers": layers},
        "stats_ms": stats_ms([t * 1e3 for t in t_all]),
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": logical, "kind": "port", "sample": sample,
                         "reference_thread_policy": {"threads": policy, "value": round(nbytes / float(np.mean(t_pol)) / 1e9, 3),
                                                     "rule": "min(physical, 8 + physical / 4), physical = logical / 2 (core/src/system/parallel.zig:41-50)"}},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------- GPU arm
MIN_SECONDS_SCALE = 1.0   # --min-seconds


def time_graph(ctx, torch, stream, launch_step, steps, warmup, min_seconds=1.0, clocks=None):
    """Captures one step into a CUDA graph on `stream` and replays it for at least `min_seconds` (and at least
    `steps` times), an event after every replay.  Returns (mean ms of the last `steps` replays, stats over all,
    clocks seen)."""
    with torch.cuda.stream(stream):
        launch_step()  # sizes the library's scratch before capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            launch_step()
        for _ in range(max(3, warmup)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(5):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        est = max(e0.elapsed_time(e1) / 5, 1e-3)
        n = int(min(20000, max(steps, min_seconds * MIN_SECONDS_SCALE * 1e3 / est)))
        mark = clocks.mark() if clocks else 0
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        evs[0].record(stream)
        for i in range(n):
            graph.replay()
            evs[i + 1].record(stream)
        stream.synchronize()
    ctx.synchronize()
    samples = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)]
    del graph
    return float(np.mean(samples[-steps:])), stats_ms(samples), (clocks.since(mark) if clocks else None)


def measured_peak_tflops():
    from talu_b200.peaks import measured_peak_tflops as f
    return f()


def time_prefill(gaf, ctx, torch, stream, rng, iters=20, clocks=None):
    """gaf4_64 prefill dequant-GEMM: x bf16 [2048, 4096], W [14336, 4096] (tcgen05 path).
    TFLOP/s = 2*M*N*K / time; the dequant work is not counted."""
    M, K, N = 2048, 4096, 14336
    ws = [gaf.Weight.from_host(ctx, *synth_weight(rng, N, K), GROUP, BITS) for _ in range(2)]
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")

    def step():
        for w in ws:
            gaf.linear(ctx, w, x, out=y)

    ms, st, clk = time_graph(ctx, torch, stream, step, iters, 3, min_seconds=1.0 if iters > 2 else 0.0, clocks=clocks)
    ms /= len(ws)
    tf = 2.0 * M * N * K / ms / 1e9
    burst, sustained, kind = measured_peak_tflops()
    for w in ws:
        w.free()
    return {"workload": "gaf4_64 prefill M=2048 K=4096 N=14336", "tflops": round(tf, 1), "ms": round(ms, 4),
            "frac_of_burst_peak": round(tf / burst, 4), "frac_of_sustained_peak": round(tf / sustained, 4),
            "peak_tflops": {"burst": burst, "sustained": sustained, "kind": f"of {kind}"},
            "stats_ms_per_two_gemms": st, "clocks": clk, "bound": "tensor"}


def check_outputs(gaf, ctx, torch, stream):
    """The timed configuration once on converter-made weights against the CPU oracle: one 8B FFN layer (gate|up and
    down, M = 1) through a launch list and through single calls.  Returns the largest relative error; raises
    when it exceeds 1e-2."""
    from oracle import gaf_oracle as oracle
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import bits_from_torch_bf16, make_weights, make_x_bf16, rel_err, torch_bf16_from_bits
    worst = 0.0
    ws, xs, ys, refs = [], [], [], []
    with torch.cuda.stream(stream):
        for i, (N, K) in enumerate(((2 * 14336, 4096), (4096, 14336))):
            p, s, b = make_weights(oracle, N, K, GROUP, BITS, seed=i)
            xb, xf = make_x_bf16(oracle, 1, K, seed=10 + i)
            ws.append(gaf.Weight.from_host(ctx, p, s, b, GROUP, BITS))
            xs.append(torch_bf16_from_bits(xb, "cuda:0"))
            ys.append(torch.zeros((1, N), dtype=torch.bfloat16, device="cuda"))
            refs.append(oracle.matmul_f32(xf, p, s, b, GROUP, BITS))
        batch = gaf.Batch(ctx, ws, xs, ys)
        batch.run()
        stream.synchronize()
        ctx.synchronize()
        for w, x, y, ref in zip(ws, xs, ys, refs):
            worst = max(worst, rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), ref))
            single = gaf.linear(ctx, w, x)
            stream.synchronize()
            ctx.synchronize()
            worst = max(worst, rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(single)), ref))
        batch.close()
        for w in ws:
            w.free()
    if not worst <= 1e-2:
        raise RuntimeError(f"output check failed: rel {worst}")
    return worst


def time_incumbent_kernel(torch, weights_host, steps=5):
    """The reference's own CUDA kernel (talu_gaffine_u4_matvec_f32, compiled unchanged into oracle/_ref/) on the
    same weights under its own launch geometry, f32 activations: the GPU baseline this path replaces."""
    from oracle import gaf_oracle as oracle
    cubin = oracle.build_ref()
    if cubin is None:
        return None
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import CubinModule, to_dev
    mod = CubinModule(cubin)
    dev = [(N, K, to_dev(p), to_dev(s), to_dev(b)) for (N, K, p, s, b) in weights_host]
    xs = {K: torch.randn((1, K), device="cuda") for K in {k for _, k, *_ in dev}}
    ys = [torch.empty((1, N), device="cuda") for N, *_ in dev]

    def step():
        for (N, K, dp, ds, db), y in zip(dev, ys):
            mod.launch("talu_gaffine_u4_matvec_f32", ((N + 7) // 8, 1), (xs[K], dp, ds, db, y, K, N, GROUP, 1, 1))

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    nbytes = sum(weight_bytes(N, K) + K * 4 + N * 4 for N, K, *_ in dev)
    return {"kernel": "talu_gaffine_u4_matvec_f32 (core/src/compute/cuda/kernels/ops/quant_ops.cu:46-93, compiled unchanged)",
            "ms_per_step": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 2), "gemvs": len(dev),
            "note": "the first two layers of the same stack, f32 activations as its contract requires, block 256 / grid ceil(N / 8)"}


def tp_parity_check(ctx, torch, dist, rank, world, stream):
    """Every rank's output of sharded linears against the UNSHARDED CPU oracle, on converter-made weights (the
    oracle's quantizer): a column-parallel -> row-parallel chain (hidden 1024, ffn 2048; M = 1, 2, 4) and one
    full-size Llama-3-70B `down` shard (8192 x 28672, M = 1), the sum over ranks taken by every path the library
    has.  Raises when any rank is beyond the path's bound (max relative error 1e-2; where every rank's partial
    sums are rounded to bf16 before the sum, 3e-2); returns the worst figure and the paths."""
    import talu_b200 as gaf
    from talu_b200.tp import SHARD_COL, SHARD_ROW
    from oracle import gaf_oracle as oracle
    if rank == 0:
        oracle.build()
    dist.barrier()
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import bits_from_torch_bf16, make_weights, make_x_bf16, rel_err, torch_bf16_from_bits
    peer = ctx.uses_peer_memory()
    paths = [("launch list, sums inside the launch", None),
             ("fused into the GEMV write-out", {"fused_allreduce": 1, "peer_allreduce": 1}),
             ("GEMV then the one-shot peer-memory kernel", {"fused_allreduce": 0, "peer_allreduce": 1}),
             ("GEMV then NCCL all-reduce", {"fused_allreduce": 0, "peer_allreduce": 0})]
    worst, report, failed = 0.0, [], False

    def to_f32(t):
        return oracle.bf16_to_f32(bits_from_torch_bf16(t))

    with torch.cuda.stream(stream):
        # ---- chain ----
        H, F = 1024, 2048
        p1, s1, b1 = make_weights(oracle, F, H, GROUP, BITS, seed=101)
        p2, s2, b2 = make_weights(oracle, H, F, GROUP, BITS, seed=102)
        w1 = gaf.Weight.from_host(ctx, p1, s1, b1, GROUP, BITS, shard=SHARD_COL, tp_rank=rank, tp_size=world)
        w2 = gaf.Weight.from_host(ctx, p2, s2, b2, GROUP, BITS, shard=SHARD_ROW, tp_rank=rank, tp_size=world)
        # ---- one full-size row-parallel shard ----
        N3, K3 = 8192, 28672
        p3, s3, b3 = make_weights(oracle, N3, K3, GROUP, BITS, seed=103)
        w3 = gaf.Weight.from_host(ctx, p3, s3, b3, GROUP, BITS, shard=SHARD_ROW, tp_rank=rank, tp_size=world)
        xb3, xf3 = make_x_bf16(oracle, 1, K3, seed=113)
        ref3 = oracle.matmul_f32(xf3, p3, s3, b3, GROUP, BITS)
        k3 = K3 // world
        x3 = torch_bf16_from_bits(np.ascontiguousarray(xb3[:, rank * k3:(rank + 1) * k3]), "cuda")
        # kernel error apart from reduction error: every rank's own partial output (no sum on the GPU), added over the
        # ranks on the host in float64, against the oracle; the GPU's sums below are then compared with that sum too
        part = gaf.linear(ctx, w3, x3)
        stream.synchronize()
        ctx.synchronize()
        psum = torch.from_numpy(to_f32(part).astype(np.float64))
        dist.all_reduce(psum, op=dist.ReduceOp.SUM)
        psum = psum.numpy()
        kernel_rel = rel_err(psum.astype(np.float32), ref3)
        reduction_rel = 0.0
        for name, opts in paths:
            for k, v in (opts or {}).items():
                ctx.set_option(k, v)
            errs = []
            for M in (1, 2, 4):
                xb, xf = make_x_bf16(oracle, M, H, seed=110 + M)
                href = oracle.matmul_f32(xf, p1, s1, b1, GROUP, BITS)
                href = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(href))      # the chain hands bf16 activations on
                yref = oracle.matmul_f32(href, p2, s2, b2, GROUP, BITS)
                x = torch_bf16_from_bits(xb, "cuda")
                h = torch.empty((M, F // world), dtype=torch.bfloat16, device="cuda")
                y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
                if opts is None:
                    b = gaf.Batch(ctx, [w1, w2], [x, h], [h, y], depends=[0, 1], reduce=[0, 1])
                    b.run()
                    stream.synchronize()
                    ctx.synchronize()
                    b.close()
                else:
                    gaf.linear(ctx, w1, x, out=h)
                    gaf.linear_allreduce(ctx, w2, h, out=y)
                    stream.synchronize()
                    ctx.synchronize()
                errs.append(rel_err(to_f32(y), yref))
                if opts is None:
                    # operations that do not depend on one another: the wait for the peers' words of a row-parallel
                    # operation is put off to the end of the following operation
                    ya, yb = torch.zeros_like(y), torch.zeros_like(y)
                    h2, h3 = torch.zeros_like(h), torch.zeros_like(h)
                    b = gaf.Batch(ctx, [w2, w1, w2, w1], [h, x, h, x], [ya, h2, yb, h3], reduce=[1, 0, 1, 0])
                    for _ in range(3):
                        b.run()
                    stream.synchronize()
                    ctx.synchronize()
                    b.close()
                    errs.append(rel_err(to_f32(ya), yref))
                    errs.append(rel_err(to_f32(yb), yref))
                    errs.append(0.0 if (torch.equal(h2, h) and torch.equal(h3, h)) else 1.0)
            y3 = torch.empty((1, N3), dtype=torch.bfloat16, device="cuda")
            if opts is None:
                b = gaf.Batch(ctx, [w3], [x3], [y3], reduce=[1])
                b.run()
                stream.synchronize()
                ctx.synchronize()
                b.close()
            else:
                gaf.linear_allreduce(ctx, w3, x3, out=y3)
                stream.synchronize()
                ctx.synchronize()
            errs.append(rel_err(to_f32(y3), ref3))
            if opts is None or opts["fused_allreduce"]:
                reduction_rel = max(reduction_rel, rel_err(to_f32(y3), psum.astype(np.float32)))
            e = torch.tensor([max(errs)], dtype=torch.float64)
            dist.all_reduce(e, op=dist.ReduceOp.MAX)            # the worst rank
            # the two-step paths round every rank's partial sums to bf16 before they are added (P + 1 roundings
            # instead of one, and NCCL rounds again at every hop): their bound is 3e-2; the paths that add fp32 partials keep the 1e-2 of the other tests
            tol = 3e-2 if (opts and not opts["fused_allreduce"]) else 1e-2
            report.append({"path": name, "rel": round(float(e.item()), 6), "tolerance": tol})
            failed = failed or not float(e.item()) <= tol
            worst = max(worst, float(e.item()))
        ctx.set_option("fused_allreduce", 1)
        ctx.set_option("peer_allreduce", 1)
        for w in (w1, w2, w3):
            w.free()
    if failed:
        raise RuntimeError(f"rank {rank}: sharded linears differ from the unsharded oracle: {report}")
    return {"rel": round(worst, 6), "peer_memory": bool(peer), "paths": report,
            "down_shard_split": {"kernel_rel": round(float(kernel_rel), 6), "reduction_rel": round(float(reduction_rel), 6),
                                 "note": "8192 x 28672 shard: float64 host sum of the ranks' own bf16 partial outputs vs the oracle "
                                         "(kernel error), and the GPU's fp32-partials sum vs that host sum (reduction and rounding)"},
            "cases": "col->row chain 1024/2048 at M = 1, 2, 4; 8192 x 28672 row-parallel shard at M = 1; every rank compared"}


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
    weights, weights_host = [], []
    for li in range(layers):
        for name, N, K in shapes:
            p, s, b = synth_weight(rng, N, K)
            weights.append((name, gaf.Weight.from_host(ctx, p, s, b, GROUP, BITS)))
            if li < 2:
                weights_host.append((N, K, p, s, b))
    ring_bytes = sum(weight_bytes(w.N, w.K) for _, w in weights)
    wl = [w for _, w in weights]

    def make_io(M):
        xs = {K: torch.randn((M, K), device="cuda").to(torch.bfloat16) for K in (4096, 14336)}
        ys = [torch.empty((M, w.N), dtype=torch.bfloat16, device="cuda") for w in wl]
        return xs, ys

    if args.quick and args.case == "prefill":
        print(json.dumps({"quick": True, "prefill": time_prefill(gaf, ctx, torch, stream, rng, iters=2)}))
        return
    if args.quick and args.case == "stack70b":
        from talu_b200 import tp_bench
        r = tp_bench.measure(args, existing_ctx=ctx, existing_stream=stream, M=args.m, quick=True)
        print(json.dumps({"quick": True, "workload": "llama3_70b_stack", "M": args.m, "layers": r["layers"],
                          "ms_per_step": r["ms"], "gbs": round(r["bytes"] / r["ms"] / 1e6, 2)}))
        return
    if args.quick:
        # small case for profilers: one launch list (or the separate launches with --separate), not a bench value
        M = args.m
        if args.prefetch_units >= 0:
            ctx.set_option("prefetch_units", args.prefetch_units)
        xs, ys = make_io(M)
        with torch.cuda.stream(stream):
            if args.separate or M > 8:
                def step():
                    for i, (w, y) in enumerate(zip(wl, ys)):
                        gaf.hint_next_weight(ctx, wl[(i + 1) % len(wl)])
                        gaf.linear(ctx, w, xs[w.K], out=y)
            else:
                batch = gaf.Batch(ctx, wl, [xs[w.K] for w in wl], ys)
                step = batch.run
            for _ in range(max(1, args.warmup)):
                step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                step()
            e1.record(stream)
            stream.synchronize()
        ctx.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        nbytes = sum(launch_bytes(w.N, w.K, M) for w in wl)
        print(json.dumps({"quick": True, "M": M, "mode": "separate" if (args.separate or M > 8) else "launch list",
                          "gbs": round(nbytes / ms / 1e6, 2), "ms_per_step": ms}))
        return

    peak, peak_kind = measured_peak_hbm()
    parity_rel = check_outputs(gaf, ctx, torch, stream)
    results, lists = {}, {}
    from talu_b200.clocks import ClockSampler
    clocks = ClockSampler(dev)

    def frac(gbs):
        return {"gbs": round(gbs, 2), "frac_of_measured_hbm": round(gbs / peak, 4), "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4)}

    with clocks:
        for M in (1, 2, 4, 8, 16):
            xs, ys = make_io(M)
            nbytes = sum(launch_bytes(w.N, w.K, M) for w in wl)

            def separate():
                # a decoder knows its layer order: each call names the weight the following call streams
                for i, (w, y) in enumerate(zip(wl, ys)):
                    gaf.hint_next_weight(ctx, wl[(i + 1) % len(wl)])
                    gaf.linear(ctx, w, xs[w.K], out=y)

            ms, st, clk = time_graph(ctx, torch, stream, separate, args.steps, args.warmup, clocks=clocks)
            results[M] = {"ms_per_step": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes, "stats_ms": st, "clocks": clk}
            if M <= 8:
                b = gaf.Batch(ctx, wl, [xs[w.K] for w in wl], ys)
                ms, st, clk = time_graph(ctx, torch, stream, b.run, args.steps, args.warmup, clocks=clocks)
                lists[M] = {"independent": {"ms_per_step": ms, "gbs": nbytes / ms / 1e6, "stats_ms": st, "clocks": clk,
                                            "one_launch": b.one_launch}}
                b.close()
                b = gaf.Batch(ctx, wl, [xs[w.K] for w in wl], ys, depends=[0] + [1] * (len(wl) - 1))
                ms, st, clk = time_graph(ctx, torch, stream, b.run, args.steps, args.warmup, min_seconds=0.5, clocks=clocks)
                lists[M]["chained"] = {"ms_per_step": ms, "gbs": nbytes / ms / 1e6, "stats_ms": st}
                b.close()

        # ---- cfg2 as written: gate and up as separate weights (three GEMVs per layer) ----
        un_layers = min(layers, 6)
        un = []
        for _ in range(un_layers):
            for N, K in ((14336, 4096), (14336, 4096), (4096, 14336)):
                un.append(gaf.Weight.from_host(ctx, *synth_weight(rng, N, K), GROUP, BITS))
        xs, _ = make_io(1)
        uys = [torch.empty((1, w.N), dtype=torch.bfloat16, device="cuda") for w in un]
        unbytes = sum(launch_bytes(w.N, w.K, 1) for w in un)

        def un_separate():
            for i, (w, y) in enumerate(zip(un, uys)):
                gaf.hint_next_weight(ctx, un[(i + 1) % len(un)])
                gaf.linear(ctx, w, xs[w.K], out=y)

        ms_s, st_s, _ = time_graph(ctx, torch, stream, un_separate, args.steps, args.warmup, min_seconds=0.5, clocks=clocks)
        b = gaf.Batch(ctx, un, [xs[w.K] for w in un], uys)
        ms_l, st_l, _ = time_graph(ctx, torch, stream, b.run, args.steps, args.warmup, min_seconds=0.5, clocks=clocks)
        b.close()
        unstacked = {"layers": un_layers, "gemvs_per_layer": 3,
                     "separate_launches": {**frac(unbytes / ms_s / 1e6), "ms_per_step": round(ms_s, 5), "stats_ms": st_s},
                     "launch_list": {**frac(unbytes / ms_l / 1e6), "ms_per_step": round(ms_l, 5), "stats_ms": st_l}}
        for w in un:
            w.free()

        # ---- cfg1 (latency-bound: 2.4 MB per GEMV) and the cfg3 scheme sweep (K = N = 4096, ring >= 1 GB) ----
        def sweep_case(N, K, G, bits, M, ring_target):
            per = weight_bytes(N, K, G, bits)
            n = max(8, int(ring_target // per))
            ws_ = [gaf.Weight.from_host(ctx, *synth_weight(rng, N, K, G, bits), G, bits) for _ in range(n)]
            x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
            ys_ = [torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in ws_]
            nb = n * launch_bytes(N, K, M, G, bits)

            def sep():
                for i, (w, y) in enumerate(zip(ws_, ys_)):
                    gaf.hint_next_weight(ctx, ws_[(i + 1) % n])
                    gaf.linear(ctx, w, x, out=y)

            ms, st, _ = time_graph(ctx, torch, stream, sep, args.steps, args.warmup, min_seconds=0.3, clocks=clocks)
            out = {"gemvs": n, "ring_gb": round(n * per / 1e9, 3),
                   "separate_launches": {**frac(nb / ms / 1e6), "us_per_gemv": round(ms * 1e3 / n, 3), "stats_ms": st}}
            b_ = gaf.Batch(ctx, ws_, [x] * n, ys_)
            if b_.one_launch:
                ms, st, _ = time_graph(ctx, torch, stream, b_.run, args.steps, args.warmup, min_seconds=0.3, clocks=clocks)
                out["launch_list"] = {**frac(nb / ms / 1e6), "us_per_gemv": round(ms * 1e3 / n, 3), "stats_ms": st}
            b_.close()
            for w in ws_:
                w.free()
            return out

        cfg1 = sweep_case(4096, 1024, 64, 4, 1, 0.6e9)
        cfg1["note"] = "N=4096 K=1024 M=1: 2.4 MB per GEMV, latency-bound; reported for completeness, not against the roofline"
        cfg3 = {}
        for bits, G in ((4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)):
            for M in (1, 8):
                cfg3[f"gaf{bits}_{G}_M{M}"] = sweep_case(4096, 4096, G, bits, M, 1.0e9)

        # ---- end to end through the C ABI with host buffers (pinned), M = 1 ----
        # all activations of a step in one page-locked block, all outputs in another (24 views each): per step the x
        # block goes up, the launch list runs, the y block comes back; host wall clock around submit + wait
        from types import SimpleNamespace
        from talu_b200 import tp_bench
        e2e = tp_bench.time_e2e(ctx, torch, None, 1, SimpleNamespace(weights=wl, reduce=[0] * len(wl)), 1, max(args.steps, 100))
        e2e_ms = e2e["ms_per_step"]
        h2d, d2h = e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]
        e2e_gbs = results[1]["bytes"] / e2e_ms / 1e6
        e2e_mode = ("tgaf_host_batch_submit (recorded list: x block up, ONE launch list, y block down)" if e2e["one_launch"]
                    else "tgaf_host_batch_submit (recorded list of queued calls)")

        prefill = time_prefill(gaf, ctx, torch, stream, rng, clocks=clocks)
        # the multi-GPU workload on this one GPU, so that the N > 1 lines have their N = 1 reference
        st70 = tp_bench.measure(args, existing_ctx=ctx, existing_stream=stream, also_m=(64,))
        stack70b = {"workload": "llama3_70b_stack", "layers": st70["layers"], "ms_per_step": round(st70["ms"], 5),
                    **frac(st70["bytes"] / st70["ms"] / 1e6), "stats_ms": st70["stats"], "submission": st70["submission"],
                    "separate_launches": st70.get("separate")}
        # the skinny case of the same stack (64 activation rows: the tcgen05 GEMM with one 128-row activation half)
        sk = st70["also"][64]
        stack70b["m64"] = {"ms_per_step": round(sk["ms"], 5), **frac(sk["bytes"] / sk["ms"] / 1e6), "stats_ms": sk["stats"]}
    incumbent = time_incumbent_kernel(torch, weights_host)

    head = lists[1]["independent"]
    gemvs_per_step = len(wl)
    achieved = head["gbs"]
    from oracle import gaf_oracle as oracle
    logical, policy = oracle.logical_cpu_count(), oracle.reference_thread_count()
    cstack = cpu_stack(ffn_shapes(min(layers, 4)))
    cbytes = sum(launch_bytes(N, K, 1) for N, K, *_ in cstack)
    n_cpu = max(2, int(args.cpu_seconds / 0.02 / max(1, len(cstack) // 2)))
    t_all = cpu_time_step(oracle, cstack, logical, n_cpu, 1)
    t_pol = cpu_time_step(oracle, cstack, policy, max(2, n_cpu // 2), 1)
    cpu_gbs = cbytes / float(np.mean(t_all)) / 1e9

    out = {
        "metric": METRIC, "value": round(head["gbs"], 2), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(head["ms_per_step"], 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama3_8b_ffn", "scheme": "gaf4_64", "M": 1, "layers": layers,
                   "gemvs_per_step": gemvs_per_step, "gate_up_stacked": True,
                   "submission": "one launch list per step (tgaf_batch_run): 24 GEMVs, each with its own activations, one kernel launch",
                   "l2": f"distinct weights per GEMV, ring {ring_bytes / 1e9:.2f} GB > 126 MB L2 (no flush needed)",
                   "timing": "CUDA graph replay for >= 1 s, an event per step; value = mean of the last --steps steps"},
        "stats_ms": head["stats_ms"],
        "output_check": {"rel_err_vs_oracle": round(parity_rel, 6), "tolerance": 1e-2,
                         "what": "one FFN layer of converter-made weights, M = 1, launch list and single calls"},
        "decode": {f"M{m}": {"separate_launches": {**frac(r["gbs"]), "ms_per_step": round(r["ms_per_step"], 5), "stats_ms": r["stats_ms"], "clocks": r["clocks"]},
                             **({"launch_list": {**frac(lists[m]["independent"]["gbs"]), "ms_per_step": round(lists[m]["independent"]["ms_per_step"], 5),
                                                 "stats_ms": lists[m]["independent"]["stats_ms"], "clocks": lists[m]["independent"]["clocks"]},
                                 "launch_list_every_gemv_waits_for_its_predecessor": {**frac(lists[m]["chained"]["gbs"]),
                                                                                       "ms_per_step": round(lists[m]["chained"]["ms_per_step"], 5)}}
                                if m in lists else {})}
                   for m, r in results.items()},
        "cfg2_gate_and_up_as_separate_weights": unstacked,
        "cfg1": cfg1, "cfg3": cfg3,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                     "peak_kind": f"of {peak_kind}", "traffic": NCU_TRAFFIC_PER_GEMV * gemvs_per_step,
                     "algorithmic_bytes": results[1]["bytes"],
                     "note": "per launch = one list of all the step's GEMVs: achieved = algorithmic bytes of the step / its time; "
                             "traffic = ncu dram bytes (read + written) of a 4-GEMV list, per GEMV, times the GEMVs of this list "
                             "(traffic grows in proportion to the weights streamed)"},
        "cpu_baseline": {"value": round(cpu_gbs, 3), "unit": "GB/s", "cores": logical, "kind": "port",
                         "sample": f"{len(t_all)} passes over the first {len(cstack)} matrices of the same stack ({cbytes / 1e6:.0f} MB per pass), M=1, f32 activations",
                         "reference_thread_policy": {"threads": policy, "value": round(cbytes / float(np.mean(t_pol)) / 1e9, 3)}},
        "incumbent_gpu_kernel": incumbent,
        "e2e": {"value": round(e2e_gbs, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms, 4), "stats_ms": e2e["stats_ms"],
                "note": e2e_mode + " + tgaf_synchronize per step, host wall clock; the 24 x buffers are views of one page-locked block, the 24 y buffers of another"},
        "prefill": prefill,
        "llama3_70b_stack_1gpu": stack70b,
        "gpu_launches": args.steps,
        "gpu_launches_note": "kernel launches inside the timed K steps of the headline: one launch list per step (24 GEMVs each)",
        "clocks": {**clocks.summary(), "sm_mhz": (head["clocks"] or {}).get("sm_mhz_median", clocks.summary()["sm_mhz"]),
                   "sm_mhz_all_cases": clocks.summary()["sm_mhz"],
                   "note": "sm_mhz = median while the headline case (M = 1 launch list) ran; reasons = seen at any time during the bench"},
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
    ap.add_argument("--separate", action="store_true", help="with --quick: separate launches instead of one launch list")
    ap.add_argument("--prefetch-units", type=int, default=-1,
                    help="with --quick --separate: units per CTA of the next weight a launch pulls into L2 (library default 2)")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="length of every timed graph-replay run (shorter only for launch listings under a profiler)")
    ap.add_argument("--quick", action="store_true",
                    help="one configuration only, no end-to-end and no CPU leg (small case for profilers; not a bench value)")
    args = ap.parse_args()
    global MIN_SECONDS_SCALE
    MIN_SECONDS_SCALE = args.min_seconds
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        from talu_b200 import tp_bench
        tp_bench.run(args, parity_check=tp_parity_check)
        return
    run_single(args)


if __name__ == "__main__":
    main()
