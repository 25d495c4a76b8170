"""The Llama-3-70B-shaped linear stack in gaf4_64 (qkv, o, gate|up, down per layer), whole on one GPU or
column- / row-sharded over the ranks (one process per GPU) with the sum over ranks on the row-parallel
outputs.  Strong scaling: the stack is the same at every N.  Used by bench.py for its N > 1 line and for the
one-GPU figure of the same workload."""
from __future__ import annotations

import json
import os
import time

import numpy as np

from . import gaf
from .clocks import ClockSampler
from .peaks import measured_peak_hbm
from .tp import LLAMA3_70B_LINEARS, SHARD_ROW, shard_slice

GROUP, BITS = 64, 4
HIDDEN = 8192
METRIC = "gaf4_64 decode GEMV HBM GB/s"


def _weight_bytes(N, K):
    return N * K * BITS // 8 + 2 * N * (K // GROUP) * 2


def stack_bytes(layers, M):
    """Whole-job algorithmic bytes of one step: the full (unsharded) stack once, activations in and out."""
    return layers * sum(_weight_bytes(N, K) + M * K * 2 + M * N * 2 for (N, K, _) in LLAMA3_70B_LINEARS.values())


def _stats_ms(samples):
    a = np.sort(np.asarray(samples, np.float64))
    return {"min": round(float(a[0]), 5), "p50": round(float(np.percentile(a, 50)), 5),
            "p90": round(float(np.percentile(a, 90)), 5), "mean": round(float(a.mean()), 5), "n": int(a.size)}


def _check_allreduce(ctx, torch, rank, world, stream):
    """Every rank can compute every rank's tile, so each checks the sum it gets.  On the peer-memory path
    the sum is fp32 in rank order, rounded once: the check is exact.  Sizes vary from call to call so
    that both exchange phases and different CTA counts are used."""
    exact = ctx.uses_peer_memory()
    with torch.cuda.stream(stream):
        for it, (n, dt) in enumerate([(8192, torch.bfloat16), (8, torch.bfloat16), (4096, torch.float32),
                                      (8192 * 16, torch.bfloat16), (8192, torch.bfloat16), (24, torch.bfloat16),
                                      (8192 * 16, torch.float32), (8192 * 3, torch.bfloat16)] * 3):
            tiles = [((torch.arange(n, device="cuda", dtype=torch.float32) * (0.37 + it) % 251.0) - 125.0 + 1.5 * r).to(dt)
                     for r in range(world)]
            mine = tiles[rank].clone()
            ctx.allreduce(mine)
            acc = torch.zeros(n, device="cuda", dtype=torch.float32)
            for r in range(world):
                acc += tiles[r].float()
            want = acc.to(dt)
            stream.synchronize()
            ctx.synchronize()
            if exact:
                ok = torch.equal(mine, want)
            else:
                ok = torch.allclose(mine.float(), want.float(), rtol=2e-2, atol=1.0)
            if not ok:
                bad = (mine != want).nonzero()[:4].flatten().tolist()
                raise RuntimeError(f"rank {rank}: all-reduce mismatch at call {it} (n={n}, {dt}), first bad indices {bad}")


class Stack:
    """`layers` decoder layers' linears, this rank's shards.  One layer's random codes are generated on the host
    and uploaded once per layer: every layer is its own device buffers (timing does not depend on the values)."""

    def __init__(self, ctx, layers, rank, world):
        self.ctx, self.layers, self.rank, self.world = ctx, layers, rank, world
        rng = np.random.default_rng(1234)
        host = []
        for name, (N, K, kind) in LLAMA3_70B_LINEARS.items():
            sl = shard_slice(N, K, GROUP, BITS, kind, rank, world)
            packed = rng.integers(0, 2 ** 32, size=(sl.n, sl.k * BITS // 32), dtype=np.uint32)
            scales = (np.full((sl.n, sl.k // GROUP), 0.0053, np.float32).view(np.uint32) >> 16).astype(np.uint16)
            biases = (np.full((sl.n, sl.k // GROUP), -0.04, np.float32).view(np.uint32) >> 16).astype(np.uint16)
            host.append((name, kind, packed, scales, biases))
        self.ws = []
        for _ in range(layers):
            for name, kind, p, s, b in host:
                self.ws.append((name, kind, gaf.Weight.from_host(ctx, p, s, b, GROUP, BITS)))
        self.weights = [w for _, _, w in self.ws]
        self.reduce = [1 if (kind == SHARD_ROW and world > 1) else 0 for _, kind, _ in self.ws]

    def free(self):
        for w in self.weights:
            w.free()
        self.ws, self.weights = [], []


def _time_graph(ctx, torch, dist, world, stream, launch_step, steps, warmup, min_seconds):
    """Captures one step into a CUDA graph and replays it for at least `min_seconds` (the same number of replays
    on every rank), an event after every replay; barrier + synchronize on both sides.  Returns (mean ms of the
    last `steps` replays, max over ranks; this rank's per-step statistics)."""
    with torch.cuda.stream(stream):
        launch_step()
        stream.synchronize()
        ctx.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
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
        n = torch.tensor([int(min(20000, max(steps, min_seconds * 1e3 / est)))])
        if world > 1:
            dist.all_reduce(n, op=dist.ReduceOp.MAX)     # the same replay count everywhere: the steps hold collectives
        n = int(n.item())
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        evs[0].record(stream)
        for i in range(n):
            graph.replay()
            evs[i + 1].record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    ctx.synchronize()
    samples = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)]
    ms = torch.tensor([float(np.mean(samples[-steps:]))])
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)     # max over ranks (device-timed on every rank)
    # the captured graph may refer to the communicator: release it here, before the caller lets the communicator go
    del graph
    torch.cuda.synchronize()
    return float(ms.item()), _stats_ms(samples)


def _time_stack(ctx, torch, dist, world, stream, stack, M, steps, warmup, min_seconds, want_separate, want_no_reduce):
    """One step = every linear of the stack once, each with its own activations.  M <= 4: one launch list; above:
    separate launches.  Returns a dict."""
    xs = [torch.randn((M, w.K), device="cuda").to(torch.bfloat16) for w in stack.weights]
    ys = [torch.empty((M, w.N), dtype=torch.bfloat16, device="cuda") for w in stack.weights]
    ws = stack.weights

    def separate():
        for i, (w, x, y, red) in enumerate(zip(ws, xs, ys, stack.reduce)):
            gaf.hint_next_weight(ctx, ws[(i + 1) % len(ws)])
            if red:
                gaf.linear_allreduce(ctx, w, x, out=y)
            else:
                gaf.linear(ctx, w, x, out=y)

    out = {"separate": None, "no_reduce_ms": None}
    if M <= 4 or (M <= 8 and not any(stack.reduce)):
        batch = gaf.Batch(ctx, ws, xs, ys, reduce=stack.reduce if any(stack.reduce) else None)
        out["submission"] = ("one launch list per step (tgaf_batch_run), one kernel launch" if batch.one_launch
                             else "tgaf_batch_run, its calls one after the other")
        out["launches_per_step"] = 1 if batch.one_launch else len(ws)
        out["ms"], out["stats"] = _time_graph(ctx, torch, dist, world, stream, batch.run, steps, warmup, min_seconds)
        batch.close()
        if want_no_reduce and any(stack.reduce):
            # the same list without the sums over ranks: the difference is what the exchanges cost
            b2 = gaf.Batch(ctx, ws, xs, ys)
            out["no_reduce_ms"], _ = _time_graph(ctx, torch, dist, world, stream, b2.run, steps, warmup, min(min_seconds, 0.3))
            b2.close()
        if want_separate:
            ms, st = _time_graph(ctx, torch, dist, world, stream, separate, steps, warmup, min(min_seconds, 0.3))
            out["separate"] = {"ms_per_step": round(ms, 5), "stats_ms": st}
    else:
        out["submission"] = "separate launches"
        out["launches_per_step"] = len(ws)
        out["ms"], out["stats"] = _time_graph(ctx, torch, dist, world, stream, separate, steps, warmup, min_seconds)
    return out


def time_e2e(ctx, torch, dist, world, stack, M, steps):
    """End to end on every rank through the recorded host batch: all activations in one page-locked block, all
    outputs in another; per step the x block goes up, the launch list runs (sums over ranks inside), the y block
    comes back, one wait.  Host wall clock per step, max over ranks of the mean."""
    ws = stack.weights
    xn = sum(M * w.K for w in ws)
    yn = sum(M * w.N for w in ws)
    hx = torch.randn(xn).to(torch.bfloat16).pin_memory()
    hy = torch.empty(yn, dtype=torch.bfloat16).pin_memory()
    hx_np = hx.view(torch.int16).numpy().view(np.uint16)
    hy_np = hy.view(torch.int16).numpy().view(np.uint16)
    xv, yv, xo, yo = [], [], 0, 0
    for w in ws:
        xv.append(hx_np[xo: xo + M * w.K].reshape(M, w.K))
        yv.append(hy_np[yo: yo + M * w.N].reshape(M, w.N))
        xo += M * w.K
        yo += M * w.N
    hb = gaf.HostBatch(ctx, ws, xv, yv, reduce=stack.reduce if any(stack.reduce) else None)
    hb.record()
    one = hb.one_launch

    def step():
        hb.submit()
        ctx.synchronize()

    for _ in range(5):
        step()
    n = max(steps, 100)
    if world > 1:
        dist.barrier()
    samples = []
    for _ in range(n):
        t0 = time.perf_counter()
        step()
        samples.append((time.perf_counter() - t0) * 1e3)
    if world > 1:
        dist.barrier()
    t = torch.tensor([float(np.mean(samples[-steps:]))])
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    hb.close()
    return {"ms_per_step": float(t.item()), "stats_ms": _stats_ms(samples), "one_launch": one,
            "h2d_bytes_per_step": world * xn * 2, "d2h_bytes_per_step": world * yn * 2}


def measure(args, existing_ctx=None, existing_stream=None, M=1, quick=False, parity_check=None, also_m=()):
    """Runs the stack on this rank (all ranks call it together).  Returns a dict: ms (max over ranks), bytes
    (whole job, per step), layers, stats, submission, separate, and for N > 1 the one-GPU time of the same
    workload (measured by rank 0 on its GPU before the communicator exists), the exchange cost, the end-to-end
    leg and what `parity_check` returned."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if existing_ctx is None:
        torch.cuda.set_device(local)
    if world > 1:
        # control plane (id hand-over, barriers, max of timings) over gloo; the data path is the
        # library's own communicator
        dist.init_process_group("gloo")
    stream = existing_stream or torch.cuda.Stream()
    ctx = existing_ctx or gaf.Context(local, stream=stream.cuda_stream)
    layers = 2 if quick else (args.layers if args.layers != 12 else 8)   # 8 layers: 3.85 GB, 481 MB per rank at N = 8
    steps, warmup = args.steps, max(3, args.warmup)
    min_seconds = 0.0 if quick else float(getattr(args, "min_seconds", 1.0))
    res = {"layers": layers, "world": world, "rank": rank, "steps": steps, "warmup": warmup, "bytes": stack_bytes(layers, M)}

    if world > 1:
        # the same workload on ONE GPU, in this run: rank 0 holds the whole stack for a moment, the others wait
        one = torch.zeros(1, dtype=torch.float64)
        if rank == 0:
            whole = Stack(ctx, layers, 0, 1)
            r1 = _time_stack(ctx, torch, None, 1, stream, whole, M, steps, warmup, 0.5, False, False)
            whole.free()
            one[0] = r1["ms"]
        dist.broadcast(one, src=0)
        res["one_gpu_ms"] = float(one.item())

        ids = [gaf.make_comm_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init(ids[0], rank, world)
        _check_allreduce(ctx, torch, rank, world, stream)
        res["allreduce"] = ("inside the GEMV launch over NVLink peer memory (plain peer stores, fp32 partial tiles summed in rank order)"
                            if ctx.uses_peer_memory() else "NCCL")
        if parity_check is not None:
            res["tp_parity"] = parity_check(ctx, torch, dist, rank, world, stream)

    stack = Stack(ctx, layers, rank, world)
    with ClockSampler(local) as clocks:
        r = _time_stack(ctx, torch, dist if world > 1 else None, world, stream, stack, M, steps, warmup, min_seconds,
                        want_separate=(M == 1 and not quick), want_no_reduce=(world > 1))
    res.update(r)
    res["clocks"] = clocks.summary()
    if world > 1 and r.get("no_reduce_ms"):
        n_red = sum(stack.reduce)
        res["exchange_us"] = round((r["ms"] - r["no_reduce_ms"]) * 1e3 / n_red, 3)
    res["also"] = {}
    for m2 in also_m:
        r2 = _time_stack(ctx, torch, dist if world > 1 else None, world, stream, stack, m2, steps, warmup, min_seconds, False, False)
        r2["bytes"] = stack_bytes(layers, m2)
        res["also"][m2] = r2
    res["e2e"] = time_e2e(ctx, torch, dist, world, stack, M, steps) if (world > 1 and M <= 4) else None
    torch.cuda.synchronize()
    stack.free()
    if world > 1:
        dist.barrier()
        ctx._lib.tgaf_comm_destroy(ctx._h)
        dist.destroy_process_group()
    return res


def run(args, parity_check=None):
    M = 1
    r = measure(args, M=M, parity_check=parity_check)
    if r["rank"] != 0:
        return
    world, ms, total = r["world"], r["ms"], r["bytes"]
    value = total / ms / 1e6
    peak, kind = measured_peak_hbm()
    e2e = r["e2e"]
    print(json.dumps({
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
        "steps": r["steps"], "warmup": r["warmup"], "ms_per_step": round(ms, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama3_70b_stack", "scheme": "gaf4_64", "M": M, "layers": r["layers"],
                   "parallelism": f"tp{world}",
                   "sharding": "qkv, gate|up column-parallel; o, down row-parallel + sum over ranks (fp32 partial tiles, one rounding)",
                   "allreduce": r.get("allreduce"), "submission": r["submission"],
                   "l2": f"distinct layers per step, {total / world / 1e6:.0f} MB per rank (> 126 MB L2)",
                   "timing": "CUDA graph replay for >= 1 s, an event per step, max over ranks; value = mean of the last --steps steps"},
        "stats_ms": r["stats"],
        "same_workload_1gpu": {"ms_per_step": round(r["one_gpu_ms"], 5), "gbs": round(total / r["one_gpu_ms"] / 1e6, 2),
                               "speedup": round(r["one_gpu_ms"] / ms, 3),
                               "note": "the whole stack on rank 0's GPU in this run, same submission, before the communicator exists"},
        "exchange": {"us_per_sum": r.get("exchange_us"), "sums_per_step": 2 * r["layers"],
                     "ms_per_step_without_sums": None if r.get("no_reduce_ms") is None else round(r["no_reduce_ms"], 5),
                     "note": "step time minus the time of the same launch list with the sums over ranks switched off, per sum"},
        "separate_launches": r.get("separate"),
        "tp_parity": r.get("tp_parity"),
        "roofline": {"bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(value / world / peak, 4), "peak_kind": f"of {kind}", "traffic": None,
                     "note": "per-GPU share of the aggregate; exchange time included"},
        "cpu_baseline": None,
        "e2e": None if e2e is None else {
            "value": round(total / e2e["ms_per_step"] / 1e6, 2), "unit": "GB/s", "ms_per_step": round(e2e["ms_per_step"], 5),
            "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
            "stats_ms": e2e["stats_ms"], "one_launch": e2e["one_launch"],
            "note": "per rank and step: tgaf_host_batch_submit (recorded list with the row-parallel sums) + tgaf_synchronize; "
                    "x block pinned host -> device, launch list, y block -> pinned host; host wall clock, max over ranks"},
        "gpu_launches": r["launches_per_step"] * r["steps"] * world,
        "clocks": r["clocks"],
    }))
