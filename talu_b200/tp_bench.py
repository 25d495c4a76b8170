"""Multi-GPU leg of bench.py: the Llama-3-70B-shaped linear stack in gaf4_64,
column- / row-sharded over the ranks (one process per GPU), NCCL allreduce on the
row-parallel outputs.  Strong scaling: the stack is the same at every N."""
from __future__ import annotations

import json
import os

import numpy as np

from . import gaf
from .tp import LLAMA3_70B_LINEARS, SHARD_ROW, shard_slice

GROUP, BITS = 64, 4
HIDDEN = 8192


def _weight_bytes(N, K):
    return N * K * BITS // 8 + 2 * N * (K // GROUP) * 2


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


def _check_fused(ctx, torch, dist, rank, world, stream, ws, xs):
    """Row-parallel linears: the one-kernel path (fp32 partial tiles summed in rank order) against the two-step
    path (bf16 outputs, then all-reduce) within the bf16 tolerance, and bit-identical results on all ranks."""
    with torch.cuda.stream(stream):
        for name, kind, w in ws[:8]:
            if kind != SHARD_ROW:
                continue
            for rep in range(3):
                y1 = gaf.linear_allreduce(ctx, w, xs[w.K])
                ctx.set_option("fused_allreduce", 0)
                y2 = gaf.linear_allreduce(ctx, w, xs[w.K])
                ctx.set_option("fused_allreduce", 1)
                stream.synchronize()
                ctx.synchronize()
                a, b = y1.float(), y2.float()
                scale = max(float(b.abs().max()), 1e-6)
                err = float((a - b).abs().max()) / scale
                if not err <= 1e-2:
                    raise RuntimeError(f"rank {rank}: fused {name} differs from the two-step path: rel {err}")
                mine = y1.view(torch.int16).to(torch.int32).cpu()
                ref = mine.clone()
                dist.broadcast(ref, src=0)
                if not torch.equal(mine, ref):
                    raise RuntimeError(f"rank {rank}: fused {name} is not bit-identical to rank 0's")


def measure(args, existing_ctx=None, existing_stream=None, M=1):
    """Runs the stack on this rank (all ranks call it together) and returns (ms per step over ranks,
    whole-job bytes per step, launches per rank, layers, world)."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    debug = os.environ.get("TGAF_BENCH_DEBUG") == "1"

    def note(msg):
        if debug:
            import sys
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    if debug:
        import faulthandler
        faulthandler.dump_traceback_later(60, exit=True)   # where are we if nothing moves for a minute
    if existing_ctx is None:
        torch.cuda.set_device(local)
    if world > 1:
        # control plane (id hand-over, barriers, max of timings) over gloo; the data path is the
        # library's own NCCL communicator
        dist.init_process_group("gloo")
    note("process group up")
    stream = existing_stream or torch.cuda.Stream()
    ctx = existing_ctx or gaf.Context(local, stream=stream.cuda_stream)
    if world > 1:
        ids = [gaf.make_comm_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        note("comm id exchanged")
        ctx.comm_init(ids[0], rank, world)
        note("communicator initialised")

        _check_allreduce(ctx, torch, rank, world, stream)
        note(f"all-reduce checked (peer memory: {ctx.uses_peer_memory()})")

    layers = args.layers if args.layers != 12 else 4          # distinct layers in the ring (1.9 GB over all ranks)
    rng = np.random.default_rng(1234)                          # same seed on every rank: same full weights
    ws = []
    for _ in range(layers):
        for name, (N, K, kind) in LLAMA3_70B_LINEARS.items():
            sl = shard_slice(N, K, GROUP, BITS, kind, rank, world)
            # only this rank's slice is generated (timing does not depend on the values)
            packed = rng.integers(0, 2 ** 32, size=(sl.n, sl.k * BITS // 32), dtype=np.uint32)
            scales = (np.full((sl.n, sl.k // GROUP), 0.0053, np.float32).view(np.uint32) >> 16).astype(np.uint16)
            biases = (np.full((sl.n, sl.k // GROUP), -0.04, np.float32).view(np.uint32) >> 16).astype(np.uint16)
            ws.append((name, kind, gaf.Weight.from_host(ctx, packed, scales, biases, GROUP, BITS)))
    xs = {k: torch.randn((M, k), device="cuda").to(torch.bfloat16) for k in {w.K for _, _, w in ws}}
    ys = [torch.empty((M, w.N), dtype=torch.bfloat16, device="cuda") for _, _, w in ws]

    def step():
        for i, ((name, kind, w), y) in enumerate(zip(ws, ys)):
            gaf.hint_next_weight(ctx, ws[(i + 1) % len(ws)][2])
            if kind == SHARD_ROW and world > 1:
                gaf.linear_allreduce(ctx, w, xs[w.K], out=y)   # partial sums of the row-parallel output -> full [M, 8192]
            else:
                gaf.linear(ctx, w, xs[w.K], out=y)

    kind_ar = None
    if world > 1:
        kind_ar = "fused into the GEMV write-out over NVLink peer memory" if ctx.uses_peer_memory() else "NCCL"
    steps, warmup = args.steps, max(3, args.warmup)
    note(f"{len(ws)} weights uploaded")
    if world > 1:
        _check_fused(ctx, torch, dist, rank, world, stream, ws, xs)
        note("fused linear + all-reduce checked against the two-step path")
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        note("eager step done")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            step()
        note("graph captured")
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        note("warm-up done")
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps])
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)     # max over ranks (device-timed on every rank)
    ms = float(ms.item())
    note(f"timed: {ms} ms/step")

    # end to end on every rank: each launch's x comes from page-locked host memory and its y goes back there,
    # copies on the launching stream inside the timed region, one wait per step
    e2e = None
    if world > 1 and M == 1:
        hx = {k: torch.randn((M, k)).to(torch.bfloat16).pin_memory() for k in xs}
        hy = [torch.empty((M, w.N), dtype=torch.bfloat16).pin_memory() for _, _, w in ws]

        def e2e_step():
            for i, ((name, kind, w), y, yh) in enumerate(zip(ws, ys, hy)):
                xs[w.K].copy_(hx[w.K], non_blocking=True)
                gaf.hint_next_weight(ctx, ws[(i + 1) % len(ws)][2])
                if kind == SHARD_ROW:
                    gaf.linear_allreduce(ctx, w, xs[w.K], out=y)
                else:
                    gaf.linear(ctx, w, xs[w.K], out=y)
                yh.copy_(y, non_blocking=True)
            stream.synchronize()

        e2e_steps = max(3, min(steps, 20))
        with torch.cuda.stream(stream):
            for _ in range(3):
                e2e_step()
            dist.barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(stream)
            for _ in range(e2e_steps):
                e2e_step()
            f1.record(stream)
            stream.synchronize()
            dist.barrier()
        t = torch.tensor([f0.elapsed_time(f1) / e2e_steps])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"ms_per_step": float(t.item()),
               "h2d_bytes_per_step": world * sum(M * w.K * 2 for _, _, w in ws),
               "d2h_bytes_per_step": world * sum(M * w.N * 2 for _, _, w in ws)}
        note(f"end to end: {e2e['ms_per_step']} ms/step")

    # whole-job algorithmic bytes: the full (unsharded) stack once per step
    total = 0
    for _ in range(layers):
        for name, (N, K, kind) in LLAMA3_70B_LINEARS.items():
            total += _weight_bytes(N, K) + M * K * 2 + M * N * 2
    # the captured graph refers to the communicator: release it before the communicator goes
    del graph
    torch.cuda.synchronize()
    for _, _, w in ws:
        w.free()
    if world > 1:
        dist.barrier()
        ctx._lib.tgaf_comm_destroy(ctx._h)
        note("communicator destroyed")
        dist.destroy_process_group()
    if debug:
        import faulthandler
        faulthandler.cancel_dump_traceback_later()
    return ms, total, len(ws), layers, world, rank, steps, warmup, kind_ar, e2e


def run(args):
    ms, total, per_rank_launches, layers, world, rank, steps, warmup, allreduce_kind, e2e = measure(args)
    M = 1
    value = total / ms / 1e6
    if rank == 0:
        from bench import measured_peak_hbm
        peak, kind = measured_peak_hbm()
        print(json.dumps({
            "metric": "gaf4_64 decode GEMV HBM GB/s", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3_70b_stack", "scheme": "gaf4_64", "M": M, "layers": layers,
                       "parallelism": f"tp{world}", "sharding": "qkv, gate|up column-parallel; o, down row-parallel + all-reduce (bf16 tiles, fp32 sums)",
                       "allreduce": allreduce_kind,
                       "l2": "distinct layers per step, ring larger than L2 on every rank",
                       "timing": "CUDA graph replay, CUDA events, max over ranks"},
            "roofline": {"bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(value / world / peak, 4), "peak_kind": f"of {kind}", "traffic": None,
                         "note": "per-GPU share of the aggregate; allreduce time included"},
            "cpu_baseline": None,
            "e2e": None if e2e is None else {
                "value": round(total / e2e["ms_per_step"] / 1e6, 2), "unit": "GB/s", "ms_per_step": round(e2e["ms_per_step"], 5),
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "note": "per launch and rank: pinned host x -> device, linear (row-parallel ones with the sum over ranks), y -> pinned host; one wait per step"},
            "gpu_launches": per_rank_launches * steps * world,
        }))
