"""Launch lists (tgaf_batch_*): the linears of a decoder step as one call, one kernel launch when the list qualifies.
Against the CPU oracle (rel <= 1e-2 per linear, 2e-2 through a dependent pair) and against the same calls made one by
one; run to run the bits must not change."""
import numpy as np
import pytest

from helpers import TOL_BF16, bits_from_torch_bf16, make_weights, make_x_bf16, rel_err, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gaf():
    import talu_b200
    return talu_b200


@pytest.fixture(scope="module")
def ctx(gaf):
    c = gaf.Context(0)
    yield c
    c.close()


def _f32(oracle, t):
    return oracle.bf16_to_f32(bits_from_torch_bf16(t))


@pytest.mark.parametrize("M", [1, 2, 4])
def test_independent_list_in_one_launch(gaf, ctx, oracle, M):
    """Six weights of different shapes (ragged N, K below and above one activation block, a K that is split over many
    CTAs), each with its own activations: one launch, every output against the oracle and the one-by-one calls."""
    import torch
    shapes = [(1000, 2048), (4096, 1024), (384, 14336), (2048, 4096), (130, 512), (3000, 8192)]
    G = 64
    ws, xs, refs = [], [], []
    for i, (N, K) in enumerate(shapes):
        p, s, b = make_weights(oracle, N, K, G, 4, seed=100 + i)
        xb, xf = make_x_bf16(oracle, M, K, seed=200 + i)
        ws.append(gaf.Weight.from_host(ctx, p, s, b, G, 4))
        xs.append(torch_bf16_from_bits(xb, "cuda:0"))
        refs.append(oracle.matmul_f32(xf, p, s, b, G, 4))
    ys = [torch.full((M, w.N), float("nan"), dtype=torch.bfloat16, device="cuda:0") for w in ws]
    batch = gaf.Batch(ctx, ws, xs, ys)
    assert batch.one_launch
    batch.run()
    ctx.synchronize()
    first = [y.clone() for y in ys]
    for y, ref, w, x in zip(ys, refs, ws, xs):
        assert rel_err(_f32(oracle, y), ref) <= TOL_BF16
        single = gaf.linear(ctx, w, x)
        ctx.synchronize()
        assert rel_err(_f32(oracle, y), _f32(oracle, single)) <= TOL_BF16
    for rep in range(3):                       # counters and tagged words are back at zero: same bits every run
        for y in ys:
            y.fill_(float("nan"))
        batch.run()
        ctx.synchronize()
        for y, f in zip(ys, first):
            assert torch.equal(y, f), rep
    batch.close()
    for w in ws:
        w.free()


def test_dependent_pair_and_graph_replay(gaf, oracle):
    """x of the second operation is the first one's output (depends = [0, 1]): the second waits for the first to be
    complete on the whole GPU.  Also replayed from a CUDA graph."""
    import torch
    stream = torch.cuda.Stream()
    ctx = gaf.Context(0, stream=stream.cuda_stream)
    try:
        d, h, G, M = 1024, 4096, 64, 1
        p1, s1, b1 = make_weights(oracle, h, d, G, 4, seed=1)
        p2, s2, b2 = make_weights(oracle, d, h, G, 4, seed=2)
        xb, xf = make_x_bf16(oracle, M, d, seed=3)
        w1, w2 = gaf.Weight.from_host(ctx, p1, s1, b1, G, 4), gaf.Weight.from_host(ctx, p2, s2, b2, G, 4)
        with torch.cuda.stream(stream):
            x = torch_bf16_from_bits(xb, "cuda:0")
            mid = torch.zeros((M, h), dtype=torch.bfloat16, device="cuda:0")
            y = torch.zeros((M, d), dtype=torch.bfloat16, device="cuda:0")
            batch = gaf.Batch(ctx, [w1, w2], [x, mid], [mid, y], depends=[0, 1])
            assert batch.one_launch
            batch.run()
            stream.synchronize()
            ctx.synchronize()
            mid_ref = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(oracle.matmul_f32(xf, p1, s1, b1, G, 4)))
            assert rel_err(_f32(oracle, mid), mid_ref) <= TOL_BF16
            y_ref = oracle.matmul_f32(_f32(oracle, mid), p2, s2, b2, G, 4)    # from the GPU's own intermediate: one linear's budget
            assert rel_err(_f32(oracle, y), y_ref) <= TOL_BF16
            y0 = y.clone()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                batch.run()
            for rep in range(3):
                y.zero_()
                mid.zero_()
                g.replay()
                stream.synchronize()
                assert torch.equal(y, y0), rep
            del g
        batch.close()
        w1.free()
        w2.free()
    finally:
        ctx.close()


def test_list_that_does_not_qualify_runs_call_by_call(gaf, ctx, oracle):
    """Mixed code widths (and M > 4): not one launch, same results, same entry points."""
    import torch
    pa, sa, ba = make_weights(oracle, 512, 1024, 64, 4, seed=7)
    pb, sb, bb = make_weights(oracle, 256, 1024, 32, 8, seed=8)
    wa, wb = gaf.Weight.from_host(ctx, pa, sa, ba, 64, 4), gaf.Weight.from_host(ctx, pb, sb, bb, 32, 8)
    for M in (1, 6):
        xb, xf = make_x_bf16(oracle, M, 1024, seed=9 + M)
        x = torch_bf16_from_bits(xb, "cuda:0")
        ya = torch.zeros((M, 512), dtype=torch.bfloat16, device="cuda:0")
        yb = torch.zeros((M, 256), dtype=torch.bfloat16, device="cuda:0")
        batch = gaf.Batch(ctx, [wa, wb], [x, x], [ya, yb])
        assert not batch.one_launch
        batch.run()
        ctx.synchronize()
        assert rel_err(_f32(oracle, ya), oracle.matmul_f32(xf, pa, sa, ba, 64, 4)) <= TOL_BF16
        assert rel_err(_f32(oracle, yb), oracle.matmul_f32(xf, pb, sb, bb, 32, 8)) <= TOL_BF16
        batch.close()
    with pytest.raises(gaf.GafError):
        gaf.Batch(ctx, [wa, wb], [x, x], [ya, yb], depends=[1, 0])      # the first operation cannot depend on anything
    wa.free()
    wb.free()


def test_list_with_sums_over_the_ranks_on_a_one_rank_communicator(gaf, oracle):
    """reduce flags on a communicator of ONE rank: the exchange code of the launch list runs (push to the own region,
    wait for the own words, add, write y), including the form in which an operation's wait for its words is put off
    to the end of the following independent operation, and many replays go round all data phases of the exchange."""
    import torch
    c = gaf.Context(0)
    try:
        try:
            c.comm_init(gaf.make_comm_id(), 0, 1)
        except gaf.GafError as e:
            pytest.skip(f"no NCCL on this machine: {e}")
        assert c.uses_peer_memory()
        G = 64
        shapes = [(1024, 2048), (2048, 1024), (640, 4096), (1024, 2048), (384, 1024)]
        reduce = [1, 0, 1, 1, 0]
        for M in (1, 2):
            ws, xs, refs = [], [], []
            for i, (N, K) in enumerate(shapes):
                p, s, b = make_weights(oracle, N, K, G, 4, seed=300 + i)
                xb, xf = make_x_bf16(oracle, M, K, seed=400 + i + M)
                ws.append(gaf.Weight.from_host(c, p, s, b, G, 4))
                xs.append(torch_bf16_from_bits(xb, "cuda:0"))
                refs.append(oracle.matmul_f32(xf, p, s, b, G, 4))
            ys = [torch.full((M, w.N), float("nan"), dtype=torch.bfloat16, device="cuda:0") for w in ws]
            batch = gaf.Batch(c, ws, xs, ys, reduce=reduce)
            assert batch.one_launch
            first = None
            for rep in range(9):
                for y in ys:
                    y.fill_(float("nan"))
                batch.run()
                c.synchronize()
                if first is None:
                    first = [y.clone() for y in ys]
                    for y, ref in zip(ys, refs):
                        assert rel_err(_f32(oracle, y), ref) <= TOL_BF16
                else:
                    for y, f in zip(ys, first):
                        assert torch.equal(y, f), rep
            batch.close()
            for w in ws:
                w.free()
    finally:
        c.close()


def test_recorded_host_batch_is_two_block_copies_around_one_launch(gaf, oracle):
    """tgaf_host_batch_create on page-locked buffers: views of ONE block travel as one copy each way around one
    launch list; separate allocations still work (one copy per buffer).  New activations in the same buffers give
    new results on the next submit."""
    import torch
    stream = torch.cuda.Stream()
    c = gaf.Context(0, stream=stream.cuda_stream)
    try:
        G, M = 64, 1
        shapes = [(1000, 2048), (2048, 1024), (384, 4096)]
        ws, prm = [], []
        for i, (N, K) in enumerate(shapes):
            p, s, b = make_weights(oracle, N, K, G, 4, seed=500 + i)
            ws.append(gaf.Weight.from_host(c, p, s, b, G, 4))
            prm.append((p, s, b))
        xn, yn = sum(M * w.K for w in ws), sum(M * w.N for w in ws)
        for one_block in (True, False):
            if one_block:
                hx = torch.zeros(xn, dtype=torch.int16).pin_memory().numpy().view(np.uint16)
                hy = torch.zeros(yn, dtype=torch.int16).pin_memory().numpy().view(np.uint16)
                xv, yv, xo, yo = [], [], 0, 0
                for w in ws:
                    xv.append(hx[xo: xo + M * w.K].reshape(M, w.K))
                    yv.append(hy[yo: yo + M * w.N].reshape(M, w.N))
                    xo, yo = xo + M * w.K, yo + M * w.N
            else:
                xv = [torch.zeros((M, w.K), dtype=torch.int16).pin_memory().numpy().view(np.uint16) for w in ws]
                yv = [torch.zeros((M, w.N), dtype=torch.int16).pin_memory().numpy().view(np.uint16) for w in ws]
            hb = gaf.HostBatch(c, ws, xv, yv).record()
            assert hb.one_launch
            for rep in range(3):
                xfs = []
                for i, (w, x) in enumerate(zip(ws, xv)):
                    xb, xf = make_x_bf16(oracle, M, w.K, seed=600 + 10 * rep + i)
                    x[...] = xb
                    xfs.append(xf)
                for y in yv:
                    y[...] = 0
                hb.submit()
                c.synchronize()
                for (p, s, b), xf, y in zip(prm, xfs, yv):
                    assert rel_err(oracle.bf16_to_f32(y), oracle.matmul_f32(xf, p, s, b, G, 4)) <= TOL_BF16, (one_block, rep)
            hb.close()
        for w in ws:
            w.free()
    finally:
        c.close()


@pytest.mark.parametrize("M", [1, 3, 5, 8])
def test_full_grid_list_takes_its_activations_through_the_ring(gaf, ctx, oracle, M):
    """Llama-3-8B FFN shapes on all SMs: every operation gives each CTA dozens of units, so the launch quantises the
    activations once at its start and the copy warps stream them into the ring stages beside the weights (one
    activation row: integer-dot instance; three: the int8-MMA instance with an unused fourth row; five and eight: its
    two-column-set form, which exists for such lists only).  Every output against the oracle; same bits on every run."""
    import torch
    G = 64
    shapes = [(28672, 4096), (4096, 14336), (20480, 4608)]
    ws, xs, refs = [], [], []
    for i, (N, K) in enumerate(shapes):
        p, s, b = make_weights(oracle, N, K, G, 4, seed=700 + i)
        xb, xf = make_x_bf16(oracle, M, K, seed=800 + i + M)
        ws.append(gaf.Weight.from_host(ctx, p, s, b, G, 4))
        xs.append(torch_bf16_from_bits(xb, "cuda:0"))
        refs.append(oracle.matmul_f32(xf, p, s, b, G, 4))
    ys = [torch.full((M, w.N), float("nan"), dtype=torch.bfloat16, device="cuda:0") for w in ws]
    batch = gaf.Batch(ctx, ws, xs, ys)
    assert batch.one_launch
    first = None
    for rep in range(4):
        for y in ys:
            y.fill_(float("nan"))
        batch.run()
        ctx.synchronize()
        if first is None:
            first = [y.clone() for y in ys]
            for y, ref in zip(ys, refs):
                assert rel_err(_f32(oracle, y), ref) <= TOL_BF16
        else:
            for y, f in zip(ys, first):
                assert torch.equal(y, f), rep
    batch.close()
    for w in ws:
        w.free()


@pytest.mark.parametrize("M", [1, 3])
def test_list_whose_operations_have_fewer_units_than_the_grid(gaf, ctx, oracle, M):
    """One grid serves the whole list, sized for its largest operation: in the small operations (4, 32 and 128 units of
    128 rows x 256 packed bytes against a grid of 148 CTAs) some CTAs have no units and pass straight on, and the
    ranges with one unit more rotate from operation to operation.  The second half repeats the list with the second
    operation reading the first one's output (the grid-wide counter between them is reached by every CTA, with or
    without units).  Every output against the oracle; same bits on every run."""
    import torch
    G = 64
    shapes = [(8192, 8192), (256, 1024), (1024, 2048), (8192, 1024), (20480, 4608)]
    ws, xs, refs = [], [], []
    for i, (N, K) in enumerate(shapes):
        p, s, b = make_weights(oracle, N, K, G, 4, seed=1100 + i)
        xb, xf = make_x_bf16(oracle, M, K, seed=1200 + i + M)
        ws.append(gaf.Weight.from_host(ctx, p, s, b, G, 4))
        xs.append(torch_bf16_from_bits(xb, "cuda:0"))
        refs.append(oracle.matmul_f32(xf, p, s, b, G, 4))
    ys = [torch.full((M, w.N), float("nan"), dtype=torch.bfloat16, device="cuda:0") for w in ws]
    batch = gaf.Batch(ctx, ws, xs, ys)
    assert batch.one_launch
    first = None
    for rep in range(4):
        for y in ys:
            y.fill_(float("nan"))
        batch.run()
        ctx.synchronize()
        if first is None:
            first = [y.clone() for y in ys]
            for y, ref in zip(ys, refs):
                assert rel_err(_f32(oracle, y), ref) <= TOL_BF16
        else:
            for y, f in zip(ys, first):
                assert torch.equal(y, f), rep
    batch.close()
    # a chain through small operations: y0 = W[8192 x 1024] x0 (128 units), y1 = W[2048 x 8192] y0, y2 = W[1024 x 2048] y1 (32 units)
    pm, sm, bm = make_weights(oracle, 2048, 8192, G, 4, seed=1300)
    mid_w = gaf.Weight.from_host(ctx, pm, sm, bm, G, 4)
    y0 = torch.full((M, 8192), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    y1 = torch.full((M, 2048), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    y2 = torch.full((M, 1024), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    chain = gaf.Batch(ctx, [ws[3], mid_w, ws[2]], [xs[3], y0, y1], [y0, y1, y2], depends=[0, 1, 1])
    assert chain.one_launch
    p2, s2, b2 = make_weights(oracle, 1024, 2048, G, 4, seed=1100 + 2)
    kept = None
    for rep in range(3):
        for y in (y0, y1, y2):
            y.fill_(float("nan"))
        chain.run()
        ctx.synchronize()
        if kept is None:
            kept = [y.clone() for y in (y0, y1, y2)]
            assert rel_err(_f32(oracle, y0), refs[3]) <= TOL_BF16
            # each link from the GPU's own input: one linear's budget
            assert rel_err(_f32(oracle, y1), oracle.matmul_f32(_f32(oracle, y0), pm, sm, bm, G, 4)) <= TOL_BF16
            assert rel_err(_f32(oracle, y2), oracle.matmul_f32(_f32(oracle, y1), p2, s2, b2, G, 4)) <= TOL_BF16
        else:
            for y, f in zip((y0, y1, y2), kept):
                assert torch.equal(y, f), rep
    chain.close()
    mid_w.free()
    for w in ws:
        w.free()


@pytest.mark.parametrize("M", [1, 2, 4])
def test_list_of_8bit_weights(gaf, ctx, oracle, M):
    """gaf8_64 weights: one launch of the integer kernel's 8-bit instances (dot products at one row, the int8 MMA on the
    code bytes above; activations through the ring stages where the operation is large enough); against the oracle."""
    import torch
    G = 64
    shapes = [(4096, 4096), (1000, 2048), (8192, 4096), (512, 14336)]
    ws, xs, refs = [], [], []
    for i, (N, K) in enumerate(shapes):
        p, s, b = make_weights(oracle, N, K, G, 8, seed=900 + i)
        xb, xf = make_x_bf16(oracle, M, K, seed=950 + i + M)
        ws.append(gaf.Weight.from_host(ctx, p, s, b, G, 8))
        xs.append(torch_bf16_from_bits(xb, "cuda:0"))
        refs.append(oracle.matmul_f32(xf, p, s, b, G, 8))
    ys = [torch.full((M, w.N), float("nan"), dtype=torch.bfloat16, device="cuda:0") for w in ws]
    batch = gaf.Batch(ctx, ws, xs, ys)
    assert batch.one_launch
    for rep in range(3):
        for y in ys:
            y.fill_(float("nan"))
        batch.run()
        ctx.synchronize()
        for y, ref in zip(ys, refs):
            assert rel_err(_f32(oracle, y), ref) <= TOL_BF16, rep
    batch.close()
    for w in ws:
        w.free()
