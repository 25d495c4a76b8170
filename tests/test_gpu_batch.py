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
