"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Bit-exact for dequantized weights; matmul
within the stated tolerance (written beside each check)."""
import json

import numpy as np
import pytest

from helpers import (TOL_BF16, TOL_F32, bits_from_torch_bf16, make_weights, make_x_bf16, rel_err,
                     torch_bf16_from_bits)

pytestmark = pytest.mark.gpu

SCHEMES = [(4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)]


@pytest.fixture(scope="module")
def gaf():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import talu_b200
    return talu_b200


@pytest.fixture(scope="module")
def ctx(gaf):
    c = gaf.Context(0)
    yield c
    c.close()


def _run_bf16(gaf, ctx, oracle, N, K, G, bits, M, seed=0, host=False):
    import torch
    p, s, b = make_weights(oracle, N, K, G, bits, seed)
    xb, xf = make_x_bf16(oracle, M, K, seed + 1)
    w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
    if host:
        y_bits = gaf.linear_host(ctx, w, xb)
    else:
        x = torch_bf16_from_bits(xb, "cuda:0")
        y = gaf.linear(ctx, w, x)
        ctx.synchronize()
        y_bits = bits_from_torch_bf16(y)
    w.free()
    ref = oracle.matmul_f32(xf, p, s, b, G, bits)
    ref_bf16 = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(ref))
    return oracle.bf16_to_f32(y_bits), ref_bf16


@pytest.mark.parametrize("bits,G", SCHEMES)
def test_dequant_bit_exact(gaf, ctx, oracle, bits, G):
    """Dequantized weights are bit-exact with the reference CPU dequant."""
    N, K = 257, 16 * G
    p, s, b = make_weights(oracle, N, K, G, bits, seed=bits + G)
    w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
    d_host = gaf.dequant_f32_host(ctx, w)
    d_dev = gaf.dequant_f32(ctx, w)
    ctx.synchronize()
    ref = oracle.dequant_f32(p, s, b, G, bits)
    assert (d_host.view(np.uint32) == ref.view(np.uint32)).all()
    assert (d_dev.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()
    w.free()


def test_dequant_bit_exact_f16_scales_and_4096(gaf, ctx, oracle):
    """Scheme sweep shape (K = N = 4096) and f16 scale/bias patterns."""
    rng = np.random.default_rng(5)
    for bits, G in SCHEMES:
        p, s, b = make_weights(oracle, 4096, 4096, G, bits, seed=11)
        w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
        d = gaf.dequant_f32_host(ctx, w)
        ref = oracle.dequant_f32(p, s, b, G, bits)
        assert (d.view(np.uint32) == ref.view(np.uint32)).all(), (bits, G)
        w.free()
    p, _, _ = make_weights(oracle, 64, 256, 64, 4, seed=3)
    s16 = rng.standard_normal((64, 4)).astype(np.float16).view(np.uint16)
    b16 = rng.standard_normal((64, 4)).astype(np.float16).view(np.uint16)
    w = gaf.Weight.from_host(ctx, p, s16, b16, 64, 4, sdtype=gaf.SCALES_F16)
    d = gaf.dequant_f32_host(ctx, w)
    ref = oracle.dequant_f32(p, s16, b16, 64, 4, sdtype=oracle.SCALES_F16)
    assert (d.view(np.uint32) == ref.view(np.uint32)).all()
    w.free()


def test_reference_known_answers_through_c_abi(gaf, ctx, oracle, kats):
    """The reference's own matmul and CUDA self-test vectors, through the raw
    f32 entry point that mirrors its kernel wrapper."""
    import torch
    from test_oracle_kats import _build_matmul_case, _h
    for k in kats["matmul"]:
        x, packed, scales, biases, want = _build_matmul_case(k)
        dev = "cuda:0"
        tx = torch.from_numpy(x).to(dev)
        tp = torch.from_numpy(packed.view(np.int32)).to(dev)
        ts = torch.from_numpy(scales.view(np.int16)).to(dev)
        tb = torch.from_numpy(biases.view(np.int16)).to(dev)
        out = torch.zeros((k["M"], k["N"]), dtype=torch.float32, device=dev)
        gaf.gaffine_matvec_f32(ctx, k["bits"], tx, tp, ts, tb, out, k["K"], k["N"], k["group"], k["sdtype"], k["M"])
        ctx.synchronize()
        assert np.allclose(out.cpu().numpy(), want, atol=k["tol"]), k["src"]
    for k in kats["cuda_selftest"]:
        dev = "cuda:0"
        tx = torch.tensor(k["input"], dtype=torch.float32, device=dev)
        tp = torch.from_numpy(np.array([_h(w) for w in k["packed"]], np.uint32).view(np.int32)).to(dev)
        ts = torch.from_numpy(np.array([_h(w) for w in k["scales"]], np.uint16).view(np.int16)).to(dev)
        tb = torch.from_numpy(np.array([_h(w) for w in k["biases"]], np.uint16).view(np.int16)).to(dev)
        out = torch.zeros((len(k["input"]), k["out_dim"]), dtype=torch.float32, device=dev)
        gaf.gaffine_matvec_f32(ctx, 4, tx, tp, ts, tb, out, k["in_dim"], k["out_dim"], k["group"], k["sdtype"],
                               len(k["input"]))
        ctx.synchronize()
        assert np.allclose(out.cpu().numpy(), np.array(k["expect"]), atol=k["tol"]), k["src"]


def test_cfg1_gemv_gaf4_64(gaf, ctx, oracle):
    """N=4096, K=1024, M=1, gaf4_64: the reference's CPU-runnable case.  rel <= 1e-2."""
    y, ref = _run_bf16(gaf, ctx, oracle, 4096, 1024, 64, 4, 1, seed=0)
    assert rel_err(y, ref) <= TOL_BF16


@pytest.mark.parametrize("bits,G", SCHEMES)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 8])
def test_cfg3_scheme_sweep(gaf, ctx, oracle, bits, G, M):
    """K = N = 4096, M in {1, 8}, every scheme.  rel <= 1e-2."""
    y, ref = _run_bf16(gaf, ctx, oracle, 4096, 4096, G, bits, M, seed=20 + bits + G)
    assert rel_err(y, ref) <= TOL_BF16


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
def test_cfg2_llama8b_ffn(gaf, ctx, oracle, N, K, M):
    """Llama-3-8B FFN shapes (gate/up and down), gaf4_64, M in {1, 4, 16}.  rel <= 1e-2."""
    y, ref = _run_bf16(gaf, ctx, oracle, N, K, 64, 4, M, seed=N % 97)
    assert rel_err(y, ref) <= TOL_BF16


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 15, 16, 17, 33])
def test_ragged_shapes(gaf, ctx, oracle, M):
    """Row counts around the tile edges, N not a multiple of 16 (and odd)."""
    for N, K, G, bits in [(3, 256, 64, 4), (17, 512, 32, 4), (1001, 1024, 128, 4), (31, 256, 32, 8), (130, 768, 64, 8)]:
        y, ref = _run_bf16(gaf, ctx, oracle, N, K, G, bits, M, seed=M)
        assert rel_err(y, ref) <= TOL_BF16, (N, K, G, bits, M)


def test_f32_contract(gaf, ctx, oracle):
    """The reference's f32-in / f32-out contract, tolerance 1e-3 (its policy for f32 matmul)."""
    import torch
    for bits, G, N, K, M in [(4, 64, 1024, 2048, 1), (4, 32, 515, 1024, 7), (8, 64, 512, 1024, 16), (4, 128, 256, 4096, 12),
                             (4, 32, 300, 1024, 12), (4, 32, 300, 1024, 16)]:
        p, s, b = make_weights(oracle, N, K, G, bits, seed=G + M)
        x = np.random.default_rng(M).standard_normal((M, K), dtype=np.float32)
        w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
        y = gaf.linear(ctx, w, torch.from_numpy(x).to("cuda:0"))
        ctx.synchronize()
        y_host = gaf.linear_host(ctx, w, x)
        truth = oracle.matmul_f64(x, p, s, b, G, bits)
        assert rel_err(y.cpu().numpy(), truth) <= TOL_F32, (bits, G, N, K, M)
        assert (y_host == y.cpu().numpy()).all()
        w.free()


def test_generic_kernel_matches(gaf, ctx, oracle):
    """Shapes outside the fast path (group 8 / 16, K = one group) and the forced generic path."""
    for N, K, G, bits, M in [(5, 8, 8, 4, 2), (9, 48, 16, 4, 3), (6, 16, 4, 8, 1), (33, 64, 16, 8, 4)]:
        y, ref = _run_bf16(gaf, ctx, oracle, N, K, G, bits, M, seed=K)
        assert rel_err(y, ref) <= TOL_BF16, (N, K, G, bits, M)
    ctx.set_option("force_generic", 1)
    try:
        y, ref = _run_bf16(gaf, ctx, oracle, 300, 1024, 64, 4, 3, seed=8)
        assert rel_err(y, ref) <= TOL_BF16
    finally:
        ctx.set_option("force_generic", 0)


def test_host_entry_point_equals_device_entry_point(gaf, ctx, oracle):
    yd, ref = _run_bf16(gaf, ctx, oracle, 2048, 1024, 64, 4, 4, seed=2)
    yh, _ = _run_bf16(gaf, ctx, oracle, 2048, 1024, 64, 4, 4, seed=2, host=True)
    assert (yd == yh).all()
    assert rel_err(yh, ref) <= TOL_BF16


def test_queued_host_calls_equal_waited_ones(gaf, ctx, oracle):
    """tgaf_linear_bf16_host_async: several calls queued on page-locked buffers, one wait, same bits as the
    call that waits (the staging buffers are shared between the queued calls in stream order)."""
    import torch
    ws, xs, want = [], [], []
    for i, (N, K, M) in enumerate([(1000, 2048, 1), (384, 1024, 3), (2048, 512, 16)]):
        p, s, b = make_weights(oracle, N, K, 64, 4, seed=60 + i)
        w = gaf.Weight.from_host(ctx, p, s, b, 64, 4)
        xb, _ = make_x_bf16(oracle, M, K, 70 + i)
        want.append(gaf.linear_host(ctx, w, xb).copy())
        ws.append(w)
        xs.append(xb)
    pinned_x = [torch.from_numpy(x.view(np.int16)).pin_memory() for x in xs]
    pinned_y = [torch.empty((x.shape[0], w.N), dtype=torch.int16).pin_memory() for x, w in zip(xs, ws)]
    for rep in range(2):
        for y in pinned_y:
            y.zero_()
        for w, x, y in zip(ws, pinned_x, pinned_y):
            gaf.linear_host(ctx, w, x.numpy().view(np.uint16), out=y.numpy().view(np.uint16), wait=False)
        ctx.synchronize()
        for y, ref in zip(pinned_y, want):
            assert np.array_equal(y.numpy().view(np.uint16), ref), rep
    # the same list through one crossing of the ABI
    batch = gaf.HostBatch(ctx, ws, [x.numpy().view(np.uint16) for x in pinned_x], [y.numpy().view(np.uint16) for y in pinned_y])
    for rep in range(3):
        for y in pinned_y:
            y.zero_()
        batch.submit()
        ctx.synchronize()
        for y, ref in zip(pinned_y, want):
            assert np.array_equal(y.numpy().view(np.uint16), ref), rep
    # ... and recorded once, replayed per step: needs a context on a stream of its own
    with pytest.raises(gaf.GafError):
        batch.record()                      # this context runs on torch's default stream
    stream = torch.cuda.Stream()
    ctx2 = gaf.Context(0, stream=stream.cuda_stream)
    try:
        batch2 = gaf.HostBatch(ctx2, ws, [x.numpy().view(np.uint16) for x in pinned_x],
                               [y.numpy().view(np.uint16) for y in pinned_y]).record()
        for rep in range(3):
            for y in pinned_y:
                y.zero_()
            batch2.submit()
            ctx2.synchronize()
            for y, ref in zip(pinned_y, want):
                assert np.array_equal(y.numpy().view(np.uint16), ref), rep
        batch2.close()
    finally:
        ctx2.close()
    for w in ws:
        w.free()


def test_split_k_is_deterministic_and_tunable(gaf, ctx, oracle):
    """Any number of persistent CTAs (hence any cut of row groups across CTAs) agrees
    within tolerance, and a given cut gives the same bits on every run (partials are
    added in slot order)."""
    import torch
    p, s, b = make_weights(oracle, 520, 8192, 64, 4, seed=4)
    xb, xf = make_x_bf16(oracle, 3, 8192, 9)
    w = gaf.Weight.from_host(ctx, p, s, b, 64, 4)
    x = torch_bf16_from_bits(xb, "cuda:0")
    ref = oracle.matmul_f32(xf, p, s, b, 64, 4)
    try:
        with pytest.raises(gaf.GafError) as ei:      # more CTAs than SMs could not all be resident: refused
            ctx.set_option("gemv_ctas", 500)
        assert ei.value.invalid_argument
        for ctas in [0, 1, 2, 3, 7, 33, 79, 80, 148]:
            ctx.set_option("gemv_ctas", ctas)
            y1 = gaf.linear(ctx, w, x).clone()
            y2 = gaf.linear(ctx, w, x).clone()
            ctx.synchronize()
            assert torch.equal(y1, y2), ctas
            assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y1)), ref) <= TOL_BF16, ctas
    finally:
        ctx.set_option("gemv_ctas", 0)
    w.free()


def test_next_weight_hint_changes_no_result(gaf, ctx, oracle):
    """The next-weight hint only warms L2: with it, without it, at any depth, with a next weight of
    another scheme, or with a hinted weight that is freed before the call, outputs keep their bits."""
    import torch
    pa, sa, ba = make_weights(oracle, 1000, 2048, 64, 4, seed=21)
    pb, sb, bb = make_weights(oracle, 300, 1024, 32, 8, seed=22)
    wa = gaf.Weight.from_host(ctx, pa, sa, ba, 64, 4)
    wb = gaf.Weight.from_host(ctx, pb, sb, bb, 32, 8)
    try:
        for M in (1, 2, 5, 16):
            xab, xaf = make_x_bf16(oracle, M, 2048, 30 + M)
            xbb, xbf = make_x_bf16(oracle, M, 1024, 40 + M)
            xa, xb = torch_bf16_from_bits(xab, "cuda:0"), torch_bf16_from_bits(xbb, "cuda:0")
            ya0, yb0 = gaf.linear(ctx, wa, xa).clone(), gaf.linear(ctx, wb, xb).clone()
            assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(ya0)), oracle.matmul_f32(xaf, pa, sa, ba, 64, 4)) <= TOL_BF16
            assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(yb0)), oracle.matmul_f32(xbf, pb, sb, bb, 32, 8)) <= TOL_BF16
            for depth in (0, 1, 3, 4096):
                ctx.set_option("prefetch_units", depth)
                gaf.hint_next_weight(ctx, wb)
                ya = gaf.linear(ctx, wa, xa)
                gaf.hint_next_weight(ctx, wa)
                yb = gaf.linear(ctx, wb, xb)
                ctx.synchronize()
                assert torch.equal(ya, ya0) and torch.equal(yb, yb0), (M, depth)
        # a hint whose weight goes away before the call is dropped with it
        pc, sc, bc = make_weights(oracle, 128, 512, 64, 4, seed=23)
        wc = gaf.Weight.from_host(ctx, pc, sc, bc, 64, 4)
        gaf.hint_next_weight(ctx, wc)
        wc.free()
        ya = gaf.linear(ctx, wa, xa)
        ctx.synchronize()
        assert torch.equal(ya, ya0)
    finally:
        ctx.set_option("prefetch_units", 2)
        gaf.hint_next_weight(ctx, None)
    wa.free()
    wb.free()


def test_one_rank_communicator_runs_the_peer_memory_kernels(gaf, oracle):
    """A communicator of one rank still takes the peer-memory paths (its own region is the only slot), so the
    all-reduce kernel and the GEMV with the all-reduce fused into its write-out are exercised on one GPU:
    a sum over one rank must return the operand's bits, call after call (both exchange phases)."""
    import torch
    ctx1 = gaf.Context(0)
    try:
        try:
            ctx1.comm_init(gaf.make_comm_id(), 0, 1)
        except gaf.GafError as e:  # no libnccl: nothing to test
            pytest.skip(f"no NCCL on this machine: {e}")
        assert ctx1.uses_peer_memory()
        for it, (n, dt) in enumerate([(8192, torch.bfloat16), (8, torch.bfloat16), (4096, torch.float32),
                                      (8192 * 16, torch.bfloat16), (24, torch.bfloat16), (8192 * 16, torch.float32)] * 2):
            t = (torch.randn(n, device="cuda") * (1 + it)).to(dt)
            want = t.clone()
            ctx1.allreduce(t)
            ctx1.synchronize()
            assert torch.equal(t, want), (it, n, dt)
        big = torch.randn(1 << 20, device="cuda")          # larger than a slot: the library collective
        want = big.clone()
        ctx1.allreduce(big)
        ctx1.synchronize()
        assert torch.equal(big, want)
        for (N, K, G) in [(8192, 1024, 64), (300, 2048, 64), (4096, 3584, 128), (1000, 512, 32)]:
            p, s, b = make_weights(oracle, N, K, G, 4, seed=N + K)
            w = gaf.Weight.from_host(ctx1, p, s, b, G, 4)
            for M in (1, 2, 4):
                xb, xf = make_x_bf16(oracle, M, K, 5 + M)
                x = torch_bf16_from_bits(xb, "cuda:0")
                y0 = gaf.linear(ctx1, w, x).clone()
                for rep in range(3):
                    y1 = gaf.linear_allreduce(ctx1, w, x)
                    ctx1.synchronize()
                    assert torch.equal(y0, y1), (N, K, G, M, rep)
                for ctas in (1, 7, 148):
                    ctx1.set_option("gemv_ctas", ctas)
                    y2 = gaf.linear_allreduce(ctx1, w, x)
                    ctx1.synchronize()
                    ctx1.set_option("gemv_ctas", 0)
                    assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y2)), oracle.matmul_f32(xf, p, s, b, G, 4)) <= TOL_BF16
            w.free()
        # the FFN operator with the sum over ranks riding in its down projection (one launch at M = 1)
        pg, sg, bg = make_weights(oracle, 2 * 1024, 512, 64, 4, seed=77)
        pd, sd, bd = make_weights(oracle, 512, 1024, 64, 4, seed=78)
        wgu, wd = gaf.Weight.from_host(ctx1, pg, sg, bg, 64, 4), gaf.Weight.from_host(ctx1, pd, sd, bd, 64, 4)
        for M in (1, 2):
            xb, _ = make_x_bf16(oracle, M, 512, 90 + M)
            x = torch_bf16_from_bits(xb, "cuda:0")
            y0 = gaf.ffn_swiglu(ctx1, wgu, wd, x).clone()
            for rep in range(3):
                y1 = gaf.ffn_swiglu(ctx1, wgu, wd, x, allreduce=True)
                ctx1.synchronize()
                assert torch.equal(y0, y1), (M, rep)
        wgu.free()
        wd.free()
        ctx1._lib.tgaf_comm_destroy(ctx1._h)
    finally:
        ctx1.close()


@pytest.mark.parametrize("d_model,d_ff,G", [(512, 1024, 64), (1024, 2816, 64), (256, 384, 32), (4096, 14336, 64), (512, 1536, 128)])
def test_ffn_swiglu_operator(gaf, ctx, oracle, d_model, d_ff, G):
    """The FFN operator (gate|up, silu-mul, down) against the oracle's restatement of SwiGLU.forward: the
    one-launch path (M <= 2), the three-kernel path (M = 5, and M = 1 with the option off) and repeat calls."""
    import torch
    pg, sg, bg = make_weights(oracle, 2 * d_ff, d_model, G, 4, seed=d_ff)
    pd, sd, bd = make_weights(oracle, d_model, d_ff, G, 4, seed=d_ff + 1)
    wgu = gaf.Weight.from_host(ctx, pg, sg, bg, G, 4)
    wd = gaf.Weight.from_host(ctx, pd, sd, bd, G, 4)
    try:
        for M in (1, 2, 5):
            xb, xf = make_x_bf16(oracle, M, d_model, 50 + M)
            xf = xf * 8.0   # weights of N(0, 0.02^2): larger activations put the gate values where silu bends
            xb = oracle.f32_to_bf16_rne(xf)
            xf = oracle.bf16_to_f32(xb)
            ref = oracle.ffn_swiglu_f32(xf, (pg, sg, bg), (pd, sd, bd), G, 4)
            x = torch_bf16_from_bits(xb, "cuda:0")
            y1 = gaf.ffn_swiglu(ctx, wgu, wd, x).clone()
            y2 = gaf.ffn_swiglu(ctx, wgu, wd, x).clone()
            ctx.set_option("ffn_one_launch", 0)
            y3 = gaf.ffn_swiglu(ctx, wgu, wd, x).clone()
            ctx.set_option("ffn_one_launch", 1)
            ctx.synchronize()
            assert torch.equal(y1, y2), M
            # two chained linears + activation: twice the per-linear bf16 budget
            for y in (y1, y3):
                assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), ref) <= 2 * TOL_BF16, (M, d_model, d_ff)
    finally:
        ctx.set_option("ffn_one_launch", 1)
    wgu.free()
    wd.free()


def test_linearity_at_full_size(gaf, ctx, oracle):
    """Size-independent property at the benchmark's full shape: y(2x) = 2 y(x) exactly
    (scaling by two is exact in bf16 and in every partial sum)."""
    import torch
    N, K = 14336, 4096
    p, s, b = make_weights(oracle, N, K, 64, 4, seed=6)
    xb, _ = make_x_bf16(oracle, 4, K, 3)
    w = gaf.Weight.from_host(ctx, p, s, b, 64, 4)
    x = torch_bf16_from_bits(xb, "cuda:0")
    y1 = gaf.linear(ctx, w, x)
    y2 = gaf.linear(ctx, w, x * 2)
    ctx.synchronize()
    assert torch.equal(y1 * 2, y2)
    w.free()


def test_invalid_arguments_are_status_codes(gaf, ctx, oracle):
    """Host-side validation mirrors the reference wrapper's tests
    (gaffine_u4_matvec.zig:145-170): bad group alignment, bad dtype tag, zero rows."""
    import torch
    dev = "cuda:0"
    buf = torch.zeros(4096, dtype=torch.float32, device=dev)
    for args in [(16, 8, 12, 1, 1), (16, 8, 8, 7, 1), (16, 8, 8, 1, 0)]:
        with pytest.raises(gaf.GafError) as ei:
            gaf.gaffine_matvec_f32(ctx, 4, buf, buf, buf, buf, buf, *args)
        assert ei.value.invalid_argument
    p, s, b = make_weights(oracle, 8, 64, 32, 4)
    with pytest.raises(gaf.GafError):
        gaf.Weight.from_host(ctx, p, s, b, 12, 4)            # group not a multiple of 8
    with pytest.raises(gaf.GafError):
        gaf.Weight.from_host(ctx, p, s, b, 32, 4, sdtype=5)  # bad scales dtype
    with pytest.raises(gaf.GafError):
        gaf.Weight.from_host(ctx, p, s, b, 32, 5)            # bits
    w = gaf.Weight.from_host(ctx, p, s, b, 32, 4)
    with pytest.raises(gaf.GafError):
        gaf.linear(ctx, w, torch.zeros((2, 32), dtype=torch.bfloat16, device=dev))  # wrong K
    w.free()
    # the context is still usable after every rejected call
    y, ref = _run_bf16(gaf, ctx, oracle, 64, 256, 64, 4, 1)
    assert rel_err(y, ref) <= TOL_BF16


@pytest.mark.parametrize("P", [2, 4, 8])
def test_tensor_parallel_shards_on_one_gpu(gaf, ctx, oracle, P):
    """tgaf_weight_upload's column / row sharding: every rank's shard is uploaded in turn on
    this one GPU; column-parallel outputs are concatenated, row-parallel partials are summed
    on the host, and both must match the unsharded oracle.  rel <= 1e-2."""
    import torch
    from talu_b200 import tp
    G, bits, M = 64, 4, 2
    hidden, ffn = 1024, 2048
    up = make_weights(oracle, ffn, hidden, G, bits, seed=31)
    down = make_weights(oracle, hidden, ffn, G, bits, seed=32)
    xb, xf = make_x_bf16(oracle, M, hidden, seed=33)
    x = torch_bf16_from_bits(xb, "cuda:0")
    # column-parallel: rows of `up`
    h_parts = []
    for r in range(P):
        w = gaf.Weight.from_host(ctx, *up, G, bits, shard=gaf.SHARD_COL, tp_rank=r, tp_size=P)
        assert (w.N, w.K) == (ffn // P, hidden)
        h_parts.append(gaf.linear(ctx, w, x))
        ctx.synchronize()
        w.free()
    h = torch.cat(h_parts, dim=1)
    h_ref = oracle.matmul_f32(xf, *up, G, bits)
    assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(h)), h_ref) <= TOL_BF16
    # row-parallel: columns of `down`, fed with the matching slice of h (f32 entry point: exact partial sums)
    hf = oracle.bf16_to_f32(bits_from_torch_bf16(h))
    y = np.zeros((M, hidden), np.float64)
    for r in range(P):
        w = gaf.Weight.from_host(ctx, *down, G, bits, shard=gaf.SHARD_ROW, tp_rank=r, tp_size=P)
        assert (w.N, w.K) == (hidden, ffn // P)
        sl = tp.shard_slice(hidden, ffn, G, bits, tp.SHARD_ROW, r, P)
        part = gaf.linear_host(ctx, w, np.ascontiguousarray(hf[:, sl.k0:sl.k1]))
        y += part
        w.free()
    y_ref = oracle.matmul_f64(hf, *down, G, bits)
    assert rel_err(y, y_ref) <= TOL_F32
    with pytest.raises(gaf.GafError):
        gaf.Weight.from_host(ctx, *down, G, bits, shard=gaf.SHARD_ROW, tp_rank=0, tp_size=5)   # K not divisible
    with pytest.raises(gaf.GafError):
        gaf.Weight.from_host(ctx, *up, G, bits, shard=gaf.SHARD_COL, tp_rank=3, tp_size=3)     # rank out of range


def _prefill_case(gaf, ctx, oracle, M, N, K, G, seed):
    import torch
    p, s, b = make_weights(oracle, N, K, G, 4, seed)
    xb, xf = make_x_bf16(oracle, M, K, seed + 1)
    w = gaf.Weight.from_host(ctx, p, s, b, G, 4)
    y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
    ctx.synchronize()
    got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
    w.free()
    ref = oracle.matmul_f32(xf, p, s, b, G, 4)
    return got, ref


@pytest.mark.parametrize("M,N,K,G", [(17, 256, 128, 64), (64, 1024, 2048, 64), (100, 300, 512, 128), (129, 256, 256, 32),
                                     (256, 256, 128, 64), (128, 512, 1024, 64), (300, 1000, 512, 32),
                                     (515, 768, 2048, 128), (1024, 2048, 4096, 64)])
def test_prefill_tensor_core_gemm(gaf, ctx, oracle, M, N, K, G):
    """Prefill / skinny-M dequant-GEMM (tcgen05 path, M > 16): full tiles, ragged M and N, every group size.
    Weights are rounded to bf16 after the affine (one rounding), fp32 accumulate, bf16 out.  rel <= 1e-2."""
    got, ref = _prefill_case(gaf, ctx, oracle, M, N, K, G, seed=M + N)
    assert rel_err(got, ref) <= TOL_BF16, (M, N, K, G, rel_err(got, ref))


def test_prefill_cfg4_full_size(gaf, ctx, oracle):
    """The prefill benchmark shape: M=2048, K=4096, N=14336, gaf4_64.  rel <= 1e-2 against the CPU oracle
    on every one of the 29M outputs."""
    got, ref = _prefill_case(gaf, ctx, oracle, 2048, 14336, 4096, 64, seed=4)
    assert rel_err(got, ref) <= TOL_BF16, rel_err(got, ref)


def test_8bit_codes_on_the_integer_dot_product_kernel(gaf, ctx, oracle):
    """gaf8_32 / gaf8_64 at one to four bf16 activation rows run on the integer kernel (a packed word IS four unsigned
    bytes: dot products at one and two rows, the int8 MMA at three and four): K split over many CTAs, ragged N, bf16
    and f16 scale patterns; gaf8_128 stays on the tensor-core GEMV.  rel <= 1e-2 against the oracle."""
    rng = np.random.default_rng(5)
    for N, K, G, M, f16 in [(2048, 4096, 64, 1, False), (1000, 8192, 32, 2, False), (4096, 14336, 64, 1, True),
                            (520, 2048, 32, 1, True), (384, 1024, 128, 2, False), (2048, 4096, 64, 4, False),
                            (1000, 8192, 32, 3, True), (4096, 14336, 64, 4, True), (130, 512, 64, 3, False)]:
        p, s, b = make_weights(oracle, N, K, G, 8, seed=N + M)
        sd_lib, sd_or = gaf.SCALES_BF16, oracle.SCALES_BF16
        if f16:
            s = (oracle.bf16_to_f32(s) * (1 + rng.uniform(0, 2 ** -8, s.shape))).astype(np.float16).view(np.uint16)
            b = (oracle.bf16_to_f32(b) * (1 + rng.uniform(0, 2 ** -8, b.shape))).astype(np.float16).view(np.uint16)
            sd_lib, sd_or = gaf.SCALES_F16, oracle.SCALES_F16
        xb, xf = make_x_bf16(oracle, M, K, seed=M + 3)
        w = gaf.Weight.from_host(ctx, p, s, b, G, 8, sdtype=sd_lib)
        y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
        ctx.synchronize()
        ref = oracle.matmul_f32(xf, p, s, b, G, 8, sdtype=sd_or)
        assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), ref) <= TOL_BF16, (N, K, G, M, f16)
        w.free()


def test_gemm_min_m_option_moves_the_hand_over(gaf, oracle):
    """"gemm_min_m" = the activation rows from which the tensor-core GEMM takes over from the decode GEMVs (default 17).
    With it lowered, M = 5, 8 and 16 run on the GEMM: same results within the same bound."""
    import torch
    c = gaf.Context(0)
    try:
        with pytest.raises(gaf.GafError):
            c.set_option("gemm_min_m", 0)
        with pytest.raises(gaf.GafError):
            c.set_option("gemm_min_m", 18)
        for M, N, K, G in [(5, 300, 1024, 64), (8, 1024, 2048, 32), (16, 512, 4096, 128)]:
            p, s, b = make_weights(oracle, N, K, G, 4, seed=M)
            xb, xf = make_x_bf16(oracle, M, K, seed=M + 1)
            w = gaf.Weight.from_host(c, p, s, b, G, 4)
            x = torch_bf16_from_bits(xb, "cuda:0")
            ref = oracle.matmul_f32(xf, p, s, b, G, 4)
            outs = []
            for mn in (17, 5):
                c.set_option("gemm_min_m", mn)
                y = gaf.linear(c, w, x)
                c.synchronize()
                got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
                assert rel_err(got, ref) <= TOL_BF16, (M, N, K, G, mn)
                outs.append(y)
            w.free()
    finally:
        c.close()


def test_embedding_lookup_and_lm_head(gaf, ctx, oracle):
    """Embedding rows (bit-exact gather-dequant with the multiplier) and the lm_head shape: one GEMV over a
    vocabulary-sized table."""
    import torch
    vocab, hidden, G = 32000, 2048, 64
    p, s, b = make_weights(oracle, vocab, hidden, G, 4, seed=77)
    w = gaf.Weight.from_host(ctx, p, s, b, G, 4)
    ids = np.array([0, 5, 31999, 17, 17, 12345], np.uint32)
    for mult in (1.0, 45.25):
        got = gaf.embedding_lookup_f32(ctx, w, ids, mult)
        ctx.synchronize()
        ref = oracle.gather_dequant_f32(p, s, b, G, 4, ids, mult)
        assert (got.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()
    with pytest.raises(gaf.GafError) as ei:
        gaf.embedding_lookup_f32(ctx, w, [3, vocab])
    assert ei.value.invalid_argument
    # lm_head: logits[1, vocab] = h[1, hidden] @ table^T
    xb, xf = make_x_bf16(oracle, 1, hidden, seed=5)
    y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
    ctx.synchronize()
    ref = oracle.matmul_f32(xf, p, s, b, G, 4)
    assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), ref) <= TOL_BF16
    w.free()
