"""Parity against outputs of the reference ITSELF: its own CUDA kernels for this path
(core/src/compute/cuda/kernels/ops/quant_ops.cu, compiled unchanged into oracle/_ref/ by `make -C oracle ref`)
run on the same GPU under the reference's launch geometry (block 256, grid (ceil(N / 8), M),
core/src/compute/cuda/gaffine_u4_matvec.zig:87-96) on the benchmark's seeded inputs.  These pin the random-data
matmul that none of the reference's tests hold a vector for: the C-ABI entry points, the sideload kernels and
the CPU oracle must all agree with the reference kernel.  Tolerances are written beside each check."""
import numpy as np
import pytest

from helpers import (TOL_BF16, TOL_F32, CubinModule, bits_from_torch_bf16, make_weights, make_x_bf16, matvec_u4,
                     matvec_u4_fused, rel_err, to_dev, torch_bf16_from_bits)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_mod(oracle):
    cubin = oracle.build_ref()
    if cubin is None:
        pytest.skip("oracle/_ref/talu_ref_quant_sm_100.cubin has not been built (needs a talu checkout: make -C oracle ref)")
    return CubinModule(cubin)


@pytest.fixture(scope="module")
def gaf():
    import talu_b200
    return talu_b200


@pytest.fixture(scope="module")
def ctx(gaf):
    c = gaf.Context(0)
    yield c
    c.close()


def _max_rel(y, ref):
    return float(np.abs(np.asarray(y, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


# cfg1 (the reference's CPU-runnable case), one Llama-3-8B gate matrix and its down matrix, the other group sizes
CASES = [(4096, 1024, 64, 1), (14336, 4096, 64, 1), (14336, 4096, 64, 4), (4096, 14336, 64, 2), (4096, 4096, 32, 1),
         (4096, 4096, 128, 8), (1001, 1024, 128, 3)]


@pytest.mark.parametrize("N,K,G,M", CASES)
def test_f32_entry_points_against_the_reference_kernel(gaf, ctx, oracle, ref_mod, N, K, G, M):
    """tgaf_linear_f32, tgaf_gaffine_u4_matvec_f32 (the wrapper-shaped entry) and the CPU oracle against the
    reference kernel on f32 activations: max |y - y_ref| / max |y_ref| <= 1e-3 (the reference's f32 policy)."""
    import torch
    p, s, b = make_weights(oracle, N, K, G, 4, seed=N % 89 + G)
    x = np.random.default_rng(K + M).standard_normal((M, K), dtype=np.float32)
    y_ref = matvec_u4(ref_mod, x, p, s, b, G).astype(np.float64)
    assert np.isfinite(y_ref).all()
    w = gaf.Weight.from_host(ctx, p, s, b, G, 4)
    y1 = gaf.linear(ctx, w, torch.from_numpy(x).cuda())
    dx, dp, ds, db = to_dev(x), to_dev(p), to_dev(s), to_dev(b)
    y2 = torch.zeros((M, N), device="cuda")
    gaf.gaffine_matvec_f32(ctx, 4, dx, dp, ds, db, y2, K, N, G, 1, M)
    ctx.synchronize()
    assert _max_rel(y1.cpu().numpy(), y_ref) <= TOL_F32
    assert _max_rel(y2.cpu().numpy(), y_ref) <= TOL_F32
    # the oracle's restatements: the CUDA kernel's per-element arithmetic, the CPU micro-kernels, the f64 truth
    assert _max_rel(oracle.matvec_cuda_semantics(x, p, s, b, G), y_ref) <= 1e-4
    assert _max_rel(oracle.matmul_f32(x, p, s, b, G, 4), y_ref) <= TOL_F32
    assert _max_rel(oracle.matmul_f64(x, p, s, b, G, 4), y_ref) <= TOL_F32
    w.free()


@pytest.mark.parametrize("N,K,G,M", CASES[:4])
def test_bf16_path_against_the_reference_kernel(gaf, ctx, oracle, ref_mod, N, K, G, M):
    """The bf16 operator (bf16 in, fp32 accumulate, bf16 out) against the reference kernel fed the same
    activations widened to f32, its output rounded to bf16: rel <= 1e-2."""
    p, s, b = make_weights(oracle, N, K, G, 4, seed=N % 89 + G)
    xb, xf = make_x_bf16(oracle, M, K, seed=K + M)
    y_ref = matvec_u4(ref_mod, xf, p, s, b, G)
    y_ref = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(y_ref))
    w = gaf.Weight.from_host(ctx, p, s, b, G, 4)
    y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
    ctx.synchronize()
    assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), y_ref) <= TOL_BF16
    w.free()


def test_sideload_kernels_against_the_reference_kernels(oracle, ref_mod):
    """The three sideload symbols against the reference's kernels of the same names, same arguments, same
    geometry: matvec, fused q|k|v, fused gate|up.  1e-3 of the largest output (f32 in, f32 out)."""
    from talu_b200 import build
    cubin, _ = build.build_sideload()
    ours = CubinModule(cubin)
    rng = np.random.default_rng(17)
    for N, K, G, M in [(4096, 1024, 64, 1), (14336, 4096, 64, 1), (300, 1024, 32, 3)]:
        p, s, b = make_weights(oracle, N, K, G, 4, seed=N % 83)
        x = rng.standard_normal((M, K), dtype=np.float32)
        assert _max_rel(matvec_u4(ours, x, p, s, b, G), matvec_u4(ref_mod, x, p, s, b, G).astype(np.float64)) <= TOL_F32
    for symbol, dims, K in [("talu_gaffine_u4_matvec_qkv_f32", [(4096, 64), (1024, 64), (1024, 64)], 4096),
                            ("talu_gaffine_u4_matvec_gate_up_f32", [(14336, 64), (14336, 64)], 4096),
                            ("talu_gaffine_u4_matvec_qkv_f32", [(100, 32), (37, 128), (64, 64)], 1024)]:
        x = rng.standard_normal((1, K), dtype=np.float32)
        parts = [(*make_weights(oracle, n, K, G, 4, seed=n + i), G) for i, (n, G) in enumerate(dims)]
        got = matvec_u4_fused(ours, symbol, x, parts, K)
        want = matvec_u4_fused(ref_mod, symbol, x, parts, K)
        for a, r in zip(got, want):
            assert np.isfinite(r).all()
            assert _max_rel(a, r.astype(np.float64)) <= TOL_F32, symbol


def test_f16_scales_against_the_reference_kernel(gaf, ctx, oracle, ref_mod):
    """f16 scale / bias patterns (tag 0, core/src/compute/cuda/gaffine_u4_matvec.zig:13-14) through the decode
    GEMVs and the tensor-core GEMM: f32 entry <= 1e-3, bf16 operator <= 1e-2 against the reference kernel."""
    import torch
    rng = np.random.default_rng(23)
    for N, K, G, M in [(1024, 2048, 64, 1), (1024, 2048, 64, 4), (512, 1024, 32, 12), (512, 2048, 128, 64), (768, 1024, 64, 200)]:
        p, s, b = make_weights(oracle, N, K, G, 4, seed=N + M)
        # the same scales / biases as f16 patterns (more mantissa bits than bf16 holds)
        s16 = (oracle.bf16_to_f32(s) * (1 + rng.uniform(0, 2 ** -8, s.shape))).astype(np.float16).view(np.uint16)
        b16 = (oracle.bf16_to_f32(b) * (1 + rng.uniform(0, 2 ** -8, b.shape))).astype(np.float16).view(np.uint16)
        xb, xf = make_x_bf16(oracle, M, K, seed=M)
        y_ref = matvec_u4(ref_mod, xf, p, s16, b16, G, tag=0).astype(np.float64)
        w = gaf.Weight.from_host(ctx, p, s16, b16, G, 4, sdtype=gaf.SCALES_F16)
        y32 = gaf.linear(ctx, w, torch.from_numpy(xf).cuda())
        y16 = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
        ctx.synchronize()
        assert _max_rel(y32.cpu().numpy(), y_ref) <= TOL_F32, (N, K, G, M)
        assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y16)), y_ref) <= TOL_BF16, (N, K, G, M)
        # and the CPU oracle agrees with the reference kernel on f16 patterns too
        assert _max_rel(oracle.matmul_f32(xf, p, s16, b16, G, 4, sdtype=oracle.SCALES_F16), y_ref) <= TOL_F32
        w.free()


def test_embedding_lookup_against_the_reference_kernel(gaf, ctx, oracle, ref_mod):
    """talu_embedding_lookup_gaffine_u4_f32 (quant_ops.cu:12-44; one token per launch, grid ceil(hidden / 256))
    against tgaf_embedding_lookup_f32: the same bits."""
    import torch
    vocab, hidden, G = 1000, 2048, 64
    p, s, b = make_weights(oracle, vocab, hidden, G, 4, seed=71)
    w = gaf.Weight.from_host(ctx, p, s, b, G, 4)
    dp, ds, db = to_dev(p), to_dev(s), to_dev(b)
    ids = [0, 7, 999, 512]
    got = gaf.embedding_lookup_f32(ctx, w, ids, 3.5)
    ctx.synchronize()
    for i, tok in enumerate(ids):
        out = torch.zeros(hidden, device="cuda")
        import ctypes
        fn_args = (out, dp, ds, db, vocab, hidden, tok, G, 1)
        # the multiplier is a float argument: pass its bits through a one-element tensor-free path
        vals = tuple(a.data_ptr() if hasattr(a, "data_ptr") else int(a) for a in fn_args) + (3.5,)
        types = tuple(ctypes.c_void_p if hasattr(a, "data_ptr") else ctypes.c_uint32 for a in fn_args) + (ctypes.c_float,)
        cu = ref_mod._cu
        if "emb" not in ref_mod._fns:
            ref_mod._fns["emb"] = ref_mod._ok(cu.cuModuleGetFunction(ref_mod.mod, b"talu_embedding_lookup_gaffine_u4_f32"))
        (err,) = cu.cuLaunchKernel(ref_mod._fns["emb"], (hidden + 255) // 256, 1, 1, 256, 1, 1, 0,
                                   torch.cuda.current_stream().cuda_stream, (vals, types), 0)
        assert int(err) == 0, err
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int32), got[i].view(torch.int32)), tok
    w.free()
