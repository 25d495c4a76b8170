"""GPU tests of the callers' forms of the operator (bias rows, the gelu variant of the gated FFN, a converted
checkpoint file taken to a sharded linear), the BASELINE 70B-stack shapes at full size, and the library's
failure paths: a bounded device-side wait that runs out by design, and context create / destroy leaving no
device memory behind."""
import numpy as np
import pytest

from helpers import (TOL_BF16, TOL_F32, bits_from_torch_bf16, make_weights, make_x_bf16, rel_err,
                     torch_bf16_from_bits)

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


# Llama-3-70B-shaped decoder-layer linears: qkv, o, gate (= up), down
CFG5 = [(10240, 8192), (8192, 8192), (28672, 8192), (8192, 28672)]


@pytest.mark.parametrize("M", [1, 64])
@pytest.mark.parametrize("N,K", CFG5)
def test_cfg5_llama70b_shapes_full_size(gaf, ctx, oracle, N, K, M):
    """The 70B-stack matrices at full size, gaf4_64, M = 1 (decode GEMV) and M = 64 (skinny tensor-core
    path), every output against the CPU oracle.  rel <= 1e-2."""
    p, s, b = make_weights(oracle, N, K, 64, 4, seed=N % 101 + M)
    xb, xf = make_x_bf16(oracle, M, K, seed=K % 97 + M)
    w = gaf.Weight.from_host(ctx, p, s, b, 64, 4)
    y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
    ctx.synchronize()
    got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
    w.free()
    ref = oracle.matmul_f32(xf, p, s, b, 64, 4)
    assert rel_err(got, ref) <= TOL_BF16, rel_err(got, ref)


@pytest.mark.parametrize("bits,G", [(4, 64), (8, 32), (8, 64), (8, 128)])
@pytest.mark.parametrize("M", [17, 64, 300])
def test_prefill_sizes_every_scheme(gaf, ctx, oracle, bits, G, M):
    """M > 16 for 4-bit and 8-bit codes (the reference's matmulGaffineU8Prefill,
    core/src/compute/cpu/matmul_prefill.zig:488-569, takes any M): rel <= 1e-2 against the oracle."""
    N, K = 1024, 2048
    p, s, b = make_weights(oracle, N, K, G, bits, seed=bits * G + M)
    xb, xf = make_x_bf16(oracle, M, K, seed=M)
    w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
    y = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
    ctx.synchronize()
    got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
    w.free()
    assert rel_err(got, oracle.matmul_f32(xf, p, s, b, G, bits)) <= TOL_BF16


def test_linear_with_bias_rows(gaf, ctx, oracle):
    """Linear.forward with its optional bias (core/src/inference/backend/cpu/executor/model.zig:98-139):
    y = x W^T + bias, bf16 (rel <= 1e-2) and f32 (<= 1e-3) forms, decode and prefill sizes, bias = None."""
    import torch
    for N, K, G, bits, M in [(1000, 1024, 64, 4, 1), (512, 2048, 32, 8, 5), (768, 1024, 128, 4, 40)]:
        p, s, b = make_weights(oracle, N, K, G, bits, seed=N)
        bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
        xb, xf = make_x_bf16(oracle, M, K, seed=M)
        w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
        dbias = torch.from_numpy(bias).cuda()
        y16 = gaf.linear_bias(ctx, w, torch_bf16_from_bits(xb, "cuda:0"), dbias)
        y32 = gaf.linear_bias(ctx, w, torch.from_numpy(xf).cuda(), dbias)
        y0 = gaf.linear_bias(ctx, w, torch_bf16_from_bits(xb, "cuda:0"), None)
        y1 = gaf.linear(ctx, w, torch_bf16_from_bits(xb, "cuda:0"))
        ctx.synchronize()
        ref = oracle.matmul_f32(xf, p, s, b, G, bits) + bias[None, :]
        assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y16)), ref) <= TOL_BF16
        assert rel_err(y32.cpu().numpy(), oracle.matmul_f64(xf, p, s, b, G, bits) + bias[None, :]) <= TOL_F32
        assert torch.equal(y0, y1)
        w.free()


@pytest.mark.parametrize("d_model,d_ff,G", [(512, 1024, 64), (1024, 2816, 32)])
def test_ffn_gelu_variant(gaf, ctx, oracle, d_model, d_ff, G):
    """The gated FFN with the reference's use_gelu activation (tanh-form gelu(gate) * up,
    core/src/compute/cpu/activation.zig:22-27; CUDA talu_gelu_mul_f32, reduction_ops.cu:59-72): the
    one-launch path (M = 1) and the three-kernel path, against the oracle.  Two chained linears: 2e-2."""
    import torch
    pg, sg, bg = make_weights(oracle, 2 * d_ff, d_model, G, 4, seed=d_ff)
    pd, sd, bd = make_weights(oracle, d_model, d_ff, G, 4, seed=d_ff + 1)
    wgu = gaf.Weight.from_host(ctx, pg, sg, bg, G, 4)
    wd = gaf.Weight.from_host(ctx, pd, sd, bd, G, 4)
    try:
        for M in (1, 3):
            xb, xf = make_x_bf16(oracle, M, d_model, 50 + M)
            xb = oracle.f32_to_bf16_rne(xf * 8.0)
            xf = oracle.bf16_to_f32(xb)
            ref = oracle.ffn_swiglu_f32(xf, (pg, sg, bg), (pd, sd, bd), G, 4, gelu=True)
            ref_silu = oracle.ffn_swiglu_f32(xf, (pg, sg, bg), (pd, sd, bd), G, 4)
            x = torch_bf16_from_bits(xb, "cuda:0")
            y1 = gaf.ffn_swiglu(ctx, wgu, wd, x, activation=gaf.ACT_GELU).clone()
            ctx.set_option("ffn_one_launch", 0)
            y2 = gaf.ffn_swiglu(ctx, wgu, wd, x, activation=gaf.ACT_GELU).clone()
            ctx.set_option("ffn_one_launch", 1)
            ctx.synchronize()
            for y in (y1, y2):
                got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
                assert rel_err(got, ref) <= 2 * TOL_BF16, M
                assert rel_err(got, ref_silu) > 2 * TOL_BF16, "the activation made no difference"
        with pytest.raises(gaf.GafError):
            ctx._check(ctx._lib.tgaf_ffn_gated_bf16(ctx._h, wgu._h, wd._h, x.data_ptr(), 1, 7, y1.data_ptr()))
    finally:
        ctx.set_option("ffn_one_launch", 1)
    wgu.free()
    wd.free()


def test_safetensors_file_to_sharded_linear(gaf, ctx, oracle, tmp_path):
    """A converted checkpoint as the reference writes it (<base>.weight U32, .scales / .biases BF16,
    core/src/converter/grouped_affine.zig:565-593) read from disk, bits / group size inferred from the shapes
    (core/src/models/load/transforms.zig:75-155), uploaded whole and as column / row shards of two ranks, and
    run: sharded results re-assembled on the host match the unsharded oracle."""
    import torch
    from talu_b200.safetensors_gaf import SafetensorsGaf, write_safetensors
    hidden, ffn, G = 1024, 2048, 64
    up = make_weights(oracle, ffn, hidden, G, 4, seed=5)
    down = make_weights(oracle, hidden, ffn, G, 8, seed=6)
    path = tmp_path / "model.safetensors"
    tensors = {}
    for base, (p, s, b) in (("mlp.up_proj", up), ("mlp.down_proj", down)):
        tensors[f"{base}.weight"] = ("U32", p)
        tensors[f"{base}.scales"] = ("BF16", s)
        tensors[f"{base}.biases"] = ("BF16", b)
    write_safetensors(path, tensors)
    f = SafetensorsGaf(path)
    xb, xf = make_x_bf16(oracle, 2, hidden, seed=9)
    x = torch_bf16_from_bits(xb, "cuda:0")
    # whole
    w = f.upload(ctx, "mlp.up_proj", expected_dim=hidden)
    assert (w.N, w.K, w.group, w.bits) == (ffn, hidden, G, 4)
    h = gaf.linear(ctx, w, x)
    ctx.synchronize()
    h_ref = oracle.matmul_f32(xf, *up, G, 4)
    assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(h)), h_ref) <= TOL_BF16
    w.free()
    # column shards of up, row shards of the 8-bit down
    parts = []
    for r in range(2):
        w = f.upload(ctx, "mlp.up_proj", shard_kind=gaf.SHARD_COL, tp_rank=r, tp_size=2, expected_dim=hidden)
        assert (w.N, w.K) == (ffn // 2, hidden)
        parts.append(gaf.linear(ctx, w, x))
        ctx.synchronize()
        w.free()
    hcat = torch.cat(parts, dim=1)
    assert torch.equal(hcat, h)
    hf = oracle.bf16_to_f32(bits_from_torch_bf16(h))
    y = np.zeros((2, hidden))
    for r in range(2):
        w = f.upload(ctx, "mlp.down_proj", shard_kind=gaf.SHARD_ROW, tp_rank=r, tp_size=2, expected_dim=ffn)
        assert (w.N, w.K, w.bits) == (hidden, ffn // 2, 8)
        y += gaf.linear_host(ctx, w, np.ascontiguousarray(hf[:, r * ffn // 2:(r + 1) * ffn // 2]))
        w.free()
    assert rel_err(y, oracle.matmul_f64(hf, *down, G, 8)) <= TOL_F32
    f.close()


def test_bounded_wait_runs_out_and_the_context_survives(gaf, oracle):
    """The give-up path of a device-side wait, without a fault: a one-rank communicator whose all-reduce kernel
    is told to wait also for a rank that does not exist, with a short poll limit.  The kernel returns by
    itself, tgaf_synchronize reports TGAF_ERR_DEVICE_FLAG, and the next calls on the context succeed."""
    import torch
    c = gaf.Context(0)
    try:
        try:
            c.comm_init(gaf.make_comm_id(), 0, 1)
        except gaf.GafError as e:
            pytest.skip(f"no NCCL on this machine: {e}")
        assert c.uses_peer_memory()
        t = torch.randn(4096, device="cuda").to(torch.bfloat16)
        want = t.clone()
        c.allreduce(t)
        c.synchronize()
        assert torch.equal(t, want)
        c.set_option("wait_limit", 2000)
        c.set_option("peer_expect_absent_rank", 1)
        c.allreduce(t)
        with pytest.raises(gaf.GafError) as ei:
            c.synchronize()
        assert ei.value.status == 7 and "0x100" in ei.value.message          # TGAF_ERR_DEVICE_FLAG, the peer wait's code
        c.set_option("peer_expect_absent_rank", 0)
        c.set_option("wait_limit", 0)
        for _ in range(3):                                                   # both exchange phases
            t = want.clone()
            c.allreduce(t)
            c.synchronize()
            assert torch.equal(t, want)
        p, s, b = make_weights(oracle, 512, 1024, 64, 4, seed=1)
        w = gaf.Weight.from_host(c, p, s, b, 64, 4)
        xb, xf = make_x_bf16(oracle, 1, 1024, seed=2)
        y = gaf.linear_allreduce(c, w, torch_bf16_from_bits(xb, "cuda:0"))
        c.synchronize()
        assert rel_err(oracle.bf16_to_f32(bits_from_torch_bf16(y)), oracle.matmul_f32(xf, p, s, b, 64, 4)) <= TOL_BF16
        w.free()
        c._lib.tgaf_comm_destroy(c._h)
    finally:
        c.close()


def test_contexts_leave_no_device_memory_behind(gaf, oracle):
    """Create / use / destroy in a loop: cudaMemGetInfo returns to where it started (every scratch buffer a
    context grows - partial sums, counters, tagged split-K words, staging, FFN intermediates - is freed)."""
    import torch
    torch.cuda.synchronize()
    p, s, b = make_weights(oracle, 2048, 1024, 64, 4, seed=3)
    pg, sg_, bg = make_weights(oracle, 2 * 1024, 512, 64, 4, seed=4)
    pd, sd, bd = make_weights(oracle, 512, 1024, 64, 4, seed=5)
    xb, _ = make_x_bf16(oracle, 3, 1024, seed=4)
    x = torch_bf16_from_bits(xb, "cuda:0")
    x5 = torch_bf16_from_bits(make_x_bf16(oracle, 1, 512, seed=6)[0], "cuda:0")
    y = torch.empty((3, 2048), dtype=torch.bfloat16, device="cuda")
    y5 = torch.empty((1, 512), dtype=torch.bfloat16, device="cuda")

    def cycle():
        c = gaf.Context(0)
        w = gaf.Weight.from_host(c, p, s, b, 64, 4)
        gaf.linear(c, w, x, out=y)
        gaf.linear_host(c, w, xb)
        wgu, wd = gaf.Weight.from_host(c, pg, sg_, bg, 64, 4), gaf.Weight.from_host(c, pd, sd, bd, 64, 4)
        gaf.ffn_swiglu(c, wgu, wd, x5, out=y5)
        c.synchronize()
        for t in (w, wgu, wd):
            t.free()
        c.close()

    cycle()                              # first use: module load, kernel images
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        cycle()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 >= free0 - (1 << 20), f"{(free0 - free1) / 2 ** 20:.1f} MiB lost over five contexts"
