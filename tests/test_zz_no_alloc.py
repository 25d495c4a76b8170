"""The allocation-free entry point, tgaf_linear_bf16_fixed_scratch.

A host that has handed the rest of the device's memory to its own KV cache cannot let the
matmul call cudaMalloc in the middle of a token step (it synchronises the device and may
fail).  This entry point runs the same streaming GEMV on a fixed scratch array inside the
library image.  Here it is called through the C ABI twice in a row (the second call finds
the scratch exactly as the first one left it) and must give the same output as the regular
entry point, within the tolerance the other parity tests use (max relative error 1e-2);
over-sized problems must be refused with a status code.  The file name sorts last so that a
run that stops at the first failure has already gone through every other test."""
import ctypes as C

import numpy as np
import pytest

from helpers import TOL_BF16, bits_from_torch_bf16, make_weights, make_x_bf16, rel_err, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gaf():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import talu_b200
    return talu_b200


def test_fixed_scratch_matches_regular_entry_point_twice(gaf, oracle):
    import torch
    ctx = gaf.Context(0)
    try:
        # K split over many CTAs (partial sums and arrival counters in use), ragged N, M on both tile sizes
        for (N, K, G, bits, M) in [(4096, 14336, 64, 4, 1), (1000, 8192, 64, 4, 5), (2048, 4096, 128, 8, 16),
                                   (520, 2048, 32, 4, 19)]:
            p, s, b = make_weights(oracle, N, K, G, bits, seed=N + M)
            xb, xf = make_x_bf16(oracle, M, K, seed=7)
            w = gaf.Weight.from_host(ctx, p, s, b, G, bits)
            x = torch_bf16_from_bits(xb, "cuda:0")
            y_ref = gaf.linear(ctx, w, x)
            ctx.synchronize()
            ref = oracle.bf16_to_f32(bits_from_torch_bf16(y_ref))
            want = oracle.matmul_f32(xf, p, s, b, G, bits)
            for call in range(2):
                y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda:0")
                st = ctx._lib.tgaf_linear_bf16_fixed_scratch(ctx._h, w._h, C.c_void_p(x.data_ptr()), M,
                                                             C.c_void_p(y.data_ptr()))
                assert st == 0, ctx._lib.tgaf_last_error(ctx._h)
                ctx.synchronize()
                got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
                assert rel_err(got, ref) <= TOL_BF16, (N, K, G, bits, M, call)     # same as the regular entry point
                assert rel_err(got, want) <= TOL_BF16, (N, K, G, bits, M, call)    # and as the CPU oracle
            w.free()
    finally:
        ctx.close()


def test_fixed_scratch_refuses_what_does_not_fit(gaf, oracle):
    import torch
    ctx = gaf.Context(0)
    try:
        # 600k output rows at M = 16 need far more than 8 MiB of partial sums
        N, K, G, bits, M = 600_000, 256, 32, 4, 16
        rng = np.random.default_rng(0)
        p = rng.integers(0, 2 ** 32, size=(N, K // 8), dtype=np.uint32)
        sb = np.zeros((N, K // G), np.uint16)
        w = gaf.Weight.from_host(ctx, p, sb, sb, G, bits)
        x = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda:0")
        y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda:0")
        st = ctx._lib.tgaf_linear_bf16_fixed_scratch(ctx._h, w._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(y.data_ptr()))
        assert st == 5                                                  # TGAF_ERR_UNSUPPORTED
        assert b"fixed" in ctx._lib.tgaf_last_error(ctx._h)
        assert ctx._lib.tgaf_linear_bf16_fixed_scratch(ctx._h, w._h, None, M, C.c_void_p(y.data_ptr())) == 1
        # the regular entry point still takes it, and the context is still usable
        gaf.linear(ctx, w, x, out=y)
        ctx.synchronize()
        w.free()
    finally:
        ctx.close()


def test_fixed_scratch_allocates_nothing(gaf, oracle):
    """The property the entry point exists for: free device memory (cudaMemGetInfo) is the same before and
    after its calls.  The first call on a device is made beforehand (it looks the fixed array's address up,
    which is also when the driver materialises the library's image on that device).  The measured calls use a
    shape whose split-K scratch on the regular path (4 MiB of tagged words) is larger than anything this
    fresh context holds, so a call that grew the context's scratch would show as lost memory."""
    import torch
    ctx = gaf.Context(0)
    try:
        rng = np.random.default_rng(1)
        small = gaf.Weight.from_host(ctx, *make_weights(oracle, 256, 1024, 64, 4, seed=1), 64, 4)
        N, K, G, M = 65536, 512, 64, 4
        p = rng.integers(0, 2 ** 32, size=(N, K // 8), dtype=np.uint32)
        s = np.full((N, K // G), 0x3C00, np.uint16)        # bf16 2^-7
        b = np.full((N, K // G), 0xBD80, np.uint16)        # bf16 -2^-4
        big = gaf.Weight.from_host(ctx, p, s, b, G, 4)
        xs = torch_bf16_from_bits(make_x_bf16(oracle, 4, 1024, seed=2)[0], "cuda:0")
        ys = torch.empty((4, 256), dtype=torch.bfloat16, device="cuda:0")
        xb, xf = make_x_bf16(oracle, M, K, seed=3)
        x = torch_bf16_from_bits(xb, "cuda:0")
        y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda:0")
        call = lambda w, xi, yi, m: ctx._lib.tgaf_linear_bf16_fixed_scratch(ctx._h, w._h, C.c_void_p(xi.data_ptr()), m,
                                                                            C.c_void_p(yi.data_ptr()))
        assert call(small, xs, ys, 1) == 0                 # first call on the device: set-up
        assert call(small, xs, ys, 4) == 0                 # and the first launch of the kernel the measured calls use
        ctx.synchronize()
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        for _ in range(2):
            assert call(big, x, y, M) == 0, ctx._lib.tgaf_last_error(ctx._h)
        ctx.synchronize()
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0, f"{free0 - free1} bytes of device memory went during allocation-free calls"
        got = oracle.bf16_to_f32(bits_from_torch_bf16(y))
        assert rel_err(got, oracle.matmul_f32(xf, p, s, b, G, 4)) <= TOL_BF16
        small.free()
        big.free()
    finally:
        ctx.close()
