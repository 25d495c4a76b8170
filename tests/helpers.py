"""Shared helpers for the parity tests: seeded inputs of the benchmark's shapes
and the error measure used everywhere.

Weights ~ N(0, 0.02^2) fp32 (seed per matrix) quantized with the oracle's
restatement of talu's converter; activations ~ N(0, 1) rounded to bf16 (RNE)."""
from __future__ import annotations

import numpy as np

TOL_BF16 = 1e-2   # max relative error, bf16 out / fp32 accumulate (the stated target)
TOL_F32 = 1e-3    # the reference's policy for f32 matmul results


def make_weights(oracle, N, K, group, bits, seed=0):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    return oracle.quantize(w, group, bits)


def make_x_bf16(oracle, M, K, seed=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    xb = oracle.f32_to_bf16_rne(x)
    return xb, oracle.bf16_to_f32(xb)


def rel_err(y, ref):
    """max_ij |y - ref| / max(|ref_ij|, rms(ref row i)): relative error that does not
    blow up on the outputs that happen to be near zero."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    den = np.maximum(np.abs(ref), np.maximum(rms, 1e-30))
    return float((np.abs(y - ref) / den).max())


def torch_bf16_from_bits(bits_u16, device):
    import torch
    return torch.from_numpy(bits_u16.view(np.int16)).to(device).view(torch.bfloat16)


def bits_from_torch_bf16(t):
    import torch
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


class CubinModule:
    """A cubin loaded the way talu's registry loads one (cuModuleLoadData + cuModuleGetFunction) and launched
    the way its wrappers launch (cuLaunchKernel, block 256, no dynamic shared memory;
    core/src/compute/cuda/gaffine_u4_matvec.zig:87-96).  Arguments: torch tensors (passed as device
    pointers) and Python ints (passed as u32)."""

    def __init__(self, path):
        import torch
        from cuda.bindings import driver as cu
        self._cu = cu
        torch.cuda.init()
        torch.zeros(1, device="cuda")                      # the primary context talu's backend would also use
        self.mod = self._ok(cu.cuModuleLoadData(open(path, "rb").read()))
        self._fns = {}

    @staticmethod
    def _ok(res):
        assert int(res[0]) == 0, res[0]
        return res[1] if len(res) == 2 else res[1:]

    def launch(self, symbol, grid, args, block=256):
        import ctypes
        import torch
        cu = self._cu
        if symbol not in self._fns:
            self._fns[symbol] = self._ok(cu.cuModuleGetFunction(self.mod, symbol.encode()))
        vals = tuple(a.data_ptr() if hasattr(a, "data_ptr") else int(a) for a in args)
        types = tuple(ctypes.c_void_p if hasattr(a, "data_ptr") else ctypes.c_uint32 for a in args)
        stream = torch.cuda.current_stream().cuda_stream
        (err,) = cu.cuLaunchKernel(self._fns[symbol], grid[0], grid[1], 1, block, 1, 1, 0, stream, (vals, types), 0)
        assert int(err) == 0, err


def to_dev(a):
    """numpy u32 / u16 / f32 array -> torch device tensor of the same bits."""
    import torch
    a = np.ascontiguousarray(a)
    view = {np.dtype(np.uint32): np.int32, np.dtype(np.uint16): np.int16}.get(a.dtype)
    return torch.from_numpy(a.view(view) if view else a).cuda()


def matvec_u4(mod, x, packed, scales, biases, group, tag=1, symbol="talu_gaffine_u4_matvec_f32"):
    """One launch of the ten-argument matvec kernel under the reference's geometry: grid (ceil(N / 8), M)."""
    import torch
    M, K = x.shape
    N = packed.shape[0]
    dx, dp, ds, db = to_dev(x), to_dev(packed), to_dev(scales), to_dev(biases)
    dy = torch.full((M, N), float("nan"), device="cuda")
    mod.launch(symbol, ((N + 7) // 8, M), (dx, dp, ds, db, dy, K, N, group, tag, M))
    torch.cuda.synchronize()
    return dy.cpu().numpy()


def matvec_u4_fused(mod, symbol, x, parts, in_dim, tag=1):
    """The fused q|k|v (three parts) or gate|up (two parts) launch: per part (packed, scales, biases, group);
    grid.x = ceil(sum of the output dims / 8) (gaffine_u4_matvec_qkv.zig:193-198, _gate_up.zig:79-85)."""
    import torch
    M = x.shape[0]
    dx = to_dev(x)
    args, outs, total = [dx], [], 0
    keep = []
    for packed, scales, biases, group in parts:
        n = packed.shape[0]
        dp, ds, db = to_dev(packed), to_dev(scales), to_dev(biases)
        dy = torch.full((M, n), float("nan"), device="cuda")
        keep += [dp, ds, db]
        args += [dp, ds, db, dy, n, group, tag]
        outs.append(dy)
        total += n
    args += [in_dim, M]
    mod.launch(symbol, ((total + 7) // 8, M), tuple(args))
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in outs]
