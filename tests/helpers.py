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
