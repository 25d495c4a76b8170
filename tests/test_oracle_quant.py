"""Quantizer and dequant of the CPU oracle: the reference's qualitative tests
(core/src/converter/grouped_affine.zig:793-1073), an independent numpy
restatement of the same lines (bit-exact), and determinism across threads."""
import numpy as np
import pytest

SCHEMES = [(4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)]


def np_quantize(w, G, bits):
    """numpy restatement of quantizeRowSlice (grouped_affine.zig:448-501)."""
    N, K = w.shape
    maxq = np.float32(15.0 if bits == 4 else 255.0)
    vpw = 8 if bits == 4 else 4
    g = w.reshape(N, K // G, G)
    lo = g.min(axis=2)
    hi = g.max(axis=2)
    rng = (hi - lo).astype(np.float32)
    scale = np.where(rng > 0, (rng / maxq).astype(np.float32), np.float32(0))
    bias = lo
    with np.errstate(divide="ignore", invalid="ignore"):
        norm = ((g - bias[..., None]).astype(np.float32) / scale[..., None]).astype(np.float32)
    # @round: half away from zero
    # (floor(|x| + 0.5) is evaluated in f64 so that it equals roundf exactly)
    r = np.sign(norm) * np.floor(np.abs(norm).astype(np.float64) + 0.5)
    q = np.clip(r, 0, float(maxq))
    q = np.where(scale[..., None] > 0, q, 0).astype(np.uint32).reshape(N, K // vpw, vpw)
    shifts = (np.arange(vpw, dtype=np.uint32) * bits)
    packed = np.bitwise_or.reduce(q << shifts, axis=2).astype(np.uint32)
    s16 = (scale.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    b16 = (bias.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return packed, s16, b16


def np_dequant(packed, s16, b16, G, bits):
    N = packed.shape[0]
    vpw = 8 if bits == 4 else 4
    mask = np.uint32(0xF if bits == 4 else 0xFF)
    shifts = (np.arange(vpw, dtype=np.uint32) * bits)
    q = ((packed[:, :, None] >> shifts) & mask).reshape(N, -1).astype(np.float32)
    s = (s16.astype(np.uint32) << 16).view(np.float32)
    b = (b16.astype(np.uint32) << 16).view(np.float32)
    return (q * np.repeat(s, G, axis=1)).astype(np.float32) + np.repeat(b, G, axis=1)


@pytest.mark.parametrize("bits,G", SCHEMES)
def test_quantizer_matches_numpy_restatement(oracle, bits, G):
    rng = np.random.default_rng(bits * 1000 + G)
    w = (rng.standard_normal((24, 4 * G), dtype=np.float32) * np.float32(0.02))
    w[3, :G] = 0.0            # zero group -> scale 0, all codes 0
    w[5, G:2 * G] = 0.125     # constant group -> range 0
    p, s, b = oracle.quantize(w, G, bits, nthreads=1)
    p2, s2, b2 = np_quantize(w, G, bits)
    assert (p == p2).all() and (s == s2).all() and (b == b2).all()
    assert s[3, 0] == 0 and (p[3, : G // (8 if bits == 4 else 4)] == 0).all()
    assert s[5, 1] == 0
    # thread count does not change a bit
    p3, s3, b3 = oracle.quantize(w, G, bits, nthreads=5)
    assert (p == p3).all() and (s == s3).all() and (b == b3).all()


def test_quantizer_reference_qualitative(oracle):
    # single row 4-bit: ramp 0..63, two groups of 32 -> non-zero scales (:793-837)
    w = np.arange(64, dtype=np.float32)[None, :]
    p, s, b = oracle.quantize(w, 32, 4, nthreads=1)
    assert s[0, 0] != 0 and s[0, 1] != 0
    # 8-bit ramp*0.1 (:839-881)
    w8 = (np.arange(32, dtype=np.float32) * np.float32(0.1))[None, :]
    p8, s8, b8 = oracle.quantize(w8, 32, 8, nthreads=1)
    assert s8[0, 0] != 0
    codes = (p8[0, :, None] >> (np.arange(4, dtype=np.uint32) * 8)) & 0xFF
    assert codes.reshape(-1)[0] == 0 and codes.reshape(-1)[-1] == 255
    # all zeros -> scale 0, bias 0 (:939-977)
    pz, sz, bz = oracle.quantize(np.zeros((1, 32), np.float32), 32, 4, nthreads=1)
    assert sz[0, 0] == 0 and bz[0, 0] == 0 and (pz == 0).all()
    # negative values -> negative bias (sign bit set) (:979-1021)
    wn = -(np.arange(32, dtype=np.float32) + 1)[None, :]
    pn, sn, bn = oracle.quantize(wn, 32, 4, nthreads=1)
    assert bn[0, 0] & 0x8000 and sn[0, 0] != 0
    # mixed sign: bias negative, scale positive (:1023-1073)
    wm = (np.arange(32, dtype=np.float32) - 16)[None, :]
    pm, sm, bm = oracle.quantize(wm, 32, 4, nthreads=1)
    assert bm[0, 0] & 0x8000 and not (sm[0, 0] & 0x8000) and sm[0, 0] != 0


@pytest.mark.parametrize("bits,G", SCHEMES)
def test_dequant_matches_numpy_and_bounds(oracle, bits, G):
    rng = np.random.default_rng(99 + bits + G)
    w = rng.standard_normal((16, 8 * G), dtype=np.float32) * np.float32(0.02)
    p, s, b = oracle.quantize(w, G, bits, nthreads=2)
    d = oracle.dequant_f32(p, s, b, G, bits, nthreads=3)
    assert (d.view(np.uint32) == np_dequant(p, s, b, G, bits).view(np.uint32)).all()
    # reconstruction error: half a step plus bf16 truncation of scale and bias
    step = (w.reshape(16, -1, G).max(2) - w.reshape(16, -1, G).min(2)) / (15 if bits == 4 else 255)
    maxq = 15 if bits == 4 else 255
    bound = np.repeat(0.5 * step + (maxq * step + np.abs(w.reshape(16, -1, G).min(2))) * 2.0 ** -7, G, axis=1)
    assert (np.abs(d - w) <= bound + 1e-7).all()


def test_matmul_agrees_with_f64_truth(oracle):
    rng = np.random.default_rng(3)
    for bits, G in SCHEMES:
        N, K = 33, 4 * G           # odd N exercises the single-column kernel
        w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
        p, s, b = oracle.quantize(w, G, bits, nthreads=1)
        for M in (1, 3, 4, 9):
            x = rng.standard_normal((M, K), dtype=np.float32)
            y = oracle.matmul_f32(x, p, s, b, G, bits, nthreads=2)
            t = oracle.matmul_f64(x, p, s, b, G, bits, nthreads=2)
            assert np.abs(y - t).max() <= 1e-4 * max(1.0, np.abs(t).max())


def test_matmul_rejects_bad_arguments(oracle):
    x = np.ones((1, 16), np.float32)
    p = np.zeros((2, 2), np.uint32)
    sb = np.zeros((2, 2), np.uint16)
    with pytest.raises(oracle.OracleError):
        oracle.matmul_f32(x, p, sb, sb, 12, 4)      # group not a multiple of 8
    with pytest.raises(oracle.OracleError):
        oracle.matmul_f32(x, p, sb, sb, 8, 4, sdtype=7)
