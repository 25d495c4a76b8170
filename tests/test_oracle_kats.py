"""The CPU oracle against every known-answer vector the reference's own unit
tests and CUDA start-up self-tests hold for the grouped-affine path
(tests/golden/reference_kats.json names the reference test behind each)."""
import numpy as np
import pytest


def _h(s):
    return int(s, 16)


def _x(kind, M, K, group):
    if kind == "ones":
        return np.ones((M, K), np.float32)
    if kind == "ramp1":
        return np.tile(np.arange(1, K + 1, dtype=np.float32), (M, 1))
    if kind == "row_index_plus1":
        return np.repeat(np.arange(1, M + 1, dtype=np.float32)[:, None], K, axis=1)
    if kind == "group_index_plus1":
        return np.tile((np.arange(K) // group + 1).astype(np.float32), (M, 1))
    raise KeyError(kind)


def test_nibble_and_byte_order(oracle, kats):
    for k in kats["nibbles"]:
        assert oracle.extract_nibbles(_h(k["word"])).tolist() == k["expect"], k["src"]
    for k in kats["bytes"]:
        assert oracle.extract_bytes(_h(k["word"])).tolist() == k["expect"], k["src"]
    for k in kats["nibbles32"]:
        out = oracle.extract32_nibbles(np.array(k["bytes"], np.uint8))
        for idx, want in k["expect_prefix"].items():
            assert out[int(idx)] == want, k["src"]
        # zero and all-ones inputs (simd/arch/root.zig:127-150)
    assert not oracle.extract32_nibbles(np.zeros(16, np.uint8)).any()
    assert (oracle.extract32_nibbles(np.full(16, 0xFF, np.uint8)) == 15).all()


def test_scale_bias_decode_and_bf16_trunc(oracle, kats):
    L = oracle.lib()
    for k in kats["scale_decode"]:
        assert L.gaf_scale_bias_to_f32(k["sdtype"], _h(k["bits"])) == k["expect"], k["src"]
    for k in kats["bf16_trunc"]:
        assert L.gaf_f32_to_bf16_trunc(k["value"]) == _h(k["expect"]), k["src"]
    # truncation, not rounding: 1 + 2^-8 + 2^-9 keeps only the top 16 bits
    v = np.float32(1.0 + 2.0 ** -8 + 2.0 ** -9)
    assert L.gaf_f32_to_bf16_trunc(float(v)) == 0x3F80
    assert L.gaf_f32_to_bf16_rne(float(v)) == 0x3F81
    # sign symmetry (converter/root.zig:687-696)
    p, n = L.gaf_f32_to_bf16_trunc(3.14), L.gaf_f32_to_bf16_trunc(-3.14)
    assert (p & 0x8000) == 0 and (n & 0x8000) != 0 and (p & 0x7FFF) == (n & 0x7FFF)


def test_f16_decode_matches_numpy(oracle):
    L = oracle.lib()
    bits = np.arange(0, 65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([L.gaf_f16_to_f32(int(b)) for b in bits[::37]], np.float32)
    w = want[::37]
    both_nan = np.isnan(w) & np.isnan(got)
    assert ((w == got) | both_nan).all()


def test_dequant_kats(oracle, kats):
    for k in kats["dequant"]:
        packed = np.array([[_h(w) for w in k["packed"]]], np.uint32)
        s = np.array([[_h(w) for w in k["scales"]]], np.uint16)
        b = np.array([[_h(w) for w in k["biases"]]], np.uint16)
        out = oracle.dequant_f32(packed, s, b, k["group"], k["bits"], k["sdtype"], nthreads=1)
        assert np.allclose(out, k["expect_all"], atol=k["tol"]), k["src"]


def test_dot_kats(oracle, kats):
    for k in kats["dot"]:
        K, G = k["K"], k["group"]
        vpw = 8 if k["bits"] == 4 else 4
        a = np.full(K, k["x_all"], np.float32)
        w = np.full(K // vpw, _h(k["word"]), np.uint32)
        s = np.full(K // G, k["scale"], np.float32)
        b = np.full(K // G, k["bias"], np.float32)
        fn = oracle.dot_u4 if k["bits"] == 4 else oracle.dot_u8
        assert abs(fn(a, w, s, b, G) - k["expect"]) <= k["tol"], k["src"]


def _build_matmul_case(k):
    M, K, N, G, bits = k["M"], k["K"], k["N"], k["group"], k["bits"]
    vpw = 8 if bits == 4 else 4
    x = _x(k["x"], M, K, G)
    if "words_per_row" in k:
        packed = np.array([[_h(w) for w in row] for row in k["words_per_row"]], np.uint32)
    else:
        row = [_h(w) for w in k["words"]]
        assert len(row) == K // vpw
        packed = np.tile(np.array(row, np.uint32), (N, 1))
    groups = K // G
    sc = [_h(w) for w in k["scales"]]
    bi = [_h(w) for w in k["biases"]]
    if len(sc) == 1:
        sc, bi = sc * groups, bi * groups
    scales = np.tile(np.array(sc, np.uint16), (N, 1))
    biases = np.tile(np.array(bi, np.uint16), (N, 1))
    if "expect" in k:
        want = np.array(k["expect"], np.float32)
    elif "expect_rows_times" in k:
        want = np.repeat((np.arange(1, M + 1, dtype=np.float32) * k["expect_rows_times"])[:, None], N, axis=1)
    else:
        want = np.full((M, N), k["expect_all"], np.float32)
    return x, packed, scales, biases, want


@pytest.mark.parametrize("nthreads", [1, 3])
def test_matmul_kats(oracle, kats, nthreads):
    for k in kats["matmul"]:
        x, packed, scales, biases, want = _build_matmul_case(k)
        got = oracle.matmul_f32(x, packed, scales, biases, k["group"], k["bits"], k["sdtype"], nthreads=nthreads)
        assert np.allclose(got, want, atol=k["tol"]), (k["src"], got)
        truth = oracle.matmul_f64(x, packed, scales, biases, k["group"], k["bits"], k["sdtype"], nthreads=1)
        assert np.allclose(truth, want, atol=k["tol"]), k["src"]


def test_cuda_selftest_vectors(oracle, kats):
    for k in kats["cuda_selftest"]:
        x = np.array(k["input"], np.float32)
        packed = np.array([[_h(w)] for w in k["packed"]], np.uint32)
        s = np.array([[_h(w)] for w in k["scales"]], np.uint16)
        b = np.array([[_h(w)] for w in k["biases"]], np.uint16)
        want = np.array(k["expect"], np.float32)
        got = oracle.matvec_cuda_semantics(x, packed, s, b, k["group"], k["sdtype"])
        assert np.allclose(got, want, atol=k["tol"]), k["src"]
        got2 = oracle.matmul_f32(x, packed, s, b, k["group"], 4, k["sdtype"], nthreads=1)
        assert np.allclose(got2, want, atol=k["tol"]), k["src"]


def test_4x2_equals_1x2(oracle):
    """kernel4x2 and kernel1x2 agree to 1e-3 (matmul_prefill.zig:1560-1672): the
    first four rows of an M=5 problem go through 4x2, the same rows submitted
    one at a time go through 1x2."""
    rng = np.random.default_rng(7)
    K, N, G = 128, 6, 32
    w = rng.standard_normal((N, K), dtype=np.float32) * 0.02
    packed, s, b = oracle.quantize(w, G, 4, nthreads=1)
    x = rng.standard_normal((5, K), dtype=np.float32)
    full = oracle.matmul_f32(x, packed, s, b, G, 4, nthreads=1)
    for m in range(5):
        one = oracle.matmul_f32(x[m:m + 1], packed, s, b, G, 4, nthreads=1)
        assert np.allclose(full[m], one[0], atol=1e-3)


def test_validate_shape_rules(oracle):
    """gaffine_u4_matvec.zig:145-170 (bad group alignment, bad dtype tag) and the
    loader's limits (transforms.zig:158-185)."""
    ok = oracle.validate_shape
    assert ok(8, 16, 8, 4, 1) == 0
    assert ok(8, 16, 12, 4, 1) != 0        # group not a multiple of 8
    assert ok(8, 16, 8, 4, 7) != 0         # bad scales dtype tag
    assert ok(0, 16, 8, 4, 1) != 0
    assert ok(8, 20, 8, 4, 1) != 0         # K not a multiple of the group
    assert ok(8, 16, 8, 5, 1) != 0         # bits
    assert ok(4, 32 * 1025, 32, 4, 1) != 0  # more than 1024 groups
    assert ok(4, 32 * 1024, 32, 4, 1) == 0


def test_gather_decode_kats(oracle, kats):
    for k in kats["gather"]:
        packed = np.array([[_h(w) for w in row] for row in k["packed"]], np.uint32)
        s = np.array([[_h(w) for w in row] for row in k["scales"]], np.uint16)
        b = np.array([[_h(w) for w in row] for row in k["biases"]], np.uint16)
        out = oracle.gather_dequant_f32(packed, s, b, k["group"], k["bits"], k["ids"], sdtype=k["sdtype"])
        assert np.allclose(out, k["expect_all"], atol=k["tol"]), k["src"]
    # an index outside the table is the reference's error.InvalidTokenId (quant_decode.zig:155,194)
    k = kats["gather"][0]
    packed = np.array([[_h(w) for w in row] for row in k["packed"]], np.uint32)
    sb = np.zeros((2, 1), np.uint16)
    with pytest.raises(oracle.InvalidTokenId):
        oracle.gather_dequant_f32(packed, sb, sb, 8, 4, [2], sdtype=0)
