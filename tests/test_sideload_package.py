"""The sideload package for talu's own kernel registry (kernels_sm_100.cubin + manifest_sm_100.json):
the manifest against the rules talu's loader applies (CPU), the three kernels under talu's fixed launch
geometry against the oracle, the reference's CUDA self-test vectors and the reference's own kernels (GPU)."""
import hashlib
import json
import re

import numpy as np
import pytest

from helpers import CubinModule, matvec_u4, matvec_u4_fused

SYMBOLS = {"gaffine_u4_matvec_f32": "talu_gaffine_u4_matvec_f32",            # gaffine_u4_matvec.zig:12-13
           "gaffine_u4_matvec_qkv_f32": "talu_gaffine_u4_matvec_qkv_f32",    # gaffine_u4_matvec_qkv.zig:13-14
           "gaffine_u4_matvec_gate_up_f32": "talu_gaffine_u4_matvec_gate_up_f32"}  # gaffine_u4_matvec_gate_up.zig:12-13


@pytest.fixture(scope="module")
def package():
    from talu_b200 import build
    return build.build_sideload()


def test_manifest_passes_the_reference_loader_rules(package):
    cubin, manifest = package
    doc = json.loads(manifest.read_text())
    # core/src/compute/cuda/manifest.zig:12-19 (no unknown fields) and :54-73
    assert set(doc) == {"schema_version", "kernel_abi_version", "arch", "driver_min", "sha256", "kernels"}
    assert doc["schema_version"] == 1 and doc["kernel_abi_version"] == 1
    assert doc["arch"] == "sm_100" and doc["driver_min"]            # arch tag "sm_{major}{minor}", sideload.zig:46-49
    assert re.fullmatch(r"[0-9a-f]{64}", doc["sha256"])
    assert doc["sha256"] == hashlib.sha256(cubin.read_bytes()).hexdigest()   # verified before cuModuleLoadData, sideload.zig:78-122
    assert cubin.name == "kernels_sm_100.cubin" and manifest.name == "manifest_sm_100.json"   # sideload.zig:24-32
    ops = [k["op"] for k in doc["kernels"]]
    assert len(ops) == len(set(ops)) and ops
    for k in doc["kernels"]:
        assert set(k) == {"op", "symbol"}
        assert re.fullmatch(r"[a-z0-9_]+", k["op"]) and not re.search(r"_v\\d+$", k["op"])          # manifest.zig:88-95
        assert k["symbol"].startswith("talu_") and re.fullmatch(r"[a-z0-9_]+", k["symbol"])        # manifest.zig:97-103
        assert not re.search(r"_v\\d+$", k["symbol"])
    for op, sym in SYMBOLS.items():
        assert {"op": op, "symbol": sym} in doc["kernels"]


def _case_arrays(case, part=None):
    src = part or case
    N, K = case["out_dim"], case["in_dim"]
    packed = np.array([int(v, 16) for v in src["packed"]], np.uint32).reshape(N, K // 8)
    scales = np.array([int(v, 16) for v in src["scales"]], np.uint16).reshape(N, K // case["group"])
    biases = np.array([int(v, 16) for v in src["biases"]], np.uint16).reshape(N, K // case["group"])
    return packed, scales, biases


@pytest.mark.gpu
def test_kernel_under_the_reference_launch_geometry(package, oracle, kats):
    """Loaded the way talu loads it (cuModuleLoadData + cuModuleGetFunction) and launched the way talu
    launches it: block 256, grid (ceil(out_dim / 8), batch_rows), no dynamic shared memory, ten arguments
    (gaffine_u4_matvec.zig:74-96)."""
    cubin, _ = package
    mod = CubinModule(cubin)
    # the vectors talu's own start-up self-test holds (smoke_checks.zig)
    for case in kats["cuda_selftest"]:
        x = np.array(case["input"], np.float32)
        packed, scales, biases = _case_arrays(case)
        y = matvec_u4(mod, x, packed, scales, biases, case["group"], case["sdtype"])
        assert np.allclose(y, np.array(case["expect"], np.float32), atol=case["tol"]), case["src"]
    # random matrices, both load paths (16-byte steps; word steps when K is not a multiple of 32 or G = 8-multiples)
    rng = np.random.default_rng(3)
    for (N, K, G, M) in [(300, 1024, 64, 3), (129, 4096, 128, 1), (64, 96, 32, 2), (40, 72, 24, 2)]:
        w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float32)
        p, s, b = oracle.quantize(w, G, 4)
        x = rng.standard_normal((M, K), dtype=np.float32)
        ref = oracle.matmul_f64(x, p, s, b, G, 4)
        y = matvec_u4(mod, x, p, s, b, G)
        scale = np.maximum(np.abs(ref).max(), 1e-6)
        assert np.abs(y - ref).max() / scale <= 1e-3, (N, K, G, M)     # the reference's f32 policy


@pytest.mark.gpu
def test_fused_kernels_under_the_reference_launch_geometry(package, oracle, kats):
    """talu_gaffine_u4_matvec_qkv_f32 (24 arguments) and talu_gaffine_u4_matvec_gate_up_f32 (17), grid.x =
    ceil(sum of output dims / 8): the reference's self-test and probe vectors, then random matrices with
    different output sizes and group sizes per part against the float64 truth."""
    cubin, _ = package
    mod = CubinModule(cubin)
    for case in kats["cuda_selftest_fused"]:
        x = np.array(case["input"], np.float32)
        parts = [(*_case_arrays(case, p), case["group"]) for p in case["parts"]]
        outs = matvec_u4_fused(mod, case["symbol"], x, parts, case["in_dim"], case["sdtype"])
        for p, y in zip(case["parts"], outs):
            assert np.allclose(y, np.array(p["expect"], np.float32), atol=case["tol"]), (case["src"], p["name"])
    rng = np.random.default_rng(5)
    for symbol, dims, K, M in [("talu_gaffine_u4_matvec_qkv_f32", [(512, 64), (131, 32), (128, 128)], 1024, 1),
                               ("talu_gaffine_u4_matvec_qkv_f32", [(40, 24), (9, 8), (17, 72)], 72, 3),
                               ("talu_gaffine_u4_matvec_gate_up_f32", [(1000, 64), (1000, 64)], 2048, 1),
                               ("talu_gaffine_u4_matvec_gate_up_f32", [(77, 32), (50, 128)], 256, 2)]:
        x = rng.standard_normal((M, K), dtype=np.float32)
        parts, refs = [], []
        for n, G in dims:
            w = (rng.standard_normal((n, K), dtype=np.float32) * 0.02).astype(np.float32)
            p, s, b = oracle.quantize(w, G, 4)
            parts.append((p, s, b, G))
            refs.append(oracle.matmul_f64(x, p, s, b, G, 4))
        outs = matvec_u4_fused(mod, symbol, x, parts, K)
        for y, ref in zip(outs, refs):
            assert not np.isnan(y).any()
            assert np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-6) <= 1e-3, (symbol, dims, K, M)
