"""The sideload package for talu's own kernel registry (kernels_sm_100.cubin + manifest_sm_100.json):
the manifest against the rules talu's loader applies (CPU), the kernel under talu's fixed launch
geometry against the oracle and the reference's CUDA self-test vectors (GPU)."""
import hashlib
import json
import re

import numpy as np
import pytest


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
    assert {"op": "gaffine_u4_matvec_f32", "symbol": "talu_gaffine_u4_matvec_f32"} in doc["kernels"]   # gaffine_u4_matvec.zig:12-13


@pytest.mark.gpu
def test_kernel_under_the_reference_launch_geometry(package, oracle, kats):
    """Loaded the way talu loads it (cuModuleLoadData + cuModuleGetFunction) and launched the way talu
    launches it: block 256, grid (ceil(out_dim / 8), batch_rows), no dynamic shared memory, ten arguments
    (gaffine_u4_matvec.zig:74-96)."""
    import torch
    from cuda.bindings import driver as cu

    def ok(res):
        err = res[0]
        assert int(err) == 0, err
        return res[1] if len(res) == 2 else res[1:]

    torch.cuda.init()
    torch.zeros(1, device="cuda")                      # the primary context talu's backend would also use
    cubin, _ = package
    mod = ok(cu.cuModuleLoadData(cubin.read_bytes()))
    fn = ok(cu.cuModuleGetFunction(mod, b"talu_gaffine_u4_matvec_f32"))

    def run(x, packed, scales, biases, group, tag=1):
        M, K = x.shape
        N = packed.shape[0]
        dx = torch.from_numpy(np.ascontiguousarray(x)).cuda()
        dp = torch.from_numpy(np.ascontiguousarray(packed).view(np.int32)).cuda()
        ds = torch.from_numpy(np.ascontiguousarray(scales).view(np.int16)).cuda()
        db = torch.from_numpy(np.ascontiguousarray(biases).view(np.int16)).cuda()
        dy = torch.full((M, N), float("nan"), device="cuda")
        vals = (dx.data_ptr(), dp.data_ptr(), ds.data_ptr(), db.data_ptr(), dy.data_ptr(), K, N, group, tag, M)
        import ctypes
        types = (ctypes.c_void_p,) * 5 + (ctypes.c_uint32,) * 5
        stream = torch.cuda.current_stream().cuda_stream
        (err,) = cu.cuLaunchKernel(fn, (N + 7) // 8, M, 1, 256, 1, 1, 0, stream, (vals, types), 0)
        assert int(err) == 0, err
        torch.cuda.synchronize()
        return dy.cpu().numpy()

    # the vectors talu's own start-up self-test holds (smoke_checks.zig)
    for case in kats["cuda_selftest"]:
        x = np.array(case["input"], np.float32)
        N, K = case["out_dim"], case["in_dim"]
        packed = np.array([int(v, 16) for v in case["packed"]], np.uint32).reshape(N, K // 8)
        scales = np.array([int(v, 16) for v in case["scales"]], np.uint16).reshape(N, K // case["group"])
        biases = np.array([int(v, 16) for v in case["biases"]], np.uint16).reshape(N, K // case["group"])
        y = run(x, packed, scales, biases, case["group"], case["sdtype"])
        assert np.allclose(y, np.array(case["expect"], np.float32), atol=case["tol"]), case["src"]
    # random matrices, both load paths (16-byte steps; word steps when K is not a multiple of 32 or G = 8-multiples)
    rng = np.random.default_rng(3)
    for (N, K, G, M) in [(300, 1024, 64, 3), (129, 4096, 128, 1), (64, 96, 32, 2), (40, 72, 24, 2)]:
        w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float32)
        p, s, b = oracle.quantize(w, G, 4)
        x = rng.standard_normal((M, K), dtype=np.float32)
        ref = oracle.matmul_f64(x, p, s, b, G, 4)
        y = run(x, p, s, b, G)
        scale = np.maximum(np.abs(ref).max(), 1e-6)
        assert np.abs(y - ref).max() / scale <= 1e-3, (N, K, G, M)     # the reference's f32 policy
