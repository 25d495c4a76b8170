"""Builds talu_b200/libtalu_gaf.so from csrc/*.cu with nvcc for sm_100a.

In-tree build (no JIT cache): object files go to build/, the shared library
next to this file.  nvcc cross-compiles, so this runs on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ_DIR = ROOT / "build" / "obj"
LIB = PKG / "libtalu_gaf.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
          "--expt-relaxed-constexpr", "-I", str(ROOT / "include")]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, verbose_ptxas: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _deps_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj, ""
    cmd = [NVCC, *ARCH, *CFLAGS, "-c", str(src), "-o", str(obj)]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose_ptxas), srcs))
    objs = [o for o, _ in results]
    if verbose_ptxas:
        for _, log in results:
            sys.stderr.write(log)
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "--cudart=static", "-o", str(LIB), *map(str, objs), "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


SIDELOAD_SRC = CSRC / "sideload" / "talu_kernels_sm100.cu"
SIDELOAD_DIR = PKG / "sideload"
SIDELOAD_ARCH = "sm_100"   # talu's arch tag for B200: "sm_{major}{minor}" (core/src/compute/cuda/sideload.zig:46-49)
# op name -> symbol, as talu's wrappers name them (core/src/compute/cuda/gaffine_u4_matvec.zig:12-13)
SIDELOAD_KERNELS = [("gaffine_u4_matvec_f32", "talu_gaffine_u4_matvec_f32"),
                    # the fused decode launches (gaffine_u4_matvec_qkv.zig:13-14, gaffine_u4_matvec_gate_up.zig:12-13)
                    ("gaffine_u4_matvec_qkv_f32", "talu_gaffine_u4_matvec_qkv_f32"),
                    ("gaffine_u4_matvec_gate_up_f32", "talu_gaffine_u4_matvec_gate_up_f32")]


def build_sideload(force: bool = False) -> tuple[Path, Path]:
    """kernels_sm_100.cubin + manifest_sm_100.json, the pair talu's registry picks up from
    $TALU_CUDA_CACHE_DIR (core/src/compute/cuda/sideload.zig:24-44, manifest.zig:5-29): the manifest carries the
    SHA-256 talu verifies before cuModuleLoadData (sideload.zig:78-122)."""
    import hashlib
    import json
    SIDELOAD_DIR.mkdir(parents=True, exist_ok=True)
    cubin = SIDELOAD_DIR / f"kernels_{SIDELOAD_ARCH}.cubin"
    manifest = SIDELOAD_DIR / f"manifest_{SIDELOAD_ARCH}.json"
    if force or not cubin.exists() or cubin.stat().st_mtime < SIDELOAD_SRC.stat().st_mtime:
        cmd = [NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-cubin", str(SIDELOAD_SRC), "-o", str(cubin)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {SIDELOAD_SRC.name}:\n{r.stdout}\n{r.stderr}")
    digest = hashlib.sha256(cubin.read_bytes()).hexdigest()
    doc = {"schema_version": 1, "kernel_abi_version": 1, "arch": SIDELOAD_ARCH, "driver_min": "570.00", "sha256": digest,
           "kernels": [{"op": op, "symbol": sym} for op, sym in SIDELOAD_KERNELS]}
    manifest.write_text(json.dumps(doc, indent=2) + "\n")
    return cubin, manifest


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv))
    print(*build_sideload(force="--force" in sys.argv))
