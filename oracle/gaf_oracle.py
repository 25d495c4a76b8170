"""ctypes loader for the CPU oracle (``oracle/libgaf_oracle.so``).

TEST INFRASTRUCTURE ONLY.  Importers: the tests, the smoke check and the
benchmark's CPU-baseline / reference legs.  The product package
(``talu_b200``) never imports it.

Every function takes and returns numpy arrays; shapes follow the reference's
weight layout (packed u32 ``[N, K/vpw]``, scales / biases u16 ``[N, K/G]``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libgaf_oracle.so"

SCALES_F16 = 0
SCALES_BF16 = 1


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside this file (gcc only)."""
    srcs = [_HERE / n for n in ("gaf_oracle_exact.c", "gaf_oracle_matmul.c", "gaf_pool.c",
                                "gaf_oracle.h", "gaf_pool.h", "Makefile")]
    stale = (not _LIB_PATH.exists()) or any(
        s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in srcs if s.exists())
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


REF_CUBIN = _HERE / "_ref" / "talu_ref_quant_sm_100.cubin"


def build_ref(reference_root: str | os.PathLike = "/root/reference") -> Path | None:
    """Compile the reference's own CUDA kernels for this path, unchanged, into oracle/_ref/ (`make ref`).
    Needs a talu checkout at `reference_root`; where there is none (the GPU box) the cubin built earlier is
    used as it is.  Returns the cubin's path, or None when it neither exists nor can be built."""
    src = Path(reference_root) / "core/src/compute/cuda/kernels/ops/quant_ops.cu"
    if src.exists():
        subprocess.run(["make", "-C", str(_HERE), "ref", f"REF={reference_root}"], check=True, capture_output=True)
    return REF_CUBIN if REF_CUBIN.exists() else None


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        build()
    L = C.CDLL(str(_LIB_PATH))
    vp, sz, i32, u32 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32
    L.gaf_f32_to_bf16_trunc.restype = C.c_uint16
    L.gaf_f32_to_bf16_trunc.argtypes = [C.c_float]
    L.gaf_f32_to_bf16_rne.restype = C.c_uint16
    L.gaf_f32_to_bf16_rne.argtypes = [C.c_float]
    L.gaf_bf16_to_f32.restype = C.c_float
    L.gaf_bf16_to_f32.argtypes = [C.c_uint16]
    L.gaf_f16_to_f32.restype = C.c_float
    L.gaf_f16_to_f32.argtypes = [C.c_uint16]
    L.gaf_scale_bias_to_f32.restype = C.c_float
    L.gaf_scale_bias_to_f32.argtypes = [i32, C.c_uint16]
    L.gaf_extract_nibbles.argtypes = [u32, vp]
    L.gaf_extract_bytes.argtypes = [u32, vp]
    L.gaf_extract32_nibbles.argtypes = [vp, vp]
    L.gaf_validate_shape.restype = i32
    L.gaf_validate_shape.argtypes = [sz, sz, sz, i32, i32]
    L.gaf_quantize.restype = i32
    L.gaf_quantize.argtypes = [vp, sz, sz, sz, i32, vp, vp, vp, i32]
    L.gaf_dequant_f32.restype = i32
    L.gaf_dequant_f32.argtypes = [vp, vp, vp, i32, sz, sz, sz, i32, vp, i32]
    L.gaf_gather_dequant_f32.restype = i32
    L.gaf_gather_dequant_f32.argtypes = [vp, vp, vp, i32, sz, sz, sz, i32, vp, sz, C.c_float, vp]
    L.gaf_matmul_f32.restype = i32
    L.gaf_matmul_f32.argtypes = [vp, sz, sz, vp, vp, vp, i32, sz, sz, i32, vp, i32]
    L.gaf_matmul_f64.restype = i32
    L.gaf_matmul_f64.argtypes = [vp, sz, sz, vp, vp, vp, i32, sz, sz, i32, vp, i32]
    L.gaf_dot_u4.restype = C.c_float
    L.gaf_dot_u4.argtypes = [vp, vp, vp, vp, sz, sz]
    L.gaf_dot_u8.restype = C.c_float
    L.gaf_dot_u8.argtypes = [vp, vp, vp, vp, sz, sz]
    L.gaf_matvec_cuda_semantics_f32.restype = i32
    L.gaf_matvec_cuda_semantics_f32.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32]
    L.gaf_reference_thread_count.restype = i32
    L.gaf_logical_cpu_count.restype = i32
    L.gaf_bf16_to_f32_array.argtypes = [vp, vp, sz]
    L.gaf_f32_to_bf16_rne_array.argtypes = [vp, vp, sz]
    _lib = L
    return L


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def vpw(bits: int) -> int:
    return 8 if bits == 4 else 4


class OracleError(ValueError):
    """The oracle rejected the arguments (the reference's InvalidArgument)."""


def quantize(w: np.ndarray, group: int, bits: int, nthreads: int = 0):
    """f32 [N,K] -> (packed u32 [N,K/vpw], scales u16 [N,K/G], biases u16 [N,K/G])."""
    w = _c(w, np.float32)
    N, K = w.shape
    if bits not in (4, 8) or group <= 0 or K % group or K % vpw(bits) or group % vpw(bits):
        raise OracleError("bad quantize shape")
    packed = np.empty((N, K // vpw(bits)), np.uint32)
    scales = np.empty((N, K // group), np.uint16)
    biases = np.empty((N, K // group), np.uint16)
    nt = nthreads or logical_cpu_count()
    rc = lib().gaf_quantize(_p(w), N, K, group, bits, _p(packed), _p(scales), _p(biases), nt)
    if rc != 0:
        raise OracleError(f"gaf_quantize rc={rc}")
    return packed, scales, biases


def dequant_f32(packed, scales, biases, group: int, bits: int, sdtype: int = SCALES_BF16,
                nthreads: int = 0) -> np.ndarray:
    packed = _c(packed, np.uint32)
    scales = _c(scales, np.uint16)
    biases = _c(biases, np.uint16)
    N = packed.shape[0]
    K = packed.shape[1] * vpw(bits)
    out = np.empty((N, K), np.float32)
    nt = nthreads or logical_cpu_count()
    rc = lib().gaf_dequant_f32(_p(packed), _p(scales), _p(biases), sdtype, N, K, group, bits, _p(out), nt)
    if rc != 0:
        raise OracleError(f"gaf_dequant_f32 rc={rc}")
    return out


class InvalidTokenId(OracleError):
    """A row index is outside the table (the reference's error.InvalidTokenId)."""


def gather_dequant_f32(packed, scales, biases, group: int, bits: int, ids, multiplier: float = 1.0,
                       sdtype: int = SCALES_BF16) -> np.ndarray:
    packed = _c(packed, np.uint32)
    scales = _c(scales, np.uint16)
    biases = _c(biases, np.uint16)
    ids = _c(ids, np.uint32)
    N = packed.shape[0]
    K = packed.shape[1] * vpw(bits)
    out = np.empty((ids.size, K), np.float32)
    rc = lib().gaf_gather_dequant_f32(_p(packed), _p(scales), _p(biases), sdtype, N, K, group, bits, _p(ids),
                                      ids.size, multiplier, _p(out))
    if rc == 2:
        raise InvalidTokenId("row index out of range")
    if rc != 0:
        raise OracleError(f"gaf_gather_dequant_f32 rc={rc}")
    return out


def matmul_f32(a, packed, scales, biases, group: int, bits: int, sdtype: int = SCALES_BF16,
               nthreads: int = 0) -> np.ndarray:
    """The reference's f32-in / f32-out gaf matmul.  nthreads=0: reference thread policy."""
    a = _c(a, np.float32)
    packed = _c(packed, np.uint32)
    scales = _c(scales, np.uint16)
    biases = _c(biases, np.uint16)
    M, K = a.shape
    N = packed.shape[0]
    if packed.shape[1] * vpw(bits) != K:
        raise OracleError("K mismatch")
    out = np.empty((M, N), np.float32)
    rc = lib().gaf_matmul_f32(_p(a), M, K, _p(packed), _p(scales), _p(biases), sdtype, N, group, bits,
                              _p(out), nthreads)
    if rc != 0:
        raise OracleError(f"gaf_matmul_f32 rc={rc}")
    return out


def silu_mul_split(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """siluMulSplit, core/src/compute/cpu/activation.zig:78-94: (gate * sigmoid(gate)) * up in f32.
    (The reference's exp is a fast approximation; this uses the exact one - tolerance-level parity.)"""
    g = np.asarray(gate, np.float32)
    sig = np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))
    return ((g * sig) * np.asarray(up, np.float32)).astype(np.float32)


def gelu_mul_split(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """geluMulSplit (core/src/compute/cpu/activation.zig:22-27, :70-75): tanh-form gelu(gate) * up in f32."""
    g = np.asarray(gate, np.float32)
    inner = np.float32(0.7978845608) * (g + np.float32(0.044715) * (g * g * g))
    return ((g * np.float32(0.5) * (np.float32(1.0) + np.tanh(inner, dtype=np.float32))) * np.asarray(up, np.float32)).astype(np.float32)


def ffn_swiglu_f32(x, gate_up, down, group: int, bits: int, sdtype: int = SCALES_BF16, gelu: bool = False) -> np.ndarray:
    """SwiGLU.forward with a fused gate|up weight in the concat layout [gate rows..., up rows...]
    (core/src/inference/backend/cpu/kernels/ffn.zig:166-241, :388): y = down(act(gate(x)) * up(x)), act =
    silu, or the tanh-form gelu when `gelu` (the reference's use_gelu).  gate_up / down are (packed, scales,
    biases) triples."""
    gu = matmul_f32(x, *gate_up, group, bits, sdtype)
    d_ff = gu.shape[1] // 2
    h = (gelu_mul_split if gelu else silu_mul_split)(gu[:, :d_ff], gu[:, d_ff:])
    return matmul_f32(h, *down, group, bits, sdtype)


def matmul_f64(a, packed, scales, biases, group: int, bits: int, sdtype: int = SCALES_BF16,
               nthreads: int = 0) -> np.ndarray:
    a = _c(a, np.float32)
    packed = _c(packed, np.uint32)
    scales = _c(scales, np.uint16)
    biases = _c(biases, np.uint16)
    M, K = a.shape
    N = packed.shape[0]
    out = np.empty((M, N), np.float64)
    nt = nthreads or logical_cpu_count()
    rc = lib().gaf_matmul_f64(_p(a), M, K, _p(packed), _p(scales), _p(biases), sdtype, N, group, bits,
                              _p(out), nt)
    if rc != 0:
        raise OracleError(f"gaf_matmul_f64 rc={rc}")
    return out


def matvec_cuda_semantics(x, packed, scales, biases, group: int, sdtype: int = SCALES_BF16) -> np.ndarray:
    x = _c(x, np.float32)
    packed = _c(packed, np.uint32)
    scales = _c(scales, np.uint16)
    biases = _c(biases, np.uint16)
    rows, in_dim = x.shape
    out_dim = packed.shape[0]
    out = np.zeros((rows, out_dim), np.float32)
    rc = lib().gaf_matvec_cuda_semantics_f32(_p(x), _p(packed), _p(scales), _p(biases), _p(out),
                                             in_dim, out_dim, group, sdtype, rows)
    if rc != 0:
        raise OracleError(f"gaf_matvec_cuda_semantics_f32 rc={rc}")
    return out


def dot_u4(a, w, scales_f32, biases_f32, group: int) -> float:
    a = _c(a, np.float32); w = _c(w, np.uint32)
    s = _c(scales_f32, np.float32); b = _c(biases_f32, np.float32)
    return float(lib().gaf_dot_u4(_p(a), _p(w), _p(s), _p(b), group, a.size // group))


def dot_u8(a, w, scales_f32, biases_f32, group: int) -> float:
    a = _c(a, np.float32); w = _c(w, np.uint32)
    s = _c(scales_f32, np.float32); b = _c(biases_f32, np.float32)
    return float(lib().gaf_dot_u8(_p(a), _p(w), _p(s), _p(b), group, a.size // group))


def extract_nibbles(word: int) -> np.ndarray:
    out = np.zeros(8, np.float32)
    lib().gaf_extract_nibbles(word, _p(out))
    return out


def extract_bytes(word: int) -> np.ndarray:
    out = np.zeros(4, np.float32)
    lib().gaf_extract_bytes(word, _p(out))
    return out


def extract32_nibbles(b16) -> np.ndarray:
    src = _c(b16, np.uint8)
    out = np.zeros(32, np.uint8)
    lib().gaf_extract32_nibbles(_p(src), _p(out))
    return out


def bf16_to_f32(a) -> np.ndarray:
    a = _c(a, np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().gaf_f32_to_bf16_rne_array(_p(a), _p(out), a.size)
    return out


def f32_to_bf16_trunc(a) -> np.ndarray:
    a = _c(a, np.float32)
    return (a.view(np.uint32) >> 16).astype(np.uint16)


def reference_thread_count() -> int:
    return int(lib().gaf_reference_thread_count())


def logical_cpu_count() -> int:
    return int(lib().gaf_logical_cpu_count())


def validate_shape(N, K, group, bits, sdtype=SCALES_BF16) -> int:
    return int(lib().gaf_validate_shape(N, K, group, bits, sdtype))
