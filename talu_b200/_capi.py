"""ctypes binding of include/talu_gaf.h (the same stub a talu maintainer would
write for `bindings/python/talu/_bindings.py`)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libtalu_gaf.so"

COMM_ID_BYTES = 128

# name -> (restype, argtypes); every symbol include/talu_gaf.h declares
_vp, _i32, _u32, _u64, _i64, _cp = C.c_void_p, C.c_int32, C.c_uint32, C.c_uint64, C.c_int64, C.c_char_p
_pp = C.POINTER(C.c_void_p)
SIGNATURES = {
    "tgaf_abi_version": (_i32, []),
    "tgaf_status_string": (_cp, [_i32]),
    "tgaf_ctx_create": (_i32, [_i32, _vp, _pp]),
    "tgaf_ctx_destroy": (_i32, [_vp]),
    "tgaf_ctx_set_stream": (_i32, [_vp, _vp]),
    "tgaf_synchronize": (_i32, [_vp]),
    "tgaf_last_error": (_cp, [_vp]),
    "tgaf_ctx_set_option": (_i32, [_vp, _cp, _i64]),
    "tgaf_weight_upload": (_i32, [_vp, _vp, _vp, _vp, _u64, _u64, _u32, _u32, _u32, _u32, _u32, _u32, _pp]),
    "tgaf_weight_wrap_device": (_i32, [_vp, _vp, _vp, _vp, _u64, _u64, _u32, _u32, _u32, _pp]),
    "tgaf_weight_free": (_i32, [_vp, _vp]),
    "tgaf_weight_dims": (_i32, [_vp, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u32), C.POINTER(_u32)]),
    "tgaf_hint_next_weight": (_i32, [_vp, _vp]),
    "tgaf_linear_bf16": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_f32": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_fixed_scratch": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_host": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_f32_host": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_host_async": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_host_async_batch": (_i32, [_vp, _u32, _vp, _vp, _vp, _vp]),
    "tgaf_host_batch_create": (_i32, [_vp, _u32, _vp, _vp, _vp, _vp, C.POINTER(_vp)]),
    "tgaf_host_batch_create_reduce": (_i32, [_vp, _u32, _vp, _vp, _vp, _vp, _vp, C.POINTER(_vp)]),
    "tgaf_host_batch_uses_one_launch": (_i32, [_vp]),
    "tgaf_host_batch_submit": (_i32, [_vp, _vp]),
    "tgaf_host_batch_destroy": (_i32, [_vp, _vp]),
    "tgaf_gaffine_u4_matvec_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "tgaf_gaffine_u8_matvec_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "tgaf_dequant_f32": (_i32, [_vp, _vp, _vp]),
    "tgaf_dequant_f32_host": (_i32, [_vp, _vp, _vp]),
    "tgaf_embedding_lookup_f32": (_i32, [_vp, _vp, _vp, _u32, C.c_float, _vp]),
    "tgaf_comm_make_id": (_i32, [_vp]),
    "tgaf_comm_init": (_i32, [_vp, _vp, _u32, _u32]),
    "tgaf_comm_destroy": (_i32, [_vp]),
    "tgaf_allreduce": (_i32, [_vp, _vp, _u64, _u32]),
    "tgaf_comm_uses_peer_memory": (_i32, [_vp]),
    "tgaf_ffn_swiglu_bf16": (_i32, [_vp, _vp, _vp, _vp, _u32, _vp]),
    "tgaf_ffn_swiglu_bf16_allreduce": (_i32, [_vp, _vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_allreduce": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "tgaf_linear_bf16_bias": (_i32, [_vp, _vp, _vp, _u32, _vp, _vp]),
    "tgaf_linear_f32_bias": (_i32, [_vp, _vp, _vp, _u32, _vp, _vp]),
    "tgaf_ffn_gated_bf16": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "tgaf_watchdog_wait": (_i32, [_vp, _vp, _u32]),
    "tgaf_batch_create": (_i32, [_vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp, C.POINTER(_vp)]),
    "tgaf_batch_run": (_i32, [_vp, _vp]),
    "tgaf_batch_uses_one_launch": (_i32, [_vp]),
    "tgaf_batch_destroy": (_i32, [_vp, _vp]),
}

# tgaf_watch_fns: the three hooks of tgaf_watchdog_wait
WORK_DONE_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p)
ASYNC_ERROR_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p)
ABORT_FN = C.CFUNCTYPE(None, C.c_void_p)


class WatchFns(C.Structure):
    _fields_ = [("work_done", WORK_DONE_FN), ("async_error", ASYNC_ERROR_FN), ("abort_comm", ABORT_FN)]

_lib = None


def load() -> C.CDLL:
    """Load libtalu_gaf.so; raises ImportError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m talu_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
