"""CPU checks of the C-ABI library: it loads, exports every symbol that
include/talu_gaf.h declares, and refuses to compute without a GPU."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from talu_b200 import build, _capi
    build.build()
    return _capi.load()


def test_header_symbols_are_exported(lib):
    from talu_b200 import _capi
    header = (ROOT / "include" / "talu_gaf.h").read_text()
    declared = set(re.findall(r"\b(tgaf_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_capi.SIGNATURES), "ctypes binding and header disagree"


def test_abi_version_and_status_strings(lib):
    assert lib.tgaf_abi_version() == 1
    assert lib.tgaf_status_string(0) == b"ok"
    assert lib.tgaf_status_string(1) == b"invalid argument"


def test_no_fallback_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.tgaf_ctx_create(0, None, C.byref(h)) != 0
    assert not h.value
    import talu_b200
    with pytest.raises(talu_b200.GafError):
        talu_b200.Context(0)


def test_null_arguments_are_rejected(lib):
    assert lib.tgaf_ctx_create(0, None, None) == 1
    assert lib.tgaf_synchronize(None) == 1
    assert lib.tgaf_linear_bf16(None, None, None, 1, None) == 1
    assert lib.tgaf_weight_dims(None, None, None, None, None) == 1
    assert lib.tgaf_ctx_destroy(None) == 0
    assert lib.tgaf_weight_free(None, None) == 0
