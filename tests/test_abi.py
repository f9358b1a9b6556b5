"""CPU: libfkmoe.so loads, exports every symbol include/fkmoe.h declares, and rejects bad
arguments before touching a GPU."""

import ctypes as C
import re
from pathlib import Path

import pytest

from fastkernels_b200 import _lib
from fastkernels_b200._lib import Call, Dims

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "fkmoe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in fkmoe.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.fk_version() >= 100
    assert lib.fk_status_string(0) == b"ok"
    assert b"workspace" in lib.fk_status_string(3)


def test_workspace_bytes_scales_and_rejects_bad_dims():
    lib = _lib.load()
    small = lib.fk_moe_workspace_bytes(C.byref(Dims(1, 2048, 256, 512, 8)))
    big = lib.fk_moe_workspace_bytes(C.byref(Dims(256, 2048, 256, 512, 8)))
    assert 0 < small < big
    assert big % 256 == 0
    assert lib.fk_moe_workspace_bytes(C.byref(Dims(1, 8192, 256, 512, 8))) == 0      # hidden over the limit
    assert lib.fk_moe_workspace_bytes(C.byref(Dims(1, 2048, 2048, 512, 8))) == 0     # experts over the limit
    assert lib.fk_moe_workspace_bytes(C.byref(Dims(1, 2048, 256, 512, 9))) == 0      # top_k over the limit
    assert lib.fk_moe_workspace_bytes(None) == 0


def test_calls_reject_null_pointers_without_a_gpu():
    lib = _lib.load()
    call = Call()
    call.dims = Dims(4, 2048, 256, 512, 8)
    call.hidden_dtype = _lib.FK_BF16
    call.weight_dtype = _lib.FK_BF16
    assert lib.fk_moe_layer(C.byref(call), None) == 1        # FK_ERR_ARG: null tensors
    assert lib.fk_moe_router(C.byref(call), None) == 1
    assert lib.fk_moe_experts(C.byref(call), None) == 1
    call.weight_dtype = 7
    assert lib.fk_moe_layer(C.byref(call), None) == 2        # FK_ERR_UNSUPPORTED
    call.weight_dtype = _lib.FK_BF16
    call.dims = Dims(4, 2048, 4, 512, 8)                     # top_k > experts
    assert lib.fk_moe_layer(C.byref(call), None) == 1
    assert lib.fk_moe_layer(None, None) == 1
    with pytest.raises(RuntimeError, match="invalid argument"):
        _lib.check(1, "probe")
