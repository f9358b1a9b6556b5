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


def test_expert_parallel_entry_points_check_arguments_without_a_gpu():
    lib = _lib.load()
    b2 = lib.fk_ep_buffer_bytes(2, 32, 2048, 8, _lib.FK_BF16)
    b8 = lib.fk_ep_buffer_bytes(8, 32, 2048, 8, _lib.FK_BF16)
    # header + gathered activations (bf16) + routing (ids, weights) + partial rows (fp32), each 256-byte aligned
    assert b2 == 256 + 2 * 32 * 2048 * 2 + 2 * (2 * 32 * 8 * 4) + 2 * 32 * 2048 * 4
    assert b8 > b2 and b8 % 256 == 0
    assert lib.fk_ep_buffer_bytes(9, 32, 2048, 8, _lib.FK_BF16) == 0         # more ranks than one node has GPUs
    assert lib.fk_ep_buffer_bytes(2, 0, 2048, 8, _lib.FK_BF16) == 0
    assert lib.fk_ep_buffer_bytes(2, 32, 2048, 9, _lib.FK_BF16) == 0
    call = Call()
    call.dims = Dims(32, 2048, 256, 512, 8)
    call.hidden_dtype = call.weight_dtype = _lib.FK_BF16
    comm = _lib.EpComm()
    comm.rank, comm.world, comm.tokens_per_rank = 0, 2, 32
    assert lib.fk_moe_layer_ep(C.byref(call), C.byref(comm), None) == 1      # FK_ERR_ARG: null tensors
    assert lib.fk_moe_layer_ep(C.byref(call), None, None) == 1
    comm.tokens_per_rank = 16
    assert lib.fk_moe_layer_ep(C.byref(call), C.byref(comm), None) == 1      # token count differs from the buffers'
    assert lib.fk_ep_buffer_open(None, None) == 1
    assert lib.fk_ep_buffer_close(None) == 0 and lib.fk_ep_buffer_destroy(None) == 0
