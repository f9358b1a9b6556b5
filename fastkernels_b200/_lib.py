"""ctypes binding of libfkmoe.so (the C ABI declared in include/fkmoe.h).

There is no fallback: if the shared library is missing or a call returns a
non-zero status, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libfkmoe.so"

FK_F32, FK_BF16, FK_F16 = 0, 1, 2
FLAG_FORCE_GENERIC = 1
FLAG_FORCE_GEMV = 2
FLAG_FORCE_TENSOR = 4
FLAG_NO_FUSED_DECODE = 8
FLAG_SKIP_FOREIGN = 16
FLAG_TRACE = 64
FLAG_WIDE_PASSES = 128


class Dims(C.Structure):
    _fields_ = [("tokens", C.c_int32), ("hidden", C.c_int32), ("experts", C.c_int32),
                ("intermediate", C.c_int32), ("top_k", C.c_int32)]


class Call(C.Structure):
    _fields_ = [
        ("dims", Dims),
        ("hidden_dtype", C.c_int32), ("weight_dtype", C.c_int32),
        ("eps", C.c_float), ("norm_offset", C.c_float),
        ("flags", C.c_uint32), ("expert_base", C.c_int32),
        ("shared_token_base", C.c_int32), ("shared_token_count", C.c_int32),
        ("hidden", C.c_void_p), ("norm_weight", C.c_void_p), ("router_weight", C.c_void_p),
        ("router_bias", C.c_void_p),
        ("expert_gate_up", C.c_void_p), ("expert_down", C.c_void_p),
        ("shared_gate_up", C.c_void_p), ("shared_down", C.c_void_p), ("shared_gate", C.c_void_p),
        ("topk_ids_in", C.c_void_p), ("topk_weights_in", C.c_void_p),
        ("out", C.c_void_p), ("layer_hidden", C.c_void_p), ("logits", C.c_void_p),
        ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


EP_MAX_RANKS = 8
EP_HANDLE_BYTES = 64


class EpComm(C.Structure):          # struct fk_ep_comm
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("tokens_per_rank", C.c_int32), ("reserved", C.c_int32),
                ("base", C.c_void_p * EP_MAX_RANKS), ("bytes", C.c_size_t)]


# name -> (restype, argtypes); every symbol include/fkmoe.h declares
SIGNATURES = {
    "fk_version": (C.c_int, []),
    "fk_status_string": (C.c_char_p, [C.c_int]),
    "fk_last_cuda_error": (C.c_char_p, []),
    "fk_launch_count": (C.c_uint64, []),
    "fk_moe_layer_timed": (C.c_int, [C.POINTER(Call), C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "fk_moe_experts_timed": (C.c_int, [C.POINTER(Call), C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "fk_moe_trace_offset": (C.c_size_t, [C.POINTER(Dims)]),
    "fk_moe_workspace_bytes": (C.c_size_t, [C.POINTER(Dims)]),
    "fk_moe_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "fk_moe_router": (C.c_int, [C.POINTER(Call), C.c_void_p]),
    "fk_moe_router_noalloc": (C.c_int, [C.POINTER(Call), C.c_void_p]),
    "fk_moe_experts": (C.c_int, [C.POINTER(Call), C.c_void_p]),
    "fk_moe_layer": (C.c_int, [C.POINTER(Call), C.c_void_p]),
    "fk_moe_host_staging_bytes": (C.c_size_t, [C.POINTER(Dims), C.c_int]),
    "fk_moe_layer_host": (C.c_int, [C.POINTER(Call), C.c_void_p, C.c_size_t, C.c_void_p]),
    "fk_single_expert_mlp": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                       C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "fk_residual_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]),
    "fk_fused_swiglu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p]),
    "fk_expert_histogram": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "fk_moe_permute": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_size_t, C.c_void_p]),
    "fk_moe_layer_residual": (C.c_int, [C.POINTER(Call), C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]),
    "fk_ep_buffer_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "fk_ep_buffer_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "fk_ep_buffer_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "fk_ep_buffer_close": (C.c_int, [C.c_void_p]),
    "fk_ep_buffer_destroy": (C.c_int, [C.c_void_p]),
    "fk_moe_layer_ep": (C.c_int, [C.POINTER(Call), C.POINTER(EpComm), C.c_void_p]),
    "fk_ep_status": (C.c_int, [C.POINTER(EpComm), C.POINTER(C.c_int)]),
    "fk_ep_buffer_reset": (C.c_int, [C.c_void_p]),
    "fk_moe_layer_ep_timed": (C.c_int, [C.POINTER(Call), C.POINTER(EpComm), C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "fk_set_wait_limit_cycles": (C.c_int, [C.c_longlong]),
    "fk_moe_status": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_int)]),
}

_lib = None


def load() -> C.CDLL:
    """Load libfkmoe.so and bind every symbol; raises RuntimeError if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m fastkernels_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    text = lib.fk_status_string(status).decode()
    detail = lib.fk_last_cuda_error().decode() if status == 4 else ""
    raise RuntimeError(f"{what} failed: {text}" + (f" ({detail})" if detail else ""))
