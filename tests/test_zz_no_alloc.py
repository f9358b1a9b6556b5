"""GPU: the router entry point that brings its own scratch (fk_moe_router_noalloc) gives the same
logits, ids and weights as fk_moe_router, called twice in a row through the C ABI.

Some callers of this library cannot allocate device memory (their framework owns every byte, or their
latency budget forbids the allocator), so they cannot provide the workspace fk_moe_router wants; the
variant keeps its 4 KB of tickets inside the library.  Both run the same kernel, so the comparison is
bitwise.  The file name sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""

import ctypes as C

import pytest
import torch

from fastkernels_b200 import _lib
from fastkernels_b200._lib import Call, Dims

pytestmark = pytest.mark.gpu


def _router_call(lib, entry, hidden, norm_w, router_w, bias, workspace, dtype_code=_lib.FK_BF16):
    T, H = hidden.shape
    E = router_w.shape[0]
    logits = torch.empty(T, E, device="cuda", dtype=torch.float32)
    ids = torch.empty(T, 8, device="cuda", dtype=torch.int64)
    weights = torch.empty(T, 8, device="cuda", dtype=torch.float32)
    call = Call()
    call.dims = Dims(T, H, E, 1, 8)
    call.hidden_dtype = call.weight_dtype = dtype_code
    call.eps, call.norm_offset = 1e-6, 1.0
    call.hidden, call.norm_weight, call.router_weight = hidden.data_ptr(), norm_w.data_ptr(), router_w.data_ptr()
    call.router_bias = bias.data_ptr()
    call.logits, call.topk_ids, call.topk_weights = logits.data_ptr(), ids.data_ptr(), weights.data_ptr()
    if workspace is not None:
        call.workspace, call.workspace_bytes = workspace.data_ptr(), workspace.numel()
    status = getattr(lib, entry)(C.byref(call), torch.cuda.current_stream().cuda_stream)
    assert status == 0, lib.fk_status_string(status)
    torch.cuda.synchronize()
    return logits, ids, weights


@pytest.mark.parametrize("tokens", [1, 37, 300])
def test_router_noalloc_matches_router_twice_in_a_row(tokens):
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(tokens)
    hidden = torch.randn(tokens, 2048, generator=g, device="cuda").to(torch.bfloat16)
    norm_w = (0.02 * torch.randn(2048, generator=g, device="cuda")).to(torch.bfloat16)
    router_w = (0.02 * torch.randn(256, 2048, generator=g, device="cuda")).to(torch.bfloat16)
    bias = 0.5 * torch.randn(256, generator=g, device="cuda")
    dims = Dims(tokens, 2048, 256, 1, 8)
    ws = torch.zeros(lib.fk_moe_workspace_bytes(C.byref(dims)), dtype=torch.uint8, device="cuda")
    ref = _router_call(lib, "fk_moe_router", hidden, norm_w, router_w, bias, ws)
    for _ in range(2):                       # the shared scratch must come back clean for the second call
        got = _router_call(lib, "fk_moe_router_noalloc", hidden, norm_w, router_w, bias, None)
        for a, b in zip(got, ref):
            assert torch.equal(a, b)


@pytest.mark.parametrize("tokens", [3, 130])
def test_router_noalloc_fp32_inputs_take_the_generic_kernel(tokens):
    """fp32 activations and weights go through the shape-agnostic router kernel (4 or 8 tokens per block), which
    indexes the same built-in tickets: same answer as with a workspace, twice in a row."""
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(1000 + tokens)
    hidden = torch.randn(tokens, 2048, generator=g, device="cuda")
    norm_w = 0.02 * torch.randn(2048, generator=g, device="cuda")
    router_w = 0.02 * torch.randn(256, 2048, generator=g, device="cuda")
    bias = 0.5 * torch.randn(256, generator=g, device="cuda")
    dims = Dims(tokens, 2048, 256, 1, 8)
    ws = torch.zeros(lib.fk_moe_workspace_bytes(C.byref(dims)), dtype=torch.uint8, device="cuda")
    ref = _router_call(lib, "fk_moe_router", hidden, norm_w, router_w, bias, ws, _lib.FK_F32)
    for _ in range(2):
        got = _router_call(lib, "fk_moe_router_noalloc", hidden, norm_w, router_w, bias, None, _lib.FK_F32)
        for a, b in zip(got, ref):
            assert torch.equal(a, b)


def test_router_noalloc_rejects_more_tokens_than_its_scratch_covers():
    lib = _lib.load()
    call = Call()
    call.dims = Dims(4097, 2048, 256, 1, 8)
    call.hidden_dtype = call.weight_dtype = _lib.FK_BF16
    assert lib.fk_moe_router_noalloc(C.byref(call), None) == 1          # FK_ERR_ARG
    assert b"4096" in lib.fk_last_cuda_error()
