"""GPU: a device-side wait that runs out.  Nothing here traps, faults or spins without a limit: the wait limit is
set to (almost) nothing, the kernels give up their waits at once, finish by themselves with undefined output, raise
an error word that the host reads through the status entry points, and the next call on re-initialised scratch is
correct again."""

import ctypes as C

import pytest
import torch

from fastkernels_b200 import _lib
from fastkernels_b200.plan import MoEDecodePlan
from fastkernels_b200.spec import MoESpec
from fastkernels_b200.workloads import make_hidden, make_moe_weights
from tests.parity import check_output, oracle_layer

pytestmark = pytest.mark.gpu
REAL = MoESpec()
FK_OK, FK_ERR_TIMEOUT = 0, 5


def _status(lib, ws):
    code = C.c_int(-1)
    st = lib.fk_moe_status(ws.data_ptr(), ws.numel(), C.byref(code))
    return st, code.value


@pytest.mark.parametrize("tokens", [1, 4])
def test_single_launch_kernels_wait_runs_out_and_is_reported(tokens):
    """tokens = 1: the single-token kernel; tokens = 4: the kernel for two to four tokens."""
    lib = _lib.load()
    w = make_moe_weights(41, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
    x = make_hidden(41, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    plan = MoEDecodePlan(w, tokens)
    good = [t.clone() for t in plan.run(x)]
    torch.cuda.synchronize()
    assert _status(lib, plan.workspace) == (FK_OK, 0)
    try:
        assert lib.fk_set_wait_limit_cycles(1) == FK_OK          # every wait on another block gives up at once
        plan.run(x)                                              # returns by itself; the output is undefined
        torch.cuda.synchronize()
        st, code = _status(lib, plan.workspace)
        assert st == FK_ERR_TIMEOUT and code == 2                # 2: a single-launch decode kernel
        assert _status(lib, plan.workspace) == (FK_OK, 0)        # reading the status clears it
    finally:
        assert lib.fk_set_wait_limit_cycles(0) == FK_OK          # back to the default (about a second)
    # after a time-out the scratch is re-initialised; then the same plan is right again
    _lib.check(lib.fk_moe_workspace_init(plan.workspace.data_ptr(), plan.workspace.numel(), None), "workspace init")
    torch.cuda.synchronize()
    for _ in range(2):
        out, logits, ids, weights = plan.run(x)
        torch.cuda.synchronize()
        assert torch.equal(ids, good[2]) and torch.equal(out, good[0])
    ref = oracle_layer(x, w, 8)
    check_output(out, ref.output, torch.bfloat16)
    assert _status(lib, plan.workspace) == (FK_OK, 0)
    assert lib.fk_set_wait_limit_cycles(-5) == 1                 # FK_ERR_ARG


class _FakeExchange:
    """An fk_ep_comm over buffers of this process: rank 0 of a two-rank world whose second rank never runs."""

    def __init__(self, lib, world, tokens, hidden, top_k):
        self.lib, self.world, self.rank = lib, world, 0
        self.bytes = lib.fk_ep_buffer_bytes(2, tokens, hidden, top_k, _lib.FK_BF16)     # sized for the larger world
        self.buffers = []
        handle = C.create_string_buffer(_lib.EP_HANDLE_BYTES)
        for _ in range(2):
            ptr = C.c_void_p()
            _lib.check(lib.fk_ep_buffer_create(self.bytes, C.byref(ptr), handle), "fk_ep_buffer_create")
            self.buffers.append(ptr.value)
        self.comm = _lib.EpComm()
        self.comm.rank, self.comm.world, self.comm.tokens_per_rank, self.comm.bytes = 0, world, tokens, self.bytes
        for r in range(world):
            self.comm.base[r] = self.buffers[r]

    def error(self):
        e = C.c_int(0)
        _lib.check(self.lib.fk_ep_status(C.byref(self.comm), C.byref(e)), "fk_ep_status")
        return e.value

    def destroy(self):
        torch.cuda.synchronize()
        for b in self.buffers:
            self.lib.fk_ep_buffer_destroy(b)


def test_expert_parallel_wait_on_a_silent_peer_runs_out_and_is_reported():
    from fastkernels_b200.ep import PeerEPLayer, shard_weights
    lib = _lib.load()
    tokens = 8
    w = make_moe_weights(42, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
    x = make_hidden(42, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    ex2 = _FakeExchange(lib, 2, tokens, REAL.hidden_size, 8)
    try:
        layer = PeerEPLayer(shard_weights(w, 0, 2), ex2, tokens, capture=False, warmup=False)
        try:
            assert lib.fk_set_wait_limit_cycles(100000) == FK_OK     # about 50 microseconds
            layer.hidden.copy_(x)
            layer.launch()                                           # rank 1 never signals: both waits give up
            torch.cuda.synchronize()
            assert ex2.error() == 1                                  # the first wait that gave up: the dispatch
        finally:
            assert lib.fk_set_wait_limit_cycles(0) == FK_OK
        _status(lib, layer.workspace)
        # re-initialise the buffers, then a one-rank world on the same buffer equals the plain layer bit for bit
        for b in ex2.buffers:
            _lib.check(lib.fk_ep_buffer_reset(b), "fk_ep_buffer_reset")
        ex1 = _FakeExchange.__new__(_FakeExchange)
        ex1.lib, ex1.world, ex1.rank, ex1.bytes, ex1.buffers = lib, 1, 0, ex2.bytes, ex2.buffers
        ex1.comm = _lib.EpComm()
        ex1.comm.rank, ex1.comm.world, ex1.comm.tokens_per_rank, ex1.comm.bytes = 0, 1, tokens, ex2.bytes
        ex1.comm.base[0] = ex2.buffers[0]
        one = PeerEPLayer(shard_weights(w, 0, 1), ex1, tokens, capture=False, warmup=False)
        out, logits, ids, weights = one.run(x)
        plain = MoEDecodePlan(w, tokens, flags=_lib.FLAG_NO_FUSED_DECODE)
        want, _, want_ids, _ = plain.run(x)
        torch.cuda.synchronize()
        assert torch.equal(ids, want_ids) and torch.equal(out, want)
        assert ex1.error() == 0
    finally:
        ex2.destroy()
