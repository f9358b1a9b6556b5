"""Shared checks for the GPU parity tests."""

import torch

from oracle import moe_oracle as O
from tests.tolerances import OUT_MAX_ABS, OUT_REL_L2, default_tolerance

# a token whose k-th and (k+1)-th probabilities are closer than this may legitimately route
# differently when fp32 sums are taken in another order; such tokens are reported, not failed
TIE_MARGIN = 2e-6


def check_routing(logits, ids, weights, oracle_res, weight_dtype):
    """ids: bit-exact against the oracle's selection rule applied to our own logits (the reference
    tests do the same, tests/test_triton_moe.py:131), and against the oracle's ids wherever the cut
    is not a near-tie."""
    logits_c, ids_c, weights_c = logits.float().cpu(), ids.cpu(), weights.float().cpu()
    atol, rtol = default_tolerance(torch.float32)
    torch.testing.assert_close(logits_c, oracle_res.logits, atol=atol, rtol=rtol)
    k = ids_c.shape[-1]
    own_ids, own_w = O.route_from_logits(logits_c, k)
    assert torch.equal(ids_c, own_ids), "top-k ids differ from the oracle rule on the kernel's own logits"
    torch.testing.assert_close(weights_c, own_w, atol=1e-6, rtol=1e-5)
    clear = oracle_res.margin > TIE_MARGIN
    assert torch.equal(ids_c[clear], oracle_res.topk_ids[clear]), "top-k ids differ from the oracle"
    return int((~clear).sum())


def check_output(out, ref, weight_dtype, *, strict=True):
    out_c = out.float().cpu()
    ma, rl = O.max_abs(out_c, ref), O.rel_l2(out_c, ref)
    if weight_dtype == torch.float32:
        atol, rtol = default_tolerance(torch.float32)
        torch.testing.assert_close(out_c, ref, atol=atol, rtol=rtol)
    else:
        assert ma <= OUT_MAX_ABS, f"max-abs {ma:.3e} > {OUT_MAX_ABS}"
        assert rl <= OUT_REL_L2, f"rel-L2 {rl:.3e} > {OUT_REL_L2}"
    return ma, rl


def check_output_where_ids_agree(out, ids, ref_ids, ref_out, weight_dtype, *, what=""):
    """Outputs are compared token by token on every token whose ids equal the oracle's.  A token whose cut is a
    near-tie may route differently (fp32 sums in another order) and is left out, but never silently: at most one
    token in 64 (and at least one allowed) may be left out, and the count is printed."""
    ids_c = ids.cpu()
    same = (ids_c == ref_ids).all(dim=-1)
    excluded = int((~same).sum())
    allowed = max(1, ids_c.shape[0] // 64)
    assert excluded <= allowed, f"{what}: {excluded} of {ids_c.shape[0]} tokens route differently from the oracle (allowed {allowed})"
    assert int(same.sum()) > 0, f"{what}: no token left to compare"
    if excluded:
        print(f"{what}: {excluded} near-tie token(s) left out of the output comparison")
    return check_output(out.float().cpu()[same], ref_out[same], weight_dtype)


def oracle_layer(hidden, w, top_k, **kw):
    cpu = [None if t is None else t.detach().cpu() for t in w.tuple()]
    bias = None if w.router_bias is None else w.router_bias.cpu()
    return O.moe_update(hidden.detach().cpu(), *cpu, top_k=top_k, router_bias=bias, **kw)
