"""GPU: the two callers around the hot path -- the decode loop with a switchable MoE implementation and the
matched-operator comparison at the routed-experts-only boundary."""

import pytest
import torch

from fastkernels_b200.spec import MoESpec, synthetic_qwen36_spec

pytestmark = pytest.mark.gpu


def test_decode_runner_both_moe_impls_agree_on_a_four_layer_tiny_model():
    from fastkernels_b200.decode_runner import DecodeRunner, build_layers
    spec = synthetic_qwen36_spec()
    layers = build_layers(spec, 4, torch.float32, "cuda")
    outs = {}
    for impl in ("reference", "b200"):
        runner = DecodeRunner(layers, spec, moe_impl=impl, dtype=torch.float32, seed=3, vocab=64)
        generated, logits = runner.generate([1, 7], 3)
        torch.cuda.synchronize()
        outs[impl] = (generated, logits.clone())
        assert runner.position == 5
    assert outs["reference"][0] == outs["b200"][0]
    torch.testing.assert_close(outs["b200"][1], outs["reference"][1], atol=1e-4, rtol=1e-4)


def test_decode_runner_real_shape_two_layers_bf16():
    from fastkernels_b200.decode_runner import DecodeRunner, build_layers
    spec = MoESpec()
    layers = build_layers(spec, 2, torch.bfloat16, "cuda")
    logits = {}
    for impl in ("reference", "b200"):
        runner = DecodeRunner(layers, spec, moe_impl=impl, dtype=torch.bfloat16, seed=4, vocab=128)
        logits[impl] = runner.step(5).clone()
    torch.cuda.synchronize()
    # the residual stream passes through bf16 between layers in both arms; the kernels round nothing else
    torch.testing.assert_close(logits["b200"], logits["reference"], atol=2e-2, rtol=2e-2)


def test_decode_runner_cli_prints_the_reference_runner_keys(capsys):
    from fastkernels_b200 import decode_runner
    decode_runner.main(["--spec", "tiny", "--dtype", "float32", "--layers", "4", "--prompt-token-ids", "0,3", "--max-new-tokens", "2"])
    text = capsys.readouterr().out
    for key in ("elapsed_ms_per_position:", "elapsed_ms_per_layer_position:", "layer_positions_per_second:", "moe_impl: b200",
                "generated_token_ids:", "layers_executed: 4"):
        assert key in text


def test_routed_moe_comparison_harness(capsys):
    from fastkernels_b200 import compare_routed_moe
    res = compare_routed_moe.main(["--tokens", "2", "--iters", "3", "--warmup", "1", "--hidden-scale", "0.02"])
    text = capsys.readouterr().out
    assert "comparison_scope: routed_experts_only" in text and "fastkernels_routed_moe_tokens_per_second:" in text
    assert "vllm_available:" in text
    assert res["fastkernels_routed_max_abs_diff"] < 1e-5          # values are ~1e-4: a relative 1e-2 bound
    bigger = compare_routed_moe.main(["--tokens", "3", "--iters", "2", "--warmup", "1", "--hidden-scale", "0.2", "--seed", "1"])
    assert bigger["fastkernels_routed_max_abs_diff"] < 5e-3       # outputs of order 10 here
