"""Host-side compiler core, no GPU: the parser and the pass pipeline over the op-case corpus and over the
structural expectations the reference's own tests state (pattern -> custom_call target, pass sets per level)."""
import re

import pytest

from metalhlo_b200 import capi
from op_cases import CASES, attention_text
from oracle import interp

BY_NAME = {c[0]: c for c in CASES}


def targets(text):
    return re.findall(r'call_target_name = "(\w+)"', text)


def live_ops(text):
    return re.findall(r'= "stablehlo\.(\w+)"', text)


@pytest.mark.parametrize("name", [c[0] for c in CASES])
def test_oracle_and_compiler_accept_case(name):
    _, text, inputs = BY_NAME[name]
    outs = interp.evaluate(text, inputs)
    assert len(outs) >= 1
    for level in (0, 1, 2, 3):
        out = capi.optimize_text(text, level)
        assert "func.func @main" in out
    # the printer's output is itself parseable by both parsers (round trip)
    again = capi.optimize_text(capi.optimize_text(text, 0), 0)
    assert live_ops(again) == live_ops(capi.optimize_text(text, 0))


@pytest.mark.parametrize("name", [c[0] for c in CASES])
def test_every_case_lowers_to_a_step_list_without_a_device(name):
    _, text, _ = BY_NAME[name]
    for level in (0, 2, 3):
        steps, launches, arena = capi.plan_text(text, level)
        assert launches >= len(steps)
        assert arena >= 0
        assert all(steps), steps


def test_long_sort_plans_its_global_stages():
    _, text, _ = BY_NAME["sort_global_20000"]
    steps, launches, arena = capi.plan_text(text, 3)
    # 32768 padded keys: key build, chunk sort, (1 global stage + merge) for 16384, (2 + merge) for 32768, apply
    assert steps == ["sort"] and launches == 8
    assert arena >= 3 * 32768 * 12


def test_conditionals_become_selects():
    _, text, _ = BY_NAME["case_index_1"]
    flat = capi.optimize_text(text, 0)
    assert "stablehlo.case" not in flat and "stablehlo.if" not in flat
    assert flat.count('"stablehlo.select"') >= 3  # two for the case, one for the nested if


def test_parse_errors_report_status_3_with_a_line_number():
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text("module { func.func @main(%a: tensor<2xf32>) -> tensor<2xf32> { %0 = stablehlo.add %a, %b : tensor<2xf32>\n return %0 : tensor<2xf32> } }", 0)
    assert e.value.status == 3 and "%b" in str(e.value)
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text("this is not mlir", 0)
    assert e.value.status == 3
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text("func.func @main(%a: tensor<?xf32>) -> tensor<?xf32> { return %a : tensor<?xf32> }", 0)
    assert e.value.status == 3 and "dynamic" in str(e.value)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_o3_rewrites_patterns_to_the_reference_custom_call_targets(dt):
    # Tests/MetalHLOCoreTests/HLOOptimizerTests.swift:265-436 (attention -> fused_scaled_dot_product_attention) and
    # PassManagerTests: softmax / layer norm / rms norm / gelu / matmul+bias+activation
    expect = {
        f"pattern_softmax_{dt}": ["fused_softmax"], f"pattern_softmax_axis1_{dt}": ["fused_softmax"],
        f"pattern_layer_norm_{dt}": ["fused_layer_norm"], f"pattern_layer_norm_plain_{dt}": ["fused_layer_norm"],
        f"pattern_rms_norm_{dt}": ["fused_rms_norm"], f"pattern_gelu_{dt}": ["fused_gelu"],
        f"pattern_residual_layer_norm_{dt}": ["fused_add_layer_norm"], f"pattern_residual_rms_norm_{dt}": ["fused_add_rms_norm"],
        f"pattern_residual_table_layer_norm_side0_{dt}": ["fused_add_layer_norm"], f"pattern_residual_table_layer_norm_side1_{dt}": ["fused_add_layer_norm"],
        f"pattern_residual_table_rms_norm_{dt}": ["fused_add_rms_norm"],
        f"pattern_dense_gelu_{dt}": ["fused_matmul_bias_activation"],
        f"pattern_dense_residual_norm_{dt}": ["fused_matmul_bias_activation", "fused_add_layer_norm"],
        f"pattern_dense_residual_plain_{dt}": ["fused_matmul_bias_activation"],
        f"pattern_conv_bias_none_{dt}": ["fused_conv_bias_act"], f"pattern_conv_bias_relu_{dt}": ["fused_conv_bias_act"],
        f"pattern_conv_bias_tanh_{dt}": ["fused_conv_bias_act"], f"pattern_conv_bias_sigmoid_{dt}": ["fused_conv_bias_act"],
        f"pattern_conv_bias_silu_{dt}": ["fused_conv_bias_act"],
        f"pattern_attention_BHSD_full_{dt}": ["fused_scaled_dot_product_attention"],
        f"pattern_attention_BSHD_causal_{dt}": ["fused_scaled_dot_product_attention"],
    }
    for name, want in expect.items():
        out = capi.optimize_text(BY_NAME[name][1], 3)
        assert targets(out) == want, (name, targets(out))
        # the interior of the pattern is gone: nothing but layout ops and constants may remain
        assert set(live_ops(out)) <= {"custom_call", "transpose", "constant", "broadcast_in_dim", "reshape"}, live_ops(out)


def test_fused_configs_carry_the_values_of_the_matched_graph():
    out = capi.optimize_text(BY_NAME["pattern_layer_norm_plain_f32"][1], 3)
    assert '\\"eps\\":0.001' in out  # eps read from the graph, not the reference's hard-coded 1e-5
    out = capi.optimize_text(BY_NAME["pattern_rms_norm_f32"][1], 3)
    assert '\\"eps\\":9.99999' in out or '\\"eps\\":1e-06' in out or '\\"eps\\":1.0000000000000' in out
    text, _ = attention_text(2, 3, 48, 32, "f32", True, "BHSD", scale=0.25)
    out = capi.optimize_text(text, 3)
    assert '\\"scale\\":0.25' in out and '\\"is_causal\\":true' in out and '\\"head_dim\\":32' in out
    text, _ = attention_text(2, 3, 48, 32, "f32", False, "BHSD")
    out = capi.optimize_text(text, 3)
    assert '\\"is_causal\\":false' in out and '\\"scale\\":0.17677' in out
    out = capi.optimize_text(BY_NAME["pattern_dense_gelu_f32"][1], 3)
    assert '\\"activation\\":\\"gelu_tanh\\"' in out and '\\"has_bias\\":true' in out
    # the residual add moves into the product: one more operand, no add left
    out = capi.optimize_text(BY_NAME["pattern_dense_residual_norm_f16"][1], 3)  # a sum that feeds a norm stays with the norm
    assert "has_residual" not in out and "fused_add_layer_norm" in out and "stablehlo.add" not in out
    # Tests/MetalHLOTests/Conformance/StableHLO/OptimizationCorrectnessTests.swift:488-540: one fused_conv_bias_act call that keeps
    # the convolution's attributes and names the activation
    for act in ("none", "relu", "tanh", "sigmoid", "silu"):
        out = capi.optimize_text(BY_NAME[f"pattern_conv_bias_{act}_f32"][1], 3)
        assert f'\\"activation\\":\\"{act}\\"' in out and '\\"has_bias\\":true' in out and "stablehlo.convolution" not in out
        assert "window_strides" in out and "feature_group_count" in out
        assert capi.plan_text(BY_NAME[f"pattern_conv_bias_{act}_f32"][1], 3)[0] == ["convolution.patches", "convolution.gemm+epilogue"]
    out = capi.optimize_text(BY_NAME["pattern_dense_residual_plain_f32"][1], 3)
    assert '\\"has_residual\\":true' in out and '\\"has_bias\\":false' in out and "stablehlo.add" not in out


def test_pass_sets_per_level_follow_the_reference():
    # Sources/MetalHLO/CompilationConfig.swift:232-263: pattern fusion only at O3, producer-consumer fusion from O2
    text = BY_NAME["pattern_gelu_f32"][1]
    assert targets(capi.optimize_text(text, 0)) == []
    assert targets(capi.optimize_text(text, 1)) == []
    assert targets(capi.optimize_text(text, 2)) == ["fused_elementwise"]
    assert targets(capi.optimize_text(text, 3)) == ["fused_gelu"]
    sm = BY_NAME["pattern_softmax_f32"][1]
    assert "fused_softmax" not in targets(capi.optimize_text(sm, 2))


def test_algebraic_simplifier_rules():
    # Sources/MetalHLOCore/Optimizer/AlgebraicSimplifier.swift:68-94
    t = "tensor<4xf32>"
    prog = f"""func.func @main(%x: {t}) -> {t} {{
      %z = stablehlo.constant dense<0.0> : {t}
      %o = stablehlo.constant dense<1.0> : {t}
      %0 = stablehlo.add %x, %z : {t}
      %1 = stablehlo.multiply %0, %o : {t}
      %2 = stablehlo.subtract %1, %z : {t}
      %3 = stablehlo.divide %2, %o : {t}
      %4 = stablehlo.negate %3 : {t}
      %5 = stablehlo.negate %4 : {t}
      %6 = stablehlo.log %5 : {t}
      %7 = stablehlo.exponential %6 : {t}
      return %7 : {t}
    }}"""
    out = capi.optimize_text(prog, 1)
    assert live_ops(out) == []  # everything folds to "return %x"
    assert live_ops(capi.optimize_text(prog, 0)) != []
    tr = """func.func @main(%x: tensor<2x3xf32>) -> tensor<2x3xf32> {
      %0 = stablehlo.transpose %x, dims = [1, 0] : (tensor<2x3xf32>) -> tensor<3x2xf32>
      %1 = stablehlo.transpose %0, dims = [1, 0] : (tensor<3x2xf32>) -> tensor<2x3xf32>
      %2 = stablehlo.reshape %1 : (tensor<2x3xf32>) -> tensor<6xf32>
      %3 = stablehlo.reshape %2 : (tensor<6xf32>) -> tensor<2x3xf32>
      return %3 : tensor<2x3xf32>
    }"""
    assert live_ops(capi.optimize_text(tr, 1)) == []


def test_cse_and_dce():
    t = "tensor<8xf32>"
    prog = f"""func.func @main(%x: {t}, %y: {t}) -> {t} {{
      %0 = stablehlo.add %x, %y : {t}
      %1 = stablehlo.add %x, %y : {t}
      %dead = stablehlo.multiply %x, %x : {t}
      %2 = stablehlo.multiply %0, %1 : {t}
      return %2 : {t}
    }}"""
    assert live_ops(capi.optimize_text(prog, 2)).count("add") + targets(capi.optimize_text(prog, 2)).count("fused_elementwise") <= 2
    o1 = live_ops(capi.optimize_text(prog, 1))
    assert o1.count("multiply") == 1  # the dead multiply is gone at O1, CSE only from O2
    assert o1.count("add") == 2


def test_dot_general_layout_canonicalisation_inserts_transposes():
    # Sources/MetalHLOCore/Optimizer/Canonicalizers.swift:903-1091: lhs [batch.., M.., K..], rhs [batch.., K.., N..]
    text = BY_NAME["dot_mha_qk_f32"][1]
    out = capi.optimize_text(text, 1)
    assert live_ops(out).count("transpose") == 2
    assert "lhs_batching_dimensions = [0, 1]" in out and "rhs_contracting_dimensions = [2]" in out
    assert "transpose" not in live_ops(capi.optimize_text(text, 0))


def test_position_table_added_before_the_first_norm_is_read_by_the_norm_kernel():
    # add(gathered tokens, broadcast position table) + LayerNorm: one launch that reads the table's rows modulo its height
    from metalhlo_b200 import modules
    text = modules.gpt2_module(batch=2, seq=64, layers=1)
    text = text[0] if isinstance(text, tuple) else text
    steps, _, _ = capi.plan_text(text, 3)
    assert "fused_add_layer_norm [repeated addend]" in steps[:4] and "add" not in steps[:4]
    for dt in ("f32", "f16", "bf16"):
        for name in (f"pattern_residual_table_layer_norm_side0_{dt}", f"pattern_residual_table_layer_norm_side1_{dt}", f"pattern_residual_table_rms_norm_{dt}"):
            assert capi.plan_text(BY_NAME[name][1], 3)[0][0].endswith("[repeated addend]")


def test_complex_values_become_float_pairs_behind_the_parser():
    """tensor<..xcomplex<f32>> is read as tensor<..x2xf32>; the operations on it are rewritten so that no later stage sees
    a complex type. The reference's element-type enum has none either (Sources/CMetalHLO/include/metalhlo.h:61-75) and
    its FFT kernels take (re, im) float pairs (Compiler/CodeGenerator.swift:2701-2830)."""
    _, text, _ = BY_NAME["fft_fft_8x16"]
    flat = capi.optimize_text(text, 0)
    assert "complex" not in flat and "tensor<2x8x16x2xf32>" in flat
    assert live_ops(flat).count("fft") == 1 and "concatenate" in live_ops(flat)
    steps, launches, _ = capi.plan_text(text, 3)
    assert "fft.FFT" in steps and launches >= 2  # one launch per transformed axis
    _, text, _ = BY_NAME["fft_rfft_irfft_3x4x9"]
    steps, launches, _ = capi.plan_text(text, 3)
    assert steps == ["fft.RFFT", "fft.IRFFT"] and launches == 6
    c = "tensor<4xcomplex<f32>>"
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text(f"func.func @main(%a: {c}) -> {c} {{ %0 = stablehlo.tanh %a : {c}\n return %0 : {c} }}", 0)
    assert e.value.status == 4 and "complex" in str(e.value)
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text("func.func @main(%a: tensor<4xcomplex<i32>>) -> tensor<4xcomplex<i32>> { return %a : tensor<4xcomplex<i32>> }", 0)
    assert e.value.status == 3
    with pytest.raises(capi.MetalHLOError) as e:
        capi.plan_text("func.func @main(%a: tensor<4x6xf32>) -> tensor<4x5xcomplex<f32>> { %0 = stablehlo.fft %a, type = RFFT, length = [6] : "
                       "(tensor<4x6xf32>) -> tensor<4x5xcomplex<f32>>\n return %0 : tensor<4x5xcomplex<f32>> }", 0)
    assert e.value.status == 5 and "transforms" in str(e.value)
