"""Call inlining and static while-loop unrolling (the host-side counterpart of the reference's text transformations,
Sources/PJRTMetalHLO/PJRTExecutable.swift:458-1657), checked on the host: no `call` / `while` survives, the op counts are
what the trip counts imply, and loops without a static trip count are left alone (and later refused by the executor)."""
import re

import pytest

from metalhlo_b200 import capi
from op_cases import CASES

BY_NAME = {c[0]: c for c in CASES}


def ops(text):
    return re.findall(r'"(?:stablehlo|func|chlo)\.([a-z_]+)"', text)


def test_nested_calls_are_inlined_into_main():
    out = capi.optimize_text(BY_NAME["call_nested"][1], 0)
    got = ops(out)
    assert "call" not in got
    assert got.count("tanh") == 2 and got.count("add") == 2 and got.count("exponential") == 1


def test_fori_loop_is_unrolled_with_constant_counters():
    out = capi.optimize_text(BY_NAME["while_fori_loop"][1], 0)
    got = ops(out)
    assert "while" not in got
    assert got.count("multiply") == 5            # one body copy per iteration
    # iterations 1..4 read their counter from a fresh constant, not from a chain of scalar adds
    for value in (1, 2, 3, 4):
        assert f"dense<{value}> : tensor<i32>" in out
    opt = capi.optimize_text(BY_NAME["while_fori_loop"][1], 2)
    assert ops(opt).count("custom_call") == 1     # the whole unrolled chain fuses into one elementwise kernel


def test_countdown_loop_with_a_call_in_its_body():
    out = capi.optimize_text(BY_NAME["while_countdown_with_call"][1], 0)
    got = ops(out)
    assert "while" not in got and "call" not in got
    assert got.count("sine") == 3                 # 7, 5, 3 pass the test "> 1"; the loop stops at 1


def test_loops_without_a_static_trip_count_stay():
    text = """module {
  func.func public @main(%arg0: tensor<i32>, %arg1: tensor<8xf32>) -> (tensor<8xf32>) {
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg1) : tensor<i32>, tensor<8xf32>
     cond {
      %1 = stablehlo.compare  LT, %iterArg, %arg0,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %1 = stablehlo.add %iterArg, %c_1 : tensor<i32>
      %2 = stablehlo.add %iterArg_0, %iterArg_0 : tensor<8xf32>
      stablehlo.return %1, %2 : tensor<i32>, tensor<8xf32>
    }
    return %0#1 : tensor<8xf32>
  }
}
"""
    assert "while" in ops(capi.optimize_text(text, 0))


def test_unknown_callee_and_recursion_are_errors():
    with pytest.raises(capi.MetalHLOError) as e:
        capi.optimize_text("""module {
  func.func public @main(%arg0: tensor<4xf32>) -> (tensor<4xf32>) {
    %0 = call @missing(%arg0) : (tensor<4xf32>) -> tensor<4xf32>
    return %0 : tensor<4xf32>
  }
}
""", 0)
    assert "missing" in str(e.value)
    with pytest.raises(capi.MetalHLOError):
        capi.optimize_text("""module {
  func.func public @main(%arg0: tensor<4xf32>) -> (tensor<4xf32>) {
    %0 = call @f(%arg0) : (tensor<4xf32>) -> tensor<4xf32>
    return %0 : tensor<4xf32>
  }
  func.func private @f(%arg0: tensor<4xf32>) -> tensor<4xf32> {
    %0 = call @f(%arg0) : (tensor<4xf32>) -> tensor<4xf32>
    return %0 : tensor<4xf32>
  }
}
""", 0)
