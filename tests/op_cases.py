"""Seeded StableHLO programs that exercise the backend's operator surface one op (or one fusable pattern) at a time.

Each case is (name, module text, list of numpy inputs). The texts are written in the forms `jax.jit` prints (pretty
ops, `dims = [...]`, `contracting_dims = [..] x [..]`, reduce with `applies`) plus the generic `"stablehlo.op"(...)`
form for gather. The GPU tests run every case through the C API at several optimisation levels and compare with the
numpy oracle (oracle/interp.py); the CPU tests run the oracle and the host-side compiler on them.
"""
from __future__ import annotations

import math
import re

import numpy as np

from metalhlo_b200.modules import attention_text, func, gelu_text, layer_norm_text, softmax_text, tt  # noqa: F401

try:
    import ml_dtypes

    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    BF16 = None

NP = {"f32": np.float32, "f16": np.float16, "f64": np.float64, "i32": np.int32, "i64": np.int64, "i8": np.int8,
      "i16": np.int16, "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64, "i1": np.bool_}
if BF16 is not None:
    NP["bf16"] = BF16


def rand(rng, shape, dt, lo=-2.0, hi=2.0):
    if dt in ("f32", "f16", "f64", "bf16"):
        return rng.uniform(lo, hi, size=shape).astype(np.float32).astype(NP[dt])
    if dt == "i1":
        return rng.integers(0, 2, size=shape).astype(np.bool_)
    info = np.iinfo(NP[dt])
    return rng.integers(max(info.min, -50), min(info.max, 50) + 1, size=shape).astype(NP[dt])


def build_cases():
    rng = np.random.default_rng(20240229)
    cases = []

    def add(name, text, inputs):
        cases.append((name, text, inputs))

    # ---- unary float ops
    unary = ["abs", "negate", "exponential", "tanh", "logistic", "sine", "cosine", "floor", "ceil", "sign",
             "exponential_minus_one", "cbrt", "round_nearest_even", "round_nearest_afz"]
    positive = ["log", "sqrt", "rsqrt", "log_plus_one"]
    for dt in ("f32", "f16", "bf16"):
        if dt not in NP:
            continue
        for op in unary + positive:
            shape = (5, 37)
            x = rand(rng, shape, dt, 0.1, 3.0) if op in positive else rand(rng, shape, dt)
            t = tt(shape, dt)
            add(f"{op}_{dt}", func([t], [t], f"    %0 = stablehlo.{op} %arg0 : {t}", "%0"), [x])
    # ---- binary float ops
    for dt in ("f32", "bf16"):
        if dt not in NP:
            continue
        for op in ["add", "subtract", "multiply", "divide", "maximum", "minimum", "power", "atan2", "remainder"]:
            shape = (3, 4, 19)
            a = rand(rng, shape, dt, 0.2, 2.0) if op == "power" else rand(rng, shape, dt)
            b = rand(rng, shape, dt, 0.3, 2.0)
            t = tt(shape, dt)
            add(f"{op}_{dt}", func([t, t], [t], f"    %0 = stablehlo.{op} %arg0, %arg1 : {t}", "%0"), [a, b])
    # ---- integer ops
    for dt in ("i32", "i64", "i8", "ui8", "ui32", "i16"):
        for op in ["add", "subtract", "multiply", "divide", "remainder", "maximum", "minimum", "and", "or", "xor"]:
            shape = (4, 33)
            a, b = rand(rng, shape, dt), rand(rng, shape, dt)
            b = np.where(b == 0, 3, b).astype(NP[dt])
            t = tt(shape, dt)
            add(f"{op}_{dt}", func([t, t], [t], f"    %0 = stablehlo.{op} %arg0, %arg1 : {t}", "%0"), [a, b])
    for dt in ("i32", "ui32", "i64", "i8"):
        for op in ["shift_left", "shift_right_arithmetic", "shift_right_logical"]:
            shape = (64,)
            a = rand(rng, shape, dt)
            b = rng.integers(0, 40, size=shape).astype(NP[dt])
            t = tt(shape, dt)
            add(f"{op}_{dt}", func([t, t], [t], f"    %0 = stablehlo.{op} %arg0, %arg1 : {t}", "%0"), [a, b])
        t = tt((64,), dt)
        add(f"not_{dt}", func([t], [t], f"    %0 = stablehlo.not %arg0 : {t}", "%0"), [rand(rng, (64,), dt)])
        add(f"popcnt_{dt}", func([t], [t], f"    %0 = stablehlo.popcnt %arg0 : {t}", "%0"), [rand(rng, (64,), dt)])
        add(f"clz_{dt}", func([t], [t], f"    %0 = stablehlo.count_leading_zeros %arg0 : {t}", "%0"), [rand(rng, (64,), dt)])
        add(f"negate_{dt}", func([t], [t], f"    %0 = stablehlo.negate %arg0 : {t}", "%0"), [rand(rng, (64,), dt)])
    tb = tt((7, 9), "i1")
    for op in ["and", "or", "xor"]:
        add(f"{op}_i1", func([tb, tb], [tb], f"    %0 = stablehlo.{op} %arg0, %arg1 : {tb}", "%0"),
            [rand(rng, (7, 9), "i1"), rand(rng, (7, 9), "i1")])
    add("not_i1", func([tb], [tb], f"    %0 = stablehlo.not %arg0 : {tb}", "%0"), [rand(rng, (7, 9), "i1")])
    # ---- compare / select / clamp
    for dt in ("f32", "i32"):
        t, p = tt((6, 11), dt), tt((6, 11), "i1")
        a, b = rand(rng, (6, 11), dt), rand(rng, (6, 11), dt)
        b[0] = a[0]
        kind = "FLOAT" if dt == "f32" else "SIGNED"
        for d in ["EQ", "NE", "LT", "LE", "GT", "GE"]:
            add(f"compare_{d}_{dt}", func([t, t], [p], f"    %0 = stablehlo.compare  {d}, %arg0, %arg1,  {kind} : ({t}, {t}) -> {p}", "%0"), [a, b])
        add(f"select_{dt}", func([p, t, t], [t], f"    %0 = stablehlo.select %arg0, %arg1, %arg2 : {p}, {t}", "%0"),
            [rand(rng, (6, 11), "i1"), a, b])
        s = tt((), dt)
        add(f"clamp_{dt}", func([s, t, s], [t], f"    %0 = stablehlo.clamp %arg0, %arg1, %arg2 : ({s}, {t}, {s}) -> {t}", "%0"),
            [np.array(-1, NP[dt]), a, np.array(1, NP[dt])])
    # ---- convert
    pairs = [("f32", "f16"), ("f16", "f32"), ("f32", "bf16"), ("bf16", "f32"), ("f32", "i32"), ("i32", "f32"), ("i64", "i32"),
             ("i32", "i64"), ("i1", "f32"), ("f32", "f64"), ("f64", "f32"), ("i32", "f16"), ("ui8", "f32"), ("i32", "i8")]
    for a, b in pairs:
        if a not in NP or b not in NP:
            continue
        x = rand(rng, (5, 21), a, -40.0, 40.0) if a.startswith("f") or a == "bf16" else rand(rng, (5, 21), a)
        add(f"convert_{a}_{b}", func([tt((5, 21), a)], [tt((5, 21), b)],
                                     f"    %0 = stablehlo.convert %arg0 : ({tt((5, 21), a)}) -> {tt((5, 21), b)}", "%0"), [x])
    # ---- iota / data movement
    for dt in ("i32", "f32", "i64"):
        for dim in (0, 1, 2):
            t = tt((3, 4, 5), dt)
            add(f"iota_{dt}_{dim}", func([], [t], f"    %0 = stablehlo.iota dim = {dim} : {t}", "%0"), [])
    x = rand(rng, (3, 1, 5), "f32")
    add("broadcast_in_dim", func([tt((3, 1, 5), "f32")], [tt((2, 3, 4, 5), "f32")],
                                 f"    %0 = stablehlo.broadcast_in_dim %arg0, dims = [1, 2, 3] : ({tt((3, 1, 5), 'f32')}) -> {tt((2, 3, 4, 5), 'f32')}", "%0"), [x])
    add("broadcast_scalar", func([tt((), "f32")], [tt((4, 6), "f32")],
                                 f"    %0 = stablehlo.broadcast_in_dim %arg0, dims = [] : ({tt((), 'f32')}) -> {tt((4, 6), 'f32')}", "%0"),
        [np.array(2.5, np.float32)])
    x = rand(rng, (2, 3, 4, 5), "f32")
    t4 = tt((2, 3, 4, 5), "f32")
    add("transpose_4d", func([t4], [tt((4, 2, 5, 3), "f32")],
                             f"    %0 = stablehlo.transpose %arg0, dims = [2, 0, 3, 1] : ({t4}) -> {tt((4, 2, 5, 3), 'f32')}", "%0"), [x])
    add("transpose_then_reshape", func([t4], [tt((12, 10), "f32")],
                                       f"    %0 = stablehlo.transpose %arg0, dims = [2, 1, 0, 3] : ({t4}) -> {tt((4, 3, 2, 5), 'f32')}\n"
                                       f"    %1 = stablehlo.reshape %0 : ({tt((4, 3, 2, 5), 'f32')}) -> {tt((12, 10), 'f32')}", "%1"), [x])
    add("reshape", func([t4], [tt((6, 20), "f32")], f"    %0 = stablehlo.reshape %arg0 : ({t4}) -> {tt((6, 20), 'f32')}", "%0"), [x])
    add("reverse", func([t4], [t4], f"    %0 = stablehlo.reverse %arg0, dims = [1, 3] : {t4}", "%0"), [x])
    add("slice", func([t4], [tt((1, 2, 2, 3), "f32")],
                      f"    %0 = stablehlo.slice %arg0 [1:2, 0:3:2, 1:4:2, 0:5:2] : ({t4}) -> {tt((1, 2, 2, 3), 'f32')}", "%0"), [x])
    a, b = rand(rng, (2, 3, 4), "i32"), rand(rng, (2, 5, 4), "i32")
    add("concatenate", func([tt((2, 3, 4), "i32"), tt((2, 5, 4), "i32")], [tt((2, 8, 4), "i32")],
                            f"    %0 = stablehlo.concatenate %arg0, %arg1, dim = 1 : ({tt((2, 3, 4), 'i32')}, {tt((2, 5, 4), 'i32')}) -> {tt((2, 8, 4), 'i32')}", "%0"), [a, b])
    x2 = rand(rng, (3, 4), "f32")
    add("pad_interior", func([tt((3, 4), "f32"), tt((), "f32")], [tt((8, 9), "f32")],
                             f"    %0 = stablehlo.pad %arg0, %arg1, low = [1, 2], high = [2, 0], interior = [1, 1] : ({tt((3, 4), 'f32')}, {tt((), 'f32')}) -> {tt((8, 9), 'f32')}", "%0"),
        [x2, np.array(-7.0, np.float32)])
    add("pad_negative", func([tt((3, 4), "f32"), tt((), "f32")], [tt((4, 2), "f32")],
                             f"    %0 = stablehlo.pad %arg0, %arg1, low = [2, -1], high = [-1, -1], interior = [0, 0] : ({tt((3, 4), 'f32')}, {tt((), 'f32')}) -> {tt((4, 2), 'f32')}", "%0"),
        [x2, np.array(9.0, np.float32)])
    # ---- reduce
    x3 = rand(rng, (4, 70, 9), "f32")
    t3 = tt((4, 70, 9), "f32")
    for red, init in [("add", "0.000000e+00"), ("maximum", "0xFF800000"), ("minimum", "0x7F800000"), ("multiply", "1.000000e+00")]:
        for dims, oshape in [([1], (4, 9)), ([0, 2], (70,)), ([2], (4, 70)), ([0, 1, 2], ())]:
            xin = (x3 * 0.5 + 1.0).astype(np.float32) if red == "multiply" else x3
            if red == "multiply" and len(dims) > 1:
                continue
            add(f"reduce_{red}_{'_'.join(map(str, dims))}",
                func([t3], [tt(oshape, "f32")],
                     f"    %c = stablehlo.constant dense<{init}> : tensor<f32>\n"
                     f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.{red} across dimensions = {dims} : ({t3}, tensor<f32>) -> {tt(oshape, 'f32')}", "%0"), [xin])
    xi = rand(rng, (6, 300), "i32")
    add("reduce_add_i32", func([tt((6, 300), "i32")], [tt((6,), "i32")],
                               "    %c = stablehlo.constant dense<0> : tensor<i32>\n"
                               f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [1] : ({tt((6, 300), 'i32')}, tensor<i32>) -> {tt((6,), 'i32')}", "%0"), [xi])
    xb = rand(rng, (5, 40), "i1")
    for red, init in [("and", "true"), ("or", "false")]:
        add(f"reduce_{red}_i1", func([tt((5, 40), "i1")], [tt((5,), "i1")],
                                     f"    %c = stablehlo.constant dense<{init}> : tensor<i1>\n"
                                     f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.{red} across dimensions = [1] : ({tt((5, 40), 'i1')}, tensor<i1>) -> {tt((5,), 'i1')}", "%0"), [xb])
    # large single-output reduction (the two-level path)
    xl = rand(rng, (3, 50000), "f32")
    add("reduce_add_long", func([tt((3, 50000), "f32")], [tt((3,), "f32")],
                                "    %c = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
                                f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [1] : ({tt((3, 50000), 'f32')}, tensor<f32>) -> {tt((3,), 'f32')}", "%0"), [xl])
    # argmax the way jax.numpy.argmax lowers: variadic reduce over (values, iota) with a compare/select body
    xa = rand(rng, (7, 129), "f32")
    ta, ti = tt((7, 129), "f32"), tt((7, 129), "i32")
    add("argmax", func([ta], [tt((7,), "i32")],
                       f"    %0 = stablehlo.iota dim = 1 : {ti}\n"
                       "    %c = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
                       "    %c0 = stablehlo.constant dense<0> : tensor<i32>\n"
                       f"    %1:2 = stablehlo.reduce(%arg0 init: %c), (%0 init: %c0) across dimensions = [1] : ({ta}, {ti}, tensor<f32>, tensor<i32>) -> ({tt((7,), 'f32')}, {tt((7,), 'i32')})\n"
                       "     reducer(%a: tensor<f32>, %b: tensor<f32>) (%ai: tensor<i32>, %bi: tensor<i32>)  {\n"
                       "      %2 = stablehlo.compare  GT, %a, %b,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                       "      %3 = stablehlo.compare  NE, %a, %a,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                       "      %4 = stablehlo.or %2, %3 : tensor<i1>\n"
                       "      %5 = stablehlo.compare  EQ, %a, %b,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                       "      %6 = stablehlo.compare  LT, %ai, %bi,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>\n"
                       "      %7 = stablehlo.and %5, %6 : tensor<i1>\n"
                       "      %8 = stablehlo.or %4, %7 : tensor<i1>\n"
                       "      %9 = stablehlo.select %4, %a, %b : tensor<i1>, tensor<f32>\n"
                       "      %10 = stablehlo.select %8, %ai, %bi : tensor<i1>, tensor<i32>\n"
                       "      stablehlo.return %9, %10 : tensor<f32>, tensor<i32>\n"
                       "    }", "%1#1"), [xa])
    # reductions to very few outputs over long ranges: the split (partials in scratch memory + finish) path
    rs = np.random.default_rng(77)
    xs = rs.random((512, 2048), dtype=np.float32)
    add("reduce_add_all_split", func([tt((512, 2048), "f32")], [tt((), "f32")],
                                     "    %c = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
                                     f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [0, 1] : ({tt((512, 2048), 'f32')}, tensor<f32>) -> {tt((), 'f32')}", "%0"), [xs])
    xm = rs.standard_normal((2, 300000)).astype(np.float32)
    add("reduce_max_split", func([tt((2, 300000), "f32")], [tt((2,), "f32")],
                                 "    %c = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
                                 f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.maximum across dimensions = [1] : ({tt((2, 300000), 'f32')}, tensor<f32>) -> {tt((2,), 'f32')}", "%0"), [xm])
    xis = rs.integers(-1000, 1000, size=(1, 200000)).astype(np.int32)
    add("reduce_add_i32_split", func([tt((1, 200000), "i32")], [tt((1,), "i32")],
                                     "    %c = stablehlo.constant dense<5> : tensor<i32>\n"
                                     f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [1] : ({tt((1, 200000), 'i32')}, tensor<i32>) -> {tt((1,), 'i32')}", "%0"), [xis])
    xas = rs.standard_normal((2, 150000)).astype(np.float32)
    xas[0, [140000, 70001, 99999]] = 9.5   # ties: the first position wins
    xas[1, 149999] = 11.0                  # the very last element
    tas, tis = tt((2, 150000), "f32"), tt((2, 150000), "i32")
    add("argmax_split", func([tas], [tt((2,), "i32")],
                             f"    %0 = stablehlo.iota dim = 1 : {tis}\n"
                             "    %c = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
                             "    %c0 = stablehlo.constant dense<0> : tensor<i32>\n"
                             f"    %1:2 = stablehlo.reduce(%arg0 init: %c), (%0 init: %c0) across dimensions = [1] : ({tas}, {tis}, tensor<f32>, tensor<i32>) -> ({tt((2,), 'f32')}, {tt((2,), 'i32')})\n"
                             "     reducer(%a: tensor<f32>, %b: tensor<f32>) (%ai: tensor<i32>, %bi: tensor<i32>)  {\n"
                             "      %2 = stablehlo.compare  GT, %a, %b,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                             "      %3 = stablehlo.compare  NE, %a, %a,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                             "      %4 = stablehlo.or %2, %3 : tensor<i1>\n"
                             "      %5 = stablehlo.compare  EQ, %a, %b,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>\n"
                             "      %6 = stablehlo.compare  LT, %ai, %bi,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>\n"
                             "      %7 = stablehlo.and %5, %6 : tensor<i1>\n"
                             "      %8 = stablehlo.or %4, %7 : tensor<i1>\n"
                             "      %9 = stablehlo.select %4, %a, %b : tensor<i1>, tensor<f32>\n"
                             "      %10 = stablehlo.select %8, %ai, %bi : tensor<i1>, tensor<i32>\n"
                             "      stablehlo.return %9, %10 : tensor<f32>, tensor<i32>\n"
                             "    }", "%1#1"), [xas])
    # ---- what jax.jit emits around the straight-line ops: calls of private functions and fori_loop-style while loops
    rc = np.random.default_rng(99)
    xa, xb = rc.standard_normal((4, 8)).astype(np.float32), rc.standard_normal(8).astype(np.float32)
    add("call_nested", """module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<4x8xf32>, %arg1: tensor<8xf32>) -> (tensor<4x8xf32> {jax.result_info = ""}) {
    %0 = call @helper(%arg0, %arg1) : (tensor<4x8xf32>, tensor<8xf32>) -> tensor<4x8xf32>
    %1 = stablehlo.exponential %0 : tensor<4x8xf32>
    %2 = call @helper(%1, %arg1) : (tensor<4x8xf32>, tensor<8xf32>) -> tensor<4x8xf32>
    return %2 : tensor<4x8xf32>
  }
  func.func private @helper(%arg0: tensor<4x8xf32>, %arg1: tensor<8xf32>) -> tensor<4x8xf32> {
    %0 = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<8xf32>) -> tensor<4x8xf32>
    %1 = stablehlo.add %arg0, %0 : tensor<4x8xf32>
    %2 = call @inner(%1) : (tensor<4x8xf32>) -> tensor<4x8xf32>
    return %2 : tensor<4x8xf32>
  }
  func.func private @inner(%arg0: tensor<4x8xf32>) -> tensor<4x8xf32> {
    %0 = stablehlo.tanh %arg0 : tensor<4x8xf32>
    return %0 : tensor<4x8xf32>
  }
}
""", [xa, xb])
    add("while_fori_loop", """module @jit_loop {
  func.func public @main(%arg0: tensor<8xf32>) -> (tensor<8xf32>) {
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0) : tensor<i32>, tensor<8xf32>
     cond {
      %c_1 = stablehlo.constant dense<5> : tensor<i32>
      %1 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %1 = stablehlo.add %iterArg, %c_1 : tensor<i32>
      %cst = stablehlo.constant dense<1.500000e+00> : tensor<8xf32>
      %2 = stablehlo.multiply %iterArg_0, %cst : tensor<8xf32>
      %3 = stablehlo.convert %iterArg : (tensor<i32>) -> tensor<f32>
      %4 = stablehlo.broadcast_in_dim %3, dims = [] : (tensor<f32>) -> tensor<8xf32>
      %5 = stablehlo.add %2, %4 : tensor<8xf32>
      stablehlo.return %1, %5 : tensor<i32>, tensor<8xf32>
    }
    return %0#1 : tensor<8xf32>
  }
}
""", [xb])
    add("while_countdown_with_call", """module @jit_loop2 {
  func.func public @main(%arg0: tensor<4x8xf32>, %arg1: tensor<8xf32>) -> (tensor<4x8xf32>, tensor<i32>) {
    %c = stablehlo.constant dense<7> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %arg0, %iterArg_0 = %c) : tensor<4x8xf32>, tensor<i32>
     cond {
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %1 = stablehlo.compare  GT, %iterArg_0, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %c_1 = stablehlo.constant dense<2> : tensor<i32>
      %1 = stablehlo.subtract %iterArg_0, %c_1 : tensor<i32>
      %2 = call @step(%iterArg, %arg1) : (tensor<4x8xf32>, tensor<8xf32>) -> tensor<4x8xf32>
      stablehlo.return %2, %1 : tensor<4x8xf32>, tensor<i32>
    }
    return %0#0, %0#1 : tensor<4x8xf32>, tensor<i32>
  }
  func.func private @step(%arg0: tensor<4x8xf32>, %arg1: tensor<8xf32>) -> tensor<4x8xf32> {
    %0 = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<8xf32>) -> tensor<4x8xf32>
    %1 = stablehlo.multiply %arg0, %0 : tensor<4x8xf32>
    %2 = stablehlo.sine %1 : tensor<4x8xf32>
    return %2 : tensor<4x8xf32>
  }
}
""", [xa, xb])
    # ---- dot_general
    def dot_case(name, ashape, bshape, attrs, oshape, dt):
        if dt not in NP:
            return
        scale = 1.0 / math.sqrt(max(1, ashape[-1]))
        a = (rand(rng, ashape, "f32") * scale).astype(NP[dt]) if dt != "i32" else rand(rng, ashape, dt)
        b = rand(rng, bshape, dt)
        add(name, func([tt(ashape, dt), tt(bshape, dt)], [tt(oshape, dt)],
                       f"    %0 = stablehlo.dot_general %arg0, %arg1, {attrs} : ({tt(ashape, dt)}, {tt(bshape, dt)}) -> {tt(oshape, dt)}", "%0"), [a, b])

    for dt in ("f32", "f16", "bf16", "i32"):
        dot_case(f"dot_mk_kn_{dt}", (33, 70), (70, 45), "contracting_dims = [1] x [0]", (33, 45), dt)
        dot_case(f"dot_mk_nk_{dt}", (33, 70), (45, 70), "contracting_dims = [1] x [1]", (33, 45), dt)
        dot_case(f"dot_km_kn_{dt}", (70, 33), (70, 45), "contracting_dims = [0] x [0]", (33, 45), dt)
        dot_case(f"dot_batched_{dt}", (3, 17, 24), (3, 24, 40), "batching_dims = [0] x [0], contracting_dims = [2] x [1]", (3, 17, 40), dt)
        dot_case(f"dot_mha_qk_{dt}", (2, 9, 3, 16), (2, 11, 3, 16), "batching_dims = [0, 2] x [0, 2], contracting_dims = [3] x [3]", (2, 3, 9, 11), dt)
        dot_case(f"dot_mha_pv_{dt}", (2, 3, 9, 11), (2, 11, 3, 16), "batching_dims = [0, 1] x [0, 2], contracting_dims = [3] x [1]", (2, 3, 9, 16), dt)
        dot_case(f"dot_lead_{dt}", (4, 6, 32), (32, 24), "contracting_dims = [2] x [0]", (4, 6, 24), dt)
        dot_case(f"dot_two_contract_{dt}", (5, 4, 8), (4, 8, 7), "contracting_dims = [1, 2] x [0, 1]", (5, 7), dt)
    dot_case("dot_aligned_bf16", (256, 512), (512, 384), "contracting_dims = [1] x [0]", (256, 384), "bf16")
    dot_case("dot_aligned_f16", (256, 512), (384, 512), "contracting_dims = [1] x [1]", (256, 384), "f16")
    dot_case("dot_aligned_batched_bf16", (4, 128, 256), (4, 256, 128), "batching_dims = [0] x [0], contracting_dims = [2] x [1]", (4, 128, 128), "bf16")
    # ---- gather: embedding lookup as jnp.take / x[ids] lowers, and a windowed gather
    table = rand(rng, (50, 24), "f32")
    ids = rng.integers(0, 50, size=(4, 7)).astype(np.int32)
    ids[0, 0] = 49
    add("gather_embedding", func([tt((50, 24), "f32"), tt((4, 7), "i32")], [tt((4, 7, 24), "f32")],
                                 f"    %0 = stablehlo.reshape %arg1 : ({tt((4, 7), 'i32')}) -> {tt((4, 7, 1), 'i32')}\n"
                                 f"    %1 = \"stablehlo.gather\"(%arg0, %0) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1, 24>}}> : ({tt((50, 24), 'f32')}, {tt((4, 7, 1), 'i32')}) -> {tt((4, 7, 24), 'f32')}", "%1"),
        [table, ids])
    # token ids outside the table: start indices are clamped into it (negative ones to row 0, large ones to the last row)
    wild = np.array([[-3, 0, 49, 50, 1000, -2147483648, 2147483647]], dtype=np.int32)
    add("gather_embedding_ids_out_of_range", func([tt((50, 24), "f32"), tt((1, 7), "i32")], [tt((1, 7, 24), "f32")],
                                                  f"    %0 = stablehlo.reshape %arg1 : ({tt((1, 7), 'i32')}) -> {tt((1, 7, 1), 'i32')}\n"
                                                  f"    %1 = \"stablehlo.gather\"(%arg0, %0) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1, 24>}}> : ({tt((50, 24), 'f32')}, {tt((1, 7, 1), 'i32')}) -> {tt((1, 7, 24), 'f32')}", "%1"),
        [table, wild])
    for it, arr in (("ui8", np.array([[0, 49, 7, 200, 255]], np.uint8)), ("i16", np.array([[-5, 3, 49, 32767, -32768]], np.int16))):
        add(f"gather_embedding_{it}_ids", func([tt((50, 24), "f32"), tt((1, 5), it)], [tt((1, 5, 24), "f32")],
                                              f"    %0 = stablehlo.reshape %arg1 : ({tt((1, 5), it)}) -> {tt((1, 5, 1), it)}\n"
                                              f"    %1 = \"stablehlo.gather\"(%arg0, %0) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1, 24>}}> : ({tt((50, 24), 'f32')}, {tt((1, 5, 1), it)}) -> {tt((1, 5, 24), 'f32')}", "%1"),
            [table, arr])
    op3 = rand(rng, (3, 4, 6), "i32")
    idx = np.array([[[0, 0], [1, 0], [2, 1]], [[0, 1], [1, 1], [0, 9]]], dtype=np.int64)
    add("gather_window", func([tt((3, 4, 6), "i32"), tt((2, 3, 2), "i64")], [tt((2, 3, 2, 3), "i32")],
                              "    %0 = \"stablehlo.gather\"(%arg0, %arg1) {dimension_numbers = #stablehlo.gather<offset_dims = [2, 3], collapsed_slice_dims = [0], start_index_map = [1, 0], index_vector_dim = 2>, slice_sizes = array<i64: 1, 2, 3>, indices_are_sorted = false} : "
                              f"({tt((3, 4, 6), 'i32')}, {tt((2, 3, 2), 'i64')}) -> {tt((2, 3, 2, 3), 'i32')}", "%0"), [op3, idx])
    # ---- dynamic slicing
    xd = rand(rng, (6, 8), "f32")
    add("dynamic_slice", func([tt((6, 8), "f32"), tt((), "i32"), tt((), "i32")], [tt((2, 3), "f32")],
                              f"    %0 = stablehlo.dynamic_slice %arg0, %arg1, %arg2, sizes = [2, 3] : ({tt((6, 8), 'f32')}, tensor<i32>, tensor<i32>) -> {tt((2, 3), 'f32')}", "%0"),
        [xd, np.array(5, np.int32), np.array(2, np.int32)])
    add("dynamic_update_slice", func([tt((6, 8), "f32"), tt((2, 3), "f32"), tt((), "i32"), tt((), "i32")], [tt((6, 8), "f32")],
                                     f"    %0 = stablehlo.dynamic_update_slice %arg0, %arg1, %arg2, %arg3 : ({tt((6, 8), 'f32')}, {tt((2, 3), 'f32')}, tensor<i32>, tensor<i32>) -> {tt((6, 8), 'f32')}", "%0"),
        [xd, rand(rng, (2, 3), "f32"), np.array(1, np.int32), np.array(7, np.int32)])
    for nm, s0, s1, it in (("negative_starts", -4, -1, "i32"), ("far_starts_i64", 2 ** 40, -2 ** 40, "i64"), ("ui8_starts", 200, 3, "ui8")):
        ti_ = f"tensor<{it}>"
        add(f"dynamic_slice_{nm}", func([tt((6, 8), "f32"), tt((), it), tt((), it)], [tt((2, 3), "f32")],
                                        f"    %0 = stablehlo.dynamic_slice %arg0, %arg1, %arg2, sizes = [2, 3] : ({tt((6, 8), 'f32')}, {ti_}, {ti_}) -> {tt((2, 3), 'f32')}", "%0"),
            [xd, np.array(s0, NP[it]), np.array(s1, NP[it])])
        add(f"dynamic_update_slice_{nm}", func([tt((6, 8), "f32"), tt((2, 3), "f32"), tt((), it), tt((), it)], [tt((6, 8), "f32")],
                                               f"    %0 = stablehlo.dynamic_update_slice %arg0, %arg1, %arg2, %arg3 : ({tt((6, 8), 'f32')}, {tt((2, 3), 'f32')}, {ti_}, {ti_}) -> {tt((6, 8), 'f32')}", "%0"),
            [xd, rand(rng, (2, 3), "f32"), np.array(s0, NP[it]), np.array(s1, NP[it])])
    # ---- fusable patterns (unfused text; O3 must agree with O0)
    for dt in ("f32", "f16", "bf16"):
        if dt not in NP:
            continue
        cases.extend(pattern_cases(rng, dt))
    return cases


def pattern_cases(rng, dt):
    out = []
    shape = (6, 40, 256)
    t = tt(shape, dt)
    x = rand(rng, shape, dt)
    g = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32).astype(NP[dt])
    b = (0.1 * rng.standard_normal(256)).astype(np.float32).astype(NP[dt])
    tv = tt((256,), dt)
    body, res = softmax_text("%arg0", shape, dt, 2)
    out.append((f"pattern_softmax_{dt}", func([t], [t], body.rstrip("\n"), res), [(x.astype(np.float32) * 4).astype(NP[dt])]))
    body, res = softmax_text("%arg0", shape, dt, 1)
    out.append((f"pattern_softmax_axis1_{dt}", func([t], [t], body.rstrip("\n"), res), [x]))
    body, res = layer_norm_text("%arg0", shape, dt, "%arg1", "%arg2")
    out.append((f"pattern_layer_norm_{dt}", func([t, tv, tv], [t], body.rstrip("\n"), res), [x, g, b]))
    body, res = layer_norm_text("%arg0", shape, dt, None, None, eps=1e-3)
    out.append((f"pattern_layer_norm_plain_{dt}", func([t], [t], body.rstrip("\n"), res), [x]))
    body, res = layer_norm_text("%arg0", shape, dt, "%arg1", None, eps=1e-6, rms=True)
    out.append((f"pattern_rms_norm_{dt}", func([t, tv], [t], body.rstrip("\n"), res), [x, g]))
    # residual add feeding a norm, the sum also returned (fused_add_layer_norm / fused_add_rms_norm at O3)
    r2 = np.random.default_rng(sum(map(ord, dt)))
    xr = (0.5 * r2.standard_normal(shape)).astype(np.float32).astype(NP[dt])
    body, res = layer_norm_text("%s0", shape, dt, "%arg2", "%arg3")
    out.append((f"pattern_residual_layer_norm_{dt}", func([t, t, tv, tv], [t, t], f"    %s0 = stablehlo.add %arg0, %arg1 : {t}\n" + body.rstrip("\n"),
                                                           f"%s0, {res}"), [x, xr, g, b]))
    body, res = layer_norm_text("%s0", shape, dt, "%arg2", None, eps=1e-6, rms=True)
    out.append((f"pattern_residual_rms_norm_{dt}", func([t, t, tv], [t, t], f"    %s0 = stablehlo.add %arg0, %arg1 : {t}\n" + body.rstrip("\n"),
                                                         f"%s0, {res}"), [x, xr, g]))
    # the same with an addend that repeats over the leading axis (a position table over the batch): the norm kernel
    # reads the table's rows modulo its height, on either side of the add
    tp = tt(shape[1:], dt)
    xp = (0.5 * np.random.default_rng(7 + sum(map(ord, dt))).standard_normal(shape[1:])).astype(np.float32).astype(NP[dt])
    dims = list(range(1, len(shape)))
    for side in (0, 1):
        add = "%arg0, %p0" if side == 0 else "%p0, %arg0"
        head = (f"    %p0 = stablehlo.broadcast_in_dim %arg1, dims = {dims} : ({tp}) -> {t}\n"
                f"    %s0 = stablehlo.add {add} : {t}\n")
        body, res = layer_norm_text("%s0", shape, dt, "%arg2", "%arg3")
        out.append((f"pattern_residual_table_layer_norm_side{side}_{dt}", func([t, tp, tv, tv], [t, t], head + body.rstrip("\n"), f"%s0, {res}"),
                    [x, xp, g, b]))
    body, res = layer_norm_text("%s0", shape, dt, "%arg2", None, eps=1e-6, rms=True)
    out.append((f"pattern_residual_table_rms_norm_{dt}", func([t, tp, tv], [t, t], head + body.rstrip("\n"), f"%s0, {res}"), [x, xp, g]))
    body, res = gelu_text("%arg0", shape, dt)
    out.append((f"pattern_gelu_{dt}", func([t], [t], body.rstrip("\n"), res), [x]))
    # dense layer: x.w + b then GELU (fused_matmul_bias_activation at O3)
    w = (rng.standard_normal((256, 128)) / 16).astype(np.float32).astype(NP[dt])
    bias = (0.1 * rng.standard_normal(128)).astype(np.float32).astype(NP[dt])
    ts, tw, tbias = tt((6, 40, 128), dt), tt((256, 128), dt), tt((128,), dt)
    gb, gres = gelu_text("%2", (6, 40, 128), dt)
    body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [2] x [0] : ({t}, {tw}) -> {ts}\n"
            f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [2] : ({tbias}) -> {ts}\n"
            f"    %2 = stablehlo.add %0, %1 : {ts}\n" + gb)
    out.append((f"pattern_dense_gelu_{dt}", func([t, tw, tbias], [ts], body.rstrip("\n"), gres), [x, w, bias]))
    # projection back into the residual stream: r + (x.w + b), the sum normalised next (fused_add_layer_norm takes the sum at O3;
    # without a norm behind it the product takes the residual into its epilogue: fused_matmul_bias_activation with has_residual)
    resid = (0.5 * r2.standard_normal((6, 40, 128))).astype(np.float32).astype(NP[dt])
    g128 = (1 + 0.1 * r2.standard_normal(128)).astype(np.float32).astype(NP[dt])
    b128 = (0.1 * r2.standard_normal(128)).astype(np.float32).astype(NP[dt])
    lb, lres = layer_norm_text("%3", (6, 40, 128), dt, "%arg4", "%arg5")
    body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [2] x [0] : ({t}, {tw}) -> {ts}\n"
            f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [2] : ({tbias}) -> {ts}\n"
            f"    %2 = stablehlo.add %0, %1 : {ts}\n"
            f"    %3 = stablehlo.add %arg3, %2 : {ts}\n" + lb)
    out.append((f"pattern_dense_residual_norm_{dt}", func([t, tw, tbias, ts, tbias, tbias], [ts, ts], body.rstrip("\n"), f"%3, {lres}"),
                [x, w, bias, resid, g128, b128]))
    body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [2] x [0] : ({t}, {tw}) -> {ts}\n"
            f"    %1 = stablehlo.add %0, %arg2 : {ts}")
    out.append((f"pattern_dense_residual_plain_{dt}", func([t, tw, ts], [ts], body, "%1"), [x, w, resid]))
    for causal in (False, True):
        for layout in ("BHSD", "BSHD"):
            text, qshape = attention_text(2, 3, 48, 32, dt, causal, layout)
            q, k, v = (rand(rng, qshape, dt, -1, 1) for _ in range(3))
            out.append((f"pattern_attention_{layout}_{'causal' if causal else 'full'}_{dt}", text, [q, k, v]))
    return out


def widening_cases():
    """Control flow with branches, the dynamic_* forms with constant shape operands, bitcast_convert and
    batch_norm_inference: the operators either side of the fused hot path."""
    rng = np.random.default_rng(977)
    out = []
    t48 = tt((4, 8), "f32")
    x48 = rand(rng, (4, 8), "f32")
    y48 = rand(rng, (4, 8), "f32")
    # ---- if: lax.cond prints the generic form with two regions that capture outer values
    if_text = f"""module @jit_cond {{
  func.func public @main(%arg0: tensor<i32>, %arg1: {t48}, %arg2: {t48}) -> ({t48}, tensor<f32>) {{
    %c = stablehlo.constant dense<0> : tensor<i32>
    %p = stablehlo.compare  GT, %arg0, %c,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
    %0:2 = "stablehlo.if"(%p) ({{
      %1 = stablehlo.multiply %arg1, %arg2 : {t48}
      %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
      %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({t48}, tensor<f32>) -> tensor<f32>
      stablehlo.return %1, %2 : {t48}, tensor<f32>
    }}, {{
      %1 = stablehlo.subtract %arg1, %arg2 : {t48}
      %cst = stablehlo.constant dense<1.000000e+00> : tensor<f32>
      stablehlo.return %1, %cst : {t48}, tensor<f32>
    }}) : (tensor<i1>) -> ({t48}, tensor<f32>)
    return %0#0, %0#1 : {t48}, tensor<f32>
  }}
}}
"""
    for v in (1, 0):
        out.append((f"if_{'true' if v else 'false'}", if_text, [np.asarray(v, np.int32), x48, y48]))
    # ---- while with a data-dependent trip count (lax.while_loop): halve until the largest magnitude drops under a bound
    out.append(("while_dynamic_halving", f"""module @jit_halve {{
  func.func public @main(%arg0: {t48}) -> ({t48}, tensor<i32>) {{
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %arg0, %iterArg_0 = %c) : {t48}, tensor<i32>
     cond {{
      %1 = stablehlo.abs %iterArg : {t48}
      %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
      %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.maximum across dimensions = [0, 1] : ({t48}, tensor<f32>) -> tensor<f32>
      %cst_1 = stablehlo.constant dense<3.000000e-01> : tensor<f32>
      %3 = stablehlo.compare  GT, %2, %cst_1,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      stablehlo.return %3 : tensor<i1>
    }} do {{
      %cst = stablehlo.constant dense<5.000000e-01> : tensor<f32>
      %1 = stablehlo.broadcast_in_dim %cst, dims = [] : (tensor<f32>) -> {t48}
      %2 = stablehlo.multiply %iterArg, %1 : {t48}
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %3 = stablehlo.add %iterArg_0, %c_1 : tensor<i32>
      stablehlo.return %2, %3 : {t48}, tensor<i32>
    }}
    return %0#0, %0#1 : {t48}, tensor<i32>
  }}
}}
""", [x48]))
    # a fusable pattern (softmax) inside a loop whose exit depends on the data: sharpen until one entry dominates
    sm_body, sm_res = softmax_text("%sc", (4, 8), "f32", 1, prefix="w")
    out.append(("while_dynamic_softmax_in_body", f"""module @jit_sharpen {{
  func.func public @main(%arg0: {t48}) -> ({t48}, tensor<i32>) {{
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %arg0, %iterArg_0 = %c) : {t48}, tensor<i32>
     cond {{
      %c_1 = stablehlo.constant dense<6> : tensor<i32>
      %1 = stablehlo.compare  LT, %iterArg_0, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
      %2 = stablehlo.reduce(%iterArg init: %cst) applies stablehlo.maximum across dimensions = [0, 1] : ({t48}, tensor<f32>) -> tensor<f32>
      %cst_1 = stablehlo.constant dense<9.000000e-01> : tensor<f32>
      %3 = stablehlo.compare  LT, %2, %cst_1,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %4 = stablehlo.and %1, %3 : tensor<i1>
      stablehlo.return %4 : tensor<i1>
    }} do {{
      %cst = stablehlo.constant dense<3.000000e+00> : tensor<f32>
      %1 = stablehlo.broadcast_in_dim %cst, dims = [] : (tensor<f32>) -> {t48}
      %sc = stablehlo.multiply %iterArg, %1 : {t48}
{sm_body.rstrip(chr(10)).replace("    %", "      %")}
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %5 = stablehlo.add %iterArg_0, %c_1 : tensor<i32>
      stablehlo.return {sm_res}, %5 : {t48}, tensor<i32>
    }}
    return %0#0, %0#1 : {t48}, tensor<i32>
  }}
}}
""", [(0.2 * x48).astype(np.float32)]))
    # carried values that trade places (a result is a view of another carried value), a call and an if in the body
    out.append(("while_dynamic_swap_call_if", f"""module @jit_fib {{
  func.func public @main(%arg0: tensor<8xf32>, %arg1: tensor<8xf32>, %arg2: tensor<i32>) -> (tensor<8xf32>, tensor<8xf32>, tensor<i32>) {{
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:3 = stablehlo.while(%iterArg = %arg0, %iterArg_0 = %arg1, %iterArg_1 = %c) : tensor<8xf32>, tensor<8xf32>, tensor<i32>
     cond {{
      %1 = stablehlo.compare  LT, %iterArg_1, %arg2,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    }} do {{
      %1 = call @combine(%iterArg, %iterArg_0) : (tensor<8xf32>, tensor<8xf32>) -> tensor<8xf32>
      %c_1 = stablehlo.constant dense<2> : tensor<i32>
      %2 = stablehlo.remainder %iterArg_1, %c_1 : tensor<i32>
      %c_2 = stablehlo.constant dense<0> : tensor<i32>
      %3 = stablehlo.compare  EQ, %2, %c_2,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %4 = "stablehlo.if"(%3) ({{
        stablehlo.return %1 : tensor<8xf32>
      }}, {{
        %5 = stablehlo.negate %1 : tensor<8xf32>
        stablehlo.return %5 : tensor<8xf32>
      }}) : (tensor<i1>) -> tensor<8xf32>
      %c_3 = stablehlo.constant dense<1> : tensor<i32>
      %6 = stablehlo.add %iterArg_1, %c_3 : tensor<i32>
      stablehlo.return %iterArg_0, %4, %6 : tensor<8xf32>, tensor<8xf32>, tensor<i32>
    }}
    return %0#0, %0#1, %0#2 : tensor<8xf32>, tensor<8xf32>, tensor<i32>
  }}
  func.func private @combine(%arg0: tensor<8xf32>, %arg1: tensor<8xf32>) -> tensor<8xf32> {{
    %cst = stablehlo.constant dense<5.000000e-01> : tensor<8xf32>
    %0 = stablehlo.multiply %arg0, %cst : tensor<8xf32>
    %1 = stablehlo.add %0, %arg1 : tensor<8xf32>
    return %1 : tensor<8xf32>
  }}
}}
""", [x48[0].copy(), y48[0].copy(), np.asarray(5, np.int32)]))
    out.append(("while_dynamic_zero_trips", out[-1][1], [x48[0].copy(), y48[0].copy(), np.asarray(0, np.int32)]))
    case_text = f"""module @jit_switch {{
  func.func public @main(%arg0: tensor<i32>, %arg1: {t48}) -> ({t48}) {{
    %0 = "stablehlo.case"(%arg0) ({{
      %1 = stablehlo.negate %arg1 : {t48}
      stablehlo.return %1 : {t48}
    }}, {{
      %1 = stablehlo.tanh %arg1 : {t48}
      %2 = "stablehlo.if"(%p0) ({{
        stablehlo.return %1 : {t48}
      }}, {{
        stablehlo.return %arg1 : {t48}
      }}) : (tensor<i1>) -> {t48}
      stablehlo.return %2 : {t48}
    }}, {{
      %1 = stablehlo.abs %arg1 : {t48}
      stablehlo.return %1 : {t48}
    }}) : (tensor<i32>) -> {t48}
    return %0 : {t48}
  }}
}}
""".replace("    %0 = \"stablehlo.case\"", "    %p0 = stablehlo.constant dense<true> : tensor<i1>\n    %0 = \"stablehlo.case\"")
    for v in (0, 1, 2, 7, -3):
        out.append((f"case_index_{v}".replace("-", "m"), case_text, [np.asarray(v, np.int32), x48]))
    # ---- compare under the total order (-NaN < -inf < .. < -0 < +0 < .. < +inf < +NaN)
    special = np.array([np.nan, -np.nan, np.inf, -np.inf, 0.0, -0.0, 1.5, -1.5, 1e-30, -1e-30, 3.0, np.nan], np.float32)
    special[1] = np.float32(np.uint32(0xFFC00000).view(np.float32))  # a NaN with the sign bit set
    lhs_t, rhs_t = np.repeat(special, len(special)), np.tile(special, len(special))
    for dt in ("f32", "bf16", "f16"):
        if dt not in NP:
            continue
        tcmp, tres = tt((len(lhs_t),), dt), tt((len(lhs_t),), "i1")
        for direction in ("LT", "EQ", "GE"):
            out.append((f"compare_totalorder_{direction}_{dt}", func([tcmp, tcmp], [tres],
                        f"    %0 = stablehlo.compare  {direction}, %arg0, %arg1,  TOTALORDER : ({tcmp}, {tcmp}) -> {tres}", "%0"),
                        [lhs_t.astype(NP[dt]), rhs_t.astype(NP[dt])]))
    # ---- bitcast_convert
    bits = x48.view(np.int32)
    out.append(("bitcast_convert_f32_i32", func([t48], [tt((4, 8), "i32")],
                f"    %0 = stablehlo.bitcast_convert %arg0 : ({t48}) -> {tt((4, 8), 'i32')}", "%0"), [x48]))
    out.append(("bitcast_convert_i32_f32", func([tt((4, 8), "i32")], [t48],
                f"    %0 = stablehlo.bitcast_convert %arg0 : ({tt((4, 8), 'i32')}) -> {t48}", "%0"), [bits.copy()]))
    out.append(("bitcast_convert_transposed_ui32", func([t48], [tt((8, 4), "ui32")],
                f"    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({t48}) -> {tt((8, 4), 'f32')}\n"
                f"    %1 = stablehlo.bitcast_convert %0 : ({tt((8, 4), 'f32')}) -> {tt((8, 4), 'ui32')}", "%1"), [x48]))
    out.append(("bitcast_convert_f32_to_bytes", func([t48], [tt((4, 8, 4), "ui8")],
                f"    %0 = stablehlo.bitcast_convert %arg0 : ({t48}) -> {tt((4, 8, 4), 'ui8')}", "%0"), [x48]))
    out.append(("bitcast_convert_halves_to_f32", func([tt((4, 8, 2), "ui16")], [t48],
                f"    %0 = stablehlo.bitcast_convert %arg0 : ({tt((4, 8, 2), 'ui16')}) -> {t48}", "%0"),
                [x48.view(np.uint16).reshape(4, 8, 2).copy()]))
    # ---- dynamic_* with constant shape operands
    out.append(("dynamic_reshape", func([t48], [tt((2, 16), "f32")],
                "    %s = stablehlo.constant dense<[2, 16]> : tensor<2xi32>\n"
                f"    %0 = stablehlo.dynamic_reshape %arg0, %s : ({t48}, tensor<2xi32>) -> {tt((2, 16), 'f32')}", "%0"), [x48]))
    out.append(("dynamic_broadcast_in_dim", func([tt((8,), "f32")], [tt((3, 8, 2), "f32")],
                "    %s = stablehlo.constant dense<[3, 8, 2]> : tensor<3xi64>\n"
                f"    %0 = \"stablehlo.dynamic_broadcast_in_dim\"(%arg0, %s) <{{broadcast_dimensions = array<i64: 1>}}> : ({tt((8,), 'f32')}, tensor<3xi64>) -> {tt((3, 8, 2), 'f32')}",
                "%0"), [x48[0].copy()]))
    out.append(("dynamic_iota", func([t48], [tt((4, 8), "i32")],
                "    %s = stablehlo.constant dense<[4, 8]> : tensor<2xi32>\n"
                f"    %0 = \"stablehlo.dynamic_iota\"(%s) <{{iota_dimension = 1 : i64}}> : (tensor<2xi32>) -> {tt((4, 8), 'i32')}",
                "%0"), [x48]))
    out.append(("dynamic_pad", func([t48], [tt((7, 16), "f32")],
                "    %z = stablehlo.constant dense<-1.000000e+00> : tensor<f32>\n"
                "    %lo = stablehlo.constant dense<[1, 0]> : tensor<2xi32>\n"
                "    %hi = stablehlo.constant dense<[2, 1]> : tensor<2xi32>\n"
                "    %in = stablehlo.constant dense<[0, 1]> : tensor<2xi32>\n"
                f"    %0 = stablehlo.dynamic_pad %arg0, %z, %lo, %hi, %in : ({t48}, tensor<f32>, tensor<2xi32>, tensor<2xi32>, tensor<2xi32>) -> {tt((7, 16), 'f32')}",
                "%0"), [x48]))
    ids = rng.integers(0, 4, size=(5, 1)).astype(np.int32)
    out.append(("dynamic_gather", func([t48, tt((5, 1), "i32")], [tt((5, 8), "f32")],
                "    %s = stablehlo.constant dense<[1, 8]> : tensor<2xi32>\n"
                f"    %0 = \"stablehlo.dynamic_gather\"(%arg0, %arg1, %s) <{{dimension_numbers = #stablehlo.gather<offset_dims = [1], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 1>, indices_are_sorted = false}}> : ({t48}, {tt((5, 1), 'i32')}, tensor<2xi32>) -> {tt((5, 8), 'f32')}",
                "%0"), [x48, ids]))
    # ---- map: a scalar computation with a constant, a compare and a select, applied elementwise
    map_text = f"""module @jit_map {{
  func.func public @main(%arg0: {t48}, %arg1: {t48}) -> ({t48}) {{
    %0 = "stablehlo.map"(%arg0, %arg1) <{{dimensions = array<i64: 0, 1>}}> ({{
    ^bb0(%a: tensor<f32>, %b: tensor<f32>):
      %half = stablehlo.constant dense<5.000000e-01> : tensor<f32>
      %p = stablehlo.multiply %a, %b : tensor<f32>
      %q = stablehlo.add %p, %half : tensor<f32>
      %c = stablehlo.compare  GT, %a, %b,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %r = stablehlo.select %c, %q, %b : tensor<i1>, tensor<f32>
      stablehlo.return %r : tensor<f32>
    }}) : ({t48}, {t48}) -> {t48}
    return %0 : {t48}
  }}
}}
"""
    out.append(("map_scalar_computation", map_text, [x48, y48]))
    out.append(("get_dimension_size", func([t48], [tt((), "i32")],
                f"    %0 = stablehlo.get_dimension_size %arg0, dim = 1 : ({t48}) -> tensor<i32>", "%0"), [x48]))
    for dt in ("f32", "bf16", "f16"):
        if dt in NP:
            t = tt((5, 37), dt)
            out.append((f"erf_{dt}", func([t], [t], f"    %0 = chlo.erf %arg0 : {t} -> {t}", "%0"), [rand(rng, (5, 37), dt, -3.0, 3.0)]))
    # ---- batch_norm_inference over NHWC and NCHW feature positions
    for dt in ("f32", "bf16"):
        if dt not in NP:
            continue
        for axis, shape in ((3, (2, 5, 6, 16)), (1, (2, 16, 5, 6))):
            t, tc = tt(shape, dt), tt((16,), dt)
            x = rand(rng, shape, dt)
            scale, offset, mean = (rand(rng, (16,), dt) for _ in range(3))
            var = rand(rng, (16,), dt, 0.2, 2.0)
            out.append((f"batch_norm_inference_axis{axis}_{dt}", func([t, tc, tc, tc, tc], [t],
                        f"    %0 = \"stablehlo.batch_norm_inference\"(%arg0, %arg1, %arg2, %arg3, %arg4) <{{epsilon = 1.000000e-03 : f32, feature_index = {axis} : i64}}> : ({t}, {tc}, {tc}, {tc}, {tc}) -> {t}",
                        "%0"), [x, scale, offset, mean, var]))
    return out


def _region(kind, dt, names=("a", "b")):
    """Body region of reduce_window / scatter: one binary op on two scalars, or the assignment form of scatter."""
    st = f"tensor<{dt}>"
    head = f"    ^bb0(%{names[0]}: {st}, %{names[1]}: {st}):\n"
    if kind == "set":
        return head + f"      stablehlo.return %{names[1]} : {st}\n"
    return head + f"      %r = stablehlo.{kind} %{names[0]}, %{names[1]} : {st}\n      stablehlo.return %r : {st}\n"


def _const(dt, value):
    if dt in ("f32", "f16", "bf16", "f64"):
        if value in ("-inf", "inf"):
            bits = {"f32": "0xFF800000", "f16": "0xFC00", "bf16": "0xFF80", "f64": "0xFFF0000000000000"}[dt]
            if value == "inf":
                bits = "0x7" + bits[3:]
            return f"stablehlo.constant dense<{bits}> : tensor<{dt}>"
        return f"stablehlo.constant dense<{float(value):e}> : tensor<{dt}>"
    return f"stablehlo.constant dense<{int(value)}> : tensor<{dt}>"


def reduce_window_case(name, x, dt, kind, init, window, out_shape, strides=None, padding=None, base_dil=None, win_dil=None, pre=None):
    """One stablehlo.reduce_window in the generic form jax prints. pre = (text, shape): ops applied to %arg0 first."""
    rank = len(window)
    arr = lambda v: "array<i64: " + ", ".join(str(i) for i in v) + ">"
    props = [f"window_dimensions = {arr(window)}"]
    if strides: props.append(f"window_strides = {arr(strides)}")
    if base_dil: props.append(f"base_dilations = {arr(base_dil)}")
    if win_dil: props.append(f"window_dilations = {arr(win_dil)}")
    if padding:
        rows = ", ".join(f"[{lo}, {hi}]" for lo, hi in padding)
        props.append(f"padding = dense<[{rows}]> : tensor<{rank}x2xi64>")
    t_in = tt(x.shape, dt)
    src, t_src, body = "%arg0", t_in, ""
    if pre:
        body, t_src, src = pre[0] + "\n", tt(pre[1], dt), "%pre"
    t_out = tt(out_shape, dt)
    body += (f"    %init = {_const(dt, init)}\n"
             f"    %0 = \"stablehlo.reduce_window\"({src}, %init) <{{{', '.join(props)}}}> ({{\n{_region(kind, dt)}    }}) : ({t_src}, tensor<{dt}>) -> {t_out}")
    return (name, func([t_in], [t_out], body, "%0"), [x])


def scatter_case(name, operand, indices, updates, dt, kind, dims, idt="i32"):
    t_op, t_idx, t_upd = tt(operand.shape, dt), tt(indices.shape, idt), tt(updates.shape, dt)
    body = (f"    %0 = \"stablehlo.scatter\"(%arg0, %arg1, %arg2) <{{indices_are_sorted = false, scatter_dimension_numbers = #stablehlo.scatter<{dims}>, "
            f"unique_indices = false}}> ({{\n{_region(kind, dt)}    }}) : ({t_op}, {t_idx}, {t_upd}) -> {t_op}")
    return (name, func([t_op, t_idx, t_upd], [t_op], body, "%0"), [operand, indices, updates])


def sort_case(name, arrays, dts, dimension, direction="LT", swapped=False, compare_type=None):
    """stablehlo.sort of len(arrays) operands by the first one, the comparator a single compare as jax.lax.sort prints."""
    types = [tt(a.shape, dt) for a, dt in zip(arrays, dts)]
    block = ", ".join(f"%l{i}: tensor<{dt}>, %r{i}: tensor<{dt}>" for i, dt in enumerate(dts))
    lhs, rhs = ("%r0", "%l0") if swapped else ("%l0", "%r0")
    ctype = "TOTALORDER" if dts[0] in ("f32", "f16", "bf16", "f64") else ("UNSIGNED" if dts[0].startswith("ui") else "SIGNED")
    ctype = compare_type or ctype
    args = ", ".join(f"%arg{i}" for i in range(len(arrays)))
    results = ", ".join(f"%0#{i}" for i in range(len(arrays))) if len(arrays) > 1 else "%0"
    lhs_bind = f"%0:{len(arrays)}" if len(arrays) > 1 else "%0"
    sig_out = ", ".join(types)
    body = (f"    {lhs_bind} = \"stablehlo.sort\"({args}) <{{dimension = {dimension} : i64, is_stable = true}}> ({{\n"
            f"    ^bb0({block}):\n"
            f"      %c = stablehlo.compare  {direction}, {lhs}, {rhs},  {ctype} : (tensor<{dts[0]}>, tensor<{dts[0]}>) -> tensor<i1>\n"
            f"      stablehlo.return %c : tensor<i1>\n"
            f"    }}) : ({sig_out}) -> ({sig_out})" if len(arrays) > 1 else
            f"    {lhs_bind} = \"stablehlo.sort\"({args}) <{{dimension = {dimension} : i64, is_stable = true}}> ({{\n"
            f"    ^bb0({block}):\n"
            f"      %c = stablehlo.compare  {direction}, {lhs}, {rhs},  {ctype} : (tensor<{dts[0]}>, tensor<{dts[0]}>) -> tensor<i1>\n"
            f"      stablehlo.return %c : tensor<i1>\n"
            f"    }}) : ({sig_out}) -> {sig_out}")
    return (name, func(types, types, body, results), list(arrays))


THREEFRY_ROTATIONS = (13, 15, 26, 6, 17, 29, 16, 24)


def threefry2x32_text(n):
    """Threefry-2x32 with 20 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3") over n counters, as the
    chain of ui32 adds, shifts, ors and xors that jax.random's default generator lowers to. Arguments: key [2], counters
    x0 [n], x1 [n]; results: the two output words."""
    t, tk, ts = tt((n,), "ui32"), tt((2,), "ui32"), "tensor<ui32>"
    lines = []
    k = [0]

    def v():
        k[0] += 1
        return f"%t{k[0]}"

    def emit(text):
        lines.append("    " + text)

    def splat(value):
        c, b = v(), v()
        emit(f"{c} = stablehlo.constant dense<{value}> : {ts}")
        emit(f"{b} = stablehlo.broadcast_in_dim {c}, dims = [] : ({ts}) -> {t}")
        return b

    def binary(op, a, b):
        r = v()
        emit(f"{r} = stablehlo.{op} {a}, {b} : {t}")
        return r

    keys = []
    for i in range(2):
        sl, rs, bc = v(), v(), v()
        emit(f"{sl} = stablehlo.slice %arg0 [{i}:{i + 1}] : ({tk}) -> tensor<1xui32>")
        emit(f"{rs} = stablehlo.reshape {sl} : (tensor<1xui32>) -> {ts}")
        emit(f"{bc} = stablehlo.broadcast_in_dim {rs}, dims = [] : ({ts}) -> {t}")
        keys.append(bc)
    keys.append(binary("xor", binary("xor", keys[0], keys[1]), splat(0x1BD11BDA)))
    x0 = binary("add", "%arg1", keys[0])
    x1 = binary("add", "%arg2", keys[1])
    for group in range(5):
        for r in THREEFRY_ROTATIONS[4 * (group % 2):4 * (group % 2) + 4]:
            x0 = binary("add", x0, x1)
            rot = binary("or", binary("shift_left", x1, splat(r)), binary("shift_right_logical", x1, splat(32 - r)))
            x1 = binary("xor", rot, x0)
        x0 = binary("add", x0, keys[(group + 1) % 3])
        x1 = binary("add", binary("add", x1, keys[(group + 2) % 3]), splat(group + 1))
    return func([tk, t, t], [t, t], "\n".join(lines), f"{x0}, {x1}")


def window_scatter_sort_cases():
    rng = np.random.default_rng(4242)
    out = []
    # ---- reduce_window: pooling as flax / jax.lax.reduce_window print it
    x = rand(rng, (2, 8, 8, 4), "f32")
    out.append(reduce_window_case("reduce_window_maxpool_2x2", x, "f32", "maximum", "-inf", (1, 2, 2, 1), (2, 4, 4, 4), strides=(1, 2, 2, 1)))
    out.append(reduce_window_case("reduce_window_sum_3x3_same", x, "f32", "add", 0, (1, 3, 3, 1), (2, 8, 8, 4),
                                  padding=((0, 0), (1, 1), (1, 1), (0, 0))))
    if "bf16" in NP:
        out.append(reduce_window_case("reduce_window_sum_3x3_same_bf16", rand(rng, (2, 8, 8, 4), "bf16"), "bf16", "add", 0, (1, 3, 3, 1), (2, 8, 8, 4),
                                      padding=((0, 0), (1, 1), (1, 1), (0, 0))))
    out.append(reduce_window_case("reduce_window_maxpool_3x3_s2_pad", x, "f32", "maximum", "-inf", (1, 3, 3, 1), (2, 4, 4, 4), strides=(1, 2, 2, 1),
                                  padding=((0, 0), (0, 1), (0, 1), (0, 0))))
    # channel counts that are whole 16-byte vectors take the vector kernel
    for dt in ("bf16", "f16", "f32"):
        if dt in NP:
            xv = rand(rng, (2, 9, 9, 16), dt)
            out.append(reduce_window_case(f"reduce_window_vectors_maxpool_{dt}", xv, dt, "maximum", "-inf", (1, 3, 3, 1), (2, 5, 5, 16),
                                          strides=(1, 2, 2, 1), padding=((0, 0), (1, 1), (1, 1), (0, 0))))
            out.append(reduce_window_case(f"reduce_window_vectors_dilated_sum_{dt}", xv, dt, "add", 0.25, (1, 2, 2, 1), (2, 15, 8, 16),
                                          padding=((0, 0), (0, 0), (1, 0), (0, 0)), base_dil=(1, 2, 1, 1), win_dil=(1, 2, 2, 1)))
    out.append(reduce_window_case("reduce_window_vectors_padded_sum_nonzero_init", rand(rng, (2, 6, 6, 8), "f32"), "f32", "add", 0.5, (1, 2, 2, 1),
                                  (2, 7, 7, 8), padding=((0, 0), (1, 1), (1, 1), (0, 0))))
    out.append(reduce_window_case("reduce_window_vectors_min_window_dilation", rand(rng, (2, 9, 9, 8), "f32"), "f32", "minimum", "inf", (1, 2, 3, 1),
                                  (2, 7, 3, 8), strides=(1, 1, 2, 1), win_dil=(1, 2, 2, 1)))
    xi = rand(rng, (5, 9), "i32")
    # dilated operand (9 -> 17), dilated window (3 taps spanning 5), negative low padding: (17 - 1 + 2 - 5) / 2 + 1 = 7
    out.append(reduce_window_case("reduce_window_dilations_i32", xi, "i32", "add", 0, (2, 3), (4, 7), strides=(1, 2),
                                  padding=((0, 0), (-1, 2)), base_dil=(1, 2), win_dil=(1, 2)))
    out.append(reduce_window_case("reduce_window_min_i32", xi, "i32", "minimum", 2147483647, (3, 3), (3, 7)))
    out.append(reduce_window_case("reduce_window_nonzero_init", rand(rng, (6, 6), "f32"), "f32", "add", 0.5, (2, 2), (7, 7),
                                  padding=((1, 1), (1, 1))))
    xc = rand(rng, (3, 33), "f32")
    out.append(reduce_window_case("reduce_window_cumsum", xc, "f32", "add", 0, (1, 33), (3, 33), padding=((0, 0), (32, 0))))
    xt = rand(rng, (9, 6), "f32")
    out.append(reduce_window_case("reduce_window_of_transpose", xt, "f32", "maximum", "-inf", (2, 3), (3, 3), strides=(2, 3),
                                  pre=(f"    %pre = stablehlo.transpose %arg0, dims = [1, 0] : ({tt((9, 6), 'f32')}) -> {tt((6, 9), 'f32')}", (6, 9))))
    out.append(reduce_window_case("reduce_window_or_i1", rand(rng, (4, 10), "i1"), "i1", "or", 0, (1, 3), (4, 8)))
    # ---- select_and_scatter: the gradient of max pooling as jax prints it (GE select, add scatter)
    def sas_case(name, x, src, dt, window, strides, padding=None, select="GE", kind="add", init=0):
        arr = lambda v: "array<i64: " + ", ".join(str(i) for i in v) + ">"
        props = [f"window_dimensions = {arr(window)}", f"window_strides = {arr(strides)}"]
        if padding:
            props.append("padding = dense<[" + ", ".join(f"[{lo}, {hi}]" for lo, hi in padding) + f"]> : tensor<{len(window)}x2xi64>")
        st = f"tensor<{dt}>"
        ctype = "FLOAT" if dt[0] in "fb" else "SIGNED"
        t_x, t_s = tt(x.shape, dt), tt(src.shape, dt)
        body = (f"    %init = {_const(dt, init)}\n"
                f"    %0 = \"stablehlo.select_and_scatter\"(%arg0, %arg1, %init) <{{{', '.join(props)}}}> ({{\n"
                f"    ^bb0(%a: {st}, %b: {st}):\n      %c = stablehlo.compare  {select}, %a, %b,  {ctype} : ({st}, {st}) -> tensor<i1>\n"
                f"      stablehlo.return %c : tensor<i1>\n    }}, {{\n{_region(kind, dt, ('p', 'q'))}    }}) : ({t_x}, {t_s}, {st}) -> {t_x}")
        return (name, func([t_x, t_s], [t_x], body, "%0"), [x, src])

    img = rand(rng, (2, 8, 8, 3), "f32")
    out.append(sas_case("select_and_scatter_maxpool_grad_2x2", img, rand(rng, (2, 4, 4, 3), "f32"), "f32", (1, 2, 2, 1), (1, 2, 2, 1)))
    out.append(sas_case("select_and_scatter_overlapping_3x3", img, rand(rng, (2, 4, 4, 3), "f32"), "f32", (1, 3, 3, 1), (1, 2, 2, 1),
                        padding=((0, 0), (0, 1), (0, 1), (0, 0))))
    if "bf16" in NP:
        out.append(sas_case("select_and_scatter_maxpool_grad_bf16", rand(rng, (2, 8, 8, 3), "bf16"), rand(rng, (2, 4, 4, 3), "bf16"), "bf16",
                            (1, 2, 2, 1), (1, 2, 2, 1)))
    out.append(sas_case("select_and_scatter_minpool_i32_ties", rng.integers(0, 3, size=(6, 6)).astype(np.int32), rand(rng, (3, 3), "i32"), "i32",
                        (2, 2), (2, 2), select="LE"))
    out.append(sas_case("select_and_scatter_strict_compare", rng.integers(0, 3, size=(6, 6)).astype(np.int32), rand(rng, (5, 5), "i32"), "i32",
                        (2, 2), (1, 1), select="GT"))
    out.append(sas_case("select_and_scatter_padding_can_win", -np.abs(rand(rng, (5, 5), "f32")) - 0.1, rand(rng, (3, 3), "f32"), "f32",
                        (3, 3), (2, 2), padding=((1, 1), (1, 1))))
    # ---- scatter
    point = "inserted_window_dims = [0], scatter_dims_to_operand_dims = [0], index_vector_dim = 1"
    rows = "update_window_dims = [1], inserted_window_dims = [0], scatter_dims_to_operand_dims = [0], index_vector_dim = 1"
    base = rand(rng, (20,), "f32")
    uniq = rng.permutation(20)[:6].astype(np.int32).reshape(6, 1)
    out.append(scatter_case("scatter_set_points", base, uniq, rand(rng, (6,), "f32"), "f32", "set", point))
    out.append(scatter_case("scatter_set_points_i64_index", base, uniq.astype(np.int64), rand(rng, (6,), "f32"), "f32", "set", point, idt="i64"))
    table = rand(rng, (10, 8), "f32")
    dup = np.array([[3], [7], [3], [0], [9], [3]], np.int32)
    out.append(scatter_case("scatter_add_rows_duplicates", table, dup, rand(rng, (6, 8), "f32"), "f32", "add", rows))
    oob = np.array([[-1], [4], [10], [2], [12345], [9]], np.int32)
    out.append(scatter_case("scatter_add_rows_out_of_bounds", table, oob, rand(rng, (6, 8), "f32"), "f32", "add", rows))
    for dt, kind in (("i32", "maximum"), ("f32", "minimum"), ("f32", "multiply"), ("i8", "add"), ("i64", "add"), ("f16", "maximum"),
                     ("bf16", "add"), ("f64", "add"), ("ui8", "minimum"), ("i16", "multiply")):
        if dt not in NP:
            continue
        lo, hi = (-3, 3) if kind == "multiply" else (-2.0, 2.0)
        out.append(scatter_case(f"scatter_{kind}_{dt}_duplicates", rand(rng, (10, 8), dt, lo, hi) if dt[0] in "fb" else rand(rng, (10, 8), dt),
                                dup, rand(rng, (6, 8), dt, lo, hi) if dt[0] in "fb" else rng.integers(-3 if dt[0] == "i" else 0, 4, size=(6, 8)).astype(NP[dt]),
                                dt, kind, rows))
    batched = ("inserted_window_dims = [1], input_batching_dims = [0], scatter_indices_batching_dims = [0], "
               "scatter_dims_to_operand_dims = [1], index_vector_dim = 2")
    out.append(scatter_case("scatter_add_batched", rand(rng, (3, 10), "f32"), rng.integers(0, 10, size=(3, 4, 1)).astype(np.int32),
                            rand(rng, (3, 4), "f32"), "f32", "add", batched))
    window2d = "update_window_dims = [1, 2], scatter_dims_to_operand_dims = [0, 1], index_vector_dim = 1"
    out.append(scatter_case("scatter_add_windows_partly_outside", rand(rng, (6, 7), "i32"), np.array([[0, 0], [5, 5], [2, 6], [-1, 3]], np.int32),
                            rand(rng, (4, 2, 3), "i32"), "i32", "add", window2d))
    out.append(scatter_case("scatter_add_f32_windows_of_four", rand(rng, (6, 12), "f32"), np.array([[0, 0], [5, 9], [2, 3], [-1, 1], [3, 8], [0, 0]], np.int32),
                            rand(rng, (6, 2, 4), "f32"), "f32", "add", window2d))
    # ---- sort
    keys = rand(rng, (37,), "f32")
    keys[[3, 11]] = np.nan
    keys[5], keys[6], keys[20], keys[21] = 0.0, -0.0, np.inf, -np.inf
    keys[30] = keys[2]
    out.append(sort_case("sort_f32_special_values", [keys], ["f32"], 0))
    out.append(sort_case("sort_f32_descending", [keys], ["f32"], 0, direction="GT"))
    out.append(sort_case("sort_f32_swapped_comparator", [keys], ["f32"], 0, direction="LT", swapped=True))
    m = rng.integers(-5, 6, size=(9, 7)).astype(np.int32)
    out.append(sort_case("sort_i32_dim0_descending", [m], ["i32"], 0, direction="GT"))
    ties = rng.integers(0, 6, size=(4, 100)).astype(np.float32)
    iota = np.broadcast_to(np.arange(100, dtype=np.int32), (4, 100)).copy()
    # signed zeros: a FLOAT comparison holds them equal (the stable order keeps them as they came), TOTALORDER puts -0 first
    zeros = np.array([[0.0, -0.0, 1.0, -0.0, 0.0, -1.0, -0.0, 0.0]], dtype=np.float32)
    zpos = np.arange(8, dtype=np.int32).reshape(1, 8)
    for ctype in ("FLOAT", "TOTALORDER"):
        out.append(sort_case(f"argsort_signed_zeros_{ctype.lower()}", [zeros, zpos], ["f32", "i32"], 1, compare_type=ctype))
        out.append(sort_case(f"argsort_signed_zeros_{ctype.lower()}_descending", [zeros, zpos], ["f32", "i32"], 1, direction="GT", compare_type=ctype))
    out.append(sort_case("argsort_signed_zeros_bf16_float", [zeros.astype(NP["bf16"]), zpos], ["bf16", "i32"], 1, compare_type="FLOAT"))
    out.append(sort_case("argsort_stable_ties", [ties, iota], ["f32", "i32"], 1))
    out.append(sort_case("argsort_stable_ties_descending", [ties, iota], ["f32", "i32"], 1, direction="GT"))
    for dt in ("bf16", "ui8", "i64", "f64", "f16", "i8", "ui32"):
        if dt not in NP:
            continue
        k = rand(rng, (3, 50), dt)
        out.append(sort_case(f"sort_pairs_{dt}", [k, rand(rng, (3, 50), "f32")], [dt, "f32"], 1))
    logits = rng.integers(-6, 7, size=(5, 300)).astype(np.float32) * 0.5  # many ties
    t_l = tt((5, 300), "f32")
    out.append(("top_k_with_ties", func([t_l], [tt((5, 7), "f32"), tt((5, 7), "i32")],
                f"    %0:2 = chlo.top_k(%arg0, k = 7) : {t_l} -> ({tt((5, 7), 'f32')}, {tt((5, 7), 'i32')})", "%0#0, %0#1"), [logits]))
    if "bf16" in NP:
        lb = rand(rng, (3, 9000), "bf16")
        t_b = tt((3, 9000), "bf16")
        out.append(("top_k_long_rows_bf16", func([t_b], [tt((3, 50), "bf16"), tt((3, 50), "i32")],
                    f"    %values, %indices = chlo.top_k(%arg0, k = 50) : {t_b} -> ({tt((3, 50), 'bf16')}, {tt((3, 50), 'i32')})", "%values, %indices"), [lb]))
    counters = rng.integers(0, 1 << 32, size=(2, 1000), dtype=np.uint64).astype(np.uint32)
    out.append(("threefry2x32_random_bits", threefry2x32_text(1000),
                [np.array([0x13198A2E, 0x03707344], np.uint32), counters[0].copy(), counters[1].copy()]))
    three = [rng.integers(0, 4, size=(2, 5, 3)).astype(np.int32), rand(rng, (2, 5, 3), "f32"), rand(rng, (2, 5, 3), "i8")]
    out.append(sort_case("sort_three_operands_middle_dim", three, ["i32", "f32", "i8"], 1))
    big = rand(rng, (2, 5000), "f32")
    out.append(sort_case("sort_long_rows_shared_memory", [big, np.broadcast_to(np.arange(5000, dtype=np.int32), (2, 5000)).copy()], ["f32", "i32"], 1))
    for n in (8192, 8193, 20000):
        kk = rng.integers(-1000, 1000, size=(3, n)).astype(np.int32)
        out.append(sort_case(f"sort_global_{n}", [kk, np.broadcast_to(np.arange(n, dtype=np.int32), (3, n)).copy()], ["i32", "i32"], 1,
                             direction="GT" if n == 8193 else "LT"))
    cols = rand(rng, (9000, 3), "f32")
    out.append(sort_case("sort_global_strided_dim0", [cols], ["f32"], 0))
    return out


def conv_case(name, x, w, dt, out_shape, layout="[b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f]", window="", fgc=1, bgc=1, form="pretty"):
    """One stablehlo.convolution. form: "pretty" (what jax prints), "short" (the reference benchmarks' form, NHWC x HWIO
    only) or "generic"."""
    tx, tw, to = tt(x.shape, dt), tt(w.shape, dt), tt(out_shape, dt)
    if form == "short":
        body = f"    %0 = stablehlo.convolution %arg0, %arg1 {window}feature_group_count = {fgc} : ({tx}, {tw}) -> {to}"
    elif form == "generic":
        body = (f"    %0 = \"stablehlo.convolution\"(%arg0, %arg1) {{batch_group_count = {bgc} : i64, dimension_numbers = #stablehlo.conv<{layout}>, "
                f"feature_group_count = {fgc} : i64{window}}} : ({tx}, {tw}) -> {to}")
    else:
        body = (f"    %0 = stablehlo.convolution(%arg0, %arg1) dim_numbers = {layout}, window = {{{window}}} "
                f"{{batch_group_count = {bgc} : i64, feature_group_count = {fgc} : i64, precision_config = [#stablehlo<precision DEFAULT>, #stablehlo<precision DEFAULT>]}} "
                f": ({tx}, {tw}) -> {to}")
    return (name, func([tx, tw], [to], body, "%0"), [x, w])


def convolution_cases():
    rng = np.random.default_rng(31337)
    out = []

    def data(shape, dt, scale=1.0):
        if dt in ("i32", "i8", "i64"):
            return rng.integers(-4, 5, size=shape).astype(NP[dt])
        return (scale * rng.standard_normal(shape)).astype(np.float32).astype(NP[dt])

    same = "stride = [1, 1], pad = [[1, 1], [1, 1]], rhs_dilate = [1, 1]"
    for dt in ("f32", "bf16", "f16"):
        if dt not in NP:
            continue
        out.append(conv_case(f"conv_3x3_same_{dt}", data((2, 12, 12, 16), dt), data((3, 3, 16, 32), dt, 0.1), dt, (2, 12, 12, 32), window=same))
        out.append(conv_case(f"conv_first_layer_rgb_{dt}", data((2, 16, 16, 3), dt), data((3, 3, 3, 32), dt, 0.2), dt, (2, 8, 8, 32),
                             window="stride = [2, 2], pad = [[0, 1], [0, 1]]"))
        out.append(conv_case(f"conv_1x1_{dt}", data((2, 9, 9, 24), dt), data((1, 1, 24, 16), dt, 0.2), dt, (2, 9, 9, 16)))
    out.append(conv_case("conv_nchw_oihw_f32", data((2, 8, 10, 10), "f32"), data((16, 8, 3, 3), "f32", 0.1), "f32", (2, 16, 8, 8),
                         layout="[b, f, 0, 1]x[o, i, 0, 1]->[b, f, 0, 1]"))
    if "bf16" in NP:
        out.append(conv_case("conv_nchw_oihw_bf16", data((2, 8, 10, 10), "bf16"), data((16, 8, 3, 3), "bf16", 0.1), "bf16", (2, 16, 8, 8),
                             layout="[b, f, 0, 1]x[o, i, 0, 1]->[b, f, 0, 1]"))
    out.append(conv_case("conv_dilated_kernel_f32", data((1, 11, 11, 4), "f32"), data((3, 3, 4, 8), "f32", 0.2), "f32", (1, 7, 7, 8),
                         window="rhs_dilate = [2, 2]"))
    # the gradient-of-strided-convolution form: dilated input, negative-free padding of kernel - 1
    out.append(conv_case("conv_transposed_f32", data((1, 5, 5, 4), "f32"), data((3, 3, 4, 8), "f32", 0.2), "f32", (1, 11, 11, 8),
                         window="pad = [[2, 2], [2, 2]], lhs_dilate = [2, 2]"))
    out.append(conv_case("conv_reversed_window_f32", data((1, 8, 8, 4), "f32"), data((3, 2, 4, 8), "f32", 0.2), "f32", (1, 6, 7, 8),
                         window="reverse = [true, false]"))
    out.append(conv_case("conv_negative_padding_f32", data((1, 8, 8, 4), "f32"), data((3, 3, 4, 8), "f32", 0.2), "f32", (1, 4, 5, 8),
                         window="pad = [[-1, -1], [0, -1]]"))
    out.append(conv_case("conv_feature_groups_2_f32", data((2, 8, 8, 8), "f32"), data((3, 3, 4, 16), "f32", 0.2), "f32", (2, 6, 6, 16), fgc=2))
    if "bf16" in NP:
        out.append(conv_case("conv_feature_groups_2_bf16", data((2, 8, 8, 16), "bf16"), data((3, 3, 8, 32), "bf16", 0.1), "bf16", (2, 6, 6, 32), fgc=2))
    out.append(conv_case("conv_depthwise_f32", data((2, 8, 8, 6), "f32"), data((3, 3, 1, 6), "f32", 0.3), "f32", (2, 6, 6, 6), fgc=6))
    out.append(conv_case("conv_batch_groups_2_f32", data((4, 6, 6, 3), "f32"), data((2, 2, 3, 4), "f32", 0.3), "f32", (2, 5, 5, 4), bgc=2))
    out.append(conv_case("conv_1d_f32", data((3, 20, 5), "f32"), data((4, 5, 7), "f32", 0.3), "f32", (3, 9, 7),
                         layout="[b, 0, f]x[0, i, o]->[b, 0, f]", window="stride = [2]"))
    out.append(conv_case("conv_3d_f32", data((1, 5, 6, 7, 2), "f32"), data((2, 3, 2, 2, 4), "f32", 0.3), "f32", (1, 4, 4, 6, 4),
                         layout="[b, 0, 1, 2, f]x[0, 1, 2, i, o]->[b, 0, 1, 2, f]"))
    out.append(conv_case("conv_i32", data((1, 6, 6, 2), "i32"), data((3, 3, 2, 3), "i32"), "i32", (1, 4, 4, 3)))
    # the forms the tensor-core kernel reads without a patch matrix: 16-bit NHWC x HWIO, channels in multiples of 64
    for dt in ("f16", "bf16"):
        if dt not in NP:
            continue
        out.append(conv_case(f"conv_direct_3x3_same_{dt}", data((2, 12, 12, 64), dt), data((3, 3, 64, 96), dt, 0.06), dt, (2, 12, 12, 96), window=same))
        out.append(conv_case(f"conv_direct_wide_image_{dt}", data((1, 20, 37, 64), dt), data((3, 3, 64, 64), dt, 0.06), dt, (1, 20, 37, 64), window=same))
        out.append(conv_case(f"conv_direct_valid_5x5_{dt}", data((2, 14, 14, 128), dt), data((5, 5, 128, 200), dt, 0.03), dt, (2, 10, 10, 200)))
        out.append(conv_case(f"conv_direct_1x1_{dt}", data((3, 9, 9, 64), dt), data((1, 1, 64, 8), dt, 0.15), dt, (3, 9, 9, 8)))
        out.append(conv_case(f"conv_direct_dilated_{dt}", data((1, 17, 17, 64), dt), data((3, 3, 64, 72), dt, 0.06), dt, (1, 17, 17, 72),
                             window="pad = [[2, 2], [2, 2]], rhs_dilate = [2, 2]"))
        out.append(conv_case(f"conv_direct_uneven_padding_{dt}", data((2, 9, 10, 64), dt), data((2, 4, 64, 16), dt, 0.07), dt, (2, 11, 9, 16),
                             window="pad = [[2, 1], [0, 2]]"))
        # window strides: the downsampling 3x3 and 1x1 convolutions of a residual network, and unequal strides with a dilated filter
        out.append(conv_case(f"conv_direct_stride2_3x3_{dt}", data((2, 14, 14, 64), dt), data((3, 3, 64, 128), dt, 0.06), dt, (2, 7, 7, 128),
                             window="stride = [2, 2], pad = [[0, 1], [0, 1]]"))
        out.append(conv_case(f"conv_direct_stride2_1x1_{dt}", data((2, 37, 20, 64), dt), data((1, 1, 64, 64), dt, 0.15), dt, (2, 19, 10, 64),
                             window="stride = [2, 2]"))
        out.append(conv_case(f"conv_direct_one_pixel_image_{dt}", data((3, 1, 1, 64), dt), data((3, 3, 64, 16), dt, 0.06), dt, (3, 1, 1, 16), window=same))
        out.append(conv_case(f"conv_direct_padding_wider_than_the_filter_{dt}", data((1, 5, 4, 64), dt), data((3, 3, 64, 8), dt, 0.06), dt, (1, 15, 14, 8),
                             window="pad = [[6, 6], [6, 6]]"))
        out.append(conv_case(f"conv_direct_stride_past_the_filter_{dt}", data((2, 33, 21, 128), dt), data((1, 1, 128, 40), dt, 0.1), dt, (2, 9, 6, 40),
                             window="stride = [4, 4]"))
        out.append(conv_case(f"conv_direct_stride_3_by_2_dilated_{dt}", data((1, 40, 45, 128), dt), data((3, 2, 128, 24), dt, 0.05), dt, (1, 13, 22, 24),
                             window="stride = [3, 2], pad = [[1, 1], [1, 0]], rhs_dilate = [2, 2]"))
    out.append(conv_case("conv_mixed_layouts_f32", data((6, 6, 2, 5), "f32"), data((3, 4, 3, 5), "f32", 0.3), "f32", (4, 2, 4, 4),
                         layout="[0, 1, b, f]x[0, o, 1, i]->[0, b, f, 1]"))
    out.append(conv_case("conv_short_form_f32", data((2, 8, 8, 4), "f32"), data((3, 3, 4, 8), "f32", 0.2), "f32", (2, 8, 8, 8),
                         window="window_strides = [1, 1], padding = [[1, 1], [1, 1]], ", form="short"))
    out.append(conv_case("conv_generic_form_f32", data((2, 8, 8, 4), "f32"), data((3, 3, 4, 8), "f32", 0.2), "f32", (2, 4, 4, 8),
                         window=", padding = dense<[[1, 1], [1, 1]]> : tensor<2x2xi64>, window_strides = array<i64: 2, 2>", form="generic"))
    return out


def linalg_cases():
    """stablehlo.cholesky and stablehlo.triangular_solve in the forms jax.numpy.linalg prints, every combination of side,
    triangle and transposition."""
    rng = np.random.default_rng(77)
    out = []

    def spd(batch, n, dt):
        m = rng.standard_normal(batch + (n, n))
        return (m @ np.swapaxes(m, -1, -2) / n + 2 * np.eye(n)).astype(np.float32).astype(NP[dt])

    for dt, batch, n in (("f32", (), 5), ("f32", (3,), 33), ("f64", (2, 2), 16), ("f32", (1,), 300)) + ((("bf16", (2,), 12),) if "bf16" in NP else ()):
        t = tt(batch + (n, n), dt)
        for lower in (True, False):
            body = f"    %0 = stablehlo.cholesky %arg0, lower = {str(lower).lower()} : {t}"
            out.append((f"cholesky_{dt}_{'x'.join(map(str, batch + (n,)))}_{'lower' if lower else 'upper'}", func([t], [t], body, "%0"), [spd(batch, n, dt)]))
    for dt, batch, m, n in (("f32", (), 5, 3), ("f32", (2,), 64, 40), ("f64", (3,), 17, 9)):
        for left in (True, False):
            for lower in (True, False):
                for trans in ("NO_TRANSPOSE", "TRANSPOSE"):
                    a = (rng.standard_normal(batch + (m, m)) / m + 2 * np.eye(m)).astype(NP[dt])  # both triangles filled: only one may be read
                    bshape = batch + ((m, n) if left else (n, m))
                    b = rng.standard_normal(bshape).astype(NP[dt])
                    ta, tb = tt(batch + (m, m), dt), tt(bshape, dt)
                    body = (f"    %0 = \"stablehlo.triangular_solve\"(%arg0, %arg1) <{{left_side = {str(left).lower()}, lower = {str(lower).lower()}, "
                            f"transpose_a = #stablehlo<transpose {trans}>, unit_diagonal = false}}> : ({ta}, {tb}) -> {tb}")
                    name = f"triangular_solve_{dt}_m{m}_{'left' if left else 'right'}_{'lower' if lower else 'upper'}_{trans.lower()}"
                    out.append((name, func([ta, tb], [tb], body, "%0"), [a, b]))
    a = (rng.standard_normal((6, 6)) / 6 + 2 * np.eye(6)).astype(np.float32)
    b = rng.standard_normal((6, 4)).astype(np.float32)
    ta, tb = tt((6, 6), "f32"), tt((6, 4), "f32")
    body = (f"    %0 = \"stablehlo.triangular_solve\"(%arg0, %arg1) <{{left_side = true, lower = true, transpose_a = #stablehlo<transpose ADJOINT>, "
            f"unit_diagonal = true}}> : ({ta}, {tb}) -> {tb}")
    out.append(("triangular_solve_unit_diagonal_adjoint", func([ta, tb], [tb], body, "%0"), [a, b]))
    # the solve of a Cholesky factor: A x = b as two triangular solves, the way jax.scipy.linalg.cho_solve lowers
    n = 24
    A = spd((), n, "f32")
    rhs = rng.standard_normal((n, 5)).astype(np.float32)
    tA, tB = tt((n, n), "f32"), tt((n, 5), "f32")
    body = (f"    %l = stablehlo.cholesky %arg0, lower = true : {tA}\n"
            f"    %y = \"stablehlo.triangular_solve\"(%l, %arg1) <{{left_side = true, lower = true, transpose_a = #stablehlo<transpose NO_TRANSPOSE>, unit_diagonal = false}}> : ({tA}, {tB}) -> {tB}\n"
            f"    %0 = \"stablehlo.triangular_solve\"(%l, %y) <{{left_side = true, lower = true, transpose_a = #stablehlo<transpose TRANSPOSE>, unit_diagonal = false}}> : ({tA}, {tB}) -> {tB}")
    out.append(("cholesky_solve_f32", func([tA, tB], [tB], body, "%0"), [A, rhs]))
    return out


def custom_call_cases():
    """Modules that arrive with the reference's fused custom calls already in them: every target of its handler table
    (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift) with the backend_config keys the handlers read."""
    import json

    rng = np.random.default_rng(4242)
    out = []

    def call(target, operands, types, rt, cfg=None, extra=""):
        config = json.dumps(cfg or {}).replace('"', '\\"')
        args = ", ".join(operands)
        return f"    %0 = stablehlo.custom_call @{target}({args}) {{backend_config = \"{config}\"{extra}}} : ({', '.join(types)}) -> {rt}"

    def add(name, target, arrays, rt_shape, dt, cfg=None, extra=""):
        types = [tt(a.shape, dt) for a in arrays]
        rt = tt(rt_shape, dt)
        body = call(target, [f"%arg{i}" for i in range(len(arrays))], types, rt, cfg, extra)
        out.append((name, func(types, [rt], body, "%0"), arrays))

    for dt in ("f32", "f16") + (("bf16",) if "bf16" in NP else ()):
        r = lambda *shape, scale=1.0: (scale * rng.standard_normal(shape)).astype(np.float32).astype(NP[dt])  # noqa: E731
        x, g, b = r(6, 40, 128), (1 + 0.1 * rng.standard_normal(128)).astype(np.float32).astype(NP[dt]), r(128, scale=0.1)
        add(f"call_layer_norm_{dt}", "fused_layer_norm", [x, g, b], x.shape, dt, {"eps": 1e-3})
        add(f"call_rms_norm_{dt}", "fused_rms_norm", [x, g], x.shape, dt, {"eps": 1e-6})
        add(f"call_softmax_{dt}", "fused_softmax", [r(6, 40, 128, scale=3.0)], x.shape, dt, {"axis": -1})
        add(f"call_softmax_axis1_{dt}", "fused_softmax", [r(6, 40, 128, scale=3.0)], x.shape, dt, {"axis": 1})
        add(f"call_gelu_{dt}", "fused_gelu", [x], x.shape, dt, {"approximate": True})
        add(f"call_gelu_exact_{dt}", "fused_gelu", [x], x.shape, dt, {"approximate": False})
        add(f"call_silu_{dt}", "fused_silu", [x], x.shape, dt)
        w, bias = r(128, 256, scale=1 / 11), r(256, scale=0.1)
        add(f"call_matmul_bias_gelu_{dt}", "fused_matmul_bias_activation", [x, w, bias], (6, 40, 256), dt, {"activation": "gelu", "has_bias": True})
        add(f"call_matmul_plain_{dt}", "fused_matmul_bias_activation", [x, w], (6, 40, 256), dt, {"activation": "none", "has_bias": False})
        add(f"call_matmul_bias_residual_{dt}", "fused_matmul_bias_activation", [x, w, bias, r(6, 40, 256)], (6, 40, 256), dt,
            {"activation": "none", "has_bias": True, "has_residual": True})
        q, k, v = r(2, 3, 48, 32), r(2, 3, 80, 32), r(2, 3, 80, 32)
        add(f"call_attention_{dt}", "fused_scaled_dot_product_attention", [q, k, v], q.shape, dt, {"scale": 0.25, "is_causal": False, "head_dim": 32})
        kc, vc = r(2, 3, 48, 32), r(2, 3, 48, 32)
        add(f"call_attention_causal_{dt}", "fused_scaled_dot_product_attention", [q, kc, vc], q.shape, dt,
            {"scale": 32 ** -0.5, "is_causal": True, "head_dim": 32})
        # the handlers this backend restates as plain operators
        stats = lambda: (r(128, scale=0.3), (0.5 + rng.random(128)).astype(np.float32).astype(NP[dt]))  # noqa: E731
        mean, var = stats()
        add(f"call_batch_norm_{dt}", "fused_batch_norm", [x, g, b, mean, var], x.shape, dt, {"eps": 1e-3})
        up, down = r(128, 192, scale=1 / 11), r(192, 64, scale=1 / 14)
        for act in ("gelu", "relu", "silu", "gelu_exact"):
            add(f"call_ffn_{act}_{dt}", "fused_ffn", [x, up, down], (6, 40, 64), dt, {"activation": act, "is_gated": False})
        xr = r(2, 4, 24, 32)  # [batch, heads, sequence, head_dim]
        ang = (rng.random((24, 16)) * 6.0).astype(np.float32)
        add(f"call_rope_angles_{dt}", "fused_rope", [xr, ang.astype(NP[dt])], xr.shape, dt)
        add(f"call_rope_cos_sin_{dt}", "fused_rope", [xr, np.concatenate([np.cos(ang), np.sin(ang)], -1).astype(NP[dt])], xr.shape, dt)
        img, ker, cb = r(2, 12, 12, 8), r(3, 3, 8, 16, scale=0.2), r(16, scale=0.1)
        conv_attrs = ", window_strides = array<i64: 1, 1>, padding = dense<[[1, 1], [1, 1]]> : tensor<2x2xi64>, feature_group_count = 1 : i64"
        for act in ("relu", "none", "silu"):
            add(f"call_conv_bias_{act}_{dt}", "fused_conv_bias_act", [img, ker, cb], (2, 12, 12, 16), dt, {"activation": act, "has_bias": True}, conv_attrs)
        add(f"call_conv_strided_{dt}", "fused_conv_bias_act", [img, ker], (2, 5, 5, 16), dt, {"activation": "tanh", "has_bias": False},
            ", window_strides = array<i64: 2, 2>, padding = dense<0> : tensor<2x2xi64>")
        # the unfused chain the reference's conv-bias-act-fusion takes: convolution -> add(broadcast bias) -> activation
        ti, tk, tb, to = tt(img.shape, dt), tt(ker.shape, dt), tt(cb.shape, dt), tt((2, 12, 12, 16), dt)
        conv_line = (f"    %0 = stablehlo.convolution(%arg0, %arg1) dim_numbers = [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f], "
                     f"window = {{stride = [1, 1], pad = [[1, 1], [1, 1]]}} {{batch_group_count = 1 : i64, feature_group_count = 1 : i64}} : ({ti}, {tk}) -> {to}\n"
                     f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [3] : ({tb}) -> {to}\n"
                     f"    %2 = stablehlo.add %0, %1 : {to}\n")
        tails = {"none": ("", "%2"), "relu": (f"    %z = stablehlo.constant dense<0.0> : {to}\n    %3 = stablehlo.maximum %2, %z : {to}\n", "%3"),
                 "tanh": (f"    %3 = stablehlo.tanh %2 : {to}\n", "%3"), "sigmoid": (f"    %3 = stablehlo.logistic %2 : {to}\n", "%3"),
                 "silu": (f"    %s = stablehlo.logistic %2 : {to}\n    %3 = stablehlo.multiply %2, %s : {to}\n", "%3")}
        for act, (tail, res) in tails.items():
            out.append((f"pattern_conv_bias_{act}_{dt}", func([ti, tk, tb], [to], (conv_line + tail).rstrip("\n"), res), [img, ker, cb]))
        qd, kd, vd = r(5, 1, 64), r(5, 7, 64), r(5, 7, 64)
        add(f"call_depth_attention_{dt}", "fused_depth_attention", [qd, kd, vd], (5, 1, 64), dt, {"scale": 0.125})
        # scale 1 (the handler's default, no multiply emitted): operands shrunk so that 16-bit scores stay near one
        add(f"call_depth_attention_2d_{dt}", "fused_depth_attention", [r(5, 64, scale=0.35), r(5, 7, 64, scale=0.35), vd], (5, 64), dt, {"scale": 1.0})
    return out


def saturating_convert_cases():
    """convert from floats outside the integer type's range: saturates at its ends, NaN gives 0 (the device's rule for 32 and
    64 bits, applied to the narrower types as well)."""
    vals = np.array([np.nan, np.inf, -np.inf, 1e30, -1e30, 300.7, -300.7, 70000.5, -70000.5, 3e9, -3e9, 1e19, 2e19, -1.5, 0.9, 127.9, -128.9, 255.5],
                    dtype=np.float32)
    out = []
    for src in ("f32", "f64", "f16"):
        with np.errstate(over="ignore"):
            x = vals.astype(NP[src])  # the large values become inf in f16
        for dst in ("i8", "ui8", "i16", "ui16", "i32", "ui32", "i64", "ui64"):
            ts, td = tt(x.shape, src), tt(x.shape, dst)
            out.append((f"convert_saturates_{src}_{dst}", func([ts], [td], f"    %0 = stablehlo.convert %arg0 : ({ts}) -> {td}", "%0"), [x]))
    return out


def special_value_cases():
    """NaN, infinities, signed zeros, subnormals and integer extremes through the elementwise operators, compares and
    reductions: the places where a kernel's shortcut (a maximum that drops NaN, a division that traps) shows."""
    out = []
    nan, inf = np.nan, np.inf
    v = np.array([nan, inf, -inf, 0.0, -0.0, 1e-45, -1e-40, 88.8, -104.0, 0.5, -0.5, 1.5, 2.5, -2.5, 3.0, -7.25, 1e10, -1e10], dtype=np.float32)
    t = tt(v.shape, "f32")
    for op in ("abs", "negate", "exponential", "log", "sqrt", "rsqrt", "tanh", "logistic", "floor", "ceil", "sign", "round_nearest_even",
               "round_nearest_afz", "exponential_minus_one", "log_plus_one", "cbrt"):
        out.append((f"special_unary_{op}_f32", func([t], [t], f"    %0 = stablehlo.{op} %arg0 : {t}", "%0"), [v]))
    ti = tt(v.shape, "i1")
    out.append(("special_is_finite_f32", func([t], [ti], f"    %0 = stablehlo.is_finite %arg0 : ({t}) -> {ti}", "%0"), [v]))
    trig = np.array([nan, inf, -inf, 0.0, -0.0, 1e-40, 0.5, -3.0, 100.0, -1000.0], dtype=np.float32)
    tg = tt(trig.shape, "f32")
    for op in ("sine", "cosine"):
        out.append((f"special_unary_{op}_f32", func([tg], [tg], f"    %0 = stablehlo.{op} %arg0 : {tg}", "%0"), [trig]))
    # every pair of a short list of specials
    base = np.array([nan, inf, -inf, 0.0, -0.0, 1.0, -2.5, 3e38], dtype=np.float32)
    a, b = [x.reshape(-1).copy() for x in np.meshgrid(base, base, indexing="ij")]
    tp = tt(a.shape, "f32")
    for op in ("add", "subtract", "multiply", "divide", "maximum", "minimum", "atan2", "power", "remainder"):
        out.append((f"special_binary_{op}_f32", func([tp, tp], [tp], f"    %0 = stablehlo.{op} %arg0, %arg1 : {tp}", "%0"), [a, b]))
    tpi = tt(a.shape, "i1")
    for d in ("EQ", "NE", "LT", "LE", "GT", "GE"):
        out.append((f"special_compare_{d}_f32", func([tp, tp], [tpi], f"    %0 = stablehlo.compare {d}, %arg0, %arg1, FLOAT : ({tp}, {tp}) -> {tpi}", "%0"), [a, b]))
    lo, x, hi = [y.reshape(-1).copy() for y in np.meshgrid(np.array([nan, -1.0, 2.0], np.float32), base, np.array([nan, 1.0, -3.0], np.float32), indexing="ij")]
    tc = tt(x.shape, "f32")
    out.append(("special_clamp_f32", func([tc, tc, tc], [tc], f"    %0 = stablehlo.clamp %arg0, %arg1, %arg2 : {tc}", "%0"), [lo, x, hi]))
    # reductions over rows that hold a NaN, both infinities, or only one of them
    rows = np.array([[1.0, nan, 3.0, -2.0], [inf, 1.0, -inf, 0.0], [inf, 2.0, 5.0, inf], [-0.0, 0.0, -0.0, 0.0], [-inf, -inf, -1.0, -5.0]], dtype=np.float32)
    tr, tv = tt(rows.shape, "f32"), tt((rows.shape[0],), "f32")
    for red, init in (("add", "0.0"), ("maximum", "0xFF800000"), ("minimum", "0x7F800000"), ("multiply", "1.0")):
        body = (f"    %c = stablehlo.constant dense<{init}> : tensor<f32>\n"
                f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.{red} across dimensions = [1] : ({tr}, tensor<f32>) -> {tv}")
        out.append((f"special_reduce_{red}_f32", func([tr], [tv], body, "%0"), [rows]))
    # integers at the ends of their range
    for dt in ("i32", "i64", "i8", "ui32"):
        info = np.iinfo(NP[dt])
        ends = np.array([info.min, info.max, 0, 1, 7, info.max // 3] + ([-1, -7, info.min + 1] if info.min < 0 else [2, 250, info.max - 1]), dtype=NP[dt])
        p, q = [y.reshape(-1).copy() for y in np.meshgrid(ends, ends, indexing="ij")]
        tq = tt(p.shape, dt)
        for op in ("add", "subtract", "multiply", "divide", "remainder", "maximum", "minimum", "and", "or", "xor", "shift_left", "shift_right_arithmetic",
                   "shift_right_logical"):
            out.append((f"special_binary_{op}_{dt}", func([tq, tq], [tq], f"    %0 = stablehlo.{op} %arg0, %arg1 : {tq}", "%0"), [p, q]))
        te = tt(ends.shape, dt)
        for op in ("abs", "negate", "sign", "not", "popcnt", "count_leading_zeros"):
            if info.min == 0 and op in ("abs", "negate", "sign"):
                continue
            out.append((f"special_unary_{op}_{dt}", func([te], [te], f"    %0 = stablehlo.{op} %arg0 : {te}", "%0"), [ends]))
    return out


def more_edge_cases():
    """Special values in the 16-bit and 64-bit float types, integer compares at the ends of the range, reductions of
    integers that wrap, and tensors with no elements, no dimensions or many dimensions."""
    out = []
    nan, inf = np.nan, np.inf
    for dt in ("f16", "bf16", "f64"):
        if dt not in NP:
            continue
        big = {"f16": 60000.0, "bf16": 3e38, "f64": 1e308}[dt]
        with np.errstate(over="ignore"):
            base = np.array([nan, inf, -inf, 0.0, -0.0, 1.0, -2.5, big, -big, 6e-8], dtype=np.float64).astype(NP[dt])
        a, b = [x.reshape(-1).copy() for x in np.meshgrid(base, base, indexing="ij")]
        tp, tpi = tt(a.shape, dt), tt(a.shape, "i1")
        for op in ("add", "subtract", "multiply", "divide", "maximum", "minimum"):
            out.append((f"special_binary_{op}_{dt}", func([tp, tp], [tp], f"    %0 = stablehlo.{op} %arg0, %arg1 : {tp}", "%0"), [a, b]))
        for d in ("EQ", "LT", "GE"):
            out.append((f"special_compare_{d}_{dt}", func([tp, tp], [tpi], f"    %0 = stablehlo.compare {d}, %arg0, %arg1, FLOAT : ({tp}, {tp}) -> {tpi}", "%0"), [a, b]))
        tb = tt(base.shape, dt)
        for op in ("abs", "negate", "sqrt", "exponential", "floor", "sign", "tanh"):
            out.append((f"special_unary_{op}_{dt}", func([tb], [tb], f"    %0 = stablehlo.{op} %arg0 : {tb}", "%0"), [base]))
    for dt, ctype in (("i32", "SIGNED"), ("ui32", "UNSIGNED"), ("i64", "SIGNED"), ("ui64", "UNSIGNED"), ("i8", "SIGNED"), ("ui8", "UNSIGNED")):
        info = np.iinfo(NP[dt])
        ends = np.array([info.min, info.max, 0, 1, info.max // 2, info.max // 2 + 1, info.max - 1] + ([-1, info.min + 1] if info.min < 0 else [2, 3]), dtype=NP[dt])
        p_, q_ = [y.reshape(-1).copy() for y in np.meshgrid(ends, ends, indexing="ij")]
        tq, tqi = tt(p_.shape, dt), tt(p_.shape, "i1")
        for d in ("EQ", "NE", "LT", "LE", "GT", "GE"):
            out.append((f"special_compare_{d}_{dt}", func([tq, tq], [tqi], f"    %0 = stablehlo.compare {d}, %arg0, %arg1, {ctype} : ({tq}, {tq}) -> {tqi}", "%0"), [p_, q_]))
        rows = np.stack([ends, ends[::-1], np.full_like(ends, info.max), np.full_like(ends, info.min)])
        tr, tv = tt(rows.shape, dt), tt((rows.shape[0],), dt)
        for red, init in (("add", "0"), ("multiply", "1"), ("maximum", str(info.min)), ("minimum", str(info.max))):
            if dt == "ui64" and red in ("maximum", "minimum"):
                continue  # refused by the lowering (64-bit unsigned order)
            body = (f"    %c = stablehlo.constant dense<{init}> : tensor<{dt}>\n"
                    f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.{red} across dimensions = [1] : ({tr}, tensor<{dt}>) -> {tv}")
            out.append((f"special_reduce_{red}_{dt}", func([tr], [tv], body, "%0"), [rows]))
    # tensors with no elements, scalars, and rank 6
    rng = np.random.default_rng(4242)
    e0, e1 = tt((0, 5), "f32"), tt((3, 0), "f32")
    out.append(("empty_add", func([e0, e0], [e0], f"    %0 = stablehlo.add %arg0, %arg1 : {e0}", "%0"), [np.zeros((0, 5), np.float32)] * 2))
    out.append(("empty_reduce_to_init", func([e1], [tt((3,), "f32")],
                                             f"    %c = stablehlo.constant dense<7.0> : tensor<f32>\n"
                                             f"    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [1] : ({e1}, tensor<f32>) -> {tt((3,), 'f32')}", "%0"),
                [np.zeros((3, 0), np.float32)]))
    out.append(("empty_contraction", func([tt((4, 0), "f32"), tt((0, 6), "f32")], [tt((4, 6), "f32")],
                                          f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : ({tt((4, 0), 'f32')}, {tt((0, 6), 'f32')}) -> {tt((4, 6), 'f32')}", "%0"),
                [np.zeros((4, 0), np.float32), np.zeros((0, 6), np.float32)]))
    out.append(("empty_concatenate", func([e0, tt((2, 5), "f32")], [tt((2, 5), "f32")],
                                          f"    %0 = stablehlo.concatenate %arg0, %arg1, dim = 0 : ({e0}, {tt((2, 5), 'f32')}) -> {tt((2, 5), 'f32')}", "%0"),
                [np.zeros((0, 5), np.float32), rand(rng, (2, 5), "f32")]))
    out.append(("empty_transpose_and_broadcast", func([e1], [tt((2, 0, 3), "f32")],
                                                      f"    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({e1}) -> {tt((0, 3), 'f32')}\n"
                                                      f"    %1 = stablehlo.broadcast_in_dim %0, dims = [1, 2] : ({tt((0, 3), 'f32')}) -> {tt((2, 0, 3), 'f32')}", "%1"),
                [np.zeros((3, 0), np.float32)]))
    s0 = tt((), "f32")
    out.append(("scalar_chain", func([s0, s0], [s0, tt((), "i1")],
                                     f"    %0 = stablehlo.multiply %arg0, %arg1 : {s0}\n    %1 = stablehlo.tanh %0 : {s0}\n"
                                     f"    %2 = stablehlo.compare GT, %1, %arg1, FLOAT : ({s0}, {s0}) -> tensor<i1>", "%1, %2"),
                [np.array(0.7, np.float32), np.array(-1.3, np.float32)]))
    sh6 = (2, 3, 1, 4, 2, 5)
    t6 = tt(sh6, "f32")
    p6 = [5, 0, 3, 1, 4, 2]
    o6 = tuple(sh6[i] for i in p6)
    body = (f"    %0 = stablehlo.transpose %arg0, dims = {p6} : ({t6}) -> {tt(o6, 'f32')}\n"
            f"    %c = stablehlo.constant dense<0.0> : tensor<f32>\n"
            f"    %1 = stablehlo.reduce(%0 init: %c) applies stablehlo.add across dimensions = [1, 4] : ({tt(o6, 'f32')}, tensor<f32>) -> {tt((5, 4, 3, 1), 'f32')}\n"
            f"    %2 = stablehlo.reverse %1, dims = [0, 2] : {tt((5, 4, 3, 1), 'f32')}")
    out.append(("rank6_transpose_reduce_reverse", func([t6], [tt((5, 4, 3, 1), "f32")], body, "%2"), [rand(rng, sh6, "f32")]))
    return out


def fused_pattern_edge_cases():
    """The fusable patterns on rows that stress their kernels: masked (-inf) and constant softmax rows, single-element rows,
    constant and zero rows under the norms, activations far out on both sides."""
    out = []
    inf = np.inf
    for dt in ("f32", "f16", "bf16"):
        if dt not in NP:
            continue
        hid = 64
        rows = np.zeros((8, hid), np.float32)
        rng = np.random.default_rng(77)
        rows[0] = rng.standard_normal(hid)
        rows[1] = 3.25                                   # constant row: uniform probabilities, zero variance
        rows[2] = rng.standard_normal(hid); rows[2, 10:] = -inf   # masked tail
        rows[3] = -inf; rows[3, 5] = 0.0                 # one visible entry
        rows[4] = rng.standard_normal(hid) * 30.0        # wide range: the maximum must be subtracted
        rows[5] = 0.0
        rows[6] = np.linspace(-60, 60, hid)
        rows[7] = 1e4 if dt != "f16" else 6e4            # large constant
        x = rows.astype(NP[dt])
        shape = x.shape
        t = tt(shape, dt)
        body, res = softmax_text("%arg0", shape, dt, 1)
        out.append((f"edge_softmax_rows_{dt}", func([t], [t], body.rstrip("\n"), res), [x]))
        fin = np.where(np.isfinite(rows), rows, 0.0).astype(np.float32)
        fin[7] = 100.0
        if dt == "f16":  # the unfused program sums the squares in f16: keep a row's sum below 65504
            fin[4] /= 3.0
            fin[6] /= 3.0
            fin[7] = 25.0
        xf = fin.astype(NP[dt])
        g = np.linspace(0.5, 1.5, hid).astype(np.float32).astype(NP[dt])
        b = np.linspace(-0.2, 0.2, hid).astype(np.float32).astype(NP[dt])
        tv = tt((hid,), dt)
        body, res = layer_norm_text("%arg0", shape, dt, "%arg1", "%arg2")
        out.append((f"edge_layer_norm_rows_{dt}", func([t, tv, tv], [t], body.rstrip("\n"), res), [xf, g, b]))
        body, res = layer_norm_text("%arg0", shape, dt, "%arg1", None, eps=1e-6, rms=True)
        out.append((f"edge_rms_norm_rows_{dt}", func([t, tv], [t], body.rstrip("\n"), res), [xf, g]))
        far = np.array([[-100.0, -20.0, -9.0, -5.0, -1.0, -1e-3, 0.0, -0.0, 1e-3, 1.0, 5.0, 9.0, 20.0, 100.0, 3.0, -3.0]], np.float32).astype(NP[dt])
        tf_ = tt(far.shape, dt)
        body, res = gelu_text("%arg0", far.shape, dt)
        out.append((f"edge_gelu_far_{dt}", func([tf_], [tf_], body.rstrip("\n"), res), [far]))
        one = rng.standard_normal((5, 1)).astype(np.float32).astype(NP[dt])
        t1 = tt((5, 1), dt)
        body, res = softmax_text("%arg0", (5, 1), dt, 1)
        out.append((f"edge_softmax_single_element_rows_{dt}", func([t1], [t1], body.rstrip("\n"), res), [one]))
    return out


def contraction_edge_cases():
    """Non-finite operands through the tensor-core products and attention: a NaN or an infinity must come out in exactly the
    rows and columns it touches (inf * 0 and inf - inf included), nowhere else."""
    out = []
    rng = np.random.default_rng(555)
    for dt in ("bf16", "f16", "f32"):
        if dt not in NP:
            continue
        m, k, n = 128, 64, 128
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        a[3, 7] = np.nan
        a[10, 0] = np.inf
        a[20, 5] = np.inf; a[20, 6] = -np.inf   # inf - inf in every column of row 20 (b[5], b[6] of one sign below)
        b[5, :] = np.abs(b[5, :]) + 0.1
        b[6, :] = np.abs(b[6, :]) + 0.1
        b[0, 17] = 0.0                           # inf * 0 at (10, 17)
        b[9, 40] = np.nan
        b[11, 99] = -np.inf
        ta, tb, tc = tt((m, k), dt), tt((k, n), dt), tt((m, n), dt)
        out.append((f"edge_dot_nonfinite_{dt}", func([ta, tb], [tc], f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : ({ta}, {tb}) -> {tc}", "%0"),
                    [a.astype(NP[dt]), b.astype(NP[dt])]))
    # bias + GELU in the product's epilogue with pre-activations far out on both sides (the 16-bit epilogue evaluates the
    # tanh form two values at a time in f16 arithmetic)
    for dt in ("f16", "bf16"):
        if dt not in NP:
            continue
        m, k, n = 128, 64, 128
        x = np.zeros((m, k), np.float32)
        x[:, 0] = np.linspace(-300, 300, m)
        x[:, 1:] = 0.05 * rng.standard_normal((m, k - 1))
        w = np.zeros((k, n), np.float32)
        w[0, :] = np.linspace(0.01, 1.0, n)
        w[1:, :] = 0.1 * rng.standard_normal((k - 1, n))
        bias = np.linspace(-2, 2, n).astype(np.float32)
        tx, tw, tb_, ty = tt((m, k), dt), tt((k, n), dt), tt((n,), dt), tt((m, n), dt)
        gb, gres = gelu_text("%2", (m, n), dt)
        body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : ({tx}, {tw}) -> {ty}\n"
                f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [1] : ({tb_}) -> {ty}\n"
                f"    %2 = stablehlo.add %0, %1 : {ty}\n" + gb)
        out.append((f"edge_dense_gelu_far_{dt}", func([tx, tw, tb_], [ty], body.rstrip("\n"), gres), [x.astype(NP[dt]), w.astype(NP[dt]), bias.astype(NP[dt])]))
    return out


def window_sort_edge_cases():
    """Pooling windows that hold a NaN, an infinity or only padding; sorts of keys with ties, NaNs and signed zeros."""
    out = []
    rng = np.random.default_rng(8080)
    for dt in ("f32", "bf16"):
        if dt not in NP:
            continue
        x = rand(rng, (1, 6, 6, 8), dt).astype(np.float32)
        x[0, 0, 0, :] = np.nan
        x[0, 2, 3, 1] = np.inf
        x[0, 4, 4, 2] = -np.inf
        x[0, 5, :, 3] = 0.25   # ties along a window
        x = x.astype(NP[dt])
        out.append(reduce_window_case(f"edge_maxpool_nonfinite_{dt}", x, dt, "maximum", "-inf", (1, 3, 3, 1), (1, 3, 3, 8), strides=(1, 2, 2, 1),
                                      padding=((0, 0), (1, 0), (1, 0), (0, 0))))
        out.append(reduce_window_case(f"edge_minpool_nonfinite_{dt}", x, dt, "minimum", "inf", (1, 2, 2, 1), (1, 3, 3, 8), strides=(1, 2, 2, 1)))
        out.append(reduce_window_case(f"edge_sumpool_nonfinite_{dt}", x, dt, "add", 0, (1, 2, 2, 1), (1, 5, 5, 8)))
    # a window that lies in the padding alone gives the init value
    out.append(reduce_window_case("edge_window_in_padding_only", rand(rng, (4, 4), "f32"), "f32", "maximum", "-inf", (2, 2), (4, 4),
                                  strides=(2, 2), padding=((2, 2), (2, 2))))
    keys = np.array([[3.0, np.nan, -0.0, 0.0, 3.0, -np.inf, np.inf, 1.0, -np.nan, 1.0, 0.0, -0.0]], dtype=np.float32)
    pay = np.arange(keys.size, dtype=np.int32).reshape(keys.shape)
    out.append(sort_case("edge_sort_ties_nan_zeros_asc", [keys, pay], ["f32", "i32"], 1))
    out.append(sort_case("edge_sort_ties_nan_zeros_desc", [keys, pay], ["f32", "i32"], 1, direction="GT"))
    ik = np.array([[5, -7, 5, 2147483647, -2147483648, 0, -7, 5]], dtype=np.int32)
    out.append(sort_case("edge_sort_int_ties_stable", [ik, np.arange(8, dtype=np.int32).reshape(1, 8)], ["i32", "i32"], 1))
    return out


def shared_intermediate_cases():
    """The fusable patterns with a second reader on one of their inner values: the fusion has to leave that value alive
    (or not fire), whatever the level."""
    out = []
    rng = np.random.default_rng(3131)
    for dt in ("f32", "bf16"):
        if dt not in NP:
            continue
        shape = (4, 24, 64)
        t, red = tt(shape, dt), tt(shape[:-1], dt)
        x = rand(rng, shape, dt)
        g = (1 + 0.1 * rng.standard_normal(64)).astype(np.float32).astype(NP[dt])
        b = (0.1 * rng.standard_normal(64)).astype(np.float32).astype(NP[dt])
        tv = tt((64,), dt)
        body, res = softmax_text("%arg0", shape, dt, 2)
        for extra, et in (("%s3", t), ("%s0", red), ("%s4", red)):   # exp(x - max), the row maximum, the row sum
            out.append((f"shared_softmax_{extra[1:]}_{dt}", func([t], [t, et], body.rstrip("\n"), f"{res}, {extra}"), [x]))
        body, res = layer_norm_text("%arg0", shape, dt, "%arg1", "%arg2")
        for extra, et in (("%n1", red), ("%n3", t), ("%n8", red), ("%n10", t)):   # mean, centred value, rsqrt, normalised value
            out.append((f"shared_layer_norm_{extra[1:]}_{dt}", func([t, tv, tv], [t, et], body.rstrip("\n"), f"{res}, {extra}"), [x, g, b]))
        body, res = gelu_text("%arg0", shape, dt)
        for extra in ("%g5", "%g3"):   # tanh(...), the cubic
            out.append((f"shared_gelu_{extra[1:]}_{dt}", func([t], [t, t], body.rstrip("\n"), f"{res}, {extra}"), [x]))
        # dense + bias + gelu with the pre-activation read again; residual + norm with the sum and the variance read again
        w = (rng.standard_normal((64, 128)) / 8).astype(np.float32).astype(NP[dt])
        bias = (0.1 * rng.standard_normal(128)).astype(np.float32).astype(NP[dt])
        ts, tw, tb_ = tt((4, 24, 128), dt), tt((64, 128), dt), tt((128,), dt)
        gb, gres = gelu_text("%2", (4, 24, 128), dt)
        body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [2] x [0] : ({t}, {tw}) -> {ts}\n"
                f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [2] : ({tb_}) -> {ts}\n"
                f"    %2 = stablehlo.add %0, %1 : {ts}\n" + gb)
        out.append((f"shared_dense_preactivation_{dt}", func([t, tw, tb_], [ts, ts, ts], body.rstrip("\n"), f"{gres}, %2, %0"), [x, w, bias]))
        xr = rand(rng, shape, dt)
        lb, lres = layer_norm_text("%s0", shape, dt, "%arg2", "%arg3")
        body = f"    %s0 = stablehlo.add %arg0, %arg1 : {t}\n" + lb
        out.append((f"shared_residual_norm_variance_{dt}", func([t, t, tv, tv], [t, t, red], body.rstrip("\n"), f"{lres}, %s0, %n6"), [x, xr, g, b]))
    for dt in ("f32",):  # (16-bit attention outputs need the magnitude bound the pattern_attention cases get)
        for causal in (False, True):
            text, qshape = attention_text(2, 2, 32, 32, dt, causal, "BHSD")
            # also return the scaled scores (%1): the fused attention never materialises them
            q, k, v = (rand(rng, qshape, dt) for _ in range(3))
            m = re.search(r"return (%\w+) : (tensor<[^>]*>)", text)
            if not m:
                continue
            ts_ = tt((2, 2, 32, 32), dt)
            text2 = text.replace(m.group(0), f"return {m.group(1)}, %1 : {m.group(2)}, {ts_}")
            text2 = re.sub(r"-> \(?(tensor<[^>]*>)\)? \{", lambda mm: f"-> ({mm.group(1)}, {ts_}) {{", text2, count=1)
            out.append((f"shared_attention_scores_{'causal_' if causal else ''}{dt}", text2, [q, k, v]))
    return out


def random_program_cases(count=60, seed=20260101, dt="f32", extents=(2, 3, 4, 5, 6, 8), more=False):
    """Seeded random programs of 12 to 24 operations (elementwise chains, compares and selects, reductions broadcast back,
    transposes, reshapes, slices, concatenations): what the optimisation levels do to a program nobody wrote by hand must not
    change its result."""
    rng = np.random.default_rng(seed)
    out = []
    integer = dt != "f32"
    unary = ["abs", "negate", "not", "sign", "popcnt"] if integer else ["abs", "negate", "tanh", "logistic", "floor", "ceil", "sine", "cosine", "sign", "round_nearest_even"]
    binary = ["add", "subtract", "multiply", "maximum", "minimum", "and", "or", "xor"] if integer else ["add", "subtract", "multiply", "maximum", "minimum"]
    ctype = "SIGNED" if integer else "FLOAT"
    info = np.iinfo(NP[dt]) if integer else None
    for case in range(count):
        shape = tuple(int(x) for x in rng.choice(list(extents), size=3))
        n_in = int(rng.integers(1, 4))
        vals = [(f"%arg{i}", shape) for i in range(n_in)]  # (name, shape), all f32
        lines = []

        def emit(text, shp):
            name = f"%v{len(lines)}"
            lines.append(f"    {name} = {text}")
            vals.append((name, shp))
            return name

        def pick(shp=None):
            cands = [v for v in vals if shp is None or v[1] == shp]
            return cands[int(rng.integers(0, len(cands)))]

        for _ in range(int(rng.integers(12, 25))):
            kind = rng.choice(["unary", "binary", "binary", "select", "reduce", "transpose", "reshape", "slice", "concat", "safe"] +
                              (["pad", "clamp", "iota", "dot", "reverse", "broadcast"] if more else []))
            a, shp = pick()
            t = tt(shp, dt)
            if kind == "unary":
                emit(f"stablehlo.{rng.choice(unary)} {a} : {t}", shp)
            elif kind == "binary":
                b, _ = pick(shp)
                emit(f"stablehlo.{rng.choice(binary)} {a}, {b} : {t}", shp)
            elif kind == "safe":  # divide / sqrt / log on arguments kept away from their singularities
                b, _ = pick(shp)
                one = emit(f"stablehlo.constant dense<{'3' if integer else '1.5'}> : {t}", shp)
                den = emit(f"stablehlo.add {emit(f'stablehlo.abs {b} : {t}', shp)}, {one} : {t}", shp)
                op = "divide" if integer else str(rng.choice(["divide", "sqrt", "log", "rsqrt"]))
                if integer:  # |b| + 3 wraps to a negative number only for b near the ends: keep it positive with a mask
                    den = emit(f"stablehlo.or {emit(f'stablehlo.and {den}, {emit(f"stablehlo.constant dense<1023> : {t}", shp)} : {t}', shp)}, {one} : {t}", shp)
                emit(f"stablehlo.divide {a}, {den} : {t}" if op == "divide" else f"stablehlo.{op} {den} : {t}", shp)
            elif kind == "select":
                b, _ = pick(shp)
                c, _ = pick(shp)
                d = str(rng.choice(["LT", "GE", "EQ", "NE"]))
                p = emit(f"stablehlo.compare {d}, {a}, {b}, {ctype} : ({t}, {t}) -> {tt(shp, 'i1')}", shp)
                vals.pop()  # predicates are not operands of the float ops
                emit(f"stablehlo.select {p}, {b}, {c} : {tt(shp, 'i1')}, {t}", shp)
            elif kind == "reduce" and len(shp) >= 2:
                ax = int(rng.integers(0, len(shp)))
                red = str(rng.choice(["add", "maximum", "minimum"]))
                init = {"add": "0", "maximum": str(info.min), "minimum": str(info.max)}[red] if integer else {"add": "0.0", "maximum": "0xFF800000", "minimum": "0x7F800000"}[red]
                rs = tuple(d for i, d in enumerate(shp) if i != ax)
                c0 = emit(f"stablehlo.constant dense<{init}> : tensor<{dt}>", ())
                vals.pop()
                r = emit(f"stablehlo.reduce({a} init: {c0}) applies stablehlo.{red} across dimensions = [{ax}] : ({t}, tensor<{dt}>) -> {tt(rs, dt)}", rs)
                vals.pop()
                dims = [i for i in range(len(shp)) if i != ax]
                emit(f"stablehlo.broadcast_in_dim {r}, dims = {dims} : ({tt(rs, dt)}) -> {t}", shp)
            elif kind == "transpose" and len(shp) >= 2:
                perm = [int(x) for x in rng.permutation(len(shp))]
                emit(f"stablehlo.transpose {a}, dims = {perm} : ({t}) -> {tt(tuple(shp[i] for i in perm), dt)}", tuple(shp[i] for i in perm))
            elif kind == "reshape":
                total = int(np.prod(shp))
                facts = [d for d in tuple(extents) + (2, 3, 4) if total % d == 0] or [1]
                d0 = int(rng.choice(facts))
                ns = (d0, total // d0)
                emit(f"stablehlo.reshape {a} : ({t}) -> {tt(ns, dt)}", ns)
            elif kind == "slice" and all(d >= 2 for d in shp):
                lo = [int(rng.integers(0, d // 2)) for d in shp]
                hi = [int(rng.integers(l + 1, d + 1)) for l, d in zip(lo, shp)]
                st = [int(rng.integers(1, 3)) for _ in shp]
                ns = tuple((h - l + s_ - 1) // s_ for l, h, s_ in zip(lo, hi, st))
                spec = ", ".join(f"{l}:{h}:{s_}" for l, h, s_ in zip(lo, hi, st))
                emit(f"stablehlo.slice {a} [{spec}] : ({t}) -> {tt(ns, dt)}", ns)
            elif kind == "pad":
                lo = [int(rng.integers(-1, 3)) for _ in shp]
                hi = [int(rng.integers(-1, 3)) for _ in shp]
                it_ = [int(rng.integers(0, 2)) for _ in shp]
                ns = tuple(d + l + h + max(d - 1, 0) * i_ for d, l, h, i_ in zip(shp, lo, hi, it_))
                if all(d >= 1 for d in ns) and len(shp) >= 1:
                    c0 = emit(f"stablehlo.constant dense<{'7' if integer else '0.5'}> : tensor<{dt}>", ())
                    vals.pop()
                    emit(f"stablehlo.pad {a}, {c0}, low = {lo}, high = {hi}, interior = {it_} : ({t}, tensor<{dt}>) -> {tt(ns, dt)}", ns)
            elif kind == "clamp":
                b, _ = pick(shp)
                c, _ = pick(shp)
                lo_ = emit(f"stablehlo.minimum {b}, {c} : {t}", shp)
                vals.pop()
                hi_ = emit(f"stablehlo.maximum {b}, {c} : {t}", shp)
                vals.pop()
                emit(f"stablehlo.clamp {lo_}, {a}, {hi_} : {t}", shp)
            elif kind == "iota" and len(shp) >= 1:
                ax = int(rng.integers(0, len(shp)))
                io = emit(f"stablehlo.iota dim = {ax} : {t}", shp)
                vals.pop()
                emit(f"stablehlo.{rng.choice(['add', 'multiply', 'maximum'])} {a}, {io} : {t}", shp)
            elif kind == "reverse" and len(shp) >= 1:
                ax = sorted(set(int(x) for x in rng.integers(0, len(shp), size=2)))
                emit(f"stablehlo.reverse {a}, dims = {ax} : {t}", shp)
            elif kind == "broadcast" and len(shp) >= 1 and len(shp) <= 3:
                extra = int(rng.choice([1, 2, 3]))
                pos = int(rng.integers(0, len(shp) + 1))
                ns = shp[:pos] + (extra,) + shp[pos:]
                dims = [i if i < pos else i + 1 for i in range(len(shp))]
                emit(f"stablehlo.broadcast_in_dim {a}, dims = {dims} : ({t}) -> {tt(ns, dt)}", ns)
            elif kind == "dot" and len(shp) >= 2:
                b, bs = pick()
                if len(bs) >= 2 and bs[-1] == shp[-1] and len(bs) == len(shp) and bs[:-2] == shp[:-2]:
                    # a . b^T over the last axis, the leading axes as batch
                    nb = len(shp) - 2
                    batch = list(range(nb))
                    ns = shp[:-1] + (bs[-2],)
                    spec = (f"batching_dims = {batch} x {batch}, " if nb else "") + f"contracting_dims = [{len(shp) - 1}] x [{len(bs) - 1}]"
                    emit(f"stablehlo.dot_general {a}, {b}, {spec} : ({t}, {tt(bs, dt)}) -> {tt(ns, dt)}", ns)
            elif kind == "concat":
                b, _ = pick(shp)
                ax = int(rng.integers(0, len(shp)))
                ns = tuple(d * 2 if i == ax else d for i, d in enumerate(shp))
                emit(f"stablehlo.concatenate {a}, {b}, dim = {ax} : ({t}, {t}) -> {tt(ns, dt)}", ns)
        if not lines:
            continue
        results = [vals[-1]] + ([vals[-3]] if len(vals) > n_in + 3 else [])
        text = func([tt(shape, dt)] * n_in, [tt(r[1], dt) for r in results], "\n".join(lines), ", ".join(r[0] for r in results))
        out.append((f"random_program_{dt}_{case:02d}", text, [rand(rng, shape, dt) for _ in range(n_in)]))
    return out


def quantize_cases():
    """uniform_quantize / uniform_dequantize in the reference's two-operand form (scale as a tensor operand)."""
    rng = np.random.default_rng(909)
    out = []
    for dt, qt in (("f32", "i8"), ("f32", "i32"), ("f16", "i8"), ("f32", "ui8")):
        shape = (5, 33)
        x = (rng.uniform(-40, 40, size=shape)).astype(np.float32).astype(NP[dt])
        if qt == "ui8":
            x = np.abs(x)
        t, q = tt(shape, dt), tt(shape, qt)
        for sname, sshape in (("scalar", ()), ("per_column", (33,))):
            ts = tt(sshape, dt)
            scale = rng.uniform(0.1, 0.5, size=sshape).astype(np.float32).astype(NP[dt])
            body = (f"    %0 = stablehlo.uniform_quantize %arg0, %arg1 : ({t}, {ts}) -> {q}\n"
                    f"    %1 = stablehlo.uniform_dequantize %0, %arg1 : ({q}, {ts}) -> {t}")
            out.append((f"quantize_roundtrip_{dt}_{qt}_{sname}", func([t, ts], [q, t], body, "%0, %1"), [x, scale]))
    return out


def rng_cases():
    """stablehlo.rng_bit_generator in the forms jax.random emits under the rbg implementations: every output width, a
    Philox-shaped state of three words, and two draws chained through the state."""
    out = []
    for name, shape, dt, algo, words in (("ui32", (7, 33), "ui32", "THREE_FRY", 2), ("ui64", (129,), "ui64", "DEFAULT", 2),
                                         ("ui8", (5, 5, 5), "ui8", "PHILOX", 3), ("i16", (1001,), "i16", "DEFAULT", 2),
                                         ("i32_scalar_count", (1,), "i32", "THREE_FRY", 2), ("ui32_empty", (0,), "ui32", "DEFAULT", 2)):
        ts, to = tt((words,), "ui64"), tt(shape, dt)
        body = f"    %0, %1 = stablehlo.rng_bit_generator %arg0, algorithm = {algo} : ({ts}) -> ({ts}, {to})"
        state = np.array([0x0123456789ABCDEF, 0xFFFFFFFFFFFFFFF0, 77][:words], dtype=np.uint64)  # the counter crosses 2^64 in the larger draws
        out.append((f"rng_bit_generator_{name}", func([ts], [ts, to], body, "%0, %1"), [state]))
    ts, to = tt((2,), "ui64"), tt((64,), "ui32")
    body = (f"    %0, %1 = stablehlo.rng_bit_generator %arg0, algorithm = DEFAULT : ({ts}) -> ({ts}, {to})\n"
            f"    %2, %3 = stablehlo.rng_bit_generator %0, algorithm = DEFAULT : ({ts}) -> ({ts}, {to})\n"
            f"    %4 = stablehlo.xor %1, %3 : {to}")
    out.append(("rng_bit_generator_chained", func([ts], [ts, to], body, "%2, %4"), [np.array([42, 0], dtype=np.uint64)]))
    return out


def ct(shape, part="f32"):
    return "tensor<" + "x".join([str(d) for d in shape] + [f"complex<{part}>"]) + ">"


def fft_cases():
    """stablehlo.fft (all four kinds, one to three axes, lengths on and off the powers of two, f32 and f64 parts) and the
    operations on complex values that surround it in a jax.numpy.fft program. Complex arguments and results of @main are
    float arrays with a last axis of (re, im)."""
    rng = np.random.default_rng(1807)
    out = []

    def parts(z, shape, part):  # spectrum -> (re, im, abs) as real results
        t, c = tt(shape, part), ct(shape, part)
        return (f"    %re = stablehlo.real {z} : ({c}) -> {t}\n    %im = stablehlo.imag {z} : ({c}) -> {t}\n"
                f"    %ab = stablehlo.abs {z} : ({c}) -> {t}"), "%re, %im, %ab", [t, t, t]

    # real input -> half spectrum, one axis
    for part, cases in (("f32", ((4, 64), (3, 100), (2, 1), (5, 7), (1, 4096), (2, 8192), (2, 3000))), ("f64", ((3, 32), (2, 45)))):
        for shape in cases:
            n = shape[-1]
            hs = shape[:-1] + (n // 2 + 1,)
            body, res, rts = parts("%0", hs, part)
            text = func([tt(shape, part)], rts, f"    %0 = stablehlo.fft %arg0, type = RFFT, length = [{n}] : ({tt(shape, part)}) -> {ct(hs, part)}\n" + body, res)
            out.append((f"fft_rfft_{part}_{n}", text, [rand(rng, shape, part)]))
    # lines too long for shared memory: one launch per radix-2 pass through global scratch
    for shape, lens, kinds in (((2, 16384), [16384], ("RFFT",)), ((1, 32768), [32768], ("RFFT",)), ((3, 16384), [16384], ("FFT", "IFFT"))):
        for kind in kinds:
            n = shape[-1]
            if kind == "RFFT":
                hs = shape[:-1] + (n // 2 + 1,)
                t, c = tt(shape, "f32"), ct(hs)
                text = func([t], [c, t], f"    %0 = stablehlo.fft %arg0, type = RFFT, length = {lens} : ({t}) -> {c}\n"
                                         f"    %1 = stablehlo.fft %0, type = IRFFT, length = {lens} : ({c}) -> {t}", "%0, %1")
                out.append((f"fft_long_rfft_irfft_{n}", text, [rand(rng, shape, "f32")]))
            else:
                c = ct(shape)
                text = func([c], [c], f"    %0 = stablehlo.fft %arg0, type = {kind}, length = {lens} : ({c}) -> {c}", "%0")
                out.append((f"fft_long_{kind.lower()}_{n}", text, [rand(rng, shape + (2,), "f32")]))
    # complex -> complex, forward and back, built from two real arguments
    for kind in ("FFT", "IFFT"):
        for shape, lens in (((3, 128), [128]), ((2, 8, 16), [8, 16]), ((2, 4, 6, 8), [4, 6, 8]), ((3, 5, 12), [12]), ((2, 9, 10), [9, 10])):
            t, c = tt(shape, "f32"), ct(shape)
            body, res, rts = parts("%1", shape, "f32")
            text = func([t, t], rts, f"    %0 = stablehlo.complex %arg0, %arg1 : {c}\n"
                                     f"    %1 = stablehlo.fft %0, type = {kind}, length = {lens} : ({c}) -> {c}\n" + body, res)
            out.append((f"fft_{kind.lower()}_{'x'.join(map(str, lens))}", text, [rand(rng, shape, "f32"), rand(rng, shape, "f32")]))
    # real -> half spectrum -> real over two and three axes; the spectrum crosses the boundary as (re, im) pairs
    for shape, lens in (((2, 12, 10), [12, 10]), ((3, 8, 32), [8, 32]), ((2, 3, 4, 9), [3, 4, 9]), ((4, 16), [16]), ((4, 15), [15])):
        hs = shape[:-1] + (shape[-1] // 2 + 1,)
        t, c = tt(shape, "f32"), ct(hs)
        text = func([t], [c, t], f"    %0 = stablehlo.fft %arg0, type = RFFT, length = {lens} : ({t}) -> {c}\n"
                                 f"    %1 = stablehlo.fft %0, type = IRFFT, length = {lens} : ({c}) -> {t}", "%0, %1")
        out.append((f"fft_rfft_irfft_{'x'.join(map(str, lens))}", text, [rand(rng, shape, "f32")]))
    # a complex argument (pairs) through the generic form of the operation
    shape = (5, 16)
    c = ct(shape)
    text = func([c], [c], f'    %0 = "stablehlo.fft"(%arg0) {{fft_type = #stablehlo<fft_type FFT>, fft_length = array<i64: 16>}} : ({c}) -> {c}', "%0")
    out.append(("fft_generic_form_complex_argument", text, [rand(rng, shape + (2,), "f32")]))
    # the reference's form: no complex types, the pairs are float elements (Compiler/CodeGenerator.swift:2701-2830)
    tp, th, tr = tt((4, 16, 2), "f32"), tt((4, 9, 2), "f32"), tt((4, 16), "f32")
    out.append(("fft_float_pairs_fft", func([tp], [tp], f"    %0 = stablehlo.fft %arg0, type = FFT, length = [16] : ({tp}) -> {tp}", "%0"),
                [rand(rng, (4, 16, 2), "f32")]))
    out.append(("fft_float_pairs_rfft_irfft", func([tr], [th, tr], f"    %0 = stablehlo.fft %arg0, type = RFFT, length = [16] : ({tr}) -> {th}\n"
                                                                   f"    %1 = stablehlo.fft %0, type = IRFFT, length = [16] : ({th}) -> {tr}", "%0, %1"),
                [rand(rng, (4, 16), "f32")]))
    # arithmetic and data movement on complex values
    shape = (3, 8)
    t, c = tt(shape, "f32"), ct(shape)
    a, b = rand(rng, shape + (2,), "f32"), rand(rng, shape + (2,), "f32", 0.5, 2.0)
    for name in ("add", "subtract", "multiply", "divide"):
        out.append((f"complex_{name}", func([c, c], [c], f"    %0 = stablehlo.{name} %arg0, %arg1 : {c}", "%0"), [a, b]))
    out.append(("complex_negate", func([c], [c], f"    %0 = stablehlo.negate %arg0 : {c}", "%0"), [a]))
    body = (f"    %k = stablehlo.constant dense<(0.5, -2.0)> : {c}\n"
            f"    %l = stablehlo.constant dense<[(1.0, 0.0), (0.0, 1.0), (-1.0, 0.0), (0.0, -1.0), (2.0, 2.0), (0.5, 0.25), (3.0, -1.0), (0.0, 0.0)]> : {ct((8,))}\n"
            f"    %lb = stablehlo.broadcast_in_dim %l, dims = [1] : ({ct((8,))}) -> {c}\n"
            f"    %0 = stablehlo.multiply %arg0, %k : {c}\n"
            f"    %1 = stablehlo.add %0, %lb : {c}")
    out.append(("complex_constants_and_broadcast", func([c], [c], body, "%1"), [a]))
    tc8 = ct((8, 3))
    body = (f"    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({c}) -> {tc8}\n"
            f"    %1 = stablehlo.slice %0 [2:7:2, 0:3] : ({tc8}) -> {ct((3, 3))}\n"
            f"    %2 = stablehlo.reverse %1, dims = [0] : {ct((3, 3))}\n"
            f"    %3 = stablehlo.concatenate %1, %2, dim = 1 : ({ct((3, 3))}, {ct((3, 3))}) -> {ct((3, 6))}\n"
            f"    %4 = stablehlo.reshape %3 : ({ct((3, 6))}) -> {ct((2, 9))}")
    out.append(("complex_data_movement", func([c], [ct((2, 9))], body, "%4"), [a]))
    ti = tt(shape, "i1")
    body = (f"    %0 = stablehlo.convert %arg1 : ({t}) -> {c}\n"
            f"    %1 = stablehlo.select %arg2, %arg0, %0 : {ti}, {c}")
    out.append(("complex_convert_and_select", func([c, t, ti], [c], body, "%1"), [a, rand(rng, shape, "f32"), rand(rng, shape, "i1")]))
    return out


CASES = (build_cases() + widening_cases() + window_scatter_sort_cases() + convolution_cases() + linalg_cases() + custom_call_cases() + rng_cases()
         + fft_cases() + quantize_cases() + saturating_convert_cases() + special_value_cases() + more_edge_cases() + fused_pattern_edge_cases() + contraction_edge_cases() + window_sort_edge_cases() + shared_intermediate_cases() + random_program_cases() + random_program_cases(count=40, seed=77, dt="i32"))
