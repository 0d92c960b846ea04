"""Seeded StableHLO programs that exercise the backend's operator surface one op (or one fusable pattern) at a time.

Each case is (name, module text, list of numpy inputs). The texts are written in the forms `jax.jit` prints (pretty
ops, `dims = [...]`, `contracting_dims = [..] x [..]`, reduce with `applies`) plus the generic `"stablehlo.op"(...)`
form for gather. The GPU tests run every case through the C API at several optimisation levels and compare with the
numpy oracle (oracle/interp.py); the CPU tests run the oracle and the host-side compiler on them.
"""
from __future__ import annotations

import math

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
    for causal in (False, True):
        for layout in ("BHSD", "BSHD"):
            text, qshape = attention_text(2, 3, 48, 32, dt, causal, layout)
            q, k, v = (rand(rng, qshape, dt, -1, 1) for _ in range(3))
            out.append((f"pattern_attention_{layout}_{'causal' if causal else 'full'}_{dt}", text, [q, k, v]))
    return out


CASES = build_cases()
