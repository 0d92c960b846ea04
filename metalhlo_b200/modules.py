"""StableHLO text builders for the programs this backend is measured and tested on.

The texts follow the forms `jax.jit` prints: unfused softmax / LayerNorm / RMSNorm / tanh-GELU / attention subgraphs
(which the O3 pipeline rewrites to fused custom calls) and whole benchmark modules built from them.
"""
from __future__ import annotations

import math


def tt(shape, dt):
    return "tensor<" + "".join(f"{d}x" for d in shape) + dt + ">"


def func(args, result_types, body, ret):
    sig = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    res = ", ".join(result_types)
    return (f"module @case {{\n  func.func public @main({sig}) -> ({res}) {{\n{body}\n    return {ret} : {res}\n  }}\n}}\n")


def softmax_text(x, t, rt, axis, prefix="s"):
    """Unfused softmax over `axis` the way jax.nn.softmax lowers."""
    dims = [d for d in range(len(t)) if d != axis]
    full, red = tt(t, rt), tt([t[d] for d in dims], rt)
    return (f"    %{prefix}ninf = stablehlo.constant dense<0xFF800000> : tensor<{rt}>\n".replace("0xFF800000", {"f32": "0xFF800000", "f16": "0xFC00", "bf16": "0xFF80"}[rt])
            + f"    %{prefix}0 = stablehlo.reduce({x} init: %{prefix}ninf) applies stablehlo.maximum across dimensions = [{axis}] : ({full}, tensor<{rt}>) -> {red}\n"
            f"    %{prefix}1 = stablehlo.broadcast_in_dim %{prefix}0, dims = {dims} : ({red}) -> {full}\n"
            f"    %{prefix}2 = stablehlo.subtract {x}, %{prefix}1 : {full}\n"
            f"    %{prefix}3 = stablehlo.exponential %{prefix}2 : {full}\n"
            f"    %{prefix}zero = stablehlo.constant dense<0.000000e+00> : tensor<{rt}>\n"
            f"    %{prefix}4 = stablehlo.reduce(%{prefix}3 init: %{prefix}zero) applies stablehlo.add across dimensions = [{axis}] : ({full}, tensor<{rt}>) -> {red}\n"
            f"    %{prefix}5 = stablehlo.broadcast_in_dim %{prefix}4, dims = {dims} : ({red}) -> {full}\n"
            f"    %{prefix}6 = stablehlo.divide %{prefix}3, %{prefix}5 : {full}\n", f"%{prefix}6")


def layer_norm_text(x, shape, dt, gamma=None, beta=None, eps=1e-5, rms=False, prefix="n"):
    """Unfused LayerNorm / RMSNorm over the last axis: mean, centred variance, rsqrt, scale and shift."""
    full, red = tt(shape, dt), tt(shape[:-1], dt)
    dims = list(range(len(shape) - 1))
    n = shape[-1]
    p = prefix
    lines = [f"    %{p}zero = stablehlo.constant dense<0.000000e+00> : tensor<{dt}>",
             f"    %{p}cnt = stablehlo.constant dense<{float(n):e}> : {red}",
             f"    %{p}eps = stablehlo.constant dense<{eps:e}> : {red}"]
    cur = x
    if not rms:
        lines += [f"    %{p}0 = stablehlo.reduce({x} init: %{p}zero) applies stablehlo.add across dimensions = [{len(shape) - 1}] : ({full}, tensor<{dt}>) -> {red}",
                  f"    %{p}1 = stablehlo.divide %{p}0, %{p}cnt : {red}",
                  f"    %{p}2 = stablehlo.broadcast_in_dim %{p}1, dims = {dims} : ({red}) -> {full}",
                  f"    %{p}3 = stablehlo.subtract {x}, %{p}2 : {full}"]
        cur = f"%{p}3"
    lines += [f"    %{p}4 = stablehlo.multiply {cur}, {cur} : {full}",
              f"    %{p}5 = stablehlo.reduce(%{p}4 init: %{p}zero) applies stablehlo.add across dimensions = [{len(shape) - 1}] : ({full}, tensor<{dt}>) -> {red}",
              f"    %{p}6 = stablehlo.divide %{p}5, %{p}cnt : {red}",
              f"    %{p}7 = stablehlo.add %{p}6, %{p}eps : {red}",
              f"    %{p}8 = stablehlo.rsqrt %{p}7 : {red}",
              f"    %{p}9 = stablehlo.broadcast_in_dim %{p}8, dims = {dims} : ({red}) -> {full}",
              f"    %{p}10 = stablehlo.multiply {cur}, %{p}9 : {full}"]
    out = f"%{p}10"
    last = [len(shape) - 1]
    if gamma:
        lines += [f"    %{p}11 = stablehlo.broadcast_in_dim {gamma}, dims = {last} : ({tt((n,), dt)}) -> {full}",
                  f"    %{p}12 = stablehlo.multiply {out}, %{p}11 : {full}"]
        out = f"%{p}12"
    if beta:
        lines += [f"    %{p}13 = stablehlo.broadcast_in_dim {beta}, dims = {last} : ({tt((n,), dt)}) -> {full}",
                  f"    %{p}14 = stablehlo.add {out}, %{p}13 : {full}"]
        out = f"%{p}14"
    return "\n".join(lines) + "\n", out


def gelu_text(x, shape, dt, prefix="g"):
    """tanh-GELU as jax.nn.gelu(approximate=True) lowers: x * 0.5 * (1 + tanh(0.79788 * (x + 0.044715 x^3)))."""
    t = tt(shape, dt)
    p = prefix
    return (f"    %{p}c0 = stablehlo.constant dense<4.471500e-02> : {t}\n"
            f"    %{p}c1 = stablehlo.constant dense<0.797884583> : {t}\n"
            f"    %{p}c2 = stablehlo.constant dense<1.000000e+00> : {t}\n"
            f"    %{p}c3 = stablehlo.constant dense<5.000000e-01> : {t}\n"
            f"    %{p}0 = stablehlo.multiply {x}, {x} : {t}\n"
            f"    %{p}1 = stablehlo.multiply %{p}0, {x} : {t}\n"
            f"    %{p}2 = stablehlo.multiply %{p}c0, %{p}1 : {t}\n"
            f"    %{p}3 = stablehlo.add {x}, %{p}2 : {t}\n"
            f"    %{p}4 = stablehlo.multiply %{p}c1, %{p}3 : {t}\n"
            f"    %{p}5 = stablehlo.tanh %{p}4 : {t}\n"
            f"    %{p}6 = stablehlo.add %{p}c2, %{p}5 : {t}\n"
            f"    %{p}7 = stablehlo.multiply %{p}c3, %{p}6 : {t}\n"
            f"    %{p}8 = stablehlo.multiply {x}, %{p}7 : {t}\n", f"%{p}8")


def attention_text(B, H, S, D, dt, causal, layout="BHSD", scale=None):
    """Unfused attention: QK^T * scale, optional iota-compare causal select, softmax, PV."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if layout == "BHSD":
        qshape, qk_dims, pv_dims, oshape = (B, H, S, D), "batching_dims = [0, 1] x [0, 1], contracting_dims = [3] x [3]", \
            "batching_dims = [0, 1] x [0, 1], contracting_dims = [3] x [2]", (B, H, S, D)
    else:  # BSHD as flax MultiHeadDotProductAttention lays its tensors out
        qshape, qk_dims, pv_dims, oshape = (B, S, H, D), "batching_dims = [0, 2] x [0, 2], contracting_dims = [3] x [3]", \
            "batching_dims = [0, 1] x [0, 2], contracting_dims = [3] x [1]", (B, H, S, D)
    tq, ts = tt(qshape, dt), tt((B, H, S, S), dt)
    body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, {qk_dims} : ({tq}, {tq}) -> {ts}\n"
            f"    %sc = stablehlo.constant dense<{scale:e}> : {ts}\n"
            f"    %1 = stablehlo.multiply %0, %sc : {ts}\n")
    cur = "%1"
    if causal:
        ti, tb = tt((S, S), "i32"), tt((S, S), "i1")
        neg = {"f32": "-1.000000e+09", "f16": "-6.000000e+04", "bf16": "-1.000000e+09"}[dt]
        body += (f"    %iq = stablehlo.iota dim = 0 : {ti}\n    %ik = stablehlo.iota dim = 1 : {ti}\n"
                 f"    %m = stablehlo.compare  GE, %iq, %ik,  SIGNED : ({ti}, {ti}) -> {tb}\n"
                 f"    %mb = stablehlo.broadcast_in_dim %m, dims = [2, 3] : ({tb}) -> {tt((B, H, S, S), 'i1')}\n"
                 f"    %neg = stablehlo.constant dense<{neg}> : {ts}\n"
                 f"    %2 = stablehlo.select %mb, %1, %neg : {tt((B, H, S, S), 'i1')}, {ts}\n")
        cur = "%2"
    sm, p = softmax_text(cur, (B, H, S, S), dt, 3)
    body += sm
    body += f"    %out = stablehlo.dot_general {p}, %arg2, {pv_dims} : ({ts}, {tq}) -> {tt(oshape, dt)}\n"
    return func([tq, tq, tq], [tt(oshape, dt)], body.rstrip("\n"), "%out"), qshape




def norm_sweep_module(rows: int, hidden: int, dt: str = "bf16", eps: float = 1e-5) -> str:
    """LayerNorm(x, gamma, beta), RMSNorm(x, gamma) and softmax(4 * x) over the last axis of x [rows, hidden]."""
    shape = (rows, hidden)
    t, tv = tt(shape, dt), tt((hidden,), dt)
    ln, ln_res = layer_norm_text("%arg0", shape, dt, "%arg1", "%arg2", eps=eps, prefix="a")
    rms, rms_res = layer_norm_text("%arg0", shape, dt, "%arg1", None, eps=eps, rms=True, prefix="b")
    body = ln + rms + f"    %four = stablehlo.constant dense<4.000000e+00> : {t}\n    %x4 = stablehlo.multiply %arg0, %four : {t}\n"
    sm, sm_res = softmax_text("%x4", shape, dt, 1, prefix="c")
    body += sm
    return func([t, tv, tv], [t, t, t], body.rstrip("\n"), f"{ln_res}, {rms_res}, {sm_res}")


def mlp_softmax_module(m: int = 512, k: int = 1024, n: int = 1024, dt: str = "f32") -> str:
    """softmax(gelu_tanh(x . w + b)) over the last axis: the reference-runnable fp32 configuration."""
    tx, tw, tb, to = tt((m, k), dt), tt((k, n), dt), tt((n,), dt), tt((m, n), dt)
    body = (f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : ({tx}, {tw}) -> {to}\n"
            f"    %1 = stablehlo.broadcast_in_dim %arg2, dims = [1] : ({tb}) -> {to}\n"
            f"    %2 = stablehlo.add %0, %1 : {to}\n")
    g, gres = gelu_text("%2", (m, n), dt)
    sm, res = softmax_text(gres, (m, n), dt, 1)
    return func([tx, tw, tb], [to], (body + g + sm).rstrip("\n"), res)
