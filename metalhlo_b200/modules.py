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


def gpt2_module(batch: int = 32, seq: int = 1024, layers: int = 12, d_model: int = 768, heads: int = 12, vocab: int = 50257,
                dt: str = "f16", eps: float = 1e-5):
    """GPT-2 forward pass (pre-LN blocks, tanh-GELU MLP, causal attention, tied output embedding) in the op forms
    `jax.jit` prints. Parameters arrive as fp32 and are converted to `dt` inside the module; token ids are i32.

    Returns (text, parameter list) where the parameter list is [(name, shape, dtype)] in argument order:
    ids, wte, wpe, then per layer ln1_g, ln1_b, w_qkv, b_qkv, w_o, b_o, ln2_g, ln2_b, w_fc, b_fc, w_proj, b_proj,
    then lnf_g, lnf_b. The result is the logits tensor [batch, seq, vocab] in `dt`.
    """
    dh = d_model // heads
    params = [("ids", (batch, seq), "i32"), ("wte", (vocab, d_model), "f32"), ("wpe", (seq, d_model), "f32")]
    for i in range(layers):
        params += [(f"l{i}.ln1_g", (d_model,), "f32"), (f"l{i}.ln1_b", (d_model,), "f32"),
                   (f"l{i}.w_qkv", (d_model, 3 * d_model), "f32"), (f"l{i}.b_qkv", (3 * d_model,), "f32"),
                   (f"l{i}.w_o", (d_model, d_model), "f32"), (f"l{i}.b_o", (d_model,), "f32"),
                   (f"l{i}.ln2_g", (d_model,), "f32"), (f"l{i}.ln2_b", (d_model,), "f32"),
                   (f"l{i}.w_fc", (d_model, 4 * d_model), "f32"), (f"l{i}.b_fc", (4 * d_model,), "f32"),
                   (f"l{i}.w_proj", (4 * d_model, d_model), "f32"), (f"l{i}.b_proj", (d_model,), "f32")]
    params += [("lnf_g", (d_model,), "f32"), ("lnf_b", (d_model,), "f32")]
    arg = {name: f"%arg{i}" for i, (name, _, _) in enumerate(params)}
    lines = []
    counter = [0]

    def fresh(tag="t"):
        counter[0] += 1
        return f"%{tag}{counter[0]}"

    def emit(line):
        lines.append("    " + line)

    def cvt(name, shape):
        v = fresh("p")
        emit(f"{v} = stablehlo.convert {arg[name]} : ({tt(shape, 'f32')}) -> {tt(shape, dt)}")
        return v

    act = (batch, seq, d_model)
    t_act = tt(act, dt)

    def dense(x, xshape, w, wshape, b):
        oshape = xshape[:-1] + (wshape[1],)
        y, bb, o = fresh(), fresh(), fresh()
        emit(f"{y} = stablehlo.dot_general {x}, {w}, contracting_dims = [{len(xshape) - 1}] x [0] : ({tt(xshape, dt)}, {tt(wshape, dt)}) -> {tt(oshape, dt)}")
        emit(f"{bb} = stablehlo.broadcast_in_dim {b}, dims = [{len(oshape) - 1}] : ({tt((wshape[1],), dt)}) -> {tt(oshape, dt)}")
        emit(f"{o} = stablehlo.add {y}, {bb} : {tt(oshape, dt)}")
        return o, oshape

    def layer_norm(x, g, b, prefix):
        body, res = layer_norm_text(x, act, dt, g, b, eps=eps, prefix=prefix)
        lines.extend(body.rstrip("\n").split("\n"))
        return res

    # embeddings
    wte = cvt("wte", (vocab, d_model))
    wpe = cvt("wpe", (seq, d_model))
    idx, tok, pos, x = fresh(), fresh(), fresh(), fresh()
    emit(f"{idx} = stablehlo.reshape {arg['ids']} : ({tt((batch, seq), 'i32')}) -> {tt((batch, seq, 1), 'i32')}")
    emit(f"{tok} = \"stablehlo.gather\"({wte}, {idx}) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], collapsed_slice_dims = [0], "
         f"start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1, {d_model}>}}> : "
         f"({tt((vocab, d_model), dt)}, {tt((batch, seq, 1), 'i32')}) -> {t_act}")
    emit(f"{pos} = stablehlo.broadcast_in_dim {wpe}, dims = [1, 2] : ({tt((seq, d_model), dt)}) -> {t_act}")
    emit(f"{x} = stablehlo.add {tok}, {pos} : {t_act}")
    # causal predicate shared by all layers
    ti, tb = tt((seq, seq), "i32"), tt((seq, seq), "i1")
    ts = tt((batch, heads, seq, seq), dt)
    emit(f"%iq = stablehlo.iota dim = 0 : {ti}")
    emit(f"%ik = stablehlo.iota dim = 1 : {ti}")
    emit(f"%causal = stablehlo.compare  GE, %iq, %ik,  SIGNED : ({ti}, {ti}) -> {tb}")
    emit(f"%causalb = stablehlo.broadcast_in_dim %causal, dims = [2, 3] : ({tb}) -> {tt((batch, heads, seq, seq), 'i1')}")
    neg = "-6.000000e+04" if dt == "f16" else "-1.000000e+09"
    emit(f"%neg = stablehlo.constant dense<{neg}> : {ts}")
    emit(f"%scale = stablehlo.constant dense<{1.0 / math.sqrt(dh):e}> : {ts}")
    t_heads = tt((batch, seq, heads, dh), dt)
    for i in range(layers):
        p = {k: cvt(f"l{i}.{k}", s) for k, s in [("ln1_g", (d_model,)), ("ln1_b", (d_model,)), ("w_qkv", (d_model, 3 * d_model)),
                                                   ("b_qkv", (3 * d_model,)), ("w_o", (d_model, d_model)), ("b_o", (d_model,)),
                                                   ("ln2_g", (d_model,)), ("ln2_b", (d_model,)), ("w_fc", (d_model, 4 * d_model)),
                                                   ("b_fc", (4 * d_model,)), ("w_proj", (4 * d_model, d_model)), ("b_proj", (d_model,))]}
        hn = layer_norm(x, p["ln1_g"], p["ln1_b"], f"a{i}n")
        qkv, qkv_shape = dense(hn, act, p["w_qkv"], (d_model, 3 * d_model), p["b_qkv"])
        parts = []
        for k in range(3):
            sl, rs = fresh(), fresh()
            emit(f"{sl} = stablehlo.slice {qkv} [0:{batch}, 0:{seq}, {k * d_model}:{(k + 1) * d_model}] : ({tt(qkv_shape, dt)}) -> {t_act}")
            emit(f"{rs} = stablehlo.reshape {sl} : ({t_act}) -> {t_heads}")
            parts.append(rs)
        q, k_, v = parts
        s0, s1, s2 = fresh(), fresh(), fresh()
        emit(f"{s0} = stablehlo.dot_general {q}, {k_}, batching_dims = [0, 2] x [0, 2], contracting_dims = [3] x [3] : ({t_heads}, {t_heads}) -> {ts}")
        emit(f"{s1} = stablehlo.multiply {s0}, %scale : {ts}")
        emit(f"{s2} = stablehlo.select %causalb, {s1}, %neg : {tt((batch, heads, seq, seq), 'i1')}, {ts}")
        sm, pr = softmax_text(s2, (batch, heads, seq, seq), dt, 3, prefix=f"a{i}s")
        lines.extend(sm.rstrip("\n").split("\n"))
        o0, o1, o2 = fresh(), fresh(), fresh()
        emit(f"{o0} = stablehlo.dot_general {pr}, {v}, batching_dims = [0, 1] x [0, 2], contracting_dims = [3] x [1] : ({ts}, {t_heads}) -> {tt((batch, heads, seq, dh), dt)}")
        emit(f"{o1} = stablehlo.transpose {o0}, dims = [0, 2, 1, 3] : ({tt((batch, heads, seq, dh), dt)}) -> {t_heads}")
        emit(f"{o2} = stablehlo.reshape {o1} : ({t_heads}) -> {t_act}")
        ao, _ = dense(o2, act, p["w_o"], (d_model, d_model), p["b_o"])
        x1 = fresh()
        emit(f"{x1} = stablehlo.add {x}, {ao} : {t_act}")
        hn2 = layer_norm(x1, p["ln2_g"], p["ln2_b"], f"m{i}n")
        fc, fc_shape = dense(hn2, act, p["w_fc"], (d_model, 4 * d_model), p["b_fc"])
        gl, gres = gelu_text(fc, fc_shape, dt, prefix=f"m{i}g")
        lines.extend(gl.rstrip("\n").split("\n"))
        pj, _ = dense(gres, fc_shape, p["w_proj"], (4 * d_model, d_model), p["b_proj"])
        x2 = fresh()
        emit(f"{x2} = stablehlo.add {x1}, {pj} : {t_act}")
        x = x2
    g, b = cvt("lnf_g", (d_model,)), cvt("lnf_b", (d_model,))
    xf = layer_norm(x, g, b, "fn")
    logits = fresh("logits")
    t_logits = tt((batch, seq, vocab), dt)
    emit(f"{logits} = stablehlo.dot_general {xf}, {wte}, contracting_dims = [2] x [1] : ({t_act}, {tt((vocab, d_model), dt)}) -> {t_logits}")
    text = func([tt(s, d) for _, s, d in params], [t_logits], "\n".join(lines), logits)
    return text, params


def cnn_module(batch: int = 8, size: int = 32, channels: int = 3, width: int = 32, classes: int = 10, dt: str = "bf16", eps: float = 1e-5):
    """A small residual CNN forward pass in the op forms `jax.jit` prints for a flax model (NHWC, HWIO): 3x3 stem
    convolution with stride 2, one residual block of two 3x3 convolutions with batch-norm inference and ReLU, 2x2 max
    pooling (reduce_window), global average pooling (reduce) and a dense classifier. Parameters arrive as fp32 and are
    converted to `dt` inside the module.

    Returns (text, parameter list [(name, shape, dtype)] in argument order); the result is [batch, classes] logits in `dt`.
    """
    half = size // 2
    params = [("image", (batch, size, size, channels), "f32"), ("stem_w", (3, 3, channels, width), "f32")]
    for i in (1, 2):
        params += [(f"conv{i}_w", (3, 3, width, width), "f32"), (f"bn{i}_scale", (width,), "f32"), (f"bn{i}_offset", (width,), "f32"),
                   (f"bn{i}_mean", (width,), "f32"), (f"bn{i}_var", (width,), "f32")]
    params += [("dense_w", (width, classes), "f32"), ("dense_b", (classes,), "f32")]
    arg = {name: f"%arg{i}" for i, (name, _, _) in enumerate(params)}
    shape = {name: s for name, s, _ in params}
    lines = []
    n = [0]

    def fresh():
        n[0] += 1
        return f"%c{n[0]}"

    def emit(line):
        lines.append("    " + line)

    def cvt(name):
        if dt == "f32":
            return arg[name]
        v = fresh()
        emit(f"{v} = stablehlo.convert {arg[name]} : ({tt(shape[name], 'f32')}) -> {tt(shape[name], dt)}")
        return v

    def conv(x, xs, w, ws, stride, out_hw):
        v = fresh()
        os_ = (xs[0], out_hw, out_hw, ws[3])
        pad = "[[0, 1], [0, 1]]" if stride == 2 else "[[1, 1], [1, 1]]"
        emit(f"{v} = stablehlo.convolution({x}, {w}) dim_numbers = [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f], "
             f"window = {{stride = [{stride}, {stride}], pad = {pad}}} {{batch_group_count = 1 : i64, feature_group_count = 1 : i64}} "
             f": ({tt(xs, dt)}, {tt(ws, dt)}) -> {tt(os_, dt)}")
        return v, os_

    def bn(x, xs, i):
        v = fresh()
        stats = ", ".join(cvt(f"bn{i}_{k}") for k in ("scale", "offset", "mean", "var"))
        tc = tt((xs[3],), dt)
        emit(f"{v} = \"stablehlo.batch_norm_inference\"({x}, {stats}) <{{epsilon = {eps:e} : f32, feature_index = 3 : i64}}> "
             f": ({tt(xs, dt)}, {tc}, {tc}, {tc}, {tc}) -> {tt(xs, dt)}")
        return v

    def relu(x, xs):
        z, b, v = fresh(), fresh(), fresh()
        emit(f"{z} = stablehlo.constant dense<0.000000e+00> : tensor<{dt}>")
        emit(f"{b} = stablehlo.broadcast_in_dim {z}, dims = [] : (tensor<{dt}>) -> {tt(xs, dt)}")
        emit(f"{v} = stablehlo.maximum {x}, {b} : {tt(xs, dt)}")
        return v

    x, xs = cvt("image"), shape["image"]
    x, xs = conv(x, xs, cvt("stem_w"), shape["stem_w"], 2, half)
    x = relu(x, xs)
    skip = x
    for i in (1, 2):
        x, xs = conv(x, xs, cvt(f"conv{i}_w"), shape[f"conv{i}_w"], 1, half)
        x = bn(x, xs, i)
        if i == 2:
            s = fresh()
            emit(f"{s} = stablehlo.add {x}, {skip} : {tt(xs, dt)}")
            x = s
        x = relu(x, xs)
    ninf = {"f32": "0xFF800000", "f16": "0xFC00", "bf16": "0xFF80"}[dt]
    init, pooled = fresh(), fresh()
    ps = (xs[0], half // 2, half // 2, xs[3])
    emit(f"{init} = stablehlo.constant dense<{ninf}> : tensor<{dt}>")
    emit(f"{pooled} = \"stablehlo.reduce_window\"({x}, {init}) <{{window_dimensions = array<i64: 1, 2, 2, 1>, window_strides = array<i64: 1, 2, 2, 1>}}> ({{")
    emit(f"^bb0(%a: tensor<{dt}>, %b: tensor<{dt}>):")
    emit(f"  %m = stablehlo.maximum %a, %b : tensor<{dt}>")
    emit(f"  stablehlo.return %m : tensor<{dt}>")
    emit(f"}}) : ({tt(xs, dt)}, tensor<{dt}>) -> {tt(ps, dt)}")
    zero, summed, cnt, cb, mean = fresh(), fresh(), fresh(), fresh(), fresh()
    fs = (ps[0], ps[3])
    emit(f"{zero} = stablehlo.constant dense<0.000000e+00> : tensor<{dt}>")
    emit(f"{summed} = stablehlo.reduce({pooled} init: {zero}) applies stablehlo.add across dimensions = [1, 2] : ({tt(ps, dt)}, tensor<{dt}>) -> {tt(fs, dt)}")
    emit(f"{cnt} = stablehlo.constant dense<{float(ps[1] * ps[2]):e}> : tensor<{dt}>")
    emit(f"{cb} = stablehlo.broadcast_in_dim {cnt}, dims = [] : (tensor<{dt}>) -> {tt(fs, dt)}")
    emit(f"{mean} = stablehlo.divide {summed}, {cb} : {tt(fs, dt)}")
    logits, bb, res = fresh(), fresh(), fresh()
    ls = (fs[0], classes)
    emit(f"{logits} = stablehlo.dot_general {mean}, {cvt('dense_w')}, contracting_dims = [1] x [0] : ({tt(fs, dt)}, {tt(shape['dense_w'], dt)}) -> {tt(ls, dt)}")
    emit(f"{bb} = stablehlo.broadcast_in_dim {cvt('dense_b')}, dims = [1] : ({tt((classes,), dt)}) -> {tt(ls, dt)}")
    emit(f"{res} = stablehlo.add {logits}, {bb} : {tt(ls, dt)}")
    sig = ", ".join(f"%arg{i}: {tt(s, d)}" for i, (_, s, d) in enumerate(params))
    text = (f"module @jit_cnn {{\n  func.func public @main({sig}) -> ({tt(ls, dt)}) {{\n" + "\n".join(lines) +
            f"\n    return {res} : {tt(ls, dt)}\n  }}\n}}\n")
    return text, params
