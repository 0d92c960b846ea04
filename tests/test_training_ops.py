"""Training-shaped programs: the operator forms and known answers of the reference's training tests
(Tests/MetalHLOTests/TrainingOpsTests.swift:14-677: batched and transposed dot_general, reductions, comparisons, select,
clamp, the hand-written backward passes of a linear layer and of ReLU) and a whole forward + backward step of a two-layer
MLP with an embedding table, whose gradients are checked against torch autograd in fp64. The CPU tests pin the oracle to
the known answers; the GPU tests run the same modules through the C API at every optimisation level."""
import numpy as np
import pytest

from oracle import interp

F = np.float32

BATCHED = """
module @batched_matmul {
  func.func @main(%lhs: tensor<2x3x4xf32>, %rhs: tensor<2x4x5xf32>) -> (tensor<2x3x5xf32>) {
    %0 = stablehlo.dot_general %lhs, %rhs, #stablehlo.dot<lhs_batching_dimensions = [0], rhs_batching_dimensions = [0], lhs_contracting_dimensions = [2], rhs_contracting_dimensions = [1]> : (tensor<2x3x4xf32>, tensor<2x4x5xf32>) -> tensor<2x3x5xf32>
    return %0 : tensor<2x3x5xf32>
  }
}
"""
GRAD_W = """
module @linear_grad_w {
  func.func @main(%x: tensor<2x3xf32>, %grad_y: tensor<2x4xf32>) -> (tensor<3x4xf32>) {
    // dL/dW = x^T @ dL/dy
    %x_t = stablehlo.transpose %x, dims = [1, 0] : (tensor<2x3xf32>) -> tensor<3x2xf32>
    %grad_w = stablehlo.dot %x_t, %grad_y : (tensor<3x2xf32>, tensor<2x4xf32>) -> tensor<3x4xf32>
    return %grad_w : tensor<3x4xf32>
  }
}
"""
GRAD_X = """
module @linear_grad_x {
  func.func @main(%W: tensor<3x4xf32>, %grad_y: tensor<2x4xf32>) -> (tensor<2x3xf32>) {
    %w_t = stablehlo.transpose %W, dims = [1, 0] : (tensor<3x4xf32>) -> tensor<4x3xf32>
    %grad_x = stablehlo.dot %grad_y, %w_t : (tensor<2x4xf32>, tensor<4x3xf32>) -> tensor<2x3xf32>
    return %grad_x : tensor<2x3xf32>
  }
}
"""
RELU_BACKWARD = """
module @relu_backward {
  func.func @main(%x: tensor<6xf32>, %grad_y: tensor<6xf32>) -> (tensor<6xf32>) {
    %zero = stablehlo.constant dense<0.0> : tensor<6xf32>
    %mask = stablehlo.compare %x, %zero, GT : (tensor<6xf32>, tensor<6xf32>) -> tensor<6xi1>
    %grad_x = stablehlo.select %mask, %grad_y, %zero : (tensor<6xi1>, tensor<6xf32>, tensor<6xf32>) -> tensor<6xf32>
    return %grad_x : tensor<6xf32>
  }
}
"""
LINEAR_FULL = """
module @linear_full_backward {
  func.func @main(%x: tensor<2x3xf32>, %W: tensor<3x4xf32>, %b: tensor<4xf32>) -> (tensor<3x4xf32>, tensor<4xf32>, tensor<2x3xf32>) {
    // forward: y = relu(x @ W + b)
    %matmul = stablehlo.dot %x, %W : (tensor<2x3xf32>, tensor<3x4xf32>) -> tensor<2x4xf32>
    %b_broadcast = stablehlo.broadcast_in_dim %b, dims = [1] : (tensor<4xf32>) -> tensor<2x4xf32>
    %pre_relu = stablehlo.add %matmul, %b_broadcast : tensor<2x4xf32>
    %zero = stablehlo.constant dense<0.0> : tensor<2x4xf32>
    %y = stablehlo.maximum %pre_relu, %zero : tensor<2x4xf32>
    // backward with dL/dy = ones
    %ones = stablehlo.constant dense<1.0> : tensor<2x4xf32>
    %relu_mask = stablehlo.compare %pre_relu, %zero, GT : (tensor<2x4xf32>, tensor<2x4xf32>) -> tensor<2x4xi1>
    %zero_grad = stablehlo.constant dense<0.0> : tensor<2x4xf32>
    %grad_pre_relu = stablehlo.select %relu_mask, %ones, %zero_grad : (tensor<2x4xi1>, tensor<2x4xf32>, tensor<2x4xf32>) -> tensor<2x4xf32>
    %init = stablehlo.constant dense<0.0> : tensor<f32>
    %grad_b = stablehlo.reduce %grad_pre_relu, %init applies stablehlo.add across dimensions = [0] : (tensor<2x4xf32>, tensor<f32>) -> tensor<4xf32>
    %x_t = stablehlo.transpose %x, dims = [1, 0] : (tensor<2x3xf32>) -> tensor<3x2xf32>
    %grad_W = stablehlo.dot %x_t, %grad_pre_relu : (tensor<3x2xf32>, tensor<2x4xf32>) -> tensor<3x4xf32>
    %W_t = stablehlo.transpose %W, dims = [1, 0] : (tensor<3x4xf32>) -> tensor<4x3xf32>
    %grad_x = stablehlo.dot %grad_pre_relu, %W_t : (tensor<2x4xf32>, tensor<4x3xf32>) -> tensor<2x3xf32>
    return %grad_W, %grad_b, %grad_x : tensor<3x4xf32>, tensor<4xf32>, tensor<2x3xf32>
  }
}
"""


def unary_module(body, in_types, out_type):
    args = ", ".join(f"%a{i}: {t}" for i, t in enumerate(in_types))
    return f"module @m {{\n  func.func @main({args}) -> ({out_type}) {{\n    {body}\n    return %0 : {out_type}\n  }}\n}}\n"


# name -> (module text, inputs, expected outputs): the reference's cases with their known answers
def known_answer_cases():
    eye34 = np.eye(3, 4, dtype=F)
    lhs = np.stack([eye34, np.array([[1] * 4, [2] * 4, [3] * 4], F)])
    rhs1 = np.ones((4, 5), F)
    rhs1[:, 4] = 0
    rhs = np.stack([np.eye(4, 5, dtype=F), rhs1])
    batched_want = np.stack([np.eye(3, 5, dtype=F), np.array([[4, 4, 4, 4, 0], [8, 8, 8, 8, 0], [12, 12, 12, 12, 0]], F)])
    x23 = np.array([[1, 2, 3], [4, 5, 6]], F)
    m234 = np.arange(24, dtype=F).reshape(2, 3, 4)
    cmp_a, cmp_b = np.array([1, 2, 3, 4], F), np.array([1, 3, 2, 4], F)
    cases = {
        "batched_dot_general": (BATCHED, [lhs, rhs], [batched_want]),
        "contract_first_dims": (unary_module("%0 = stablehlo.dot_general %a0, %a1, contracting_dims = [0] x [0] : (tensor<3x2xf32>, tensor<3x4xf32>) -> tensor<2x4xf32>",
                                             ["tensor<3x2xf32>", "tensor<3x4xf32>"], "tensor<2x4xf32>"),
                                [x23.T.copy(), np.arange(12, dtype=F).reshape(3, 4)], [x23 @ np.arange(12, dtype=F).reshape(3, 4)]),
        "reduce_sum_axis": (unary_module("%z = stablehlo.constant dense<0.0> : tensor<f32>\n    %0 = stablehlo.reduce(%a0 init: %z) applies stablehlo.add across dimensions = [1] : (tensor<2x3xf32>, tensor<f32>) -> tensor<2xf32>",
                                         ["tensor<2x3xf32>"], "tensor<2xf32>"), [x23], [np.array([6, 15], F)]),
        "reduce_max_axis": (unary_module("%z = stablehlo.constant dense<0xFF800000> : tensor<f32>\n    %0 = stablehlo.reduce(%a0 init: %z) applies stablehlo.maximum across dimensions = [0] : (tensor<2x3xf32>, tensor<f32>) -> tensor<3xf32>",
                                         ["tensor<2x3xf32>"], "tensor<3xf32>"), [x23], [np.array([4, 5, 6], F)]),
        "reduce_min_axis": (unary_module("%z = stablehlo.constant dense<0x7F800000> : tensor<f32>\n    %0 = stablehlo.reduce(%a0 init: %z) applies stablehlo.minimum across dimensions = [1] : (tensor<2x3xf32>, tensor<f32>) -> tensor<2xf32>",
                                         ["tensor<2x3xf32>"], "tensor<2xf32>"), [x23], [np.array([1, 4], F)]),
        "reduce_sum_two_axes": (unary_module("%z = stablehlo.constant dense<0.0> : tensor<f32>\n    %0 = stablehlo.reduce(%a0 init: %z) applies stablehlo.add across dimensions = [0, 2] : (tensor<2x3x4xf32>, tensor<f32>) -> tensor<3xf32>",
                                             ["tensor<2x3x4xf32>"], "tensor<3xf32>"), [m234], [m234.sum(axis=(0, 2))]),
        "select_predicate": (unary_module("%0 = stablehlo.select %a0, %a1, %a2 : (tensor<4xi1>, tensor<4xf32>, tensor<4xf32>) -> tensor<4xf32>",
                                          ["tensor<4xi1>", "tensor<4xf32>", "tensor<4xf32>"], "tensor<4xf32>"),
                             [np.array([True, False, True, False]), np.array([1, 2, 3, 4], F), np.array([10, 20, 30, 40], F)], [np.array([1, 20, 3, 40], F)]),
        "clamp_tensor_bounds": (unary_module("%lo = stablehlo.constant dense<0.0> : tensor<6xf32>\n    %hi = stablehlo.constant dense<1.0> : tensor<6xf32>\n    %0 = stablehlo.clamp %lo, %a0, %hi : tensor<6xf32>",
                                             ["tensor<6xf32>"], "tensor<6xf32>"), [np.array([-1, 0, 0.5, 1, 1.5, 2], F)], [np.array([0, 0, 0.5, 1, 1, 1], F)]),
        "clamp_scalar_bounds": (unary_module("%lo = stablehlo.constant dense<-1.0> : tensor<f32>\n    %hi = stablehlo.constant dense<1.0> : tensor<f32>\n    %0 = stablehlo.clamp %lo, %a0, %hi : (tensor<f32>, tensor<4xf32>, tensor<f32>) -> tensor<4xf32>",
                                             ["tensor<4xf32>"], "tensor<4xf32>"), [np.array([-5, -0.5, 0.5, 5], F)], [np.array([-1, -0.5, 0.5, 1], F)]),
        "grad_w": (GRAD_W, [x23, np.ones((2, 4), F)], [np.array([[5] * 4, [7] * 4, [9] * 4], F)]),
        "grad_x": (GRAD_X, [eye34, np.ones((2, 4), F)], [np.ones((2, 3), F)]),
        "relu_backward": (RELU_BACKWARD, [np.array([-2, -1, 0, 1, 2, 3], F), np.ones(6, F)], [np.array([0, 0, 0, 1, 1, 1], F)]),
        "linear_full_backward": (LINEAR_FULL, [np.array([[1, 0, 0], [0, 1, 0]], F), eye34, np.array([-0.5, 0.5, -0.5, 0.5], F)],
                                 [np.array([[1, 1, 0, 1], [0, 1, 0, 1], [0, 0, 0, 0]], F), np.array([1, 2, 0, 2], F), np.array([[1, 1, 0], [0, 1, 0]], F)]),
    }
    for direction, fn in (("EQ", np.equal), ("NE", np.not_equal), ("LT", np.less), ("LE", np.less_equal), ("GT", np.greater), ("GE", np.greater_equal)):
        body = f"%0 = stablehlo.compare %a0, %a1, {direction} : (tensor<4xf32>, tensor<4xf32>) -> tensor<4xi1>"
        cases[f"compare_{direction}"] = (unary_module(body, ["tensor<4xf32>", "tensor<4xf32>"], "tensor<4xi1>"), [cmp_a, cmp_b], [fn(cmp_a, cmp_b)])
    return cases


CASES = known_answer_cases()


def mlp_step_module(batch=16, vocab=29, d=8, hidden=12, out=5):
    """Forward and backward of: h0 = table[ids]; h1 = relu(h0 . W1 + b1); y = h1 . W2 + b2; loss = mean((y - t)^2). Returns the
    loss and the gradients of W1, b1, W2, b2 and of the embedding table (a scatter-add of the rows' gradients)."""
    t = lambda *s: "tensor<" + "x".join(map(str, s)) + "xf32>"  # noqa: E731
    n = float(batch * out)
    return f"""
module @mlp_step {{
  func.func @main(%ids: tensor<{batch}xi32>, %table: {t(vocab, d)}, %w1: {t(d, hidden)}, %b1: {t(hidden)}, %w2: {t(hidden, out)}, %b2: {t(out)}, %target: {t(batch, out)})
      -> (tensor<f32>, {t(d, hidden)}, {t(hidden)}, {t(hidden, out)}, {t(out)}, {t(vocab, d)}) {{
    %idx = stablehlo.reshape %ids : (tensor<{batch}xi32>) -> tensor<{batch}x1xi32>
    %h0 = "stablehlo.gather"(%table, %idx) <{{dimension_numbers = #stablehlo.gather<offset_dims = [1], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 1>, slice_sizes = array<i64: 1, {d}>}}> : ({t(vocab, d)}, tensor<{batch}x1xi32>) -> {t(batch, d)}
    %z1 = stablehlo.dot_general %h0, %w1, contracting_dims = [1] x [0] : ({t(batch, d)}, {t(d, hidden)}) -> {t(batch, hidden)}
    %b1b = stablehlo.broadcast_in_dim %b1, dims = [1] : ({t(hidden)}) -> {t(batch, hidden)}
    %a1 = stablehlo.add %z1, %b1b : {t(batch, hidden)}
    %zero_h = stablehlo.constant dense<0.0> : {t(batch, hidden)}
    %h1 = stablehlo.maximum %a1, %zero_h : {t(batch, hidden)}
    %z2 = stablehlo.dot_general %h1, %w2, contracting_dims = [1] x [0] : ({t(batch, hidden)}, {t(hidden, out)}) -> {t(batch, out)}
    %b2b = stablehlo.broadcast_in_dim %b2, dims = [1] : ({t(out)}) -> {t(batch, out)}
    %y = stablehlo.add %z2, %b2b : {t(batch, out)}
    %diff = stablehlo.subtract %y, %target : {t(batch, out)}
    %sq = stablehlo.multiply %diff, %diff : {t(batch, out)}
    %zero = stablehlo.constant dense<0.0> : tensor<f32>
    %sum = stablehlo.reduce(%sq init: %zero) applies stablehlo.add across dimensions = [0, 1] : ({t(batch, out)}, tensor<f32>) -> tensor<f32>
    %count = stablehlo.constant dense<{n}> : tensor<f32>
    %loss = stablehlo.divide %sum, %count : tensor<f32>
    // backward
    %two_over_n = stablehlo.constant dense<{2.0 / n}> : {t(batch, out)}
    %gy = stablehlo.multiply %diff, %two_over_n : {t(batch, out)}
    %gw2 = stablehlo.dot_general %h1, %gy, contracting_dims = [0] x [0] : ({t(batch, hidden)}, {t(batch, out)}) -> {t(hidden, out)}
    %gb2 = stablehlo.reduce(%gy init: %zero) applies stablehlo.add across dimensions = [0] : ({t(batch, out)}, tensor<f32>) -> {t(out)}
    %gh1 = stablehlo.dot_general %gy, %w2, contracting_dims = [1] x [1] : ({t(batch, out)}, {t(hidden, out)}) -> {t(batch, hidden)}
    %mask = stablehlo.compare GT, %a1, %zero_h, FLOAT : ({t(batch, hidden)}, {t(batch, hidden)}) -> tensor<{batch}x{hidden}xi1>
    %ga1 = stablehlo.select %mask, %gh1, %zero_h : tensor<{batch}x{hidden}xi1>, {t(batch, hidden)}
    %gw1 = stablehlo.dot_general %h0, %ga1, contracting_dims = [0] x [0] : ({t(batch, d)}, {t(batch, hidden)}) -> {t(d, hidden)}
    %gb1 = stablehlo.reduce(%ga1 init: %zero) applies stablehlo.add across dimensions = [0] : ({t(batch, hidden)}, tensor<f32>) -> {t(hidden)}
    %gh0 = stablehlo.dot_general %ga1, %w1, contracting_dims = [1] x [1] : ({t(batch, hidden)}, {t(d, hidden)}) -> {t(batch, d)}
    %zero_table = stablehlo.constant dense<0.0> : {t(vocab, d)}
    %gtable = "stablehlo.scatter"(%zero_table, %idx, %gh0) <{{indices_are_sorted = false, scatter_dimension_numbers = #stablehlo.scatter<update_window_dims = [1], inserted_window_dims = [0], scatter_dims_to_operand_dims = [0], index_vector_dim = 1>, unique_indices = false}}> ({{
    ^bb0(%p: tensor<f32>, %q: tensor<f32>):
      %s = stablehlo.add %p, %q : tensor<f32>
      stablehlo.return %s : tensor<f32>
    }}) : ({t(vocab, d)}, tensor<{batch}x1xi32>, {t(batch, d)}) -> {t(vocab, d)}
    return %loss, %gw1, %gb1, %gw2, %gb2, %gtable : tensor<f32>, {t(d, hidden)}, {t(hidden)}, {t(hidden, out)}, {t(out)}, {t(vocab, d)}
  }}
}}
"""


def mlp_step_inputs(batch=16, vocab=29, d=8, hidden=12, out=5, seed=3):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=batch).astype(np.int32)
    ids[:4] = ids[0]  # repeated rows: their gradients must add up in the table
    return [ids, rng.standard_normal((vocab, d)).astype(F), (rng.standard_normal((d, hidden)) / np.sqrt(d)).astype(F), (0.1 * rng.standard_normal(hidden)).astype(F),
            (rng.standard_normal((hidden, out)) / np.sqrt(hidden)).astype(F), (0.1 * rng.standard_normal(out)).astype(F), rng.standard_normal((batch, out)).astype(F)]


def autograd_reference(ins):
    import torch

    ids = torch.from_numpy(ins[0]).long()
    table, w1, b1, w2, b2 = (torch.from_numpy(a).double().requires_grad_() for a in ins[1:6])
    target = torch.from_numpy(ins[6]).double()
    h1 = torch.relu(table[ids] @ w1 + b1)
    loss = ((h1 @ w2 + b2 - target) ** 2).mean()
    loss.backward()
    return [loss.detach().numpy(), w1.grad.numpy(), b1.grad.numpy(), w2.grad.numpy(), b2.grad.numpy(), table.grad.numpy()]


# ---- CPU: the oracle against the known answers and against autograd ----

@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_the_known_answers(name):
    text, ins, want = CASES[name]
    got = interp.evaluate(text, ins)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(np.asarray(g, dtype=np.float64), np.asarray(w, dtype=np.float64), err_msg=name)


def test_oracle_gradients_equal_autograd():
    ins = mlp_step_inputs()
    got = interp.evaluate(mlp_step_module(), ins)
    for g, w, name in zip(got, autograd_reference(ins), ["loss", "gw1", "gb1", "gw2", "gb2", "gtable"]):
        np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-6, err_msg=name)  # the module rounds its two constants to fp32


# ---- GPU: the same programs through the C API at every level ----

@pytest.mark.gpu
@pytest.mark.parametrize("level", [0, 1, 2, 3])
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_path_reproduces_the_known_answers(name, level):
    from metalhlo_b200 import capi

    text, ins, want = CASES[name]
    got = capi.Client().run(text, ins, opt_level=level)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.shape == w.shape
        if w.dtype == np.bool_:
            np.testing.assert_array_equal(g, w, err_msg=name)
        else:
            np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-6, err_msg=name)


@pytest.mark.gpu
@pytest.mark.parametrize("level", [0, 2, 3])
def test_cuda_gradients_equal_autograd_and_the_oracle(level):
    from metalhlo_b200 import capi
    from parity import assert_close

    for sizes in (dict(), dict(batch=256, vocab=1031, d=64, hidden=256, out=32)):
        ins = mlp_step_inputs(**sizes)
        text = mlp_step_module(**sizes)
        got = capi.Client().run(text, ins, opt_level=level)
        want = interp.evaluate(text, ins)
        auto = autograd_reference(ins)
        for g, w, a, name in zip(got, want, auto, ["loss", "gw1", "gb1", "gw2", "gb2", "gtable"]):
            assert_close(g.astype(np.float64), w, 1e-5, f"{name} O{level} vs oracle")
            np.testing.assert_allclose(g, a, rtol=1e-4, atol=1e-6 * max(1.0, float(np.abs(a).max())), err_msg=f"{name} O{level} vs autograd")
