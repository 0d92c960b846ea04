"""Batch sharding on the host: the split-axis propagation accepts the programs whose shards are independent (the GPT-2
forward pass, the norm sweep, attention, a batched product, a CNN), the rewritten shard functions evaluated by the numpy
oracle on the input shards concatenate to exactly the unsharded result, and programs that mix elements along the batch
are refused with the operator named. No GPU is needed: mhlo_b200_shard_text runs the analysis and the rewrite alone."""
import numpy as np
import pytest

from metalhlo_b200 import capi, modules
from oracle import interp


def split(arr, axis, count, index):
    return arr if axis < 0 else np.split(arr, count, axis=axis)[index]


def check_shards(text, inputs, count, input_axes=None):
    want = interp.evaluate(text, inputs)
    parts = []
    plan = None
    for index in range(count):
        shard, ia, oa = capi.shard_text(text, count, index, input_axes, n_inputs=len(inputs), n_outputs=len(want))
        assert plan is None or plan == (ia, oa)
        plan = (ia, oa)
        parts.append(interp.evaluate(shard, [split(a, ax, count, index) for a, ax in zip(inputs, ia)]))
    ia, oa = plan
    for r, ax in enumerate(oa):
        got = parts[0][r] if ax < 0 else np.concatenate([p[r] for p in parts], axis=ax)
        assert got.shape == want[r].shape
        np.testing.assert_allclose(got, want[r], rtol=1e-12, atol=1e-12)
        if ax < 0:  # a replicated result is the same on every shard
            for p in parts[1:]:
                np.testing.assert_array_equal(p[r], parts[0][r])
    return ia, oa


def gpt2_inputs(params, vocab, seed=0):
    rng = np.random.default_rng(seed)
    out = []
    for name, shape, dt in params:
        if dt == "i32":
            out.append(rng.integers(0, vocab, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            out.append(np.ones(shape, np.float32))
        else:
            out.append((0.02 * rng.standard_normal(shape)).astype(np.float32))
    return out


@pytest.mark.parametrize("count", [2, 4])
def test_gpt2_forward_splits_over_the_batch(count):
    text, params = modules.gpt2_module(batch=4, seq=16, layers=2, d_model=64, heads=2, vocab=101)
    ia, oa = check_shards(text, gpt2_inputs(params, 101), count)
    assert ia == [0] + [-1] * (len(params) - 1) and oa == [0]  # token ids split, every parameter replicated


def test_sharded_gpt2_keeps_its_fused_patterns():
    text, params = modules.gpt2_module(batch=8, seq=128, layers=2, d_model=256, heads=4, vocab=1031)
    shard, _, _ = capi.shard_text(text, 4, 3, n_inputs=len(params), n_outputs=1)
    assert "tensor<2x128xi32>" in shard and "tensor<8x" not in shard
    full_steps, _, _ = capi.plan_text(text, 3)
    shard_steps, _, _ = capi.plan_text(shard, 3)
    assert shard_steps == full_steps
    assert shard_steps.count("fused_scaled_dot_product_attention") == 2


def test_norm_sweep_and_attention_and_batched_product():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 32)).astype(np.float32)
    g, b = rng.standard_normal(32).astype(np.float32), rng.standard_normal(32).astype(np.float32)
    ia, oa = check_shards(modules.norm_sweep_module(8, 32, "f32", 1e-5), [x, g, b], 4)
    assert ia == [0, -1, -1] and oa == [0, 0, 0]
    from op_cases import attention_text

    for layout in ("BHSD", "BSHD"):
        text, qshape = attention_text(2, 3, 16, 8, "f32", True, layout)
        q, k, v = (rng.standard_normal(qshape).astype(np.float32) for _ in range(3))
        ia, oa = check_shards(text, [q, k, v], 2)
        assert ia == [0, 0, 0] and oa == [0]
    t3, tw, to = modules.tt((4, 6, 5), "f32"), modules.tt((4, 5, 7), "f32"), modules.tt((4, 6, 7), "f32")
    bmm = (f"func.func @main(%a: {t3}, %b: {tw}) -> {to} {{\n  %0 = stablehlo.dot_general %a, %b, batching_dims = [0] x [0], contracting_dims = [2] x [1] : "
           f"({t3}, {tw}) -> {to}\n  return %0 : {to}\n}}\n")
    a, bb = rng.standard_normal((4, 6, 5)).astype(np.float32), rng.standard_normal((4, 5, 7)).astype(np.float32)
    assert check_shards(bmm, [a, bb], 2) == ([0, 0], [0])


def test_square_product_falls_back_to_splitting_the_rows_of_the_first_operand():
    t = modules.tt((8, 8), "f32")
    text = (f"func.func @main(%a: {t}, %b: {t}) -> {t} {{\n  %0 = stablehlo.dot_general %a, %b, contracting_dims = [1] x [0] : ({t}, {t}) -> {t}\n"
            f"  return %0 : {t}\n}}\n")
    rng = np.random.default_rng(2)
    a, b = rng.standard_normal((8, 8)).astype(np.float32), rng.standard_normal((8, 8)).astype(np.float32)
    # both operands have the batch-sized leading extent, but B's is contracted: only A is split
    assert check_shards(text, [a, b], 4) == ([0, -1], [0])
    # a column split of B, given explicitly (the column-split product of the benchmark)
    assert check_shards(text, [a, b], 4, input_axes=[-1, 1]) == ([-1, 1], [1])


def test_cnn_splits_over_the_images():
    text, params = modules.cnn_module(batch=4, size=8, channels=3, width=8, classes=5, dt="f32")
    rng = np.random.default_rng(3)
    ins = [rng.uniform(0.5, 1.5, size=s).astype(np.float32) for _, s, _ in params]
    ia, oa = check_shards(text, ins, 2)
    assert ia[0] == 0 and set(ia[1:]) == {-1} and oa == [0]


def test_replicated_values_that_meet_the_batch_are_rederived_or_sliced():
    t, tv = modules.tt((4, 6), "f32"), modules.tt((6,), "f32")
    # %w is an argument with the batch's shape but marked replicated: its shard is cut out with a slice
    text = (f"func.func @main(%x: {t}, %w: {t}, %v: {tv}) -> ({t}, {tv}) {{\n"
            f"  %i = stablehlo.iota dim = 1 : {t}\n  %c = stablehlo.constant dense<2.0> : {t}\n"
            f"  %b = stablehlo.broadcast_in_dim %v, dims = [1] : ({tv}) -> {t}\n"
            f"  %0 = stablehlo.multiply %x, %i : {t}\n  %1 = stablehlo.add %0, %c : {t}\n  %2 = stablehlo.add %1, %b : {t}\n"
            f"  %3 = stablehlo.multiply %2, %w : {t}\n  %4 = stablehlo.negate %v : {tv}\n  return %3, %4 : {t}, {tv}\n}}\n")
    rng = np.random.default_rng(4)
    ins = [rng.standard_normal((4, 6)).astype(np.float32), rng.standard_normal((4, 6)).astype(np.float32), rng.standard_normal(6).astype(np.float32)]
    assert check_shards(text, ins, 2, input_axes=[0, -1, -1]) == ([0, -1, -1], [0, -1])
    shard, _, _ = capi.shard_text(text, 2, 1, [0, -1, -1], n_inputs=3, n_outputs=2)
    assert "stablehlo.slice" in shard and "tensor<4x6xf32>) -> tensor<2x6xf32>" in shard


@pytest.mark.parametrize("body,why", [
    ("%0 = stablehlo.reduce(%x init: %z) applies stablehlo.add across dimensions = [0] : (tensor<4x6xf32>, tensor<f32>) -> tensor<6xf32>", "reduces over the split axis"),
    ("%t = stablehlo.transpose %x, dims = [1, 0] : (tensor<4x6xf32>) -> tensor<6x4xf32>\n  %0 = stablehlo.dot_general %t, %x, contracting_dims = [1] x [0] : (tensor<6x4xf32>, tensor<4x6xf32>) -> tensor<6x6xf32>", "contracts over the split axis"),
    ("%0 = stablehlo.reverse %x, dims = [0] : tensor<4x6xf32>", "reverses the split axis"),
    ("%0 = stablehlo.slice %x [1:3, 0:6] : (tensor<4x6xf32>) -> tensor<2x6xf32>", "cuts the split axis"),
    ("%0 = stablehlo.reshape %x : (tensor<4x6xf32>) -> tensor<3x8xf32>", "regroups the split axis"),
])
def test_programs_that_mix_the_batch_are_refused(body, why):
    result = body.rsplit("-> ", 1)[1] if "->" in body else "tensor<4x6xf32>"
    text = (f"func.func @main(%x: tensor<4x6xf32>) -> {result} {{\n  %z = stablehlo.constant dense<0.0> : tensor<f32>\n  {body}\n"
            f"  return %0 : {result}\n}}\n")
    with pytest.raises(capi.MetalHLOError) as e:
        capi.shard_text(text, 2, 0)
    assert e.value.status == 4 and why in str(e.value), str(e.value)


def test_batch_that_does_not_divide_and_bad_indices():
    t = modules.tt((6, 4), "f32")
    text = f"func.func @main(%x: {t}) -> {t} {{\n  %0 = stablehlo.negate %x : {t}\n  return %0 : {t}\n}}\n"
    with pytest.raises(capi.MetalHLOError, match="does not divide"):
        capi.shard_text(text, 4, 0)
    with pytest.raises(capi.MetalHLOError):
        capi.shard_text(text, 2, 2)
    assert capi.shard_text(text, 1, 0, n_inputs=1, n_outputs=1)[1:] == ([-1], [-1])  # one shard: nothing is split
    assert capi.shard_text(text, 3, 2, n_inputs=1, n_outputs=1)[1:] == ([0], [0])


@pytest.mark.parametrize("dt", ["f32", "i32"])
def test_random_programs_split_soundly_or_are_refused(dt):
    """Seeded random programs (tests/op_cases.py): whenever the analysis accepts a split, the shards evaluated on their own
    slices concatenate to the unsharded result; whatever it does not accept is refused with MHLO_ERROR_UNSUPPORTED_OP."""
    import op_cases

    accepted = refused = 0
    for name, text, ins in op_cases.random_program_cases(count=80, seed=4321, dt=dt):
        for count in (2, 3):
            if ins[0].shape[0] % count:
                continue
            try:
                capi.shard_text(text, count, 0, n_inputs=len(ins), n_outputs=4)
            except capi.MetalHLOError as e:
                assert e.status == 4, (name, str(e))
                refused += 1
                continue
            check_shards(text, ins, count)
            accepted += 1
    assert accepted >= 5 and refused >= 10, (accepted, refused)
