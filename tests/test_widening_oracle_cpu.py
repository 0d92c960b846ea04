"""The oracle's reduce_window / scatter / sort / if / case against independent numpy formulations of the same
StableHLO semantics (the interpreter folds the body regions; numpy computes the closed form)."""
import numpy as np
import pytest

from op_cases import CASES
from oracle import interp

BY_NAME = {c[0]: c for c in CASES}


def run(name):
    _, text, inputs = BY_NAME[name]
    return interp.evaluate(text, inputs), inputs


def test_maxpool_matches_numpy_blocks():
    (got,), (x,) = run("reduce_window_maxpool_2x2")
    want = x.reshape(2, 4, 2, 4, 2, 4).max(axis=(2, 4))
    np.testing.assert_array_equal(got, want)


def test_same_padded_window_sum_matches_shifted_adds():
    (got,), (x,) = run("reduce_window_sum_3x3_same")
    padded = np.pad(x.astype(np.float64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = sum(padded[:, i:i + 8, j:j + 8, :] for i in range(3) for j in range(3))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_cumsum_window_is_a_prefix_sum():
    (got,), (x,) = run("reduce_window_cumsum")
    np.testing.assert_allclose(got, np.cumsum(x.astype(np.float64), axis=1), rtol=1e-5, atol=1e-5)


def test_nonzero_init_pads_with_the_init_value():
    (got,), (x,) = run("reduce_window_nonzero_init")
    padded = np.pad(x.astype(np.float64), 1, constant_values=0.5)
    want = 0.5 + sum(padded[i:i + 7, j:j + 7] for i in range(2) for j in range(2))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_dilated_window_sum_matches_explicit_dilation():
    (got,), (x,) = run("reduce_window_dilations_i32")
    dil = np.zeros((5, 17), np.int64)
    dil[:, ::2] = x
    padded = np.pad(dil, ((0, 0), (0, 2)))[:, 1:]  # low padding of -1 trims one column
    want = np.zeros((4, 7), np.int64)
    for o0 in range(4):
        for o1 in range(7):
            want[o0, o1] = sum(padded[o0 + w0, 2 * o1 + 2 * w1] for w0 in range(2) for w1 in range(3))
    np.testing.assert_array_equal(got, want)


def test_scatter_add_matches_add_at():
    (got,), (table, idx, upd) = run("scatter_add_rows_duplicates")
    want = table.astype(np.float64).copy()
    np.add.at(want, idx[:, 0], upd.astype(np.float64))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_scatter_skips_targets_outside_the_operand():
    (got,), (table, idx, upd) = run("scatter_add_rows_out_of_bounds")
    want = table.astype(np.float64).copy()
    for r, i in enumerate(idx[:, 0]):
        if 0 <= i < 10:
            want[i] += upd[r]
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_scatter_batched_indexes_inside_each_batch():
    (got,), (x, idx, upd) = run("scatter_add_batched")
    want = x.astype(np.float64).copy()
    for b in range(3):
        np.add.at(want[b], idx[b, :, 0], upd[b].astype(np.float64))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_sort_orders_special_values_totally():
    (got,), (keys,) = run("sort_f32_special_values")
    assert np.isnan(got[-2:]).all() and got[0] == -np.inf and got[-3] == np.inf
    zeros = np.flatnonzero(got == 0)
    assert np.signbit(got[zeros[0]]) and not np.signbit(got[zeros[1]])
    finite = got[:-2]
    assert (np.diff(finite) >= 0).all()


def test_argsort_is_stable_in_both_directions():
    (vals, order), (ties, _) = run("argsort_stable_ties")
    for r in range(4):
        np.testing.assert_array_equal(order[r], np.argsort(ties[r], kind="stable"))
    (vals, order), _ = run("argsort_stable_ties_descending")
    for r in range(4):
        np.testing.assert_array_equal(order[r], np.argsort(-ties[r], kind="stable"))


@pytest.mark.parametrize("n", [8192, 8193, 20000])
def test_long_sort_is_a_stable_permutation(n):
    (vals, order), (keys, _) = run(f"sort_global_{n}")
    k = -keys.astype(np.int64) if n == 8193 else keys.astype(np.int64)
    for r in range(3):
        np.testing.assert_array_equal(order[r], np.argsort(k[r], kind="stable"))
        np.testing.assert_array_equal(vals[r], keys[r][order[r]])


def test_branches_pick_one_region():
    (a, b), (_, x, y) = run("if_true")
    np.testing.assert_allclose(a, x.astype(np.float64) * y, rtol=1e-6)
    (a, b), (_, x, y) = run("if_false")
    np.testing.assert_allclose(a, x.astype(np.float64) - y, rtol=1e-6)
    assert float(b) == 1.0
    for v, f in ((0, np.negative), (1, np.tanh), (2, np.abs), (7, np.abs), (-3, np.abs)):
        (got,), (_, x) = run(f"case_index_{v}".replace("-", "m"))
        np.testing.assert_allclose(got, f(x.astype(np.float64)), rtol=1e-6)


def _torch_conv(x_nhwc, w_hwio, **kw):
    import torch

    x = torch.from_numpy(np.ascontiguousarray(x_nhwc.astype(np.float64))).permute(0, 3, 1, 2)
    w = torch.from_numpy(np.ascontiguousarray(w_hwio.astype(np.float64))).permute(3, 2, 0, 1)
    return torch.nn.functional.conv2d(x, w, **kw).permute(0, 2, 3, 1).numpy()


def test_convolution_matches_torch_conv2d():
    (got,), (x, w) = run("conv_3x3_same_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, padding=1), rtol=1e-9, atol=1e-9)
    (got,), (x, w) = run("conv_dilated_kernel_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, dilation=2), rtol=1e-9, atol=1e-9)
    (got,), (x, w) = run("conv_feature_groups_2_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, groups=2), rtol=1e-9, atol=1e-9)
    (got,), (x, w) = run("conv_depthwise_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, groups=6), rtol=1e-9, atol=1e-9)
    (got,), (x, w) = run("conv_short_form_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, padding=1), rtol=1e-9, atol=1e-9)
    (got,), (x, w) = run("conv_generic_form_f32")
    np.testing.assert_allclose(got, _torch_conv(x, w, padding=1, stride=2), rtol=1e-9, atol=1e-9)


def test_nchw_convolution_matches_torch_conv2d():
    import torch

    (got,), (x, w) = run("conv_nchw_oihw_f32")
    want = torch.nn.functional.conv2d(torch.from_numpy(x.astype(np.float64)), torch.from_numpy(w.astype(np.float64))).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-9)


def test_transposed_convolution_matches_torch_conv_transpose2d():
    import torch

    (got,), (x, w) = run("conv_transposed_f32")
    xt = torch.from_numpy(x.astype(np.float64)).permute(0, 3, 1, 2)
    # conv_transpose2d correlates with the flipped kernel: flip it back to express the plain dilated-input convolution
    wt = torch.from_numpy(np.ascontiguousarray(w[::-1, ::-1].astype(np.float64))).permute(2, 3, 0, 1)
    want = torch.nn.functional.conv_transpose2d(xt, wt, stride=2).permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-9)


def test_select_and_scatter_is_the_max_pool_gradient():
    import torch

    (got,), (x, src) = run("select_and_scatter_maxpool_grad_2x2")
    xt = torch.from_numpy(x.astype(np.float64)).permute(0, 3, 1, 2).requires_grad_(True)
    y = torch.nn.functional.max_pool2d(xt, 2, 2)
    y.backward(torch.from_numpy(src.astype(np.float64)).permute(0, 3, 1, 2))
    np.testing.assert_allclose(got, xt.grad.permute(0, 2, 3, 1).numpy(), rtol=1e-12, atol=1e-12)


def test_select_and_scatter_drops_windows_won_by_the_padding():
    (got,), (x, src) = run("select_and_scatter_padding_can_win")
    # every operand value is negative and the init value 0 pads the border: border windows select the padding
    assert got[0].sum() == 0 and got[:, 0].sum() == 0 or np.count_nonzero(got) < src.size


def test_threefry_module_matches_a_direct_numpy_threefry():
    from op_cases import THREEFRY_ROTATIONS

    (w0, w1), (key, x0, x1) = run("threefry2x32_random_bits")
    ks = [key[0], key[1], key[0] ^ key[1] ^ np.uint32(0x1BD11BDA)]
    a, b = x0 + ks[0], x1 + ks[1]
    for group in range(5):
        for r in THREEFRY_ROTATIONS[4 * (group % 2):4 * (group % 2) + 4]:
            a = a + b
            b = ((b << np.uint32(r)) | (b >> np.uint32(32 - r))) ^ a
        a = a + ks[(group + 1) % 3]
        b = b + ks[(group + 2) % 3] + np.uint32(group + 1)
    np.testing.assert_array_equal(w0, a)
    np.testing.assert_array_equal(w1, b)
    # the output words look uniform: every bit is set about half of the time
    bits = np.unpackbits(np.concatenate([w0, w1]).view(np.uint8))
    assert abs(bits.mean() - 0.5) < 0.01


def test_threefry_known_answer():
    """Known-answer vector of Threefry-2x32-20 from the Random123 distribution's kat_vectors: zero key and counter."""
    from op_cases import threefry2x32_text

    w0, w1 = interp.evaluate(threefry2x32_text(1), [np.zeros(2, np.uint32), np.zeros(1, np.uint32), np.zeros(1, np.uint32)])
    assert (int(w0[0]), int(w1[0])) == (0x6B200159, 0x99BA4EFE)


def test_rng_bit_generator_known_answer_and_state():
    """The generator's word pair at key 0, counter 0 is the Random123 known answer of Threefry-2x32-20; the state advances by
    the pairs used and a second draw continues the stream."""
    text = """func.func @main(%arg0: tensor<2xui64>) -> (tensor<2xui64>, tensor<4xui32>) {
  %0, %1 = stablehlo.rng_bit_generator %arg0, algorithm = THREE_FRY : (tensor<2xui64>) -> (tensor<2xui64>, tensor<4xui32>)
  return %0, %1 : tensor<2xui64>, tensor<4xui32>
}"""
    state, bits = interp.evaluate(text, [np.zeros(2, np.uint64)])
    assert (int(bits[0]), int(bits[1])) == (0x6B200159, 0x99BA4EFE)
    assert state.tolist() == [0, 2]
    state2, bits2 = interp.evaluate(text, [state])
    whole = interp.evaluate(text.replace("4xui32", "8xui32"), [np.zeros(2, np.uint64)])[1]
    np.testing.assert_array_equal(np.concatenate([bits, bits2]), whole)
    assert state2.tolist() == [0, 4]
    # 64-bit elements are a whole pair, first word low
    wide = interp.evaluate(text.replace("4xui32", "2xui64"), [np.zeros(2, np.uint64)])[1]
    assert int(wide[0]) == 0x6B200159 | (0x99BA4EFE << 32)
