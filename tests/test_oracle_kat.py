"""Pins the CPU oracle to the known-answer tests the reference holds for the fused-op arithmetic.

Each case restates the input and the expectation of a reference test (cited per test); the oracle must meet
the reference's own tolerance. CPU only.
"""
import math

import numpy as np

import oracle


def test_softmax_rows_sum_to_one_uniform_and_monotone():
    # Tests/MetalHLOCoreTests/MetalKernelTests.swift:56-102
    y = oracle.softmax(np.array([[1.0, 2.0, 3.0, 4.0], [0.0, 0.0, 0.0, 0.0]], dtype=np.float32))
    assert abs(y[0].sum() - 1.0) < 1e-5 and abs(y[1].sum() - 1.0) < 1e-5
    assert np.all(np.abs(y[1] - 0.25) < 1e-5)
    assert y[0, 3] > y[0, 2] > y[0, 1] > y[0, 0]


def test_softmax_matches_host_formula():
    # Tests/MetalHLOTests/ActivationOpsTests.swift:137-192: exp(x - max) / sum, tolerance 1e-5
    x = np.array([[1.0, 2.0, 3.0, 4.0], [-1.0, 0.0, 1.0, 2.0]], dtype=np.float32)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    np.testing.assert_allclose(oracle.softmax(x), e / e.sum(axis=1, keepdims=True), atol=1e-5)


def test_softmax_inner_axis():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 5, 4)).astype(np.float32)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    np.testing.assert_allclose(oracle.softmax(x, axis=1), e / e.sum(axis=1, keepdims=True), rtol=1e-12)


def test_layer_norm_rows_have_zero_mean_unit_std():
    # MetalKernelTests.swift:173-225: [1,2,3,4] (mean 2.5, var 1.25) and a second row; (mean 25, var 125); mean ~0, std ~1 (1e-4)
    x = np.array([[1.0, 2.0, 3.0, 4.0], [10.0, 20.0, 30.0, 40.0]], dtype=np.float32)
    y = oracle.layer_norm(x, None, None, eps=1e-5)
    for row in y:
        assert abs(row.mean()) < 1e-4
        assert abs(row.std() - 1.0) < 1e-4
    # closed form for the first row: (x - 2.5) / sqrt(1.25 + 1e-5)
    np.testing.assert_allclose(y[0], (x[0].astype(np.float64) - 2.5) / math.sqrt(1.25 + 1e-5), rtol=1e-12)


def test_layer_norm_affine():
    x = np.array([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32)
    g = np.array([2.0, 2.0, 2.0, 2.0], dtype=np.float32)
    b = np.array([1.0, 1.0, 1.0, 1.0], dtype=np.float32)
    y = oracle.layer_norm(x, g, b, eps=1e-5)
    np.testing.assert_allclose(y[0], (x[0].astype(np.float64) - 2.5) / math.sqrt(1.25 + 1e-5) * 2 + 1, rtol=1e-12)


def test_rms_norm_3_4_0_0():
    # MetalKernelTests.swift:236-274: RMS of [3,4,0,0] is 2.5 -> [1.2, 1.6, 0, 0]
    y = oracle.rms_norm(np.array([[3.0, 4.0, 0.0, 0.0]], dtype=np.float32), None, eps=1e-5)
    assert abs(y[0, 0] - 1.2) < 1e-4 and abs(y[0, 1] - 1.6) < 1e-4
    assert abs(y[0, 2]) < 1e-5 and abs(y[0, 3]) < 1e-5


def test_gelu_tanh_host_formula():
    # ActivationOpsTests.swift:252-318: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), tolerance 1e-4
    x = np.array([-2.0, -1.0, 0.0, 1.0, 2.0, 3.0], dtype=np.float32)
    want = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))) for v in x.tolist()]
    np.testing.assert_allclose(oracle.gelu(x, approximate=True), want, atol=1e-4)
    assert oracle.gelu(np.zeros(1, np.float32))[0] == 0.0


def test_silu():
    x = np.array([-3.0, 0.0, 0.5, 4.0], dtype=np.float32)
    np.testing.assert_allclose(oracle.silu(x), [v / (1 + math.exp(-v)) for v in x.tolist()], rtol=1e-12)


def test_dot_2x2():
    # Tests/MetalHLOTests/OperationTests.swift:327-348: [[1,2],[3,4]] . [[5,6],[7,8]] = [[19,22],[43,50]]
    a = np.array([[1, 2], [3, 4]], dtype=np.float32)
    b = np.array([[5, 6], [7, 8]], dtype=np.float32)
    np.testing.assert_array_equal(oracle.gemm(a, b), [[19, 22], [43, 50]])
    np.testing.assert_array_equal(oracle.gemm(a.T.copy(), b, trans_a=True), [[19, 22], [43, 50]])
    np.testing.assert_array_equal(oracle.gemm(a, b.T.copy(), trans_b=True), [[19, 22], [43, 50]])


def test_gemm_batched_matches_numpy():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 7, 5)).astype(np.float32)
    b = rng.standard_normal((3, 5, 9)).astype(np.float32)
    np.testing.assert_allclose(oracle.gemm(a, b), a.astype(np.float64) @ b.astype(np.float64), rtol=1e-12)


def test_attention_matches_manual_sdpa():
    # emitManualSDPA, Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift:245-276
    rng = np.random.default_rng(2)
    q = rng.standard_normal((2, 3, 6, 8)).astype(np.float32)
    k = rng.standard_normal((2, 3, 6, 8)).astype(np.float32)
    v = rng.standard_normal((2, 3, 6, 8)).astype(np.float32)
    scale = 1 / math.sqrt(8)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) * scale
    for causal in (False, True):
        sc = s.copy()
        if causal:
            sc[..., np.triu(np.ones((6, 6), bool), 1)] = -np.inf
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        want = np.einsum("bhqk,bhkd->bhqd", p, v.astype(np.float64))
        np.testing.assert_allclose(oracle.attention(q, k, v, scale, causal=causal), want, rtol=1e-10)
    mask = rng.standard_normal((6, 6)).astype(np.float32)
    sc = s + mask
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    np.testing.assert_allclose(oracle.attention(q, k, v, scale, mask=mask),
                               np.einsum("bhqk,bhkd->bhqd", p, v.astype(np.float64)), rtol=1e-10)


def test_cpu_f32_kernels_agree_with_fp64_oracle():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((16, 256)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    b = (0.1 * rng.standard_normal(256)).astype(np.float32)
    y = np.empty_like(x)
    oracle.cpu_layer_norm_f32(x, g, b, y)
    np.testing.assert_allclose(y, oracle.layer_norm(x, g, b), rtol=1e-4, atol=1e-5)
    oracle.cpu_rms_norm_f32(x, g, y)
    np.testing.assert_allclose(y, oracle.rms_norm(x, g), rtol=1e-4, atol=1e-5)
    oracle.cpu_softmax_f32(x, y)
    np.testing.assert_allclose(y, oracle.softmax(x), rtol=1e-4, atol=1e-7)
    oracle.cpu_gelu_f32(x, y)
    np.testing.assert_allclose(y, oracle.gelu(x), rtol=1e-4, atol=1e-6)
    a = rng.standard_normal((8, 32)).astype(np.float32)
    w = rng.standard_normal((32, 12)).astype(np.float32)
    c = np.empty((8, 12), np.float32)
    oracle.cpu_gemm_f32(a, w, c)
    np.testing.assert_allclose(c, oracle.gemm(a, w), rtol=1e-4, atol=1e-5)
    q = rng.standard_normal((2, 9, 16)).astype(np.float32)
    o = np.empty_like(q)
    for causal in (False, True):
        oracle.cpu_attention_f32(q, q, q, o, 0.25, causal)
        np.testing.assert_allclose(o, oracle.attention(q, q, q, 0.25, causal=causal), rtol=1e-4, atol=1e-5)
