"""Whole-module parity through the C API: the reference-runnable fp32 MLP+softmax configuration and a reduced GPT-2
forward pass (same graph as the full model, smaller extents) at every optimisation level against the numpy oracle."""
import numpy as np
import pytest

from metalhlo_b200 import modules
from oracle import interp
from parity import assert_close

pytestmark = pytest.mark.gpu


def client():
    from metalhlo_b200 import capi

    return capi.Client()


@pytest.mark.parametrize("level", [0, 1, 2, 3])
def test_mlp_softmax_fp32_configuration(level):
    # X [512,1024] ~ N(0,1), W [1024,1024] ~ N(0,0.02), b zeros: dot_general + bias -> tanh GELU -> softmax
    rng = np.random.default_rng(42)
    x = rng.standard_normal((512, 1024)).astype(np.float32)
    w = (0.02 * rng.standard_normal((1024, 1024))).astype(np.float32)
    b = np.zeros(1024, np.float32)
    text = modules.mlp_softmax_module()
    want = interp.evaluate(text, [x, w, b])[0]
    c = client()
    exe = c.compile(text, level)
    got = exe.execute([c.buffer(x), c.buffer(w), c.buffer(b)])[0].to_numpy()
    assert_close(got.astype(np.float64), want, 1e-5, f"O{level}")
    np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=1e-5)
    if level == 3:
        assert exe.steps == ["fused_matmul_bias_activation", "fused_softmax"]


def gpt2_inputs(params, vocab, seed=0):
    rng = np.random.default_rng(seed)
    out = []
    for name, shape, dt in params:
        if dt == "i32":
            out.append(rng.integers(0, vocab, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            out.append(np.ones(shape, np.float32))
        elif name.endswith(("ln1_b", "ln2_b", "lnf_b")):
            out.append(np.zeros(shape, np.float32))
        else:
            out.append((0.02 * rng.standard_normal(shape)).astype(np.float32))
    return out


@pytest.mark.parametrize("level", [0, 2, 3])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_reduced_gpt2_forward(level, dt):
    vocab = 1031  # not a multiple of 8: ragged logits rows like the real vocabulary
    text, params = modules.gpt2_module(batch=2, seq=128, layers=2, d_model=256, heads=4, vocab=vocab, dt=dt)
    ins = gpt2_inputs(params, vocab)
    want = interp.evaluate(text, ins)[0]
    c = client()
    exe = c.compile(text, level)
    got = exe.execute([c.buffer(a) for a in ins])[0].to_numpy().astype(np.float64)
    # ~150 chained 16-bit ops: the per-op bound of tests/parity.py does not compose, so the whole-model check is normwise
    # (relative L2 error within the 16-bit tolerance, worst element within 5 % of the logit range)
    rel_l2 = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel_l2 < 2e-2, f"gpt2 {dt} O{level}: relative L2 error {rel_l2:.3e}"
    assert np.abs(got - want).max() < 5e-2 * np.abs(want).max(), f"gpt2 {dt} O{level}"
    if level == 3:
        fused = [s for s in exe.steps if s.startswith("fused")]
        assert fused.count("fused_scaled_dot_product_attention") == 2
        # all five residual adds are fused into their norms; the first one (token rows + position table) reads the table
        # as a block of rows repeated over the batch
        assert fused.count("fused_layer_norm") == 0 and fused.count("fused_add_layer_norm") == 4
        assert fused.count("fused_add_layer_norm [repeated addend]") == 1
        assert fused.count("fused_matmul_bias_activation") == 8
    # greedy next-token ids agree wherever the oracle's top-2 margin exceeds the 16-bit resolution
    top2 = np.sort(want, axis=-1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 0.05 * np.abs(top2[..., 1]) + 1e-3
    assert np.array_equal(got.argmax(-1)[clear], want.argmax(-1)[clear])


def cnn_inputs(params):
    rng = np.random.default_rng(99)
    out = []
    for name, shape, _ in params:
        if name.endswith("_var"):
            out.append(rng.uniform(0.5, 1.5, size=shape).astype(np.float32))
        elif name.endswith("_scale"):
            out.append((1 + 0.1 * rng.standard_normal(shape)).astype(np.float32))
        elif name.endswith(("_offset", "_mean", "_b")):
            out.append((0.1 * rng.standard_normal(shape)).astype(np.float32))
        elif name == "image":
            out.append(rng.standard_normal(shape).astype(np.float32))
        else:
            fan_in = int(np.prod(shape[:-1]))
            out.append((rng.standard_normal(shape) / np.sqrt(fan_in)).astype(np.float32))
    return out


@pytest.mark.parametrize("level", [0, 2, 3])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_residual_cnn_forward(level, dt):
    """Convolution (patch matrix + GEMM), batch-norm inference, max pooling and the dense head in one module."""
    text, params = modules.cnn_module(batch=4, size=16, channels=3, width=16, classes=10, dt=dt)
    ins = cnn_inputs(params)
    want = interp.evaluate(text, ins)[0]
    c = client()
    exe = c.compile(text, level)
    got = exe.execute([c.buffer(a) for a in ins])[0].to_numpy().astype(np.float64)
    rel_l2 = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel_l2 < (1e-5 if dt == "f32" else 2e-2), f"cnn {dt} O{level}: relative L2 error {rel_l2:.3e}"
    steps = exe.steps
    assert steps.count("convolution.gemm") == 3 and steps.count("reduce_window") == 1
    assert any(s.startswith("batch_norm_inference") or s.startswith("fused_elementwise") for s in steps)
