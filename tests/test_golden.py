"""The committed fixture tests/golden/hot_path.npz (written by tests/golden/make_golden.py from the CPU oracle).

CPU: the oracle still reproduces it exactly (it cannot drift without this test noticing).
GPU: every kernel family on the hot path, and a reduced GPT-2 through the C API, matches it on the same inputs.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = np.load(os.path.join(ROOT, "tests", "golden", "hot_path.npz"))


def test_oracle_reproduces_the_fixture():
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden

    fresh = make_golden.build()
    assert sorted(fresh) == sorted(GOLDEN.files)
    for name in GOLDEN.files:
        np.testing.assert_array_equal(fresh[name], GOLDEN[name], err_msg=name)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["bfloat16", "float16", "float32"])
def test_kernels_match_the_fixture(dtype_name):
    import torch

    from metalhlo_b200 import cuda
    from parity import assert_close, rel_for, to_np

    dtype = getattr(torch, dtype_name)
    rel = rel_for(dtype)
    dev = lambda name: torch.from_numpy(GOLDEN[name]).to(dtype).cuda()  # noqa: E731  (the inputs are exact in every dtype)
    x, gamma, beta = dev("norm_x"), dev("norm_gamma"), dev("norm_beta")
    assert_close(to_np(cuda.layer_norm(x, gamma, beta, 1e-5)), GOLDEN["layer_norm"], rel, "layer_norm")
    assert_close(to_np(cuda.rms_norm(x, gamma, 1e-5)), GOLDEN["rms_norm"], rel, "rms_norm")
    assert_close(to_np(cuda.softmax((x.float() * 4).to(dtype))), GOLDEN["softmax"], rel, "softmax")
    assert_close(to_np(cuda.gemm(dev("gemm_a"), dev("gemm_b"))), GOLDEN["gemm"], rel, "gemm")
    q, k, v = dev("attn_q"), dev("attn_k"), dev("attn_v")
    for causal, key in ((False, "attention"), (True, "attention_causal")):
        assert_close(to_np(cuda.attention(q, k, v, 0.125, causal=causal)), GOLDEN[key], rel, key, row_scale=True)
    assert cuda.device_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("level", [0, 3])
def test_reduced_gpt2_matches_the_fixture(level):
    from metalhlo_b200 import capi, modules

    text, params = modules.gpt2_module(batch=1, seq=32, layers=1, d_model=64, heads=2, vocab=101, dt="f16")
    client = capi.Client()
    exe = client.compile(text, opt_level=level)
    ins = [client.buffer(GOLDEN[f"gpt2_in{i}"]) for i in range(len(params))]
    got = exe.execute(ins)[0].to_numpy().astype(np.float64)
    want = GOLDEN["gpt2_logits"]
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-2
