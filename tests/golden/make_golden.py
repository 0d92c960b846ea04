"""Writes tests/golden/hot_path.npz: seeded inputs of every kernel family on the hot path together with the outputs of
the CPU oracle (fp64), which is itself pinned by the reference's known-answer tests and interpreter suite
(tests/test_oracle_kat.py, tests/test_interp_suite.py). The fixture travels with the repository, so the GPU tests have a
fixed target that does not depend on anything outside it.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from metalhlo_b200 import modules  # noqa: E402
from oracle import interp  # noqa: E402

SEED = 42  # the reference's TestDataGenerator seed


def bf16_exact(a):
    """fp32 values that bf16 holds exactly (so that every dtype sees identical inputs)."""
    return torch.from_numpy(a).to(torch.bfloat16).float().numpy()


def build():
    rng = np.random.default_rng(SEED)
    out = {}
    x = bf16_exact(rng.standard_normal((16, 256)).astype(np.float32))
    gamma = bf16_exact((1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    beta = bf16_exact((0.1 * rng.standard_normal(256)).astype(np.float32))
    out.update(norm_x=x, norm_gamma=gamma, norm_beta=beta,
               layer_norm=oracle.layer_norm(x, gamma, beta, 1e-5), rms_norm=oracle.rms_norm(x, gamma, 1e-5),
               softmax=oracle.softmax(x * 4), gelu=oracle.gelu(x), silu=oracle.silu(x))
    a = bf16_exact((rng.standard_normal((64, 96)) / np.sqrt(96)).astype(np.float32))
    b = bf16_exact(rng.standard_normal((96, 72)).astype(np.float32))
    out.update(gemm_a=a, gemm_b=b, gemm=oracle.gemm(a, b))
    q, k, v = (bf16_exact(rng.standard_normal((1, 1, 160, 64)).astype(np.float32)) for _ in range(3))
    out.update(attn_q=q, attn_k=k, attn_v=v, attention=oracle.attention(q, k, v, 0.125, causal=False),
               attention_causal=oracle.attention(q, k, v, 0.125, causal=True))
    text, params = modules.gpt2_module(batch=1, seq=32, layers=1, d_model=64, heads=2, vocab=101, dt="f16")
    ins = []
    for name, shape, dt in params:
        if dt == "i32":
            ins.append(rng.integers(0, 101, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            ins.append(np.ones(shape, np.float32))
        else:
            ins.append((0.05 * rng.standard_normal(shape)).astype(np.float32))
    for i, arr in enumerate(ins):
        out[f"gpt2_in{i}"] = arr
    out["gpt2_logits"] = interp.evaluate(text, ins)[0]
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hot_path.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
