"""Shared helpers of the parity tests: seeded inputs and the tolerance rule.

Tolerance rule (from the north-star statement of the build): bit-exact for integer/index results,
rel <= 1e-5 for fp32 results, rel <= 2e-2 for f16/bf16 results. "rel" is applied per element as
|got - want| <= rel * (|want| + mean|want|): the second term keeps elements that sit at a zero crossing of the
fp64 result (where any finite-precision evaluation has unbounded relative error) on the same scale as the
rest of the tensor.
"""
import numpy as np

REL = {"float32": 1e-5, "float16": 2e-2, "bfloat16": 2e-2}


def rel_for(dtype) -> float:
    return REL[str(dtype).replace("torch.", "")]


def assert_close(got, want, rel, what="", row_scale=False):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return
    assert np.all(np.isfinite(got) == np.isfinite(want)), f"{what}: non-finite pattern differs"
    fin = np.isfinite(want)
    scale = np.mean(np.abs(want[fin])) if fin.any() else 0.0
    if row_scale and want.ndim >= 1:
        # attention rows that see few keys keep the magnitude of single value vectors: scale each row by itself
        scale = np.broadcast_to(np.mean(np.abs(np.where(fin, want, 0.0)), axis=-1, keepdims=True), want.shape)[fin]
    err = np.abs(got[fin] - want[fin])
    bound = rel * (np.abs(want[fin]) + scale)
    bad = err > bound
    if bad.any():
        i = int(np.argmax(err - bound))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} elements outside rel={rel}; worst got={got[fin][i]!r} "
            f"want={want[fin][i]!r} err={err[i]:.3e} bound={bound[i]:.3e}")


def to_np(t):
    """torch tensor (any float dtype, any device) -> float64 ndarray of its exact values."""
    return t.detach().to("cpu").double().numpy()
