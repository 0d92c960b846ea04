"""Shared helpers of the parity tests: seeded inputs and the tolerance rule.

Tolerance rule (from the north-star statement of the build): bit-exact for integer/index results,
rel <= 1e-5 for fp32 results, rel <= 2e-2 for f16/bf16 results. "rel" is the plain per-element bound
|got - want| <= rel * |want| for every element whose magnitude reaches the tensor's mean magnitude. Elements below
the mean (zero crossings of the fp64 result, where any finite-precision evaluation has unbounded relative error) are
held to the absolute bound rel * mean|want|, i.e. the bound is rel * max(|want|, mean|want|).

Results of a contraction evaluated in 16-bit steps (attention: 16-bit scores and probabilities feeding P.V) may instead be
given their `magnitude`: the sum of the absolute values of the contracted terms, sum_j |p_j| |v_j|, per element. That sum
is what bounds the error of any finite-precision inner product (|fl(x.y) - x.y| <= c * u * sum |x_j y_j|); against
|x.y| itself the error is unbounded wherever the terms cancel. With a magnitude the bound is
rel * max(magnitude, mean|want|).
"""
import numpy as np

REL = {"float32": 1e-5, "float16": 2e-2, "bfloat16": 2e-2}


def rel_for(dtype) -> float:
    return REL[str(dtype).replace("torch.", "")]


def error_report(got, want, rel, row_scale=False, magnitude=None):
    """Per-element accounting of one comparison: counts of elements at or above the mean magnitude (held to the plain
    relative bound) and below it (held to rel * mean), how many of each fail, and the worst plain relative error among
    the former."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    fin = np.isfinite(want)
    scale = np.mean(np.abs(want[fin])) if fin.any() else 0.0
    if row_scale and want.ndim >= 1:
        # attention rows that see few keys keep the magnitude of single value vectors: scale each row by itself
        scale = np.broadcast_to(np.mean(np.abs(np.where(fin, want, 0.0)), axis=-1, keepdims=True), want.shape)[fin]
    w, g = want[fin], got[fin]
    err = np.abs(g - w)
    large = np.abs(w) >= scale
    bound = rel * np.maximum(np.abs(w), scale)
    if magnitude is not None:
        mag = np.asarray(magnitude, dtype=np.float64)[fin]
        assert np.all(mag >= np.abs(w) * (1 - 1e-9)), "a magnitude is the sum of absolute terms: it cannot be below |want|"
        bound = np.maximum(bound, rel * mag)
    with np.errstate(divide="ignore", invalid="ignore"):
        plain = np.where(large & (np.abs(w) > 0), err / np.abs(w), 0.0)
    return {"elements": int(w.size), "large": int(large.sum()), "large_failing": int((large & (err > bound)).sum()),
            "small_failing": int((~large & (err > bound)).sum()), "worst_plain_rel": float(plain.max()) if w.size else 0.0,
            "err": err, "bound": bound, "got": g, "want": w}


def assert_close(got, want, rel, what="", row_scale=False, magnitude=None):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return
    assert np.all(np.isfinite(got) == np.isfinite(want)), f"{what}: non-finite pattern differs"
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), f"{what}: infinities differ"
    r = error_report(got, want, rel, row_scale, magnitude)
    bad = r["large_failing"] + r["small_failing"]
    if bad:
        i = int(np.argmax(r["err"] - r["bound"]))
        raise AssertionError(
            f"{what}: {bad}/{r['elements']} elements outside rel={rel} ({r['large_failing']} of the {r['large']} at or above the "
            f"mean magnitude, worst plain relative error {r['worst_plain_rel']:.3e}); worst got={r['got'][i]!r} "
            f"want={r['want'][i]!r} err={r['err'][i]:.3e} bound={r['bound'][i]:.3e}")


def to_np(t):
    """torch tensor (any float dtype, any device) -> float64 ndarray of its exact values."""
    return t.detach().to("cpu").double().numpy()
