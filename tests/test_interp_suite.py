"""Pins the module-level oracle (oracle/interp.py) to the goldens of the StableHLO interpreter suite that the
reference vendors and runs (Tests/MetalHLOTests/Conformance/StableHLO/interpret). Tolerances are the reference
runner's: exact for expect_eq, 1e-4 for expect_almost_eq (InterpretTestRunner.swift:37-45). CPU only; skipped where
the reference checkout is absent."""
import numpy as np
import pytest

from interp_suite import all_cases
from oracle import interp

CASES = all_cases()


def _skip_reason(text):
    for bad in ("complex<", "f8E", "f4E", "f6E", "i2>", "i4>", "ui2>", "ui4>", "tf32", "quant", "x?x", "<?x", "token"):
        if bad in text:
            return bad
    return None


@pytest.mark.skipif(not CASES, reason="reference checkout with the vendored suite is not present")
@pytest.mark.parametrize("case", CASES, ids=[c.id for c in CASES])
def test_oracle_matches_suite_golden(case):
    why = _skip_reason(case.text)
    if why:
        pytest.skip(f"element type outside the backend's 13 types ({why})")
    try:
        outs = interp.evaluate(case.text, [])
    except interp.Unsupported as e:
        pytest.skip(f"outside the oracle's operator surface: {e}")
    for chk in case.checks:
        got = outs[chk["value"]]
        t = interp.Scanner(chk["type"]).type()
        want = interp.dense_value(chk["dense"], t) if "dense" in chk else outs[chk["other"]]
        if t.is_float:
            tol = 0 if chk["kind"].startswith("expect_eq") else 1e-4
            if t.dtype in ("f16", "bf16"):
                want = interp.round_to(want, t.dtype)
                got = interp.round_to(got, t.dtype)
                tol = max(tol, 1e-2)
            elif t.dtype == "f32":
                got = interp.round_to(got, "f32")
                tol = max(tol, 1e-6)
            np.testing.assert_allclose(got, want, rtol=tol, atol=tol, equal_nan=True, err_msg=case.id)
        else:
            np.testing.assert_array_equal(got, want, err_msg=case.id)
