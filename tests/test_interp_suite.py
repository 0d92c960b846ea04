"""Pins the module-level oracle (oracle/interp.py) to the goldens of the StableHLO interpreter suite that the
reference vendors and runs (Tests/MetalHLOTests/Conformance/StableHLO/interpret). Tolerances are the reference
runner's: exact for expect_eq, 1e-4 for expect_almost_eq (InterpretTestRunner.swift:37-45). CPU only. The cases come
from the reference checkout when it is present and from the committed fixture otherwise; a second test checks that the
fixture still equals what the checkout gives."""
import pytest

from interp_suite import all_cases, cases_from_checkout, cases_from_fixture, skip_reason, verify
from oracle import interp

CASES = all_cases()


@pytest.mark.skipif(not CASES, reason="neither the reference checkout nor the fixture is present")
@pytest.mark.parametrize("case", CASES, ids=[c.id for c in CASES])
def test_oracle_matches_suite_golden(case):
    why = skip_reason(case.text)
    if why:
        pytest.skip(f"element type outside the backend's 13 types ({why})")
    try:
        outs = interp.evaluate(case.text, [])
    except interp.Unsupported as e:
        pytest.skip(f"outside the oracle's operator surface: {e}")
    verify(case, outs)


def test_fixture_equals_the_checkout():
    live, kept = cases_from_checkout(), cases_from_fixture()
    if not live:
        pytest.skip("no reference checkout here")
    assert kept, "tests/golden/interp_suite.json.gz is missing: run tests/golden/make_interp_suite.py"
    assert [(c.id, c.text, c.checks) for c in live] == [(c.id, c.text, c.checks) for c in kept]
