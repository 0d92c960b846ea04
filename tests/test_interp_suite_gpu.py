"""The reference-held vectors on the CUDA path: every case of the StableHLO interpreter suite the reference vendors
(Tests/MetalHLOTests/Conformance/StableHLO/interpret, run there by OfficialConformanceTests.swift through
InterpretTestRunner.swift:178-259) is compiled through the C API at O0, O1, O2 and O3, executed on the GPU and held to
the suite's own goldens with the reference runner's tolerances; the four levels must also agree with one another
(OptimizationCorrectnessTests.swift:19-24). Cases whose element types lie outside the backend's 13 are skipped, as they
are for the oracle."""
import numpy as np
import pytest

from interp_suite import all_cases, skip_reason, verify

pytestmark = pytest.mark.gpu

CASES = [c for c in all_cases() if not skip_reason(c.text)]
_client = None


def client():
    global _client
    if _client is None:
        from metalhlo_b200 import capi

        _client = capi.Client()
    return _client


# operators this backend rejects with MHLO_ERROR_UNSUPPORTED_OP; their cases are skipped, not failed
def _unsupported(err):
    return err.status_name in ("UNSUPPORTED_OP",)


@pytest.mark.skipif(not CASES, reason="neither the reference checkout nor the fixture is present")
@pytest.mark.parametrize("case", CASES, ids=[c.id for c in CASES])
def test_cuda_path_matches_suite_golden_at_every_level(case):
    from metalhlo_b200 import capi

    per_level = {}
    for level in (0, 1, 2, 3):
        try:
            outs = client().run(case.text, [], opt_level=level)
        except capi.MetalHLOError as e:
            if _unsupported(e):
                pytest.skip(f"outside the backend's operator surface: {e}")
            raise
        verify(case, outs)
        per_level[level] = outs
    for level in (1, 2, 3):
        for a, b in zip(per_level[0], per_level[level]):
            if a.dtype.kind in "fV" or str(a.dtype) == "bfloat16":
                tol = 2e-2 if a.dtype.itemsize == 2 else 1e-5  # the stated tolerance of the element type
                np.testing.assert_allclose(np.asarray(b, dtype=np.float64), np.asarray(a, dtype=np.float64), rtol=tol, atol=tol / 10,
                                           equal_nan=True, err_msg=f"{case.id}: O{level} vs O0")
            else:
                np.testing.assert_array_equal(b, a, err_msg=f"{case.id}: O{level} vs O0")


def test_the_suite_is_not_silently_empty():
    assert len(CASES) >= 290
