"""Writes tests/golden/interp_suite.json.gz: the cases of the StableHLO interpreter suite the reference vendors
(Tests/MetalHLOTests/Conformance/StableHLO/interpret/*.mlir, the files listed in tests/interp_suite.py), each as the
function rewritten to return its checked values plus the `check.expect_*` goldens. Test fixture only: it lets the GPU
box, which has no reference checkout, run the reference-held vectors through the CUDA path.

    python tests/golden/make_interp_suite.py        # needs the reference checkout (MHLO_INTERP_SUITE_DIR or ../reference)
"""
import gzip
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import interp_suite  # noqa: E402


def main():
    cases = interp_suite.cases_from_checkout()
    if not cases:
        raise SystemExit(f"no suite under {interp_suite.SUITE_DIR}")
    doc = {"source": "Tests/MetalHLOTests/Conformance/StableHLO/interpret (openxla/stablehlo interpreter suite, as vendored by the reference)",
           "cases": [{"file": c.file, "name": c.name, "text": c.text, "checks": c.checks} for c in cases]}
    with gzip.GzipFile(interp_suite.FIXTURE, "wb", mtime=0) as f:
        f.write(json.dumps(doc, sort_keys=True).encode())
    print(f"{len(cases)} cases -> {interp_suite.FIXTURE} ({os.path.getsize(interp_suite.FIXTURE)} bytes)")


if __name__ == "__main__":
    main()
