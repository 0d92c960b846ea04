"""Operator-by-operator parity of the CUDA backend against the numpy oracle: every case of tests/op_cases.py is
compiled through the C API at O0 (unfused), O2 (generic fusion) and O3 (pattern fusion) and executed on the GPU.
Integer, index and boolean results must be bit-exact; floating-point results follow the tolerance of tests/parity.py."""
import numpy as np
import pytest

from op_cases import CASES
from oracle import interp
from parity import assert_close

pytestmark = pytest.mark.gpu

_client = None


def client():
    global _client
    if _client is None:
        from metalhlo_b200 import capi

        _client = capi.Client()
    return _client


REL = {"f32": 1e-5, "f16": 2e-2, "bf16": 2e-2, "f64": 1e-12}


def dtype_tag(arr):
    return {"float32": "f32", "float16": "f16", "bfloat16": "bf16", "float64": "f64"}.get(str(arr.dtype))


@pytest.mark.parametrize("level", [0, 2, 3])
@pytest.mark.parametrize("name", [c[0] for c in CASES])
def test_case_matches_oracle(name, level):
    _, text, inputs = next(c for c in CASES if c[0] == name)
    want = interp.evaluate(text, inputs)
    got = client().run(text, inputs, opt_level=level)
    assert len(got) == len(want)
    magnitude = None
    if name.startswith("pattern_attention") and dtype_tag(got[0]) in ("f16", "bf16"):
        # sum_j p_ij |v_jd| of the same module: the scale of the terms each output element contracts (tests/parity.py)
        magnitude = interp.evaluate(text, [inputs[0], inputs[1], np.abs(inputs[2])])[0]
    for g, w in zip(got, want):
        tag = dtype_tag(g)
        if tag is None:
            np.testing.assert_array_equal(g, w.astype(g.dtype), err_msg=f"{name} O{level}")
        else:
            # the oracle carries floats in fp64: what the result type cannot hold (an overflow to inf, an underflow to 0) is
            # rounded to the type before the comparison
            with np.errstate(over="ignore"):
                w = np.asarray(w, dtype=np.float64).astype(g.dtype).astype(np.float64) if name.startswith(("special_", "empty_", "scalar_", "rank6_", "edge_")) else w
            assert_close(g.astype(np.float64), w, REL[tag], f"{name} O{level}", magnitude=magnitude)


@pytest.mark.parametrize("name", [c[0] for c in CASES if c[0].startswith("conv_")])
def test_convolution_direct_kernel_matches_oracle(name, monkeypatch):
    """Every convolution case again through the direct kernel (METALHLO_CONV_DIRECT=1 is read when the module is lowered)."""
    monkeypatch.setenv("METALHLO_CONV_DIRECT", "1")
    _, text, inputs = next(c for c in CASES if c[0] == name)
    want = interp.evaluate(text, inputs)
    exe = client().compile(text, opt_level=2, caching=False)
    assert "convolution" in exe.steps
    got = [o.to_numpy() for o in exe.execute([client().buffer(x) for x in inputs])]
    for g, w in zip(got, want):
        tag = dtype_tag(g)
        if tag is None:
            np.testing.assert_array_equal(g, w.astype(g.dtype), err_msg=name)
        else:
            assert_close(g.astype(np.float64), w, REL[tag], name)
