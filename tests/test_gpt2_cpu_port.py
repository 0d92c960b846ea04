"""The fp32 CPU forward pass that bench.py times as its CPU baseline (oracle/gpt2_cpu.py) computes the same function
as the module the GPU runs: checked against the fp64 module interpreter on a reduced model, fp32 module text."""
import numpy as np

from metalhlo_b200 import modules
from oracle import gpt2_cpu, interp


def test_cpu_port_matches_the_module_interpreter():
    text, params = modules.gpt2_module(batch=2, seq=32, layers=2, d_model=64, heads=4, vocab=211, dt="f32")
    rng = np.random.default_rng(3)
    ins = []
    for name, shape, dt in params:
        if dt == "i32":
            ins.append(rng.integers(0, 211, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            ins.append((1 + 0.1 * rng.standard_normal(shape)).astype(np.float32))
        else:
            ins.append((0.05 * rng.standard_normal(shape)).astype(np.float32))
    want = interp.evaluate(text, ins)[0]
    got = gpt2_cpu.forward(ins, heads=4)
    assert got.shape == want.shape and got.dtype == np.float32
    err = np.abs(got - want)
    assert err.max() <= 1e-4 * np.abs(want).max(), err.max()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5
