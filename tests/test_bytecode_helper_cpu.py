"""MLIR bytecode programs: the helper-process protocol of the host library (bytecode on the child's stdin, text on its
stdout, errors and time-outs reported as status 3) against fake helpers, and the clean-up the real helper applies to
what jaxlib prints, against module text in the forms JAX emits. No jaxlib and no GPU are needed: the reference does the
same conversion with a jaxlib helper (Sources/PJRTMetalHLO/PJRTExecutable.swift:23-239)."""
import importlib.util
import os
import sys
import textwrap

import pytest

from metalhlo_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "metalhlo_b200", "python", "jax_plugins", "metalhlo")
MAGIC = b"ML\xefR"

ADD = "module @m {\n  func.func @main(%a: tensor<4xf32>) -> tensor<4xf32> {\n    %0 = stablehlo.add %a, %a : tensor<4xf32>\n    return %0 : tensor<4xf32>\n  }\n}\n"


def load(name):
    spec = importlib.util.spec_from_file_location(f"mhlo_plugin_{name}", os.path.join(PKG, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture()
def helper(tmp_path, monkeypatch):
    def make(body):
        path = tmp_path / "helper.py"
        path.write_text(textwrap.dedent(body))
        monkeypatch.setenv("METALHLO_PYTHON", sys.executable)
        monkeypatch.setenv("METALHLO_BYTECODE_HELPER", str(path))
        return path

    return make


def test_text_comes_back_from_the_helper(helper):
    helper(f"""
        import sys
        data = sys.stdin.buffer.read()
        assert data[:4] == b"ML\\xefR" and len(data) == 4 + 1000, len(data)
        sys.stdout.write({ADD!r})
    """)
    assert capi.bytecode_to_text(MAGIC + bytes(1000)) == ADD


def test_large_programs_do_not_deadlock_the_two_pipes(helper):
    # 3 MB in, 5 MB out: far beyond a pipe buffer in both directions; the helper answers only after reading everything
    helper("""
        import sys
        data = sys.stdin.buffer.read()
        sys.stdout.write("// %d\\n" % len(data) + "x" * 5_000_000)
    """)
    out = capi.bytecode_to_text(MAGIC + bytes(3_000_000))
    assert out.startswith("// 3000004\n") and len(out) == len("// 3000004\n") + 5_000_000


def test_helper_failures_are_reported_with_their_message(helper, monkeypatch):
    helper("""
        import sys
        sys.stderr.write("ModuleNotFoundError: No module named 'jaxlib'\\n")
        sys.exit(3)
    """)
    with pytest.raises(capi.MetalHLOError) as e:
        capi.bytecode_to_text(MAGIC + b"x")
    assert e.value.status == 3 and "exit 3" in str(e.value) and "No module named 'jaxlib'" in str(e.value)
    helper("import sys\nsys.stdin.buffer.read()\n")
    with pytest.raises(capi.MetalHLOError, match="empty output"):
        capi.bytecode_to_text(MAGIC + b"x")
    monkeypatch.setenv("METALHLO_PYTHON", "/nonexistent/python")
    with pytest.raises(capi.MetalHLOError, match="Failed to launch Python"):
        capi.bytecode_to_text(MAGIC + b"x")
    monkeypatch.setenv("METALHLO_PYTHON", sys.executable)
    monkeypatch.setenv("METALHLO_BYTECODE_HELPER", "/nonexistent/helper.py")
    with pytest.raises(capi.MetalHLOError, match="not found"):
        capi.bytecode_to_text(MAGIC + b"x")


def test_a_helper_that_exits_without_reading_does_not_kill_the_host(helper):
    helper("import sys\nsys.stdout.write('early')\nsys.exit(0)\n")
    assert capi.bytecode_to_text(MAGIC + bytes(2_000_000)) == "early"


def test_a_helper_that_hangs_is_stopped_at_the_time_limit(helper, monkeypatch):
    import time

    helper("import time\ntime.sleep(60)\n")
    monkeypatch.setenv("METALHLO_HELPER_TIMEOUT_S", "1")
    t0 = time.perf_counter()
    with pytest.raises(capi.MetalHLOError, match="did not finish within 1 s"):
        capi.bytecode_to_text(MAGIC + b"x")
    assert time.perf_counter() - t0 < 10


def test_text_is_not_bytecode(helper):
    with pytest.raises(capi.MetalHLOError) as e:
        capi.bytecode_to_text(b"module {}")
    assert e.value.status == 10


JAX_PRINTED = '''
module @jit_f attributes {jax.uses_shape_polymorphism = false, mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  sdy.mesh @mesh = <["x"=1]>
  func.func public @main(%arg0: tensor<8x16xf32> {mhlo.layout_mode = "default", sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>}, %arg1: tensor<16xf32>) -> (tensor<8x16xf32> {jax.result_info = "result"}) {
    %0 = sdy.sharding_constraint %arg0 <@mesh, [{"x"}, {}]> : tensor<8x16xf32>
    %1 = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<16xf32>) -> tensor<8x16xf32>
    %2 = stablehlo.add %0, %1 : tensor<8x16xf32>
    %3 = stablehlo.composite "chlo.erf" %2 {decomposition = @erf_impl, version = 1 : i32} : (tensor<8x16xf32>) -> tensor<8x16xf32>
    %4 = call @inner(%3) : (tensor<8x16xf32>) -> tensor<8x16xf32>
    return %4 : tensor<8x16xf32>
  }
  func.func private @erf_impl(%arg0: tensor<8x16xf32>) -> tensor<8x16xf32> {
    %0 = stablehlo.tanh %arg0 : tensor<8x16xf32>
    return %0 : tensor<8x16xf32>
  }
  func.func private @inner(%arg0: tensor<8x16xf32>) -> tensor<8x16xf32> {
    %0 = "stablehlo.dynamic_slice"(%arg0, %c, %c) <{slice_sizes = array<i64: 8, 16>}> : (tensor<8x16xf32>, tensor<i32>, tensor<i32>) -> tensor<8x16xf32>
    return %0 : tensor<8x16xf32>
  }
}
'''


def test_clean_removes_what_jax_adds_and_the_result_parses():
    import numpy as np

    from oracle import interp

    helper_mod = load("bytecode_to_text")
    text = JAX_PRINTED.replace("(%arg0, %c, %c)", "(%arg0, %z, %z)").replace(
        '    %0 = "stablehlo.dynamic_slice"', '    %z = stablehlo.constant dense<0> : tensor<i32>\n    %0 = "stablehlo.dynamic_slice"')
    cleaned = helper_mod.clean(text)
    for gone in ("attributes {", "sdy.", "jax.result_info", "mhlo.layout_mode", "stablehlo.composite"):
        assert gone not in cleaned, gone
    assert "func.call @erf_impl(%2)" in cleaned and "stablehlo.add %arg0, %1" in cleaned
    # the backend's own front end takes it from here: calls inlined, one flat function
    flat = capi.optimize_text(cleaned, 0)
    assert "func.call" not in flat and "stablehlo.tanh" in flat
    x = np.arange(128, dtype=np.float32).reshape(8, 16) / 100
    b = np.linspace(-1, 1, 16).astype(np.float32)
    np.testing.assert_allclose(interp.evaluate(flat, [x, b])[0], np.tanh((x + b).astype(np.float64)), rtol=1e-6)


def test_the_real_helper_refuses_input_that_is_not_bytecode(monkeypatch):
    import subprocess

    res = subprocess.run([sys.executable, os.path.join(PKG, "bytecode_to_text.py")], input=b"module {}", capture_output=True)
    assert res.returncode == 2 and b"does not hold MLIR bytecode" in res.stderr


def test_plugin_package_finds_the_library_and_prepares_the_helper_environment(monkeypatch):
    pkg = load("__init__")
    monkeypatch.delenv("METALHLO_PLUGIN_PATH", raising=False)
    path = pkg.find_plugin()
    assert path.endswith("pjrt_plugin_metalhlo_b200.so") and os.path.isfile(path)
    monkeypatch.setenv("METALHLO_PLUGIN_PATH", "/nonexistent.so")
    assert pkg.find_plugin() == path  # a wrong override falls through to the in-tree build
    monkeypatch.delenv("METALHLO_PYTHON", raising=False)
    monkeypatch.delenv("METALHLO_BYTECODE_HELPER", raising=False)
    pkg.prepare_environment()
    assert os.environ["METALHLO_PYTHON"] == sys.executable
    assert os.path.isfile(os.environ["METALHLO_BYTECODE_HELPER"])
    assert pkg.PLUGIN_NAME == "metalhlo"
