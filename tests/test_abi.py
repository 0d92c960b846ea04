"""The C-ABI libraries load on a CPU-only machine and export every symbol their headers declare.

No compute call is made here; kernels are exercised by the ``gpu`` tests.
"""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "metalhlo_b200", "lib")

# header -> shared library that must export its functions
HEADERS = {
    "mhlo_cuda.h": "libmhlo_cuda.so",
    "metalhlo.h": "libCMetalHLO.so",
    "pjrt_plugin_metalhlo.h": "pjrt_plugin_metalhlo_b200.so",
    "pjrt_host.h": "libpjrt_host.so",
}
MIN_FUNCTIONS = {"pjrt_plugin_metalhlo.h": 1}


def declared_functions(header_path):
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    names = re.findall(r"\b((?:mhlo_|pjrt_host_|GetPjrtApi)\w*)\s*\(", text)
    return sorted(set(names))


@pytest.mark.parametrize("header", sorted(HEADERS))
def test_library_exports_every_declared_symbol(header):
    path = os.path.join(ROOT, "include", header)
    if not os.path.exists(path):
        pytest.skip(f"{header} not part of this build yet")
    so = os.path.join(LIBDIR, HEADERS[header])
    assert os.path.exists(so), f"{so} missing: run __graft_entry__.build()"
    lib = ctypes.CDLL(so)
    names = declared_functions(path)
    assert len(names) >= MIN_FUNCTIONS.get(header, 10)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"{HEADERS[header]} does not export {missing}"


def test_every_header_is_covered():
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        assert os.path.basename(h) in HEADERS, h


def test_python_binding_matches_header():
    from metalhlo_b200 import cuda

    declared = set(declared_functions(os.path.join(ROOT, "include", "mhlo_cuda.h")))
    assert set(cuda.declared_symbols()) == declared


def test_pjrt_host_binding_matches_header():
    from metalhlo_b200 import pjrt

    declared = set(declared_functions(os.path.join(ROOT, "include", "pjrt_host.h")))
    assert set(pjrt.declared_symbols()) == declared


def test_pjrt_host_reports_the_plugin_error_without_a_gpu():
    import torch

    from metalhlo_b200 import pjrt

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(pjrt.PjrtError, match="No CUDA device"):
        pjrt.Host()
    with pytest.raises(pjrt.PjrtError, match="dlopen failed"):
        pjrt.Host("/nonexistent/plugin.so")


def test_no_device_calls_report_status_not_crash():
    import torch

    from metalhlo_b200 import cuda

    assert cuda.lib.mhlo_cuda_version().decode().startswith("mhlo-cuda")
    assert cuda.lib.mhlo_cuda_dtype_size(cuda.BF16) == 2 and cuda.lib.mhlo_cuda_dtype_size(99) == 0
    if not torch.cuda.is_available():
        n = ctypes.c_int(-1)
        status = cuda.lib.mhlo_cuda_device_count(ctypes.byref(n))
        assert (status, n.value) == (1, 0) or (status == 0 and n.value == 0)
    # argument validation happens before any CUDA work
    assert cuda.lib.mhlo_cuda_layer_norm(cuda.BF16, None, None, None, None, 4, 8, 1e-5, None, None) == 10
    assert "null" in cuda.last_error()
    assert cuda.lib.mhlo_cuda_softmax(cuda.I32, 1, 1, 1, 1, 1, None, None) == 4
