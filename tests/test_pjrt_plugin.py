"""The PJRT plugin, driven through ``GetPjrtApi`` by its C++ self-test the way a PJRT host drives it.

The cases follow the reference's plugin tests (Tests/PJRTMetalHLOTests/PJRTPluginTests.swift:160-460): table and
version, error lifecycle, client and platform name, device attributes, host/device round trip, compile + execute
``stablehlo.add`` -> [6, 8, 10, 12], serialize / deserialize. The host-only subset runs without a GPU.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "metalhlo_b200", "lib")
PLUGIN = os.path.join(LIBDIR, "pjrt_plugin_metalhlo_b200.so")
SELFTEST = os.path.join(LIBDIR, "pjrt_selftest")

HOST_CASES = ["load", "api_version", "required_functions", "error_lifecycle", "plugin_initialize", "topology_platform_name",
              "deserialize_rejects_null"]
DEVICE_CASES = ["client_create", "platform_name", "one_device", "memory_kind_device", "device_attributes", "buffer_round_trip",
                "event_on_ready", "strided_host_buffer", "copy_raw_to_host", "compile_add", "execute_add", "executable_outputs",
                "serialize_format", "deserialize_and_execute", "fingerprint", "execute_softmax", "execute_loop_with_call", "complex_buffers_and_rfft", "compile_error_reported",
                "bytecode_refused", "delete_and_memory_stats", "client_destroy"]


def run_selftest(mode):
    assert os.path.exists(PLUGIN) and os.path.exists(SELFTEST), "PJRT plugin not built: run __graft_entry__.build()"
    res = subprocess.run([SELFTEST, PLUGIN, mode], capture_output=True, text=True, timeout=300)
    lines = res.stdout.splitlines()
    passed = [ln.split()[1] for ln in lines if ln.startswith("PASS ")]
    failed = [ln for ln in lines if ln.startswith("FAIL ")]
    return res, passed, failed


def test_plugin_table_and_errors_without_a_gpu():
    res, passed, failed = run_selftest("host")
    assert not failed, failed
    assert res.returncode == 0, res.stdout + res.stderr
    assert passed == HOST_CASES


def test_plugin_exports_only_the_entry_point():
    out = subprocess.run(["nm", "-D", "--defined-only", PLUGIN], capture_output=True, text=True, check=True).stdout
    strong = [ln.split()[-1] for ln in out.splitlines() if ln.split()[1] in ("T", "D", "B")]
    assert strong == ["GetPjrtApi"], strong


@pytest.mark.gpu
def test_plugin_end_to_end_on_the_gpu():
    res, passed, failed = run_selftest("device")
    assert not failed, failed
    assert res.returncode == 0, res.stdout + res.stderr
    assert passed == HOST_CASES + DEVICE_CASES
