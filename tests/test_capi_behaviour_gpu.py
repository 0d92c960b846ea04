"""Behaviour of the mhlo_* C API, case by case as the reference's own API tests state it
(Tests/MetalHLOTests/CAPITests.swift:15-760), followed by the failure paths: errors injected on the host (bad
arguments, wrong counts and sizes, an allocator that refuses) and a bounded device wait that runs out and is reported
as a status. No case here faults, traps or hangs the GPU.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ADD_4 = """
module @add {
  func.func @main(%a: tensor<4xf32>, %b: tensor<4xf32>) -> (tensor<4xf32>) {
    %0 = stablehlo.add %a, %b : tensor<4xf32>
    return %0 : tensor<4xf32>
  }
}
"""
MATMUL_2x3x4 = """
module @types {
  func.func @main(%a: tensor<2x3xf32>, %b: tensor<3x4xf32>) -> (tensor<2x4xf32>) {
    %0 = stablehlo.dot_general %a, %b, contracting_dims = [1] x [0] : (tensor<2x3xf32>, tensor<3x4xf32>) -> tensor<2x4xf32>
    return %0 : tensor<2x4xf32>
  }
}
"""
GEMM_256 = """
func.func @main(%a: tensor<256x256xbf16>, %b: tensor<256x256xbf16>) -> tensor<256x256xbf16> {
  %0 = stablehlo.dot_general %a, %b, contracting_dims = [1] x [0] : (tensor<256x256xbf16>, tensor<256x256xbf16>) -> tensor<256x256xbf16>
  return %0 : tensor<256x256xbf16>
}
"""


@pytest.fixture(scope="module")
def api():
    from metalhlo_b200 import capi

    return capi


@pytest.fixture()
def client(api):
    return api.Client()


def raw_execute(api, exe, inputs, fn="mhlo_execute", extra=()):
    arr = (C.c_void_p * max(len(inputs), 1))(*[b._h if b is not None else None for b in inputs])
    outs = (C.c_void_p * max(exe.output_count, 1))()
    n = C.c_int32(-1)
    status = getattr(api.lib, fn)(exe._h, arr, len(inputs), outs, C.byref(n), *extra)
    return status, [api.Buffer(outs[i], exe._client) for i in range(max(n.value, 0))] if status == 0 else []


# ---- CAPITests.swift, restated ---------------------------------------------------------------------------------------

def test_version_and_element_type_sizes(api):
    assert api.lib.mhlo_version() == b"0.2.0"                                   # :15-23
    assert [api.lib.mhlo_element_type_size(t) for t in range(9)] == [2, 4, 8, 2, 0, 1, 2, 4, 8]  # :25-36


def test_client_create_destroy_and_device_name(client):
    assert client.device_name                                                    # :38-56


def test_compile_and_counts(client):
    exe = client.compile(ADD_4)
    assert (exe.input_count, exe.output_count) == (2, 1)                          # :58-89


def test_buffer_create_read(api, client):
    data = np.array([1, 2, 3, 4], np.float32)
    b = client.buffer(data)
    assert api.lib.mhlo_buffer_rank(b._h) == 1 and b.element_type == api.F32 and b.byte_count == 16  # :91-145
    assert b.shape == (4,)
    np.testing.assert_array_equal(b.to_numpy(), data)


def test_execute_simple_add(client):
    a, b = np.array([1, 2, 3, 4], np.float32), np.array([5, 6, 7, 8], np.float32)
    outs = client.compile(ADD_4).execute([client.buffer(a), client.buffer(b)])
    assert len(outs) == 1
    np.testing.assert_array_equal(outs[0].to_numpy(), [6, 8, 10, 12])             # :147-219


def test_execute_with_timing(client):
    a = np.array([1, 2, 3, 4], np.float32)
    outs, (enc, gpu, tot) = client.compile(ADD_4).execute([client.buffer(a), client.buffer(a)], timing=True)
    assert len(outs) == 1 and enc >= 0 and gpu >= 0 and tot >= 0                  # :221-302
    assert tot >= gpu and tot < 5.0
    np.testing.assert_array_equal(outs[0].to_numpy(), 2 * a)


def test_error_handling_and_clear(api, client):
    exe = C.c_void_p(1)
    status = api.lib.mhlo_compile(client._h, b"invalid mlir text", C.byref(exe))
    assert status != 0 and not exe.value                                          # :304-328
    assert api.lib.mhlo_get_last_error()
    api.lib.mhlo_clear_error()
    assert api.lib.mhlo_get_last_error() is None


def test_tensor_types_from_executable(api, client):
    exe = client.compile(MATMUL_2x3x4)
    assert exe.input_type(0) == ((2, 3), api.F32)                                 # :330-383
    assert exe.input_type(1) == ((3, 4), api.F32)
    assert exe.output_type(0) == ((2, 4), api.F32)
    shape, rank, et = (C.c_int64 * 8)(), C.c_int32(), C.c_int()
    assert api.lib.mhlo_executable_input_type(exe._h, 2, shape, C.byref(rank), C.byref(et)) == 10
    assert api.lib.mhlo_executable_output_type(exe._h, -1, shape, C.byref(rank), C.byref(et)) == 10


def test_compile_config_init_and_use(api, client):
    cfg = api.CompileConfig(optimization_level=9, enable_caching=False, enable_debug_info=True, device_policy=3)
    api.lib.mhlo_compile_config_init(C.byref(cfg))
    assert (cfg.optimization_level, cfg.enable_caching, cfg.enable_debug_info, cfg.device_policy) == (2, True, False, 0)  # :385-394
    for level in range(4):                                                        # :396-428
        exe = client.compile(ADD_4, opt_level=level)
        assert (exe.input_count, exe.output_count) == (2, 1)
    h = C.c_void_p()
    assert api.lib.mhlo_compile_with_config(client._h, ADD_4.encode(), None, C.byref(h)) == 0 and h.value  # :430-456
    api.lib.mhlo_executable_destroy(h)
    cfg.optimization_level = 7
    assert api.lib.mhlo_compile_with_config(client._h, ADD_4.encode(), C.byref(cfg), C.byref(h)) == 10


def test_execution_statistics(client):
    exe = client.compile(ADD_4, caching=False)
    a = client.buffer(np.ones(4, np.float32))
    s = exe.stats()
    assert s.execution_count == 0                                                 # :458-543
    for _ in range(3):
        exe.execute([a, a])
    s = exe.stats()
    assert s.execution_count == 3 and s.total_execution_time_ms > 0 and s.last_execution_time_ms > 0
    assert abs(s.average_execution_time_ms - s.total_execution_time_ms / 3) < 1e-9
    exe.reset_stats()
    s = exe.stats()
    assert s.execution_count == 0 and s.total_execution_time_ms == 0 and s.average_execution_time_ms == 0


def test_ane_availability_is_a_bool(api):
    assert api.lib.mhlo_ane_available() in (True, False)                          # :545-551
    assert api.lib.mhlo_ane_available() is False  # no ANE behind this backend


def test_every_device_policy_compiles(api, client):
    for policy in range(5):                                                       # :553-586
        cfg = api.CompileConfig()
        api.lib.mhlo_compile_config_init(C.byref(cfg))
        cfg.device_policy = policy
        h = C.c_void_p()
        assert api.lib.mhlo_compile_with_config(client._h, ADD_4.encode(), C.byref(cfg), C.byref(h)) == 0, policy
        assert h.value
        api.lib.mhlo_executable_destroy(h)


def test_execute_with_profile(api, client):
    exe = client.compile(ADD_4)
    a, b = client.buffer(np.array([1, 2, 3, 4], np.float32)), client.buffer(np.array([5, 6, 7, 8], np.float32))
    prof = api.ExecutionProfile()
    status, outs = raw_execute(api, exe, [a, b], "mhlo_execute_with_profile", (C.byref(prof),))
    assert status == 0 and len(outs) == 1                                         # :588-687
    assert prof.partition_count >= 1 and prof.total_time_ms >= 0
    assert prof.gpu_partition_count + prof.ane_partition_count == prof.partition_count
    assert prof.used_ane is False and prof.ane_time_ms == 0
    np.testing.assert_array_equal(outs[0].to_numpy(), [6, 8, 10, 12])
    status, outs = raw_execute(api, exe, [a, b], "mhlo_execute_with_profile", (None,))  # :689-760: NULL profile
    assert status == 0
    np.testing.assert_array_equal(outs[0].to_numpy(), [6, 8, 10, 12])


def test_compile_n_takes_a_length(api, client):
    text = ADD_4.encode() + b"this tail is not part of the program"
    h = C.c_void_p()
    assert api.lib.mhlo_compile_n(client._h, text, len(ADD_4.encode()), C.byref(h)) == 0
    assert api.lib.mhlo_executable_input_count(h) == 2
    api.lib.mhlo_executable_destroy(h)
    assert api.lib.mhlo_compile_n(client._h, text, 20, C.byref(h)) != 0  # a truncated program does not parse


def test_uninitialized_buffer_reads_as_zero_and_runs(api, client):
    shape = (C.c_int64 * 2)(3, 5)
    h = C.c_void_p()
    assert api.lib.mhlo_buffer_create_uninitialized(client._h, shape, 2, api.I32, C.byref(h)) == 0
    b = api.Buffer(h.value, client)
    assert b.shape == (3, 5) and b.element_type == api.I32 and b.byte_count == 60
    np.testing.assert_array_equal(b.to_numpy(), np.zeros((3, 5), np.int32))
    assert api.lib.mhlo_buffer_create_uninitialized(client._h, shape, 2, 99, C.byref(h)) == 10


# ---- failure paths, injected on the host -------------------------------------------------------------------------------

def test_wrong_input_count_type_and_null_inputs(api, client):
    exe = client.compile(ADD_4)
    a = client.buffer(np.ones(4, np.float32))
    status, _ = raw_execute(api, exe, [a])
    assert status == 7 and b"expected 2, got 1" in api.lib.mhlo_get_last_error()
    wrong_shape = client.buffer(np.ones(5, np.float32))
    status, _ = raw_execute(api, exe, [a, wrong_shape])
    assert status == 7 and b"tensor<5xf32>" in api.lib.mhlo_get_last_error()
    wrong_type = client.buffer(np.ones(4, np.int32))
    status, _ = raw_execute(api, exe, [a, wrong_type])
    assert status == 7
    status, _ = raw_execute(api, exe, [a, None])
    assert status == 10
    n = C.c_int32()
    assert api.lib.mhlo_execute(None, None, 0, None, C.byref(n)) == 10
    # a good call afterwards still works: failures leave the executable usable
    assert raw_execute(api, exe, [a, a])[0] == 0


def test_buffer_size_mismatch_and_small_host_destination(api, client):
    data = np.ones(4, np.float32)
    shape = (C.c_int64 * 1)(4)
    h = C.c_void_p()
    assert api.lib.mhlo_buffer_create(client._h, data.ctypes.data, 12, shape, 1, api.F32, C.byref(h)) == 6
    assert b"expected 16" in api.lib.mhlo_get_last_error() and not h.value
    assert api.lib.mhlo_buffer_create(client._h, None, 16, shape, 1, api.F32, C.byref(h)) == 10
    b = client.buffer(data)
    small = np.empty(3, np.float32)
    assert api.lib.mhlo_buffer_to_host(b._h, small.ctypes.data, 12) == 9
    assert api.lib.mhlo_buffer_to_host(None, small.ctypes.data, 12) == 10


def test_unsupported_operation_is_reported_as_such(api, client):
    h = C.c_void_p()
    # transcendental functions of complex values are outside the operator surface
    text = (b"func.func @main(%a: tensor<8xcomplex<f32>>) -> tensor<8xcomplex<f32>> { %0 = stablehlo.tanh %a : tensor<8xcomplex<f32>>\n"
            b" return %0 : tensor<8xcomplex<f32>> }")
    status = api.lib.mhlo_compile(client._h, text, C.byref(h))
    assert status == 4 and not h.value and b"complex" in api.lib.mhlo_get_last_error()


def test_allocator_refusal_fails_the_call_and_nothing_else(api, client):
    from metalhlo_b200 import cuda

    exe = client.compile(ADD_4)
    a = client.buffer(np.array([1, 2, 3, 4], np.float32))
    try:
        cuda.lib.mhlo_cuda_debug_refuse_allocs(1)
        shape = (C.c_int64 * 1)(1 << 20)
        h = C.c_void_p()
        big = np.zeros(1 << 20, np.float32)
        assert api.lib.mhlo_buffer_create(client._h, big.ctypes.data, big.nbytes, shape, 1, api.F32, C.byref(h)) == 6
        assert b"refused" in api.lib.mhlo_get_last_error() and not h.value
        cuda.lib.mhlo_cuda_debug_refuse_allocs(1)
        status, _ = raw_execute(api, exe, [a, a])  # the output buffer cannot be allocated
        assert status == 6
    finally:
        cuda.lib.mhlo_cuda_debug_refuse_allocs(0)
    status, outs = raw_execute(api, exe, [a, a])
    assert status == 0
    np.testing.assert_array_equal(outs[0].to_numpy(), [2, 4, 6, 8])


def test_a_recorded_device_error_fails_the_execution_once(api, client):
    """The contraction kernels bound every wait and record a code instead of hanging; mhlo_execute must turn a recorded
    code into MHLO_ERROR_EXECUTION_FAILED. The word is written from the host here."""
    import torch

    from metalhlo_b200 import cuda

    g = torch.Generator().manual_seed(1)
    a = (torch.randn(256, 256, generator=g) / 16).to(torch.bfloat16)
    exe = client.compile(GEMM_256, opt_level=2)
    bufs = [client.buffer(a), client.buffer(a)]
    assert raw_execute(api, exe, bufs)[0] == 0
    for which, code in ((0, 3), (1, 8)):
        assert cuda.lib.mhlo_cuda_debug_store_device_error(which, code) == 0
        status, outs = raw_execute(api, exe, bufs)
        assert status == 8 and outs == []
        msg = api.lib.mhlo_get_last_error().decode()
        assert f"code {code if which == 0 else 100 + code}" in msg, msg
        # the word was cleared with the report: the next execution is clean and correct
        status, outs = raw_execute(api, exe, bufs)
        assert status == 0
        want = (a.double() @ a.double()).numpy()
        np.testing.assert_allclose(outs[0].to_numpy().astype(np.float64), want, rtol=2e-2, atol=2e-2 * np.abs(want).mean())
    assert cuda.device_error() == 0


def test_a_wait_that_runs_out_is_a_status_not_a_hang(api, client):
    """One CTA waits 2 ms on a barrier nobody arrives at, gives up and records its code, as every wait of the contraction
    kernels does after its limit. The context stays usable."""
    import time

    import torch

    from metalhlo_b200 import cuda

    t0 = time.perf_counter()
    assert cuda.lib.mhlo_cuda_debug_wait_expiry_probe(2_000_000, None) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert cuda.lib.mhlo_cuda_debug_wait_expiry_probe(2_000_000_000, None) == 10  # limits above one second are refused
    exe = client.compile(ADD_4)
    a = client.buffer(np.ones(4, np.float32))
    status, _ = raw_execute(api, exe, [a, a])
    assert status == 8 and "code 90" in api.lib.mhlo_get_last_error().decode()
    assert raw_execute(api, exe, [a, a])[0] == 0
    assert cuda.device_error() == 0


def test_pjrt_execute_surfaces_the_same_failure():
    from metalhlo_b200 import cuda, pjrt

    host = pjrt.Host()
    exe = host.compile(ADD_4)
    a = host.buffer(np.ones(4, np.float32))
    assert cuda.lib.mhlo_cuda_debug_store_device_error(0, 4) == 0
    with pytest.raises(pjrt.PjrtError, match="code 4"):
        exe.execute([a, a])
    np.testing.assert_array_equal(exe.execute([a, a])[0].to_numpy(), 2 * np.ones(4, np.float32))
