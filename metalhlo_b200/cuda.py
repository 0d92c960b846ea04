"""ctypes binding of ``libmhlo_cuda.so`` (declared in ``include/mhlo_cuda.h``).

This is the thin Python view of the device runtime used by the tests and the benchmark. It adds nothing to
the C ABI: every function takes raw device pointers (for example ``torch.Tensor.data_ptr()``), sizes and a
CUDA stream handle, and a non-zero status raises :class:`MhloCudaError` with the library's message.
There is no fallback: if the shared library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmhlo_cuda.so")

F16, F32, F64, BF16, I1, I8, I16, I32, I64, UI8, UI16, UI32, UI64 = range(13)


class MhloCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"mhlo_cuda status {status}: {message}")
        self.status = status


class RowTuning(C.Structure):
    _fields_ = [("threads", C.c_int32), ("vecs_per_thread", C.c_int32), ("ctas_per_sm", C.c_int32)]


class View(C.Structure):
    _fields_ = [("base", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 8),
                ("stride", C.c_int64 * 8)]


class EwInst(C.Structure):
    _fields_ = [("op", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("c", C.c_int32), ("imm", C.c_double)]


class ConvertJob(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("count", C.c_int64), ("src_dtype", C.c_int32), ("dst_dtype", C.c_int32)]


class GatherDims(C.Structure):
    _fields_ = [("n_offset_dims", C.c_int32), ("n_collapsed", C.c_int32), ("n_operand_batching", C.c_int32),
                ("n_start_index_map", C.c_int32), ("offset_dims", C.c_int32 * 8), ("collapsed_slice_dims", C.c_int32 * 8),
                ("operand_batching_dims", C.c_int32 * 8), ("start_indices_batching_dims", C.c_int32 * 8),
                ("start_index_map", C.c_int32 * 8), ("index_vector_dim", C.c_int32), ("slice_sizes", C.c_int64 * 8)]


class Window(C.Structure):
    _fields_ = [("rank", C.c_int32), ("size", C.c_int64 * 8), ("stride", C.c_int64 * 8), ("base_dilation", C.c_int64 * 8),
                ("window_dilation", C.c_int64 * 8), ("pad_low", C.c_int64 * 8)]


class Conv(C.Structure):
    _fields_ = [("n_spatial", C.c_int32), ("reverse", C.c_int32 * 6), ("batch", C.c_int64), ("in_features", C.c_int64),
                ("out_features", C.c_int64), ("feature_group_count", C.c_int64), ("batch_group_count", C.c_int64),
                ("in_size", C.c_int64 * 6), ("kernel_size", C.c_int64 * 6), ("out_size", C.c_int64 * 6), ("stride", C.c_int64 * 6),
                ("pad_low", C.c_int64 * 6), ("lhs_dilation", C.c_int64 * 6), ("rhs_dilation", C.c_int64 * 6),
                ("in_batch_stride", C.c_int64), ("in_feature_stride", C.c_int64), ("in_spatial_stride", C.c_int64 * 6),
                ("kernel_in_stride", C.c_int64), ("kernel_out_stride", C.c_int64), ("kernel_spatial_stride", C.c_int64 * 6),
                ("out_batch_stride", C.c_int64), ("out_feature_stride", C.c_int64), ("out_spatial_stride", C.c_int64 * 6)]


class ScatterDims(C.Structure):
    _fields_ = [("n_update_window_dims", C.c_int32), ("n_inserted_window_dims", C.c_int32), ("n_input_batching", C.c_int32),
                ("n_scatter_dims_to_operand", C.c_int32), ("update_window_dims", C.c_int32 * 8),
                ("inserted_window_dims", C.c_int32 * 8), ("input_batching_dims", C.c_int32 * 8),
                ("scatter_indices_batching_dims", C.c_int32 * 8), ("scatter_dims_to_operand_dims", C.c_int32 * 8),
                ("index_vector_dim", C.c_int32)]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `make -C metalhlo_b200/csrc` "
        "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no CPU fallback."
    )

lib = C.CDLL(LIB_PATH)

_vp, _i64, _i32, _f32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_size_t
_PROTOTYPES = {
    "mhlo_cuda_version": (C.c_char_p, []),
    "mhlo_cuda_last_error": (C.c_char_p, []),
    "mhlo_cuda_dtype_size": (_sz, [C.c_int]),
    "mhlo_cuda_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "mhlo_cuda_device_set": (C.c_int, [C.c_int]),
    "mhlo_cuda_device_current": (C.c_int, [C.POINTER(C.c_int)]),
    "mhlo_cuda_device_name": (C.c_int, [C.c_int, C.c_char_p, _sz]),
    "mhlo_cuda_stream_create": (C.c_int, [C.POINTER(_vp)]),
    "mhlo_cuda_stream_destroy": (C.c_int, [_vp]),
    "mhlo_cuda_stream_sync": (C.c_int, [_vp]),
    "mhlo_cuda_alloc": (C.c_int, [_sz, C.POINTER(_vp)]),
    "mhlo_cuda_free": (C.c_int, [_vp]),
    "mhlo_cuda_host_alloc": (C.c_int, [_sz, C.POINTER(_vp)]),
    "mhlo_cuda_host_free": (C.c_int, [_vp]),
    "mhlo_cuda_upload": (C.c_int, [_vp, _vp, _sz, _vp]),
    "mhlo_cuda_download": (C.c_int, [_vp, _vp, _sz, _vp]),
    "mhlo_cuda_copy": (C.c_int, [_vp, _vp, _sz, _vp]),
    "mhlo_cuda_memset": (C.c_int, [_vp, C.c_int, _sz, _vp]),
    "mhlo_cuda_event_create": (C.c_int, [C.POINTER(_vp)]),
    "mhlo_cuda_event_destroy": (C.c_int, [_vp]),
    "mhlo_cuda_event_record": (C.c_int, [_vp, _vp]),
    "mhlo_cuda_event_elapsed_ms": (C.c_int, [_vp, _vp, C.POINTER(_f32)]),
    "mhlo_cuda_layer_norm": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _i64, _i64, _f32, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_rms_norm": (C.c_int, [C.c_int, _vp, _vp, _vp, _i64, _i64, _f32, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_softmax": (C.c_int, [C.c_int, _vp, _vp, _i64, _i64, _i64, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_elementwise": (C.c_int, [C.POINTER(View), _i32, C.POINTER(EwInst), _i32, _vp, _i32, C.POINTER(_i64), _i32, _vp]),
    "mhlo_cuda_elementwise_to_view": (C.c_int, [C.POINTER(View), _i32, C.POINTER(EwInst), _i32, C.POINTER(View), _vp]),
    "mhlo_cuda_reduce": (C.c_int, [C.POINTER(View), _i32, _i32, _vp, _vp, _vp, _i32, _vp]),
    "mhlo_cuda_add_layer_norm": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, C.c_float, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_add_rms_norm": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, C.c_float, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_fft_axis": (C.c_int, [C.c_int, C.c_int, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mhlo_cuda_fft_axis_scratch_bytes": (_i64, [C.c_int, _i64, _i64, _i64]),
    "mhlo_cuda_fft_axis_long": (C.c_int, [C.c_int, C.c_int, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mhlo_cuda_add_layer_norm_rows": (C.c_int, [C.c_int, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, C.c_float, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_add_rms_norm_rows": (C.c_int, [C.c_int, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, C.c_float, C.POINTER(RowTuning), _vp]),
    "mhlo_cuda_graph_capture_begin": (C.c_int, [_vp]),
    "mhlo_cuda_graph_capture_end": (C.c_int, [_vp, C.POINTER(_vp)]),
    "mhlo_cuda_graph_launch": (C.c_int, [_vp, _vp]),
    "mhlo_cuda_graph_destroy": (C.c_int, [_vp]),
    "mhlo_cuda_ipc_export": (C.c_int, [_vp, C.c_char_p]),
    "mhlo_cuda_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(_vp)]),
    "mhlo_cuda_ipc_close": (C.c_int, [_vp]),
    "mhlo_cuda_gemm_all_gather": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), C.POINTER(_vp), _i32, _i32, _i64, _i64, _i64,
                                            _vp, _i32, _vp]),
    "mhlo_cuda_gemm_all_gather_tuned": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), C.POINTER(_vp), _i32, _i32, _i64, _i64,
                                                  _i64, _vp, _i32, _vp, _i32, _vp]),
    "mhlo_cuda_gemm_residual": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp,
                                          _vp, _vp]),
    "mhlo_cuda_event_sync": (C.c_int, [_vp]),
    "mhlo_cuda_stream_wait_event": (C.c_int, [_vp, _vp]),
    "mhlo_cuda_stream_host_callback": (C.c_int, [_vp, _vp, _vp]),
    "mhlo_cuda_conv2d_nhwc": (C.c_int, [_i32, _i32, _vp, _vp, _vp] + [_i64] * 13 + [_vp, _i32, _vp]),
    "mhlo_cuda_conv2d_nhwc_strided": (C.c_int, [_i32, _i32, _vp, _vp, _vp] + [_i64] * 15 + [_vp, _i32, _vp]),
    "mhlo_cuda_rng": (C.c_int, [_i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "mhlo_cuda_rng_bit_generator": (C.c_int, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "mhlo_cuda_peer_barrier": (C.c_int, [C.POINTER(_vp), _i32, _i32, C.c_uint64, C.c_uint64, _vp]),
    "mhlo_cuda_convert_many": (C.c_int, [C.POINTER(ConvertJob), _i32, _vp]),
    "mhlo_cuda_reduce_static_scratch": (C.c_int, [C.POINTER(View), _i32, _i32, _vp, _vp, _vp, _i32, _i32, _vp]),
    "mhlo_cuda_gather": (C.c_int, [_vp, _i32, C.POINTER(_i64), _i32, _vp, _i32, C.POINTER(_i64), _i32, C.POINTER(GatherDims),
                                   _vp, C.POINTER(_i64), _i32, _vp]),
    "mhlo_cuda_convolution": (C.c_int, [_i32, _vp, _vp, _vp, C.POINTER(Conv), _vp]),
    "mhlo_cuda_im2col": (C.c_int, [_i32, _vp, _vp, _i64, C.POINTER(Conv), _vp]),
    "mhlo_cuda_reduce_window": (C.c_int, [C.POINTER(View), C.POINTER(Window), _i32, _vp, _vp, C.POINTER(_i64), _vp]),
    "mhlo_cuda_select_and_scatter": (C.c_int, [C.POINTER(View), _vp, C.POINTER(_i64), _vp, C.POINTER(Window), _i32, _i32, _vp, _vp]),
    "mhlo_cuda_scatter": (C.c_int, [_vp, _i32, C.POINTER(_i64), _i32, _vp, _i32, C.POINTER(_i64), _i32, _vp, C.POINTER(_i64), _i32,
                                    C.POINTER(ScatterDims), _i32, _vp]),
    "mhlo_cuda_sort_scratch_bytes": (_i64, [C.POINTER(_i64), _i32, _i32]),
    "mhlo_cuda_sort": (C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i32), _i32, C.POINTER(_i64), _i32, _i32, _i32, _vp, _i64, _vp]),
    "mhlo_cuda_dynamic_slice": (C.c_int, [_vp, _i32, C.POINTER(_i64), _i32, C.POINTER(_vp), _i32, C.POINTER(_i64), _vp, _vp]),
    "mhlo_cuda_dynamic_update_slice": (C.c_int, [_vp, _i32, C.POINTER(_i64), _i32, _vp, C.POINTER(_i64), C.POINTER(_vp), _i32, _vp]),
    "mhlo_cuda_dot_strided": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "mhlo_cuda_gemm": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _i64, _i64, _i64, _i64, _i64, _vp,
                                 _i32, _vp]),
    "mhlo_cuda_cholesky": (C.c_int, [_i32, _vp, _vp, _i64, _i64, _i32, _vp]),
    "mhlo_cuda_triangular_solve": (C.c_int, [_i32, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp]),
    "mhlo_cuda_kernel_lookup": (C.c_int, [C.c_char_p, _i32, C.POINTER(_i32)]),
    "mhlo_cuda_plan_create": (C.c_int, [_vp, _i32, _i32, _i32, _i64, C.c_char_p, _i64, C.POINTER(_vp)]),
    "mhlo_cuda_plan_execute": (C.c_int, [_vp, C.POINTER(_vp), _i32, C.POINTER(_vp), _i32, _vp]),
    "mhlo_cuda_plan_destroy": (C.c_int, [_vp]),
    "mhlo_cuda_tuner_measure": (C.c_int, [_vp, C.POINTER(_vp), _i32, C.POINTER(_vp), _i32, _i32, _i32, C.POINTER(_f32)]),
    "mhlo_cuda_comm_init": (C.c_int, [_i32, C.POINTER(_vp)]),
    "mhlo_cuda_comm_size": (C.c_int, [_vp]),
    "mhlo_cuda_all_gather": (C.c_int, [_vp, C.POINTER(_vp), _i64]),
    "mhlo_cuda_comm_destroy": (C.c_int, [_vp]),
    "mhlo_cuda_gemm_tuned": (C.c_int, [_i32, _i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _i64, _i64, _i64, _i64, _i64, _vp,
                                       _i32, _vp, _vp]),
    "mhlo_cuda_device_error": (C.c_int, [C.POINTER(_i32)]),
    "mhlo_cuda_device_error_fetch": (C.c_int, [_vp]),
    "mhlo_cuda_device_error_take": (C.c_int, [C.POINTER(_i32)]),
    "mhlo_cuda_debug_store_device_error": (C.c_int, [_i32, _i32]),
    "mhlo_cuda_debug_refuse_allocs": (C.c_int, [_i32]),
    "mhlo_cuda_debug_wait_expiry_probe": (C.c_int, [C.c_uint64, _vp]),
    "mhlo_cuda_attention": (C.c_int, [_i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _vp,
                                      C.POINTER(_i64), _i64, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "mhlo_cuda_attention_tuned": (C.c_int, [_i32, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _vp, _vp,
                                            C.POINTER(_i64), _i64, _i64, _i64, _i64, _i64, _f32, _i32, _vp, _vp]),
}
for _name, (_res, _args) in _PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


def declared_symbols() -> list[str]:
    """Names bound above; the CPU test suite checks them against ``include/mhlo_cuda.h``."""
    return sorted(_PROTOTYPES)


def last_error() -> str:
    return lib.mhlo_cuda_last_error().decode()


def check(status: int) -> None:
    if status != 0:
        raise MhloCudaError(status, last_error())


def torch_dtype_code(dtype) -> int:
    import torch

    return {torch.float16: F16, torch.float32: F32, torch.float64: F64, torch.bfloat16: BF16, torch.bool: I1,
            torch.int8: I8, torch.int16: I16, torch.int32: I32, torch.int64: I64, torch.uint8: UI8}[dtype]


def _stream(stream=None) -> int:
    if stream is not None:
        return int(stream)
    import torch

    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _tuning(t):
    if t is None:
        return None
    if isinstance(t, RowTuning):
        return C.byref(t)
    return C.byref(RowTuning(*t))


def layer_norm(x, gamma, beta, eps: float = 1e-5, out=None, tuning=None, stream=None):
    """LayerNorm over the last axis of a contiguous CUDA tensor (see ``mhlo_cuda_layer_norm``)."""
    import torch

    assert x.is_cuda and x.is_contiguous()
    out = torch.empty_like(x) if out is None else out
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    check(lib.mhlo_cuda_layer_norm(torch_dtype_code(x.dtype), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), rows,
                                   hidden, eps, _tuning(tuning), _stream(stream)))
    return out


def rms_norm(x, gamma, eps: float = 1e-5, out=None, tuning=None, stream=None):
    import torch

    assert x.is_cuda and x.is_contiguous()
    out = torch.empty_like(x) if out is None else out
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    check(lib.mhlo_cuda_rms_norm(torch_dtype_code(x.dtype), _ptr(x), _ptr(gamma), _ptr(out), rows, hidden, eps,
                                 _tuning(tuning), _stream(stream)))
    return out


def add_layer_norm(x, residual, gamma, beta, eps: float = 1e-5, tuning=None, stream=None):
    """(x + residual, LayerNorm(x + residual)) in one pass (see ``mhlo_cuda_add_layer_norm``)."""
    import torch

    assert x.is_cuda and x.is_contiguous() and residual.is_contiguous()
    total, out = torch.empty_like(x), torch.empty_like(x)
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    if residual.shape != x.shape:  # a block of rows repeated down x (``mhlo_cuda_add_layer_norm_rows``)
        check(lib.mhlo_cuda_add_layer_norm_rows(torch_dtype_code(x.dtype), _ptr(x), _ptr(residual), residual.numel() // hidden, _ptr(gamma),
                                                _ptr(beta), _ptr(total), _ptr(out), rows, hidden, eps, _tuning(tuning), _stream(stream)))
        return total, out
    check(lib.mhlo_cuda_add_layer_norm(torch_dtype_code(x.dtype), _ptr(x), _ptr(residual), _ptr(gamma), _ptr(beta), _ptr(total), _ptr(out),
                                       rows, hidden, eps, _tuning(tuning), _stream(stream)))
    return total, out


def add_rms_norm(x, residual, gamma, eps: float = 1e-5, tuning=None, stream=None):
    import torch

    assert x.is_cuda and x.is_contiguous() and residual.is_contiguous()
    total, out = torch.empty_like(x), torch.empty_like(x)
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    if residual.shape != x.shape:
        check(lib.mhlo_cuda_add_rms_norm_rows(torch_dtype_code(x.dtype), _ptr(x), _ptr(residual), residual.numel() // hidden, _ptr(gamma),
                                              _ptr(total), _ptr(out), rows, hidden, eps, _tuning(tuning), _stream(stream)))
        return total, out
    check(lib.mhlo_cuda_add_rms_norm(torch_dtype_code(x.dtype), _ptr(x), _ptr(residual), _ptr(gamma), _ptr(total), _ptr(out), rows, hidden,
                                     eps, _tuning(tuning), _stream(stream)))
    return total, out


def device_error() -> int:
    """Synchronises and returns the tensor-core kernels' error word (0 = no bounded wait expired)."""
    code = C.c_int32(0)
    lib.mhlo_cuda_device_error(C.byref(code))
    return code.value


EPILOGUES = {"none": 0, "relu": 1, "gelu_tanh": 2, "gelu_erf": 3, "silu": 4, "tanh": 5, "sigmoid": 6}


def _i64s(vals):
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])


class Binding(C.Structure):
    _fields_ = [("source", C.c_int32), ("index", C.c_int32), ("offset", C.c_int64)]


class PlanOp(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("dtype", C.c_int32), ("out_dtype", C.c_int32), ("args", Binding * 6), ("dims", C.c_int64 * 6),
                ("strides", C.c_int64 * 16), ("scalars", C.c_float * 2), ("flags", C.c_int32 * 2), ("tuning", C.c_int32 * 4)]


SRC_NONE, SRC_INPUT, SRC_OUTPUT, SRC_UNIFIED, SRC_CONSTANT = range(5)


def plan_op(kernel_name, dtype, args, dims, strides=(), scalars=(), flags=(), tuning=(), out_dtype=None) -> PlanOp:
    """One op of a dispatch plan. args: (source, index, offset) triples in the kernel's argument order."""
    k = C.c_int32()
    check(lib.mhlo_cuda_kernel_lookup(kernel_name.encode(), dtype, C.byref(k)))
    op = PlanOp()
    op.kernel, op.dtype, op.out_dtype = k.value, dtype, dtype if out_dtype is None else out_dtype
    for i, a in enumerate(args):
        op.args[i] = Binding(*a)
    for name, vals in (("dims", dims), ("strides", strides), ("scalars", scalars), ("flags", flags), ("tuning", tuning)):
        arr = getattr(op, name)
        for i, v in enumerate(vals):
            arr[i] = v
    return op


class Plan:
    """mhlo_cuda_plan_*: a list of kernel dispatches with their buffer bindings, an arena and a constant pool."""

    def __init__(self, ops, n_inputs, n_outputs, arena_bytes=0, constants: bytes = b""):
        arr = (PlanOp * max(len(ops), 1))(*ops)
        h = C.c_void_p()
        check(lib.mhlo_cuda_plan_create(arr, len(ops), n_inputs, n_outputs, arena_bytes, constants if constants else None, len(constants), C.byref(h)))
        self._h = h.value

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.mhlo_cuda_plan_destroy(self._h)
            self._h = None

    def _lists(self, inputs, outputs):
        return (C.c_void_p * max(len(inputs), 1))(*[_ptr(t) for t in inputs]), (C.c_void_p * max(len(outputs), 1))(*[_ptr(t) for t in outputs])

    def execute(self, inputs, outputs, stream=None):
        ins, outs = self._lists(inputs, outputs)
        check(lib.mhlo_cuda_plan_execute(self._h, ins, len(inputs), outs, len(outputs), _stream(stream)))

    def measure(self, inputs, outputs, warmup=5, iterations=20) -> float:
        ins, outs = self._lists(inputs, outputs)
        ms = C.c_float()
        check(lib.mhlo_cuda_tuner_measure(self._h, ins, len(inputs), outs, len(outputs), warmup, iterations, C.byref(ms)))
        return ms.value


class GemmTuning(C.Structure):
    _fields_ = [("tile_n", C.c_int32), ("stages", C.c_int32), ("cta_group", C.c_int32), ("reserved", C.c_int32)]


def gemm(a, b, bias=None, epilogue: str = "none", out_dtype=None, trans_a: bool = False, trans_b: bool = False,
         out=None, stream=None, tuning=None, residual=None):
    """C[..., M, N] = act(A . B + bias) through ``mhlo_cuda_gemm`` (+ residual, without activation: ``mhlo_cuda_gemm_residual``).

    a: [batch..., M, K] (or [batch..., K, M] with trans_a), b: [batch..., K, N] (or [batch..., N, K] with trans_b);
    up to two leading batch dimensions, both operands dense CUDA tensors of the same dtype.
    """
    import torch

    assert a.is_cuda and b.is_cuda and a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype
    batch = list(a.shape[:-2])
    assert len(batch) <= 2 and list(b.shape[:-2]) == batch
    b0, b1 = ([1, 1] + batch)[-2:]
    m, k = (a.shape[-1], a.shape[-2]) if trans_a else (a.shape[-2], a.shape[-1])
    n = b.shape[-2] if trans_b else b.shape[-1]
    a_mat, b_mat = a.shape[-2] * a.shape[-1], b.shape[-2] * b.shape[-1]
    a_str = [b1 * a_mat, a_mat] + ([1, m] if trans_a else [k, 1])
    b_str = [b1 * b_mat, b_mat] + ([1, k] if trans_b else [n, 1])
    out_dtype = a.dtype if out_dtype is None else out_dtype
    if out is None:
        out = torch.empty(batch + [m, n], dtype=out_dtype, device=a.device)
    if residual is not None:  # C = A . B + bias + residual, one rounding: mhlo_cuda_gemm_residual
        assert epilogue == "none" and residual.is_contiguous() and tuple(residual.shape) == tuple(out.shape) and residual.dtype == out.dtype
        t = GemmTuning(*tuning, 0) if tuning is not None else None
        check(lib.mhlo_cuda_gemm_residual(torch_dtype_code(a.dtype), torch_dtype_code(out_dtype), _ptr(a), _i64s(a_str), _ptr(b), _i64s(b_str),
                                          _ptr(out), b0, b1, m, n, k, _ptr(bias), _ptr(residual), None if t is None else C.addressof(t),
                                          _stream(stream)))
        return out
    if tuning is not None:  # (tile_n, stages, cta_group): mhlo_cuda_gemm_tuned
        t = GemmTuning(*tuning, 0)
        check(lib.mhlo_cuda_gemm_tuned(torch_dtype_code(a.dtype), torch_dtype_code(out_dtype), _ptr(a), _i64s(a_str), _ptr(b), _i64s(b_str),
                                       _ptr(out), b0, b1, m, n, k, _ptr(bias), EPILOGUES[epilogue], C.addressof(t), _stream(stream)))
        return out
    check(lib.mhlo_cuda_gemm(torch_dtype_code(a.dtype), torch_dtype_code(out_dtype), _ptr(a), _i64s(a_str), _ptr(b),
                             _i64s(b_str), _ptr(out), b0, b1, m, n, k, _ptr(bias), EPILOGUES[epilogue], _stream(stream)))
    return out


class AttentionTuning(C.Structure):
    _fields_ = [("tile_order", C.c_int32), ("reserved", C.c_int32 * 3)]


def attention(q, k, v, scale: float, causal: bool = False, mask=None, layout: str = "BHSD", out=None, stream=None, tile_order=None):
    """Fused attention through ``mhlo_cuda_attention``. q/k/v are dense [B,H,S,D] (layout "BHSD") or [B,S,H,D] ("BSHD")."""
    import torch

    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    if layout == "BHSD":
        B, H, Sq, D = q.shape
        Sk = k.shape[2]
        strides = lambda S: [H * S * D, S * D, D]
    else:
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        strides = lambda S: [S * H * D, D, H * D]
    out = torch.empty_like(q) if out is None else out
    if tile_order is not None:  # mhlo_cuda_attention_tuned
        t = AttentionTuning(tile_order)
        check(lib.mhlo_cuda_attention_tuned(torch_dtype_code(q.dtype), _ptr(q), _i64s(strides(Sq)), _ptr(k), _i64s(strides(Sk)), _ptr(v),
                                            _i64s(strides(Sk)), _ptr(mask), _ptr(out), _i64s(strides(Sq)), B, H, Sq, Sk, D, scale,
                                            1 if causal else 0, C.addressof(t), _stream(stream)))
        return out
    check(lib.mhlo_cuda_attention(torch_dtype_code(q.dtype), _ptr(q), _i64s(strides(Sq)), _ptr(k), _i64s(strides(Sk)), _ptr(v),
                                  _i64s(strides(Sk)), _ptr(mask), _ptr(out), _i64s(strides(Sq)), B, H, Sq, Sk, D, scale,
                                  1 if causal else 0, _stream(stream)))
    return out


def softmax(x, axis: int = -1, out=None, tuning=None, stream=None):
    import math

    import torch

    assert x.is_cuda and x.is_contiguous()
    out = torch.empty_like(x) if out is None else out
    axis = axis % x.dim()
    outer = math.prod(x.shape[:axis])
    inner = math.prod(x.shape[axis + 1:])
    check(lib.mhlo_cuda_softmax(torch_dtype_code(x.dtype), _ptr(x), _ptr(out), outer, x.shape[axis], inner,
                                _tuning(tuning), _stream(stream)))
    return out
