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
