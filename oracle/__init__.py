"""CPU oracle for the parity tests — TEST INFRASTRUCTURE ONLY.

numpy/ctypes front of ``oracle/mhlo_oracle.c`` (an fp64 restatement of the arithmetic the reference lowers its
fused ops to, plus fp32 host-core kernels in the operation order of the reference's CPU partition). Only the
test-suite, the smoke test and the benchmark's CPU-baseline leg import this package; the product never does.

Every ``oracle_*`` wrapper takes array-likes holding the exact input values (any float dtype; they are
widened to fp32, which is exact for f16/bf16/f32 inputs) and returns a float64 ndarray.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmhlo_oracle.so")


def build(force: bool = False) -> str:
    """Compiles ``mhlo_oracle.c`` with the committed Makefile if the library is missing or stale."""
    src = os.path.join(_HERE, "mhlo_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(LIB_PATH)
        f32p, f64p = C.POINTER(C.c_float), C.POINTER(C.c_double)
        i64, dbl, flt, cint = C.c_int64, C.c_double, C.c_float, C.c_int
        protos = {
            "oracle_max_threads": (cint, []),
            "oracle_set_threads": (None, [cint]),
            "oracle_layer_norm": (None, [f32p, f32p, f32p, f64p, i64, i64, dbl]),
            "oracle_rms_norm": (None, [f32p, f32p, f64p, i64, i64, dbl]),
            "oracle_softmax": (None, [f32p, f64p, i64, i64, i64]),
            "oracle_gelu": (None, [f32p, f64p, i64, cint]),
            "oracle_silu": (None, [f32p, f64p, i64]),
            "oracle_gemm": (None, [f32p, f32p, f64p, i64, i64, i64, i64, cint, cint]),
            "oracle_attention": (None, [f32p, f32p, f32p, f32p, f64p, i64, i64, i64, i64, dbl, cint]),
            "cpu_layer_norm_f32": (None, [f32p, f32p, f32p, f32p, i64, i64, flt]),
            "cpu_rms_norm_f32": (None, [f32p, f32p, f32p, i64, i64, flt]),
            "cpu_softmax_f32": (None, [f32p, f32p, i64, i64]),
            "cpu_gelu_f32": (None, [f32p, f32p, i64]),
            "cpu_gemm_f32": (None, [f32p, f32p, f32p, i64, i64, i64]),
            "cpu_attention_f32": (None, [f32p, f32p, f32p, f32p, i64, i64, i64, i64, flt, cint]),
        }
        for name, (res, args) in protos.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


def max_threads() -> int:
    return lib().oracle_max_threads()


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def _f32(a):
    """Exact fp32 ndarray of a torch tensor / ndarray / list (C-contiguous)."""
    if a is None:
        return None
    if hasattr(a, "detach"):  # torch tensor
        a = a.detach().to("cpu").float().numpy()
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p32(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _p64(a):
    return a.ctypes.data_as(C.POINTER(C.c_double))


def layer_norm(x, gamma=None, beta=None, eps: float = 1e-5) -> np.ndarray:
    x, gamma, beta = _f32(x), _f32(gamma), _f32(beta)
    y = np.empty(x.shape, dtype=np.float64)
    hidden = x.shape[-1]
    rows = x.size // hidden if hidden else 0
    lib().oracle_layer_norm(_p32(x), _p32(gamma), _p32(beta), _p64(y), rows, hidden, eps)
    return y


def rms_norm(x, gamma=None, eps: float = 1e-5) -> np.ndarray:
    x, gamma = _f32(x), _f32(gamma)
    y = np.empty(x.shape, dtype=np.float64)
    hidden = x.shape[-1]
    rows = x.size // hidden if hidden else 0
    lib().oracle_rms_norm(_p32(x), _p32(gamma), _p64(y), rows, hidden, eps)
    return y


def softmax(x, axis: int = -1) -> np.ndarray:
    x = _f32(x)
    axis = axis % x.ndim
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    y = np.empty(x.shape, dtype=np.float64)
    lib().oracle_softmax(_p32(x), _p64(y), outer, x.shape[axis], inner)
    return y


def gelu(x, approximate: bool = True) -> np.ndarray:
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.float64)
    lib().oracle_gelu(_p32(x), _p64(y), x.size, 1 if approximate else 0)
    return y


def silu(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.float64)
    lib().oracle_silu(_p32(x), _p64(y), x.size)
    return y


def gemm(a, b, trans_a: bool = False, trans_b: bool = False) -> np.ndarray:
    """C[b,M,N] = A[b,M,K] . B[b,K,N] (2-D inputs are a batch of one). trans_* describe the storage."""
    a, b = _f32(a), _f32(b)
    squeeze = a.ndim == 2
    if squeeze:
        a, b = a[None], b[None]
    batch = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if trans_a else (a.shape[1], a.shape[2])
    n = b.shape[1] if trans_b else b.shape[2]
    c = np.empty((batch, m, n), dtype=np.float64)
    lib().oracle_gemm(_p32(a), _p32(b), _p64(c), batch, m, n, k, int(trans_a), int(trans_b))
    return c[0] if squeeze else c


def attention(q, k, v, scale: float, causal: bool = False, mask=None) -> np.ndarray:
    """softmax(scale * Q K^T [+ mask | causal]) V for Q [..., Sq, D], K/V [..., Sk, D]."""
    q, k, v, mask = _f32(q), _f32(k), _f32(v), _f32(mask)
    sq, d = q.shape[-2:]
    sk = k.shape[-2]
    bh = q.size // (sq * d)
    o = np.empty(q.shape, dtype=np.float64)
    lib().oracle_attention(_p32(q), _p32(k), _p32(v), _p32(mask), _p64(o), bh, sq, sk, d, scale, int(causal))
    return o


# ---- fp32 host-core kernels (what the benchmark times as the CPU baseline) --------------------------------

def cpu_layer_norm_f32(x, gamma, beta, y, eps: float = 1e-5) -> None:
    rows, hidden = x.shape
    lib().cpu_layer_norm_f32(_p32(x), _p32(gamma), _p32(beta), _p32(y), rows, hidden, eps)


def cpu_rms_norm_f32(x, gamma, y, eps: float = 1e-5) -> None:
    rows, hidden = x.shape
    lib().cpu_rms_norm_f32(_p32(x), _p32(gamma), _p32(y), rows, hidden, eps)


def cpu_softmax_f32(x, y) -> None:
    rows, cols = x.shape
    lib().cpu_softmax_f32(_p32(x), _p32(y), rows, cols)


def cpu_gelu_f32(x, y) -> None:
    lib().cpu_gelu_f32(_p32(x), _p32(y), x.size)


def cpu_gemm_f32(a, b, c) -> None:
    m, k = a.shape
    n = b.shape[1]
    lib().cpu_gemm_f32(_p32(a), _p32(b), _p32(c), m, n, k)


def cpu_attention_f32(q, k, v, o, scale: float, causal: bool) -> None:
    bh, sq, d = q.shape
    sk = k.shape[1]
    lib().cpu_attention_f32(_p32(q), _p32(k), _p32(v), _p32(o), bh, sq, sk, d, scale, int(causal))
