"""ctypes view of ``libpjrt_host.so``: a PJRT host that drives ``pjrt_plugin_metalhlo_b200.so`` through ``GetPjrtApi``
the way XLA / JAX drive a plugin (Plugin_Initialize, Client_Create, BufferFromHostBuffer, Compile, Execute,
ToHostBuffer). The parity tests and the benchmark use it to reach the plugin without jaxlib; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB = os.path.join(_HERE, "lib", "libpjrt_host.so")
PLUGIN = os.path.join(_HERE, "lib", "pjrt_plugin_metalhlo_b200.so")
for _p in (HOST_LIB, PLUGIN):
    if not os.path.exists(_p):
        raise ImportError(f"{_p} is missing: run `python -c 'import __graft_entry__ as g; g.build()'`")

lib = C.CDLL(HOST_LIB)

# PJRT_Buffer_Type values (pjrt_c_api.h)
PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13

try:
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None

_NP = {PRED: np.dtype(np.bool_), S8: np.dtype(np.int8), S16: np.dtype(np.int16), S32: np.dtype(np.int32), S64: np.dtype(np.int64),
       U8: np.dtype(np.uint8), U16: np.dtype(np.uint16), U32: np.dtype(np.uint32), U64: np.dtype(np.uint64),
       F16: np.dtype(np.float16), F32: np.dtype(np.float32), F64: np.dtype(np.float64)}
if _BF16 is not None:
    _NP[BF16] = _BF16

_vp, _i64, _sz = C.c_void_p, C.c_int64, C.c_size_t
_P = C.POINTER
_PROTOTYPES = {
    "pjrt_host_last_error": (C.c_char_p, []),
    "pjrt_host_open": (C.c_int, [C.c_char_p, _P(_vp)]),
    "pjrt_host_close": (None, [_vp]),
    "pjrt_host_api_version": (C.c_int, [_vp, _P(C.c_int), _P(C.c_int)]),
    "pjrt_host_device_count": (C.c_int, [_vp]),
    "pjrt_host_device_id": (C.c_int, [_vp, C.c_int, _P(_i64)]),
    "pjrt_host_platform_name": (C.c_int, [_vp, C.c_char_p, _sz]),
    "pjrt_host_buffer_from_host": (C.c_int, [_vp, _vp, C.c_int, _P(_i64), C.c_int, C.c_int, _P(_vp)]),
    "pjrt_host_buffer_describe": (C.c_int, [_vp, _vp, _P(C.c_int), _P(_i64), _P(C.c_int), _P(_sz)]),
    "pjrt_host_buffer_to_host": (C.c_int, [_vp, _vp, _vp, _sz]),
    "pjrt_host_buffer_to_host_start": (C.c_int, [_vp, _vp, _vp, _sz, C.POINTER(_vp)]),
    "pjrt_host_event_await": (C.c_int, [_vp, _vp]),
    "pjrt_host_buffer_destroy": (None, [_vp, _vp]),
    "pjrt_host_compile": (C.c_int, [_vp, C.c_char_p, _sz, C.c_int, C.c_int, _P(_i64), _P(_vp)]),
    "pjrt_host_executable_num_outputs": (C.c_int, [_vp]),
    "pjrt_host_executable_num_devices": (C.c_int, [_vp]),
    "pjrt_host_executable_destroy": (None, [_vp, _vp]),
    "pjrt_host_execute": (C.c_int, [_vp, _vp, _P(_vp), C.c_int, C.c_int, _P(_vp)]),
}
for _name, (_res, _args) in _PROTOTYPES.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


def declared_symbols():
    return sorted(_PROTOTYPES)


class PjrtError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise PjrtError(lib.pjrt_host_last_error().decode())


def buffer_type(dtype) -> int:
    dtype = np.dtype(dtype)
    for code, nd in _NP.items():
        if nd == dtype:
            return code
    raise TypeError(f"no PJRT buffer type for {dtype}")


class Buffer:
    def __init__(self, handle, host):
        self._h, self._host = handle, host

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None and self._host._h:
            lib.pjrt_host_buffer_destroy(self._host._h, self._h)
            self._h = None

    def describe(self):
        t, r, n = C.c_int(), C.c_int(), _sz()
        dims = (_i64 * 8)()
        _check(lib.pjrt_host_buffer_describe(self._host._h, self._h, C.byref(t), dims, C.byref(r), C.byref(n)))
        return t.value, tuple(dims[i] for i in range(r.value)), n.value

    def to_numpy(self) -> np.ndarray:
        t, shape, nbytes = self.describe()
        out = np.empty(shape, dtype=_NP[t])
        assert out.nbytes == nbytes, (out.nbytes, nbytes)
        if nbytes:
            _check(lib.pjrt_host_buffer_to_host(self._host._h, self._h, out.ctypes.data, nbytes))
        return out

    def to_host_pointer(self, ptr: int, nbytes: int) -> None:
        _check(lib.pjrt_host_buffer_to_host(self._host._h, self._h, ptr, nbytes))

    def to_host_pointer_start(self, ptr: int, nbytes: int):
        """PJRT_Buffer_ToHostBuffer without the wait; returns a callable that awaits the transfer's event (call it once)."""
        ev = _vp()
        _check(lib.pjrt_host_buffer_to_host_start(self._host._h, self._h, ptr, nbytes, C.byref(ev)))
        host = self._host

        def wait():
            _check(lib.pjrt_host_event_await(host._h, ev))

        return wait


class LoadedExecutable:
    def __init__(self, handle, host):
        self._h, self._host = handle, host

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None and self._host._h:
            lib.pjrt_host_executable_destroy(self._host._h, self._h)
            self._h = None

    @property
    def num_outputs(self) -> int:
        return lib.pjrt_host_executable_num_outputs(self._h)

    @property
    def num_devices(self) -> int:
        return lib.pjrt_host_executable_num_devices(self._h)

    def execute(self, args):
        """One device: `args` is a list of buffers, the result a list of buffers."""
        return self.execute_sharded([args])[0]

    def execute_sharded(self, per_device_args):
        """`per_device_args[d]` = the argument buffers of device d; returns the output buffers per device."""
        nd, na, no = len(per_device_args), len(per_device_args[0]), self.num_outputs
        flat = (_vp * max(nd * na, 1))(*[b._h for dev in per_device_args for b in dev])
        outs = (_vp * max(nd * no, 1))()
        _check(lib.pjrt_host_execute(self._host._h, self._h, flat, nd, na, outs))
        return [[Buffer(outs[d * no + i], self._host) for i in range(no)] for d in range(nd)]


class Host:
    """One PJRT client of the plugin at `plugin_path` (default: this package's plugin)."""

    def __init__(self, plugin_path: str = PLUGIN):
        self._h = None
        h = _vp()
        _check(lib.pjrt_host_open(plugin_path.encode(), C.byref(h)))
        self._h = h.value

    def close(self):
        if self._h:
            lib.pjrt_host_close(self._h)
            self._h = None

    def __del__(self):
        if lib is not None:
            self.close()

    @property
    def api_version(self):
        a, b = C.c_int(), C.c_int()
        _check(lib.pjrt_host_api_version(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    @property
    def platform_name(self) -> str:
        buf = C.create_string_buffer(64)
        _check(lib.pjrt_host_platform_name(self._h, buf, 64))
        return buf.value.decode()

    @property
    def device_count(self) -> int:
        return lib.pjrt_host_device_count(self._h)

    def device_id(self, index: int) -> int:
        v = _i64()
        _check(lib.pjrt_host_device_id(self._h, index, C.byref(v)))
        return v.value

    def buffer(self, array, device: int = 0) -> Buffer:
        a = np.asarray(array)
        a = a if a.flags["C_CONTIGUOUS"] else np.ascontiguousarray(a)
        dims = (_i64 * max(a.ndim, 1))(*a.shape)
        h = _vp()
        _check(lib.pjrt_host_buffer_from_host(self._h, a.ctypes.data if a.size else None, buffer_type(a.dtype), dims, a.ndim, device, C.byref(h)))
        return Buffer(h.value, self)

    def buffer_from_pointer(self, ptr: int, dtype, shape, device: int = 0) -> Buffer:
        dims = (_i64 * max(len(shape), 1))(*shape)
        h = _vp()
        _check(lib.pjrt_host_buffer_from_host(self._h, ptr, buffer_type(dtype), dims, len(shape), device, C.byref(h)))
        return Buffer(h.value, self)

    def compile(self, program, num_replicas: int = 0, num_partitions: int = 1, device_ids=None) -> LoadedExecutable:
        """`program`: StableHLO text (str) or MLIR bytecode (bytes). num_replicas = 0 sends no compile options."""
        data = program.encode() if isinstance(program, str) else bytes(program)
        ids = None
        if device_ids is not None:
            ids = (_i64 * len(device_ids))(*device_ids)
        h = _vp()
        _check(lib.pjrt_host_compile(self._h, data, len(data), num_replicas, num_partitions, ids, C.byref(h)))
        return LoadedExecutable(h.value, self)
