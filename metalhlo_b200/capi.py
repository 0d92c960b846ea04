"""ctypes view of ``libCMetalHLO.so`` — the ``mhlo_*`` C API declared in ``include/metalhlo.h``.

``Client`` / ``Executable`` / ``Buffer`` mirror the reference's Swift types of the same names
(Sources/MetalHLO/{Client,Executable,Buffer}.swift): ``Client().compile(mlir, opt_level)`` gives an executable,
``executable.execute([buffers])`` returns new output buffers, ``buffer.to_numpy()`` copies back. Errors raise
``MetalHLOError`` carrying the C status code. Nothing here computes: every call goes through the C ABI.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libCMetalHLO.so")
if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'`")

C.CDLL(os.path.join(_HERE, "lib", "libmhlo_cuda.so"), mode=C.RTLD_GLOBAL)
lib = C.CDLL(LIB_PATH)

STATUS_NAMES = ["OK", "NO_DEVICE", "UNSUPPORTED_DEVICE", "PARSE_FAILED", "UNSUPPORTED_OP", "COMPILATION_FAILED",
                "BUFFER_FAILED", "INPUT_MISMATCH", "EXECUTION_FAILED", "TRANSFER_FAILED", "INVALID_ARGUMENT"]
F16, F32, F64, BF16, I1, I8, I16, I32, I64, UI8, UI16, UI32, UI64 = range(13)

try:
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None

_NP = {F16: np.dtype(np.float16), F32: np.dtype(np.float32), F64: np.dtype(np.float64), I1: np.dtype(np.bool_),
       I8: np.dtype(np.int8), I16: np.dtype(np.int16), I32: np.dtype(np.int32), I64: np.dtype(np.int64),
       UI8: np.dtype(np.uint8), UI16: np.dtype(np.uint16), UI32: np.dtype(np.uint32), UI64: np.dtype(np.uint64)}
if _BF16 is not None:
    _NP[BF16] = _BF16


def np_dtype(code: int) -> np.dtype:
    if code == BF16 and _BF16 is None:
        return np.dtype(np.uint16)  # raw bits
    return _NP[code]


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    for code, nd in _NP.items():
        if nd == dt:
            return code
    raise TypeError(f"no MHLO element type for {dt}")


class CompileConfig(C.Structure):
    _fields_ = [("optimization_level", C.c_int), ("enable_caching", C.c_bool), ("enable_debug_info", C.c_bool),
                ("device_policy", C.c_int)]


class ExecutionStats(C.Structure):
    _fields_ = [("execution_count", C.c_int64), ("total_execution_time_ms", C.c_double),
                ("last_execution_time_ms", C.c_double), ("average_execution_time_ms", C.c_double)]


class ExecutionProfile(C.Structure):
    _fields_ = [("partition_count", C.c_int32), ("gpu_partition_count", C.c_int32), ("ane_partition_count", C.c_int32),
                ("gpu_time_ms", C.c_double), ("ane_time_ms", C.c_double), ("transfer_time_ms", C.c_double),
                ("total_time_ms", C.c_double), ("used_ane", C.c_bool)]


_vp, _i32, _i64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
_P = C.POINTER
_PROTOTYPES = {
    "mhlo_version": (C.c_char_p, []),
    "mhlo_get_last_error": (C.c_char_p, []),
    "mhlo_clear_error": (None, []),
    "mhlo_element_type_size": (_sz, [C.c_int]),
    "mhlo_free_string": (None, [_vp]),
    "mhlo_client_create": (C.c_int, [_P(_vp)]),
    "mhlo_client_destroy": (None, [_vp]),
    "mhlo_client_device_name": (_vp, [_vp]),
    "mhlo_compile_config_init": (None, [_P(CompileConfig)]),
    "mhlo_ane_available": (C.c_bool, []),
    "mhlo_compile": (C.c_int, [_vp, C.c_char_p, _P(_vp)]),
    "mhlo_compile_n": (C.c_int, [_vp, C.c_char_p, _sz, _P(_vp)]),
    "mhlo_compile_with_config": (C.c_int, [_vp, C.c_char_p, _P(CompileConfig), _P(_vp)]),
    "mhlo_executable_destroy": (None, [_vp]),
    "mhlo_executable_input_count": (_i32, [_vp]),
    "mhlo_executable_output_count": (_i32, [_vp]),
    "mhlo_executable_input_type": (C.c_int, [_vp, _i32, _P(_i64), _P(_i32), _P(C.c_int)]),
    "mhlo_executable_output_type": (C.c_int, [_vp, _i32, _P(_i64), _P(_i32), _P(C.c_int)]),
    "mhlo_executable_get_stats": (C.c_int, [_vp, _P(ExecutionStats)]),
    "mhlo_executable_reset_stats": (None, [_vp]),
    "mhlo_buffer_create": (C.c_int, [_vp, _vp, _sz, _P(_i64), _i32, C.c_int, _P(_vp)]),
    "mhlo_buffer_create_uninitialized": (C.c_int, [_vp, _P(_i64), _i32, C.c_int, _P(_vp)]),
    "mhlo_buffer_destroy": (None, [_vp]),
    "mhlo_buffer_shape": (None, [_vp, _P(_i64), _P(_i32)]),
    "mhlo_buffer_rank": (_i32, [_vp]),
    "mhlo_buffer_element_type": (C.c_int, [_vp]),
    "mhlo_buffer_byte_count": (_sz, [_vp]),
    "mhlo_buffer_to_host": (C.c_int, [_vp, _vp, _sz]),
    "mhlo_execute": (C.c_int, [_vp, _P(_vp), _i32, _P(_vp), _P(_i32)]),
    "mhlo_execute_with_timing": (C.c_int, [_vp, _P(_vp), _i32, _P(_vp), _P(_i32), _P(C.c_double), _P(C.c_double),
                                           _P(C.c_double)]),
    "mhlo_execute_with_profile": (C.c_int, [_vp, _P(_vp), _i32, _P(_vp), _P(_i32), _P(ExecutionProfile)]),
    "mhlo_b200_optimize_text": (C.c_int, [C.c_char_p, _i32, _P(_vp)]),
    "mhlo_b200_plan_text": (C.c_int, [C.c_char_p, _i32, _P(_vp), _P(_i32), _P(_i64)]),
    "mhlo_b200_plan_intervals": (C.c_int, [_P(_i64), _P(_i32), _P(_i32), _i32, _P(_i64), _P(_i64)]),
    "mhlo_b200_plan_memory_text": (C.c_int, [C.c_char_p, _i32, _P(_vp), _P(_i64)]),
    "mhlo_b200_bytecode_to_text": (C.c_int, [C.c_char_p, _sz, _P(_vp)]),
    "mhlo_b200_device_count": (_i32, []),
    "mhlo_b200_client_create_on_device": (C.c_int, [_i32, _P(_vp)]),
    "mhlo_b200_compile_sharded": (C.c_int, [_vp, C.c_char_p, _P(CompileConfig), _i32, _i32, _P(_i32), _i32, _P(_vp)]),
    "mhlo_b200_executable_sharding": (C.c_int, [_vp, _P(_i32), _P(_i32), _P(_i32), _P(_i32)]),
    "mhlo_b200_shard_text": (C.c_int, [C.c_char_p, _i32, _i32, _P(_i32), _i32, _P(_vp), _P(_i32), _P(_i32)]),
    "mhlo_b200_executable_optimized_text": (_vp, [_vp]),
    "mhlo_b200_executable_launch_count": (_i32, [_vp]),
    "mhlo_b200_executable_arena_bytes": (_i64, [_vp]),
    "mhlo_b200_executable_graph_replays": (_i64, [_vp]),
    "mhlo_b200_executable_steps": (_vp, [_vp]),
    "mhlo_b200_buffer_device_pointer": (_vp, [_vp]),
    "mhlo_b200_execute_on_device": (C.c_int, [_vp, _P(_vp), _P(_vp), _vp]),
    "mhlo_b200_tuning_open": (C.c_int, [C.c_char_p]),
    "mhlo_b200_tuning_count": (_i64, []),
    "mhlo_b200_tuning_tune_row_kernel": (C.c_int, [_vp, C.c_char_p, C.c_int, _i64, _i64, _i32, _P(_vp)]),
    "mhlo_b200_tuning_tune_gemm": (C.c_int, [_vp, C.c_int, C.c_int, _i64, _i64, _i64, _i64, C.c_bool, C.c_bool, _i32, _P(_vp)]),
    "mhlo_b200_tuning_tune_attention": (C.c_int, [_vp, C.c_int, _i64, _i64, _i64, _i64, _i64, C.c_bool, C.c_bool, _i32, _P(_vp)]),
    "mhlo_b200_tuning_merge_json": (C.c_int, [C.c_char_p, C.c_bool, _P(_i32)]),
    "mhlo_b200_tuning_to_json": (_vp, []),
    "mhlo_b200_tuning_save": (C.c_int, []),
    "mhlo_b200_tuning_import": (C.c_int, [C.c_char_p, C.c_bool, _P(_i32)]),
    "mhlo_b200_tuning_prune": (_i32, [C.c_double]),
    "mhlo_b200_tuning_clear": (None, []),
}
for _name, (_res, _args) in _PROTOTYPES.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


def declared_symbols():
    return sorted(_PROTOTYPES)


class MetalHLOError(RuntimeError):
    def __init__(self, status: int):
        msg = lib.mhlo_get_last_error()
        self.status = status
        self.status_name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"MHLO_ERROR_{self.status_name}: {msg.decode() if msg else ''}")


def _check(status: int) -> None:
    if status != 0:
        raise MetalHLOError(status)


def _take_string(ptr) -> str:
    if not ptr:
        return ""
    s = C.string_at(ptr).decode()
    lib.mhlo_free_string(ptr)
    return s


def plan_intervals(sizes, firsts, lasts):
    """The static memory planner alone: (offsets, arena bytes) for buffers with the given sizes and inclusive live ranges."""
    n = len(sizes)
    offs, total = (_i64 * max(n, 1))(), _i64()
    _check(lib.mhlo_b200_plan_intervals((_i64 * max(n, 1))(*sizes), (_i32 * max(n, 1))(*firsts), (_i32 * max(n, 1))(*lasts), n, offs, C.byref(total)))
    return list(offs)[:n], total.value


def plan_memory(mlir: str, opt_level: int = 3):
    """Arena plan of a module: ([(bytes, first step, last step, offset)], arena bytes). Host only."""
    out, arena = _vp(), _i64()
    _check(lib.mhlo_b200_plan_memory_text(mlir.encode(), opt_level, C.byref(out), C.byref(arena)))
    rows = [tuple(int(x) for x in line.split()) for line in _take_string(out.value).splitlines() if line.strip()]
    return rows, arena.value


def bytecode_to_text(bytecode: bytes) -> str:
    """MLIR bytecode -> StableHLO text through the helper process (host only)."""
    out = _vp()
    _check(lib.mhlo_b200_bytecode_to_text(bytecode, len(bytecode), C.byref(out)))
    return _take_string(out.value)


def optimize_text(mlir: str, opt_level: int = 3) -> str:
    """Parse + pass pipeline on the host only (no GPU); returns the optimised module text."""
    out = _vp()
    _check(lib.mhlo_b200_optimize_text(mlir.encode(), opt_level, C.byref(out)))
    return _take_string(out.value)


def plan_text(mlir: str, opt_level: int = 3):
    """Lowering on the host only (no GPU): (step labels, kernel launches per execution, arena bytes)."""
    out, launches, arena = _vp(), _i32(0), _i64(0)
    _check(lib.mhlo_b200_plan_text(mlir.encode(), opt_level, C.byref(out), C.byref(launches), C.byref(arena)))
    return _take_string(out.value).splitlines(), launches.value, arena.value


def shard_text(mlir: str, count: int, index: int, input_axes=None, n_inputs: int = 64, n_outputs: int = 16):
    """Host only: the function that computes shard `index` of `count`, and the split axis of every argument / result."""
    out = _vp()
    ia, oa = (_i32 * n_inputs)(*([-2] * n_inputs)), (_i32 * n_outputs)(*([-2] * n_outputs))
    axes = (_i32 * len(input_axes))(*input_axes) if input_axes is not None else None
    _check(lib.mhlo_b200_shard_text(mlir.encode(), count, index, axes, len(input_axes) if input_axes is not None else 0, C.byref(out), ia, oa))
    return _take_string(out.value), [a for a in ia if a != -2], [a for a in oa if a != -2]


class tuning:
    """The process tuning database (mhlo_b200_tuning_*): measured launch configurations keyed by operation, shape,
    dtype and device name, persisted as JSON."""

    @staticmethod
    def open(path: str) -> None:
        _check(lib.mhlo_b200_tuning_open(path.encode()))

    @staticmethod
    def count() -> int:
        return int(lib.mhlo_b200_tuning_count())

    @staticmethod
    def merge(document: dict, overwrite: bool = False) -> int:
        import json

        taken = _i32(0)
        _check(lib.mhlo_b200_tuning_merge_json(json.dumps(document).encode(), overwrite, C.byref(taken)))
        return taken.value

    @staticmethod
    def to_dict() -> dict:
        import json

        return json.loads(_take_string(lib.mhlo_b200_tuning_to_json()))

    @staticmethod
    def save() -> None:
        _check(lib.mhlo_b200_tuning_save())

    @staticmethod
    def import_file(path: str, overwrite: bool = False) -> int:
        taken = _i32(0)
        _check(lib.mhlo_b200_tuning_import(path.encode(), overwrite, C.byref(taken)))
        return taken.value

    @staticmethod
    def prune(max_age_days: float) -> int:
        return int(lib.mhlo_b200_tuning_prune(max_age_days))

    @staticmethod
    def clear() -> None:
        lib.mhlo_b200_tuning_clear()

    @staticmethod
    def tune_row_kernel(client, kernel: str, element_type: int, rows: int, hidden: int, max_trials: int = 0) -> dict:
        import json

        out = _vp()
        _check(lib.mhlo_b200_tuning_tune_row_kernel(client._h, kernel.encode(), element_type, rows, hidden, max_trials, C.byref(out)))
        return json.loads(_take_string(out.value))


def _tune_gemm(client, element_type, batch, m, n, k, out_element_type=None, a_transposed=False, b_transposed=False, max_trials=0) -> dict:
    import json

    out = _vp()
    _check(lib.mhlo_b200_tuning_tune_gemm(client._h, element_type, element_type if out_element_type is None else out_element_type, batch, m, n, k,
                                          a_transposed, b_transposed, max_trials, C.byref(out)))
    return json.loads(_take_string(out.value))


def _tune_attention(client, element_type, batch, heads, seq_q, seq_k, head_dim, causal=False, bshd=False, max_trials=0) -> dict:
    import json

    out = _vp()
    _check(lib.mhlo_b200_tuning_tune_attention(client._h, element_type, batch, heads, seq_q, seq_k, head_dim, causal, bshd, max_trials, C.byref(out)))
    return json.loads(_take_string(out.value))


tuning.tune_gemm = staticmethod(_tune_gemm)
tuning.tune_attention = staticmethod(_tune_attention)


class Buffer:
    def __init__(self, handle, client):
        self._h, self._client = handle, client

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # lib is None while the interpreter shuts down
            lib.mhlo_buffer_destroy(self._h)
            self._h = None

    @property
    def shape(self):
        rank = lib.mhlo_buffer_rank(self._h)
        arr = (_i64 * max(rank, 1))()
        r = _i32()
        lib.mhlo_buffer_shape(self._h, arr, C.byref(r))
        return tuple(arr[i] for i in range(r.value))

    @property
    def element_type(self) -> int:
        return lib.mhlo_buffer_element_type(self._h)

    @property
    def byte_count(self) -> int:
        return lib.mhlo_buffer_byte_count(self._h)

    @property
    def device_pointer(self) -> int:
        return lib.mhlo_b200_buffer_device_pointer(self._h) or 0

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=np_dtype(self.element_type))
        _check(lib.mhlo_buffer_to_host(self._h, out.ctypes.data if out.size else C.c_void_p(1), max(out.nbytes, 0)))
        return out


class Executable:
    def __init__(self, handle, client):
        self._h, self._client = handle, client

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.mhlo_executable_destroy(self._h)
            self._h = None

    @property
    def input_count(self) -> int:
        return lib.mhlo_executable_input_count(self._h)

    @property
    def output_count(self) -> int:
        return lib.mhlo_executable_output_count(self._h)

    def _type(self, fn, i):
        shape = (_i64 * 8)()
        rank, et = _i32(), C.c_int()
        _check(fn(self._h, i, shape, C.byref(rank), C.byref(et)))
        return tuple(shape[d] for d in range(rank.value)), et.value

    def input_type(self, i):
        return self._type(lib.mhlo_executable_input_type, i)

    def output_type(self, i):
        return self._type(lib.mhlo_executable_output_type, i)

    def execute(self, inputs, timing: bool = False):
        n = len(inputs)
        arr = (_vp * max(n, 1))(*[b._h for b in inputs])
        outs = (_vp * max(self.output_count, 1))()
        n_out = _i32()
        if timing:
            enc, gpu, tot = C.c_double(), C.c_double(), C.c_double()
            _check(lib.mhlo_execute_with_timing(self._h, arr, n, outs, C.byref(n_out), C.byref(enc), C.byref(gpu), C.byref(tot)))
            return [Buffer(outs[i], self._client) for i in range(n_out.value)], (enc.value, gpu.value, tot.value)
        _check(lib.mhlo_execute(self._h, arr, n, outs, C.byref(n_out)))
        return [Buffer(outs[i], self._client) for i in range(n_out.value)]

    def execute_on_device(self, input_ptrs, output_ptrs, stream: int = 0) -> None:
        ins = (_vp * max(len(input_ptrs), 1))(*input_ptrs)
        outs = (_vp * max(len(output_ptrs), 1))(*output_ptrs)
        _check(lib.mhlo_b200_execute_on_device(self._h, ins, outs, stream))

    @property
    def sharding(self):
        """(shard count, shard index, split axis per input, split axis per output); -1 = replicated."""
        n, k = _i32(), _i32()
        ia, oa = (_i32 * max(self.input_count, 1))(), (_i32 * max(self.output_count, 1))()
        _check(lib.mhlo_b200_executable_sharding(self._h, C.byref(n), C.byref(k), ia, oa))
        return n.value, k.value, list(ia)[:self.input_count], list(oa)[:self.output_count]

    def stats(self) -> ExecutionStats:
        s = ExecutionStats()
        _check(lib.mhlo_executable_get_stats(self._h, C.byref(s)))
        return s

    def reset_stats(self) -> None:
        lib.mhlo_executable_reset_stats(self._h)

    @property
    def optimized_text(self) -> str:
        return _take_string(lib.mhlo_b200_executable_optimized_text(self._h))

    @property
    def launch_count(self) -> int:
        return lib.mhlo_b200_executable_launch_count(self._h)

    @property
    def arena_bytes(self) -> int:
        return lib.mhlo_b200_executable_arena_bytes(self._h)

    @property
    def graph_replays(self) -> int:
        return int(lib.mhlo_b200_executable_graph_replays(self._h))

    @property
    def steps(self):
        return [s for s in _take_string(lib.mhlo_b200_executable_steps(self._h)).split("\n") if s]


class Client:
    def __init__(self, device: int | None = None):
        h = _vp()
        if device is None:
            _check(lib.mhlo_client_create(C.byref(h)))
        else:
            _check(lib.mhlo_b200_client_create_on_device(device, C.byref(h)))
        self._h = h.value

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.mhlo_client_destroy(self._h)
            self._h = None

    @property
    def device_name(self) -> str:
        return _take_string(lib.mhlo_client_device_name(self._h))

    def compile(self, mlir: str, opt_level: int | None = None, caching: bool = True) -> Executable:
        h = _vp()
        if opt_level is None:
            _check(lib.mhlo_compile(self._h, mlir.encode(), C.byref(h)))
        else:
            cfg = CompileConfig()
            lib.mhlo_compile_config_init(C.byref(cfg))
            cfg.optimization_level = opt_level
            cfg.enable_caching = caching
            _check(lib.mhlo_compile_with_config(self._h, mlir.encode(), C.byref(cfg), C.byref(h)))
        return Executable(h.value, self)

    def compile_sharded(self, mlir: str, count: int, index: int, opt_level: int = 3, input_axes=None) -> Executable:
        """Shard `index` of `count` equal batch shards of the program (mhlo_b200_compile_sharded)."""
        h = _vp()
        cfg = CompileConfig()
        lib.mhlo_compile_config_init(C.byref(cfg))
        cfg.optimization_level = opt_level
        axes = (_i32 * len(input_axes))(*input_axes) if input_axes is not None else None
        _check(lib.mhlo_b200_compile_sharded(self._h, mlir.encode(), C.byref(cfg), count, index, axes,
                                             len(input_axes) if input_axes is not None else 0, C.byref(h)))
        return Executable(h.value, self)

    def buffer(self, array, element_type: int | None = None) -> Buffer:
        """Host array -> device buffer. torch tensors are accepted (bf16 included)."""
        if hasattr(array, "detach"):
            import torch

            t = array.detach().cpu().contiguous()
            codes = {torch.float16: F16, torch.float32: F32, torch.float64: F64, torch.bfloat16: BF16, torch.bool: I1,
                     torch.int8: I8, torch.int16: I16, torch.int32: I32, torch.int64: I64, torch.uint8: UI8}
            code = codes[t.dtype]
            shape, ptr, nbytes = tuple(t.shape), t.data_ptr(), t.numel() * t.element_size()
            keep = t
        else:
            a = np.asarray(array)
            a = a if a.flags['C_CONTIGUOUS'] else np.ascontiguousarray(a)  # keeps 0-d arrays 0-d
            code = dtype_code(a.dtype) if element_type is None else element_type
            shape, ptr, nbytes = a.shape, a.ctypes.data, a.nbytes
            keep = a
        sh = (_i64 * max(len(shape), 1))(*shape)
        h = _vp()
        _check(lib.mhlo_buffer_create(self._h, ptr if nbytes else None, nbytes, sh, len(shape), code, C.byref(h)))
        del keep
        return Buffer(h.value, self)

    def run(self, mlir: str, inputs, opt_level: int | None = None):
        """compile + execute + copy back: the one-call path the parity tests use."""
        exe = self.compile(mlir, opt_level)
        outs = exe.execute([self.buffer(x) for x in inputs])
        return [o.to_numpy() for o in outs]
