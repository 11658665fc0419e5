"""ctypes view of the C ABI declared in ``include/kge_b200.h``.

This is the thinnest possible host side: it builds the plain structs the C
functions take and turns status codes back into the exceptions the reference's
binding raises (``ValueError`` for std::invalid_argument, ``RuntimeError``
otherwise; src/lib.cpp, src/poplar_kge.cpp:39-47,121-123).  There is no
fallback: if ``libkge_b200.so`` has not been built, loading fails.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "libkge_b200.so"

OK, INVALID_ARGUMENT, RUNTIME_ERROR, DEVICE_STATUS, LOGIC_ERROR = range(5)
F32, U32, F16 = 0, 1, 2
SET_STRING, SET_BOOL, SET_FLOAT, SET_UNSIGNED = 0, 1, 2, 3
L1, L2, DOT = 0, 1, 2

#: every entry point include/kge_b200.h declares
SYMBOLS = (
    "kge_create", "kge_destroy", "kge_last_error", "kge_run", "kge_variable_count",
    "kge_variable_info", "kge_comm_handle_bytes", "kge_comm_export", "kge_comm_connect",
    "kge_stage_batch", "kge_train_staged", "kge_last_run_stats", "kge_set_kernel_timing",
    "kge_kernel_time_count", "kge_kernel_time", "kge_debug_fetch",
    "kge_op_pairwise", "kge_op_pairwise_grad", "kge_op_gather_rows", "kge_op_scatter_add_rows",
    "kge_op_scatter_add_rows_noalloc", "kge_op_tc_gemm", "kge_op_tc_planes",
    "kge_microbench_rows", "kge_microbench_scores", "kge_op_tc_planes_bf16",
    "kge_op_activation", "kge_op_all_to_all",
)


class Setting(C.Structure):
    _fields_ = [("key", C.c_char_p), ("type", C.c_int), ("s", C.c_char_p), ("f", C.c_double),
                ("u", C.c_ulonglong)]


class Array(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int), ("rank", C.c_int),
                ("shape", C.POINTER(C.c_size_t)), ("data", C.c_void_p)]


_lib: Optional[C.CDLL] = None


def load_library() -> C.CDLL:
    """Load ``libkge_b200.so``; raises if it has not been built (no other path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python distributed-kge-poplar_b200/build.py`")
    lib = C.CDLL(str(LIB_PATH))
    fp, u32p, vp, sz = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.c_void_p, C.c_size_t
    lib.kge_create.argtypes = [C.POINTER(Setting), sz, C.c_char_p, C.POINTER(vp)]
    lib.kge_destroy.argtypes = [vp]
    lib.kge_destroy.restype = None
    lib.kge_last_error.argtypes = [vp]
    lib.kge_last_error.restype = C.c_char_p
    lib.kge_run.argtypes = [vp, C.c_char_p, C.POINTER(Array), sz, C.c_char_p]
    lib.kge_variable_count.argtypes = [vp, C.POINTER(sz)]
    lib.kge_variable_info.argtypes = [vp, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_int),
                                      C.POINTER(C.c_int), C.POINTER(sz)]
    lib.kge_comm_handle_bytes.argtypes = []
    lib.kge_comm_handle_bytes.restype = sz
    lib.kge_comm_export.argtypes = [vp, vp]
    lib.kge_comm_connect.argtypes = [vp, vp, sz]
    lib.kge_stage_batch.argtypes = [vp, C.POINTER(Array), sz]
    lib.kge_train_staged.argtypes = [vp, C.c_float, fp]
    lib.kge_last_run_stats.argtypes = [vp, fp, C.POINTER(C.c_ulonglong)]
    lib.kge_set_kernel_timing.argtypes = [vp, C.c_int]
    lib.kge_kernel_time_count.argtypes = [vp, C.POINTER(sz)]
    lib.kge_kernel_time.argtypes = [vp, sz, C.POINTER(C.c_char_p), fp, C.POINTER(C.c_ulonglong)]
    lib.kge_debug_fetch.argtypes = [vp, C.c_char_p, sz, fp, sz, C.POINTER(sz)]
    lib.kge_op_pairwise.argtypes = [C.c_int, fp, fp, sz, sz, sz, fp]
    lib.kge_op_pairwise_grad.argtypes = [C.c_int, fp, fp, fp, sz, sz, sz, fp, fp]
    lib.kge_op_gather_rows.argtypes = [fp, sz, sz, u32p, sz, fp]
    lib.kge_op_scatter_add_rows.argtypes = [fp, u32p, sz, sz, sz, fp]
    lib.kge_op_scatter_add_rows_noalloc.argtypes = [vp, vp, sz, sz, sz, vp, vp]
    lib.kge_op_tc_gemm.argtypes = [vp, C.c_int, C.c_int, u32p, sz, sz, fp, C.c_int, sz, sz, sz, sz, sz, C.c_int, fp,
                                   C.c_int, C.c_int, fp]
    lib.kge_op_tc_planes.argtypes = [fp, C.c_int, C.c_int, sz, sz, fp, C.c_int, sz, sz, sz, sz, sz, C.c_int, fp, C.c_int,
                                     C.c_int, C.c_int, C.c_int, fp, fp]
    lib.kge_op_tc_planes_bf16.argtypes = [fp, C.c_int, sz, sz, fp, C.c_int, sz, sz, sz, sz, sz, C.c_int, C.c_int, C.c_int, fp, fp]
    lib.kge_microbench_rows.argtypes = [C.c_int, sz, sz, u32p, sz, C.c_int, fp]
    lib.kge_microbench_scores.argtypes = [C.c_int, sz, sz, sz, C.c_int, fp]
    lib.kge_op_activation.argtypes = [C.c_int, fp, fp, sz, sz, fp, fp]
    lib.kge_op_all_to_all.argtypes = [fp, sz, sz, fp]
    _lib = lib
    return lib


def _raise(status: int, message: bytes) -> None:
    text = (message or b"").decode("utf-8", "replace")
    if status == INVALID_ARGUMENT:
        raise ValueError(text)
    raise RuntimeError(text)


def _flatten_settings(settings: Mapping[str, Any]):
    keep, out = [], []
    for key, value in settings.items():
        if isinstance(value, Mapping):  # training.learning_rate_modifiers
            for name, v in value.items():
                out.append((f"{key}.{name}", SET_FLOAT, None, float(v), 0))
        elif isinstance(value, (bool, np.bool_)):
            out.append((key, SET_BOOL, None, 0.0, int(value)))
        elif isinstance(value, str):
            out.append((key, SET_STRING, value, 0.0, 0))
        elif isinstance(value, (float, np.floating)):
            out.append((key, SET_FLOAT, None, float(value), 0))
        elif isinstance(value, (int, np.integer)):
            if value < 0:
                raise ValueError(f"Key '{key}' holds a negative integer")
            out.append((key, SET_UNSIGNED, None, 0.0, int(value)))
        else:
            raise ValueError(f"Key '{key}' holds value of unexpected type.")
    array = (Setting * len(out))()
    for i, (key, typ, s, f, u) in enumerate(out):
        kb = key.encode()
        sb = s.encode() if s is not None else None
        keep += [kb, sb]
        array[i] = Setting(kb, typ, sb, f, u)
    return array, keep


_DTYPES = {np.dtype(np.float32): F32, np.dtype(np.uint32): U32, np.dtype(np.float16): F16,
           np.dtype(np.int16): F16}


def _pack_arrays(arrays: Mapping[str, np.ndarray]):
    packed = (Array * len(arrays))()
    keep = []
    for i, (name, a) in enumerate(arrays.items()):
        if not isinstance(a, np.ndarray) or not a.flags.c_contiguous:
            raise ValueError(f"'{name}' must be a C-contiguous numpy array")
        if a.dtype not in _DTYPES:
            raise ValueError(f"'{name}' has an element type other than float32, uint32, float16")
        shape = (C.c_size_t * max(1, a.ndim))(*a.shape)
        nb = name.encode()
        keep += [shape, nb, a]
        packed[i] = Array(nb, _DTYPES[a.dtype], a.ndim, shape, a.ctypes.data)
    return packed, keep


class CEngine:
    """One engine handle.  Methods mirror the C functions one to one."""

    def __init__(self, settings: Mapping[str, Any], artefact_dir: str = ""):
        self._lib = load_library()
        self._handle = C.c_void_p()
        flat, keep = _flatten_settings(settings)
        status = self._lib.kge_create(flat, len(flat), artefact_dir.encode(), C.byref(self._handle))
        del keep
        if status != OK:
            _raise(status, self._lib.kge_last_error(None))

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.kge_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        if status != OK:
            _raise(status, self._lib.kge_last_error(self._handle))

    def run(self, command: str, arrays: Mapping[str, np.ndarray], name: Optional[str] = None) -> None:
        packed, keep = _pack_arrays(arrays)
        self._check(self._lib.kge_run(self._handle, command.encode(), packed, len(arrays),
                                      name.encode() if name is not None else None))
        del keep

    def variables(self) -> Dict[str, Tuple[int, ...]]:
        count = C.c_size_t()
        self._check(self._lib.kge_variable_count(self._handle, C.byref(count)))
        out = {}
        for i in range(count.value):
            name, dtype, rank = C.c_char_p(), C.c_int(), C.c_int()
            shape = (C.c_size_t * 4)()
            self._check(self._lib.kge_variable_info(self._handle, i, C.byref(name), C.byref(dtype),
                                                    C.byref(rank), shape))
            out[name.value.decode()] = tuple(shape[: rank.value])
        return out

    def comm_export(self) -> bytes:
        buf = C.create_string_buffer(self._lib.kge_comm_handle_bytes())
        self._check(self._lib.kge_comm_export(self._handle, buf))
        return buf.raw

    def comm_connect(self, all_handles: bytes, world_size: int) -> None:
        buf = C.create_string_buffer(all_handles, len(all_handles))
        self._check(self._lib.kge_comm_connect(self._handle, buf, world_size))

    def stage_batch(self, arrays: Mapping[str, np.ndarray]) -> None:
        packed, keep = _pack_arrays(arrays)
        self._check(self._lib.kge_stage_batch(self._handle, packed, len(arrays)))
        del keep

    def train_staged(self, learning_rate: float, loss: Optional[np.ndarray] = None) -> None:
        ptr = loss.ctypes.data_as(C.POINTER(C.c_float)) if loss is not None else None
        self._check(self._lib.kge_train_staged(self._handle, learning_rate, ptr))

    def last_run_stats(self) -> Tuple[float, int]:
        ms, launches = C.c_float(), C.c_ulonglong()
        self._check(self._lib.kge_last_run_stats(self._handle, C.byref(ms), C.byref(launches)))
        return ms.value, launches.value

    def set_kernel_timing(self, on: bool) -> None:
        self._check(self._lib.kge_set_kernel_timing(self._handle, int(on)))

    def kernel_times(self) -> Dict[str, Tuple[float, int]]:
        """{kernel name: (total device ms, launches)} since timing was switched on."""
        count = C.c_size_t()
        self._check(self._lib.kge_kernel_time_count(self._handle, C.byref(count)))
        out = {}
        for i in range(count.value):
            name, ms, launches = C.c_char_p(), C.c_float(), C.c_ulonglong()
            self._check(self._lib.kge_kernel_time(self._handle, i, C.byref(name), C.byref(ms), C.byref(launches)))
            out[name.value.decode()] = (ms.value, launches.value)
        return out

    def debug_fetch(self, what: str, shard: int, capacity: int) -> np.ndarray:
        out = np.empty(capacity, np.float32)
        count = C.c_size_t()
        self._check(self._lib.kge_debug_fetch(self._handle, what.encode(), shard,
                                              out.ctypes.data_as(C.POINTER(C.c_float)), capacity,
                                              C.byref(count)))
        return out[: count.value]


# -- single operators ---------------------------------------------------------

def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _op_check(status: int) -> None:
    if status != OK:
        _raise(status, load_library().kge_last_error(None))


def op_pairwise(fn: int, a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty((a.shape[0], b.shape[0]), np.float32)
    _op_check(load_library().kge_op_pairwise(fn, _fp(a), _fp(b), a.shape[0], b.shape[0], a.shape[1], _fp(out)))
    return out


def op_pairwise_grad(fn: int, a, b, grad_out) -> Tuple[np.ndarray, np.ndarray]:
    a, b, g = _f32(a), _f32(b), _f32(grad_out)
    ga, gb = np.zeros_like(a), np.zeros_like(b)
    _op_check(load_library().kge_op_pairwise_grad(fn, _fp(a), _fp(b), _fp(g), a.shape[0], b.shape[0],
                                                  a.shape[1], _fp(ga), _fp(gb)))
    return ga, gb


def op_gather_rows(table, indices) -> np.ndarray:
    table = _f32(table)
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    out = np.empty((idx.size, table.shape[1]), np.float32)
    _op_check(load_library().kge_op_gather_rows(_fp(table), table.shape[0], table.shape[1],
                                                idx.ctypes.data_as(C.POINTER(C.c_uint32)), idx.size, _fp(out)))
    return out


def op_scatter_add_rows(grad_rows, indices, rows: int) -> np.ndarray:
    g = _f32(grad_rows)
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    out = np.zeros((rows, g.shape[1]), np.float32)
    _op_check(load_library().kge_op_scatter_add_rows(_fp(g), idx.ctypes.data_as(C.POINTER(C.c_uint32)),
                                                     idx.size, rows, g.shape[1], _fp(out)))
    return out


def op_scatter_add_rows_noalloc(grad_rows_ptr: int, indices_ptr: int, n: int, rows: int, width: int,
                                grad_table_ptr: int, stream_ptr: int = 0) -> None:
    """The allocation-free scatter-add on caller-owned DEVICE buffers (raw addresses); queued on
    ``stream_ptr`` (a cudaStream_t as an integer, 0 = default stream), not waited for."""
    _op_check(load_library().kge_op_scatter_add_rows_noalloc(grad_rows_ptr, indices_ptr, n, rows, width,
                                                             grad_table_ptr, stream_ptr or None))


def op_tc_gemm(a, b, m: int, n: int, k: int, a_transposed: bool = False, b_transposed: bool = False, a_gather=None,
               epilogue: int = 0, x=None, splits: int = 1, tile_n: int = 128) -> np.ndarray:
    """Tensor-core contraction out[z, m, n] (see kge_op_tc_gemm); ``a`` may be float16 or float32."""
    a = np.ascontiguousarray(a)
    if a.dtype not in (np.float16, np.float32):
        a = a.astype(np.float32)
    b = _f32(b)
    gather = np.ascontiguousarray(a_gather, dtype=np.uint32) if a_gather is not None else None
    xx = _f32(x) if x is not None else None
    out = np.empty((splits, m, n), np.float32)
    _op_check(load_library().kge_op_tc_gemm(
        a.ctypes.data, int(a.dtype == np.float16), int(a_transposed),
        gather.ctypes.data_as(C.POINTER(C.c_uint32)) if gather is not None else None, a.shape[0], a.shape[1],
        _fp(b), int(b_transposed), b.shape[0], b.shape[1], m, n, k, epilogue, _fp(xx) if xx is not None else None,
        splits, tile_n, _fp(out)))
    return out


def op_tc_planes(a, b, m: int, n: int, k: int, a_mn_major: bool = False, b_mn_major: bool = False, a_exact: bool = False,
                 epilogue: int = 0, x=None, splits: int = 1, tile_n: int = 128, hi_is_cleared: bool = False, repeat: int = 0):
    """Plane-fed tensor-core contraction out[m, n] (see kge_op_tc_planes); returns (out, mean_us)."""
    a, b = _f32(a), _f32(b)
    xx = _f32(x) if x is not None else None
    out = np.empty((m, n), np.float32)
    mean_us = C.c_float(0.0)
    _op_check(load_library().kge_op_tc_planes(
        _fp(a), int(a_mn_major), int(a_exact), a.shape[0], a.shape[1], _fp(b), int(b_mn_major), b.shape[0], b.shape[1],
        m, n, k, epilogue, _fp(xx) if xx is not None else None, splits, tile_n, int(hi_is_cleared), repeat,
        C.byref(mean_us), _fp(out)))
    return out, float(mean_us.value)


def op_tc_planes_bf16(a, b, m: int, n: int, k: int, a_mn_major: bool = False, b_mn_major: bool = False, splits: int = 1,
                      tile_n: int = 128, repeat: int = 0):
    """bf16 tensor-core contraction out[m, n] (see kge_op_tc_planes_bf16); returns (out, mean_us)."""
    a, b = _f32(a), _f32(b)
    out = np.empty((m, n), np.float32)
    mean_us = C.c_float(0.0)
    _op_check(load_library().kge_op_tc_planes_bf16(_fp(a), int(a_mn_major), a.shape[0], a.shape[1], _fp(b), int(b_mn_major),
                                                   b.shape[0], b.shape[1], m, n, k, splits, tile_n, repeat, C.byref(mean_us), _fp(out)))
    return out, float(mean_us.value)


def microbench_rows(kind: int, table_rows: int, d: int, indices, repeat: int = 20) -> float:
    """Mean device microseconds of the step's row gather (kind 0) or row-wise Adam scatter (kind 1)."""
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    us = C.c_float(0.0)
    _op_check(load_library().kge_microbench_rows(kind, table_rows, d, idx.ctypes.data_as(C.POINTER(C.c_uint32)), idx.size, repeat, C.byref(us)))
    return float(us.value)


def microbench_scores(fn: int, m: int, n: int, k: int, repeat: int = 50) -> float:
    """Mean device microseconds of m x n scores, k deep (fn: 0 L1, 1 L2, 2 dot, 3 L2 on the tensor cores)."""
    us = C.c_float(0.0)
    _op_check(load_library().kge_microbench_scores(fn, m, n, k, repeat, C.byref(us)))
    return float(us.value)


def op_activation(kind: int, x, grad_out) -> Tuple[np.ndarray, np.ndarray]:
    x, g = _f32(x), _f32(grad_out)
    x2 = x.reshape(-1, x.shape[-1]) if x.ndim > 1 else x.reshape(1, -1)
    y, gx = np.empty_like(x2), np.empty_like(x2)
    _op_check(load_library().kge_op_activation(kind, _fp(x2), _fp(g.reshape(x2.shape)), x2.shape[0],
                                               x2.shape[1], _fp(y), _fp(gx)))
    return y.reshape(x.shape), gx.reshape(x.shape)


def op_all_to_all(blocks) -> np.ndarray:
    """blocks [n_shard, n_shard, block...] -> out[dst, src] = blocks[src, dst]."""
    a = _f32(blocks)
    n = a.shape[0]
    block = int(np.prod(a.shape[2:])) if a.ndim > 2 else 1
    out = np.empty_like(a)
    _op_check(load_library().kge_op_all_to_all(_fp(a), n, block, _fp(out)))
    return out
