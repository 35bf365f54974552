"""ctypes binding of the C oracle (oracle/cb_oracle.c).  TEST INFRASTRUCTURE ONLY:
used by the tests and by the CPU-baseline leg of the benchmark."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libcb_oracle.so")


class Fmt(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("grid", "mode", "k_bits", "n_sub", "type_size", "scale_coding")]


_lib = None


def load(build: bool = True):
    global _lib
    if _lib is not None:
        return _lib
    if build and (not os.path.exists(LIB_PATH)
                  or os.path.getmtime(LIB_PATH) < os.path.getmtime(os.path.join(HERE, "cb_oracle.c"))):
        subprocess.check_call(["make", "-s", "-C", HERE])
    lib = ctypes.CDLL(LIB_PATH)
    lib.gbo_num_threads.restype = ctypes.c_int
    _lib = lib
    return lib


def _fmt(grid, mode, k_bits, n_sub, type_size, scale_coding) -> Fmt:
    return Fmt(0 if grid == "fp4" else 1, {"product": 0, "signed": 1, "full": 2}[mode or ("signed" if n_sub == 1 else "product")],
               k_bits, n_sub, type_size, 0 if grid == "fp8" else (2 if scale_coding == "v2" else 1))


def _p(a, t=ctypes.c_void_p):
    return None if a is None else a.ctypes.data_as(t)


def num_threads() -> int:
    return load().gbo_num_threads()


def linear(x, qw, cb, cb_row_offset, *, N, K, k_bits, n_sub, type_size, grid, mode=None,
           scale_coding="v1", compose=None, weight_scale=None, global_scale=None) -> np.ndarray:
    lib = load()
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, K)
    qw = np.ascontiguousarray(qw)
    cb = np.ascontiguousarray(cb, dtype=np.float32)
    off = None if cb_row_offset is None else np.ascontiguousarray(cb_row_offset, dtype=np.int32)
    comp = None if compose is None else np.ascontiguousarray(compose, dtype=np.float32)
    ws = None if weight_scale is None else np.ascontiguousarray(weight_scale, dtype=np.float32)
    y = np.empty((x.shape[0], N), dtype=np.float32)
    f = _fmt(grid, mode, k_bits, n_sub, type_size, scale_coding)
    lib.gbo_linear(_p(x), ctypes.c_int64(x.shape[0]), _p(qw), ctypes.c_int64(qw.strides[0]), _p(cb), _p(off),
                   _p(comp), _p(ws), ctypes.c_float(1.0 if global_scale is None else global_scale),
                   ctypes.byref(f), ctypes.c_int64(N), ctypes.c_int64(K), _p(y))
    return y


def reconstruct(qw, cb, cb_row_offset, *, N, K, k_bits, n_sub, type_size, grid, mode=None,
                scale_coding="v1", compose=None, weight_scale=None) -> np.ndarray:
    lib = load()
    qw = np.ascontiguousarray(qw)
    cb = np.ascontiguousarray(cb, dtype=np.float32)
    off = None if cb_row_offset is None else np.ascontiguousarray(cb_row_offset, dtype=np.int32)
    comp = None if compose is None else np.ascontiguousarray(compose, dtype=np.float32)
    ws = None if weight_scale is None else np.ascontiguousarray(weight_scale, dtype=np.float32)
    out = np.empty((N, K), dtype=np.float32)
    f = _fmt(grid, mode, k_bits, n_sub, type_size, scale_coding)
    lib.gbo_reconstruct(_p(qw), ctypes.c_int64(qw.strides[0]), _p(cb), _p(off), _p(comp), _p(ws),
                        ctypes.byref(f), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(0),
                        ctypes.c_int64(N), _p(out))
    return out


def act_qdq(x, grid: str, scale_rule: str = "div") -> np.ndarray:
    lib = load()
    x = np.ascontiguousarray(x, dtype=np.float32)
    K = x.shape[-1]
    out = np.empty_like(x)
    fn = lib.gbo_fp4_act_qdq if grid == "fp4" else lib.gbo_fp8_act_qdq
    fn(_p(x), ctypes.c_int64(x.size // K), ctypes.c_int64(K), ctypes.c_int(1 if scale_rule == "div" else 0), _p(out))
    return out
