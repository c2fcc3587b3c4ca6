"""Builds and binds ``loops.c`` (oracle; test infrastructure).

``build()`` compiles the C restatement with gcc into ``oracle/_build/liboracle.so``
(-O2 -fopenmp, no fast-math: IEEE float32 semantics must hold for the bit-exact
cases).  The wrappers take NumPy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "loops.c")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", "-o", OUT, src]
    subprocess.run(cmd, check=True, capture_output=True)
    return OUT


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.oracle_vec_sum_f32.restype = C.c_double
        _lib.oracle_masked_sum_f32.restype = C.c_double
        _lib.oracle_threads.restype = C.c_int
    return _lib


def threads() -> int:
    return int(lib().oracle_threads())


def set_threads(n: int) -> int:
    """Use `n` OpenMP threads from now on (whatever OMP_NUM_THREADS says); returns the count in effect."""
    lib().oracle_set_threads(C.c_int(int(n)))
    return threads()


def host_cores() -> int:
    """Cores this process may run on (the affinity mask, not the machine's total)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _p(a):
    return C.c_void_p(a.ctypes.data)


def vec_add(a, b):
    a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
    c = np.empty_like(a)
    lib().oracle_vec_add_f32(_p(a), _p(b), _p(c), C.c_int64(a.size))
    return c


def vec_sum(a, init=0.0):
    a = np.ascontiguousarray(a, np.float32)
    return float(lib().oracle_vec_sum_f32(_p(a), C.c_int64(a.size), C.c_double(init)))


def masked_sum(a, mask, init=0.0):
    a = np.ascontiguousarray(a, np.float32)
    m = np.ascontiguousarray(mask).view(np.uint8)
    return float(lib().oracle_masked_sum_f32(_p(a), _p(m), C.c_int64(a.size), C.c_double(init)))


def spmv(data, indptr, indices, x, nrows=None):
    nrows = len(indptr) - 1 if nrows is None else nrows
    y = np.empty(nrows, np.float32)
    lib().oracle_spmv_f32(_p(data), _p(indptr), _p(indices), _p(x), _p(y), C.c_int64(0), C.c_int64(nrows))
    return y


def gemv(alpha, A, x):
    y = np.empty(A.shape[0], np.float32)
    lib().oracle_gemv_f32(C.c_float(alpha), _p(A), C.c_int64(A.strides[0] // 4), _p(x), _p(y),
                          C.c_int64(0), C.c_int64(A.shape[0]), C.c_int64(A.shape[1]))
    return y


def spmm(data, indptr, indices, B, nrows=None):
    nrows = len(indptr) - 1 if nrows is None else nrows
    Cm = np.empty((nrows, B.shape[1]), np.float32)
    lib().oracle_spmm_f32(_p(data), _p(indptr), _p(indices), _p(B), C.c_int64(B.strides[0] // 4), _p(Cm),
                          C.c_int64(Cm.strides[0] // 4), C.c_int64(0), C.c_int64(nrows), C.c_int(B.shape[1]))
    return Cm
