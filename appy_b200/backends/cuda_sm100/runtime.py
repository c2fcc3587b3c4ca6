"""ctypes binding of libappy_sm100.so (declarations: include/appy_sm100.h).

Every wrapper raises ``RuntimeError`` carrying ``appy_last_error()`` when the C
function returns a non-zero status.  There is no fallback: if the library is
missing it is built in-tree with nvcc, and if that fails the import raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_LIB = None
_LOCK = threading.Lock()

c_void_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); used for loading and by the symbol test
SIGNATURES = {
    "appy_init": (C.c_int, [C.c_int]),
    "appy_shutdown": (C.c_int, []),
    "appy_last_error": (C.c_char_p, []),
    "appy_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "appy_device_info": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   C.POINTER(C.c_int), C.POINTER(C.c_size_t)]),
    "appy_get_stream": (C.c_int, [C.c_int, c_void_pp]),
    "appy_sync": (C.c_int, [C.c_void_p]),
    "appy_launch_count": (C.c_int64, []),
    "appy_reset_launch_count": (None, []),
    "appy_malloc": (C.c_int, [c_void_pp, C.c_size_t]),
    "appy_free": (C.c_int, [C.c_void_p]),
    "appy_trim": (C.c_int, []),
    "appy_memset": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "appy_register_host": (C.c_int, [C.c_void_p, C.c_size_t]),
    "appy_unregister_host": (C.c_int, [C.c_void_p]),
    "appy_mirror": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp, C.POINTER(C.c_int)]),
    "appy_evict": (C.c_int, [C.c_void_p]),
    "appy_h2d_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "appy_d2h_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "appy_host_cells": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "appy_h2d_staged": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "appy_d2d_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "appy_compile": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, c_void_pp]),
    "appy_compile_check": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_size_t)]),
    "appy_compile_image": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_size_t),
                                     C.POINTER(C.c_int)]),
    "appy_compile_log": (C.c_char_p, []),
    "appy_kernel_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   C.POINTER(C.c_int)]),
    "appy_occupancy": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.POINTER(C.c_int)]),
    "appy_launch": (C.c_int, [C.c_void_p, C.c_uint, C.c_uint, C.c_size_t, c_void_pp, C.c_void_p]),
    "appy_time_launches": (C.c_int, [C.c_void_p, C.c_uint, C.c_uint, C.c_size_t, c_void_pp,
                                     C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "appy_workspace": (C.c_int, [C.c_void_p, c_void_pp, C.POINTER(C.c_size_t)]),
    "appy_scratch": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp]),
    "appy_partition_range": (C.c_int, [C.c_int64, C.c_int64, C.c_int, C.c_int64,
                                       C.POINTER(C.c_int64)]),
    "appy_partition_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int,
                                      C.POINTER(C.c_int64)]),
    "appy_partition_rows_weighted": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int64,
                                               C.POINTER(C.c_int64)]),
    "appy_row_histogram": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.POINTER(C.c_int64),
                                     C.POINTER(C.c_int64), C.c_void_p]),
    "appy_p2p_create": (C.c_int, [C.c_int, C.c_int, c_void_pp, C.c_void_p]),
    "appy_p2p_open": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint, c_void_pp]),
    "appy_p2p_open_local": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint, c_void_pp]),
    "appy_p2p_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "appy_p2p_destroy": (C.c_int, [C.c_void_p]),
    "appy_p2p_combine": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "appy_probe_row_gather_f32": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_void_p,
                                            C.c_void_p]),
    "appy_probe_gather_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "appy_p2p_flush": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "appy_vec_add_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "appy_sum_f32": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]),
    "appy_sum_f32_noalloc": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "appy_masked_sum_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int,
                                      C.c_void_p]),
    "appy_spmv_csr_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "appy_gemv_f32": (C.c_int, [C.c_float, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "appy_spmm_csr_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                    C.c_void_p]),
}


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "libappy_sm100.so")


def template_dir() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "csrc", "templates")


def lib() -> C.CDLL:
    """Load (building first if needed) the shared library; never falls back."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not os.path.exists(path):
            from ... import build as _build
            _build.build()
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


class AppyRuntimeError(RuntimeError):
    pass


def check(status: int) -> None:
    if status != 0:
        msg = lib().appy_last_error()
        raise AppyRuntimeError((msg or b"").decode("utf-8", "replace") or f"libappy_sm100 error {status}")


# --------------------------------------------------------------------------- helpers

_init_done: set[int] = set()


def init(device: int = 0) -> None:
    if device not in _init_done:
        check(lib().appy_init(device))
        _init_done.add(device)
    else:
        check(lib().appy_init(device))


def device_count() -> int:
    n = C.c_int(0)
    try:
        check(lib().appy_device_count(C.byref(n)))
    except AppyRuntimeError:
        return 0
    return n.value


def device_info(device: int = 0) -> dict:
    sm, l2, cc = C.c_int(), C.c_int(), C.c_int()
    mem = C.c_size_t()
    check(lib().appy_device_info(device, C.byref(sm), C.byref(l2), C.byref(cc), C.byref(mem)))
    return {"sm_count": sm.value, "l2_bytes": l2.value, "cc": cc.value, "total_mem": mem.value}


def stream(which: int = 0) -> int:
    s = C.c_void_p()
    check(lib().appy_get_stream(which, C.byref(s)))
    return s.value or 0


def sync(stream_: int = 0) -> None:
    check(lib().appy_sync(C.c_void_p(stream_)))


def malloc(nbytes: int) -> int:
    p = C.c_void_p()
    check(lib().appy_malloc(C.byref(p), nbytes))
    return p.value


def free(dptr: int) -> None:
    check(lib().appy_free(C.c_void_p(dptr)))


def mirror(hptr: int, nbytes: int) -> tuple[int, bool]:
    p = C.c_void_p()
    created = C.c_int()
    check(lib().appy_mirror(C.c_void_p(hptr), nbytes, C.byref(p), C.byref(created)))
    return p.value, bool(created.value)


def h2d(dptr: int, hptr: int, nbytes: int, stream_: int = 0) -> None:
    check(lib().appy_h2d_async(C.c_void_p(dptr), C.c_void_p(hptr), nbytes, C.c_void_p(stream_)))


def h2d_staged(dptr: int, hptr: int, nbytes: int, stream_: int = 0) -> None:
    check(lib().appy_h2d_staged(C.c_void_p(dptr), C.c_void_p(hptr), nbytes, C.c_void_p(stream_)))


def d2h(hptr: int, dptr: int, nbytes: int, stream_: int = 0) -> None:
    check(lib().appy_d2h_async(C.c_void_p(hptr), C.c_void_p(dptr), nbytes, C.c_void_p(stream_)))


def host_cells() -> tuple[int, int, int]:
    """(host address, device address, bytes) of the current device's page of mapped pinned memory."""
    h, d, n = C.c_void_p(), C.c_void_p(), C.c_size_t()
    check(lib().appy_host_cells(C.byref(h), C.byref(d), C.byref(n)))
    return h.value, d.value, n.value


def workspace(stream_: int = 0) -> int:
    p = C.c_void_p()
    check(lib().appy_workspace(C.c_void_p(stream_), C.byref(p), None))
    return p.value


def scratch(stream_: int, nbytes: int) -> int:
    """Grow-only scratch buffer of the current device for kernels queued on `stream_`."""
    p = C.c_void_p()
    check(lib().appy_scratch(C.c_void_p(stream_), nbytes, C.byref(p)))
    return p.value


def nvrtc_options(extra: list[str] | None = None) -> bytes:
    opts = ["-I" + template_dir()]
    if extra:
        opts += extra
    return "\n".join(opts).encode()


def default_cache_dir() -> str | None:
    d = os.environ.get("APPY_CACHE_DIR")
    if d == "":
        return None
    if d is None:
        d = os.path.join(os.path.expanduser("~"), ".cache", "appy_sm100")
    try:
        os.makedirs(d, exist_ok=True)
    except OSError:
        return None
    return d


def compile_kernel(src: str, name: str, extra_opts: list[str] | None = None) -> int:
    h = C.c_void_p()
    cache = default_cache_dir()
    check(lib().appy_compile(src.encode(), name.encode(), nvrtc_options(extra_opts),
                             cache.encode() if cache else None, C.byref(h)))
    return h.value


def compile_check(src: str, name: str, extra_opts: list[str] | None = None) -> int:
    """NVRTC-only compile (no GPU needed); returns cubin size, raises with the log on error."""
    n = C.c_size_t()
    check(lib().appy_compile_check(src.encode(), name.encode(), nvrtc_options(extra_opts), C.byref(n)))
    return n.value


def compile_image(src: str, name: str, extra_opts: list[str] | None = None, cache_dir: str | None = None):
    """(cubin size, came from the on-disk cache) — the compile step of `compile_kernel` without loading."""
    n, hit = C.c_size_t(), C.c_int()
    check(lib().appy_compile_image(src.encode(), name.encode(), nvrtc_options(extra_opts),
                                   cache_dir.encode() if cache_dir else None, C.byref(n), C.byref(hit)))
    return n.value, bool(hit.value)


def kernel_info(handle: int) -> dict:
    regs, smem, mt = C.c_int(), C.c_int(), C.c_int()
    check(lib().appy_kernel_info(C.c_void_p(handle), C.byref(regs), C.byref(smem), C.byref(mt)))
    return {"regs": regs.value, "static_smem": smem.value, "max_threads": mt.value}


def occupancy(handle: int, block: int, dyn_smem: int = 0) -> int:
    n = C.c_int()
    check(lib().appy_occupancy(C.c_void_p(handle), block, dyn_smem, C.byref(n)))
    return n.value


class ArgPack:
    """Kernel arguments marshalled once into ctypes storage; reusable across launches."""

    __slots__ = ("values", "ptrs")

    def __init__(self, ctypes_values):
        self.values = list(ctypes_values)
        n = len(self.values)
        self.ptrs = (C.c_void_p * max(n, 1))()
        for i, v in enumerate(self.values):
            self.ptrs[i] = C.cast(C.pointer(v), C.c_void_p)


def launch(handle: int, grid: int, block: int, args: ArgPack, dyn_smem: int = 0, stream_: int = 0) -> None:
    # argtypes are declared, so plain ints convert without building ctypes objects first
    if (_LIB or lib()).appy_launch(handle, grid, block, dyn_smem, args.ptrs, stream_ or None) != 0:
        check(-1)


def time_launches(handle: int, grid: int, block: int, args: ArgPack, dyn_smem: int = 0,
                  stream_: int = 0, warmup: int = 2, iters: int = 10) -> float:
    ms = C.c_float()
    check(lib().appy_time_launches(C.c_void_p(handle), grid, block, dyn_smem, args.ptrs,
                                   C.c_void_p(stream_), warmup, iters, C.byref(ms)))
    return ms.value / iters


def launch_count() -> int:
    return int(lib().appy_launch_count())


def partition_range(lo: int, hi: int, parts: int, align: int = 1) -> list[int]:
    out = (C.c_int64 * (parts + 1))()
    check(lib().appy_partition_range(lo, hi, parts, align, out))
    return list(out)


def partition_rows(indptr, parts: int, row_cost: int = 0) -> list[int]:
    """Contiguous row split balanced by non-zeros plus `row_cost` per row; `indptr` is a host numpy
    int32/int64 array."""
    import numpy as np
    ip = np.ascontiguousarray(indptr)
    if ip.dtype not in (np.int32, np.int64):
        ip = ip.astype(np.int64)
    out = (C.c_int64 * (parts + 1))()
    check(lib().appy_partition_rows_weighted(C.c_void_p(ip.ctypes.data), ip.dtype.itemsize, len(ip) - 1, parts,
                                             row_cost, out))
    return list(out)


def row_histogram(d_indptr: int, idx_bytes: int, nrows: int, stream_: int = 0) -> tuple[list[int], int]:
    counts = (C.c_int64 * 32)()
    mx = C.c_int64()
    check(lib().appy_row_histogram(C.c_void_p(d_indptr), idx_bytes, nrows, counts, C.byref(mx),
                                   C.c_void_p(stream_)))
    return list(counts), mx.value
