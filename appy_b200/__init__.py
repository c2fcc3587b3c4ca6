"""appy_b200 — a B200-native execution backend for APPy-style annotated loops.

Public surface (same names and meaning as the reference's ``appy`` package,
appy/__init__.py:67-151)::

    @appy_b200.jit                      # or @jit(dump_code=True, ...)
    def kernel(a, b):
        c = np.empty_like(a)
        #pragma parallel for simd
        for i in range(a.shape[0]):
            c[i] = a[i] + b[i]
        return c

Annotated loops are compiled to CUDA C kernels for sm_100a and launched through
libappy_sm100.so; everything else in the function stays interpreted Python.
Scalars are passed by value, ``shared(...)`` scalars are copied back, arrays are
updated in place.
"""
from __future__ import annotations

import inspect
import textwrap

from . import dispatcher
from .frontend.static_rewrite import RUNTIME_NAME, rewrite_function_source

__all__ = ["jit", "prange", "range", "vidx", "to_gpu", "to_cpu", "shader", "cpu_shader", "set_default_options"]

_builtin_range = range


def _kernel_launch(loop_source, loop_name, scope, global_scope, options):
    """Runtime stub called in place of an annotated loop (appy/__init__.py:18-35)."""
    dispatcher.codegen(options.get("backend"), loop_source, loop_name, scope, global_scope, options)


def set_default_options(options: dict) -> None:
    options.setdefault("backend", None)
    options.setdefault("dry_run", False)
    options.setdefault("dump_code", False)
    options.setdefault("dump_code_to_file", None)
    options.setdefault("verbose_static_rewrite", False)
    options.setdefault("verbose_block_loop", False)


def rewrite_loops(fn, **options):
    import sys
    source = textwrap.dedent(inspect.getsource(fn))
    if options.get("shader"):
        raise NotImplementedError("shader mode is outside the scope of the cuda_sm100 backend")
    newcode = rewrite_function_source(source, options)
    if options.get("verbose_static_rewrite"):
        print("[Static Rewrite] new code:\n", newcode)
    code = compile(newcode, filename=f"<appy_b200:{fn.__name__}>", mode="exec")
    import numpy
    fn.__globals__["numpy"] = numpy
    fn.__globals__[RUNTIME_NAME] = sys.modules[__name__]
    namespace: dict = {}
    exec(code, fn.__globals__, namespace)
    new_fn = namespace[fn.__name__]
    new_fn.__wrapped__ = fn
    return new_fn


def jit(fn=None, **options):
    set_default_options(options)
    if fn is not None:
        return rewrite_loops(fn, **options)

    def jit_with_args(fn1):
        return rewrite_loops(fn1, **options)

    return jit_with_args


def shader(fn=None, **options):
    options["shader"] = True
    return jit(fn, **options)


def cpu_shader(fn=None, **options):
    raise NotImplementedError("the CPU (numba) backend is outside the scope of the cuda_sm100 backend")


def vidx(start, stepsize, bound=None):
    if bound:
        return slice(start, min(bound, start + stepsize))
    return slice(start, start + stepsize)


class prange(object):
    """1-D parallel iterator; outside a jitted function it is ``range``."""

    def __new__(cls, *args, shared=None):
        return _builtin_range(*args)


def range(*args, parallel=False, simd=False):  # noqa: A001 - same name as the reference
    return _builtin_range(*args)


def to_gpu(*args):
    out = [_to_gpu(a) for a in args]
    return out[0] if len(out) == 1 else out


def _to_gpu(a):
    import numpy as np
    import torch
    if isinstance(a, np.ndarray):
        from .backends.cuda_sm100.codegen import to_device
        return to_device(a)
    if isinstance(a, torch.Tensor):
        return a.to("cuda")
    if isinstance(a, list):
        return torch.tensor(a).to("cuda")
    if isinstance(a, (int, float)):
        return a
    raise AssertionError("Unsupported type to transfer to GPU")


def resident(*arrays):
    """Declare NumPy arrays resident: a loop uploads such an array the first time it uses it and then
    trusts its device copy until ``touch`` says that the host copy was written.  Without this every call
    uploads every NumPy argument, as the reference's generated host code does
    (appy/backends/triton/passes/host_passes/gen_data_movement.py:14-96).  Returns its argument(s)."""
    from .backends.cuda_sm100 import codegen
    return codegen.resident(*arrays)


def touch(*arrays):
    """The host copies of these resident arrays were modified: upload them again at their next use."""
    from .backends.cuda_sm100 import codegen
    codegen.touch(*arrays)


def release(*arrays):
    """Undo ``resident``: the arrays are uploaded on every call again."""
    from .backends.cuda_sm100 import codegen
    codegen.release(*arrays)


def to_cpu(*args):
    out = [_to_cpu(a) for a in args]
    return out[0] if len(out) == 1 else out


def _to_cpu(a):
    import torch
    if isinstance(a, torch.Tensor):
        return a.item() if a.ndim == 0 else a.to("cpu").numpy()
    return a
