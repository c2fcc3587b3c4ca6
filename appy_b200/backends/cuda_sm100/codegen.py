"""Plugin entry of the cuda_sm100 backend.

    codegen(loop_source, loop_name, val_map, options) -> (f, code_src)

is the boundary the reference's dispatcher calls for its Triton backend
(appy/backends/triton/codegen.py:9,73, selected in appy/dispatcher.py:19-43): `f` takes
the non-module values of `val_map` positionally, in `val_map` order, mutates arrays in
place and returns nothing; `code_src` is the generated source (here: CUDA C).

What differs underneath: the generated host function of the reference copies every
NumPy / CPU-tensor argument with ``tensor.to('cuda')`` and back with ``copy_`` on each
call (appy/backends/triton/passes/host_passes/gen_data_movement.py:14-96) and launches
``_kernel[grid](..., num_warps=4)`` (host_passes/gen_kernel_launch.py:56-69).  Here `f`
is a ``CompiledLoop``: it keeps device mirrors of host arrays in the shim's residency
cache, pins large host buffers that are seen repeatedly, copies asynchronously on a
stream, specialises the kernel on what decides the code (dtypes, ranks, pointer
alignment, stride divisibility, overlap of stored arrays with others) and can time
candidate launch configurations once per specialisation (the block-size autotuner).
CUDA tensors are used in place and never copied or synchronised.
"""
from __future__ import annotations

import ast
import ctypes as C
import hashlib
import json
import os
import sys
import types as _types

import numpy as np

from ...frontend.loop_normalize import normalize
from ...utils import pretty_dump
from . import dtypes as T
from . import runtime as rt
from .lower import ArgInfo, KernelPlan, Lowering, stored_arrays

code_cache: dict = {}          # (loop_source, signature, options) -> CompiledLoop
_PIN_MIN_BYTES = 1 << 20
_seen_host: dict = {}          # host ptr -> times seen (for the pin-on-second-use policy)
_tune_cache: dict | None = None


def _is_torch(v) -> bool:
    t = sys.modules.get("torch")
    return t is not None and isinstance(v, t.Tensor)


_SIMPLE_KINDS = {bool: ("S", "bool"), int: ("S", "pyint"), float: ("S", "pyfloat"), np.bool_: ("S", "bool"),
                 _types.ModuleType: ("M",)}


_TORCH_TENSOR = None      # torch.Tensor once torch has been imported


def _kind_of(v) -> tuple:
    """Signature entry of one argument: decides which kernel source is generated.
    Arrays: ("A", where, dtype object, rank); scalars: ("S", kind); modules: ("M",)."""
    global _TORCH_TENSOR
    t = type(v)
    k = _SIMPLE_KINDS.get(t)
    if k is not None:
        return k
    if t is _TORCH_TENSOR:
        return ("A", v.device.type, v.dtype, v.ndim)
    if t is np.ndarray:
        return ("A", "np", v.dtype, v.ndim)
    if _TORCH_TENSOR is None and "torch" in sys.modules:
        _TORCH_TENSOR = sys.modules["torch"].Tensor
        if t is _TORCH_TENSOR:
            return ("A", v.device.type, v.dtype, v.ndim)
    if _is_torch(v):
        return ("A", v.device.type, v.dtype, v.ndim)
    if isinstance(v, np.ndarray):
        return ("A", "np", v.dtype, v.ndim)
    if isinstance(v, np.generic):
        return ("S", str(v.dtype))
    if isinstance(v, bool):
        return ("S", "bool")
    if isinstance(v, int):
        return ("S", "pyint")
    if isinstance(v, float):
        return ("S", "pyfloat")
    if isinstance(v, _types.ModuleType):
        return ("M",)
    raise TypeError(f"Unsupported argument of type {type(v).__name__} in a parallel loop")


def _elem_type(dtype):
    if isinstance(dtype, np.dtype):
        return T.from_numpy(dtype)
    return T.from_torch(dtype)


def _scalar_type(kind: str):
    if kind == "bool":
        return T.BOOL
    if kind == "pyint":
        return T.WEAK_INT
    if kind == "pyfloat":
        return T.WEAK_FLOAT
    return T.from_numpy(np.dtype(kind))


_CT = {("b", 8): C.c_bool, ("i", 8): C.c_int8, ("i", 16): C.c_int16, ("i", 32): C.c_int32, ("i", 64): C.c_int64,
       ("u", 8): C.c_uint8, ("u", 16): C.c_uint16, ("u", 32): C.c_uint32, ("u", 64): C.c_uint64,
       ("f", 32): C.c_float, ("f", 64): C.c_double}


def _tune_store() -> dict:
    global _tune_cache
    if _tune_cache is None:
        _tune_cache = {}
        d = rt.default_cache_dir()
        if d:
            try:
                with open(os.path.join(d, "autotune.json")) as fh:
                    _tune_cache = json.load(fh)
            except (OSError, ValueError):
                _tune_cache = {}
    return _tune_cache


def _tune_save() -> None:
    d = rt.default_cache_dir()
    if not d or _tune_cache is None:
        return
    try:
        tmp = os.path.join(d, f"autotune.json.{os.getpid()}")
        with open(tmp, "w") as fh:
            json.dump(_tune_cache, fh)
        os.replace(tmp, os.path.join(d, "autotune.json"))
    except OSError:
        pass


def _torch_stream(torch, device: int) -> int:
    """Raw handle of torch's current stream (kernels on CUDA tensors must order with torch)."""
    try:
        return torch._C._cuda_getCurrentRawStream(device)
    except AttributeError:
        return torch.cuda.current_stream().cuda_stream


_cell_turn = [0]        # which 512-byte window of the page of host cells the next call uses
_cell_pages: dict = {}  # device -> (host address, device address, bytes) of its page of host cells


class _Array:
    """One array argument resolved for a launch."""
    __slots__ = ("name", "obj", "host", "dptr", "nbytes", "shape", "strides", "itemsize", "tmp", "hptr",
                 "pinnable", "cell")


class _DevView:
    """Minimal __cuda_array_interface__ holder so torch can wrap a device mirror without copying."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


_IDENTITY = {"+": 0, "*": 1}


class Variant:
    def __init__(self, plan: KernelPlan):
        self.plan = plan
        self.handles: dict = {}       # tunables tuple -> kernel handle
        self.tun = {k: v[0] for k, v in plan.tunables.items()}      # defaults: first candidate of each
        self.choice: dict = {}        # shape class -> tunables settled for it
        self.last_tun = self.tun
        self.lo_code = compile(ast.Expression(body=plan.lo_expr), "<lo>", "eval")
        self.hi_code = compile(ast.Expression(body=plan.hi_expr), "<hi>", "eval")

    def handle(self, tun: dict) -> int:
        key = tuple(sorted(tun.items()))
        h = self.handles.get(key)
        if h is None:
            opts = [f"-D{k}={v}" for k, v in tun.items()] + list(self.plan.info.get("nvrtc", []))
            h = rt.compile_kernel(self.plan.source, self.plan.name, opts)
            self.handles[key] = h
        return h

    def post_handle(self, tun: dict) -> int:
        """The plan's second kernel (same source, same options), launched after the main one."""
        key = ("post",) + tuple(sorted(tun.items()))
        h = self.handles.get(key)
        if h is None:
            opts = [f"-D{k}={v}" for k, v in tun.items()] + list(self.plan.info.get("nvrtc", []))
            h = rt.compile_kernel(self.plan.source, self.plan.post, opts)
            self.handles[key] = h
        return h


class CompiledLoop:
    def __init__(self, loop_source: str, loop_name: str, names: list, signature: tuple, options: dict):
        self.loop_source = loop_source
        self.loop_name = loop_name
        fn = options.get("_fn")
        self.kernel_name = f"{fn}_{loop_name}" if fn and str(fn).isidentifier() else loop_name
        self.names = names                  # val_map names, modules included
        self.signature = signature
        self.options = dict(options)
        self.variants: dict = {}
        self.arg_names = [n for n, s in zip(names, signature) if s[0] != "M"]
        self.arg_sigs = [s for s in signature if s[0] != "M"]
        ndims = {n: s[3] for n, s in zip(names, signature) if s[0] == "A"}
        self.ir = normalize(loop_source, lambda nm: ndims.get(nm))
        self.stored = stored_arrays([self.ir.loop])
        self.last_variant: Variant | None = None
        self.last_source: str | None = None
        self.memo: dict = {}
        self.has_device_args = any(sg[0] == "A" and sg[1] == "cuda" for sg in self.arg_sigs)
        # Scalars whose value only flows into the arithmetic (not into any range bound) do not shape the
        # launch: records are shared across their values and the value is patched into the arguments.
        in_ranges = set()
        for n in ast.walk(self.ir.loop):
            if isinstance(n, ast.For) and isinstance(n.iter, ast.Call):
                for arg in n.iter.args:
                    in_ranges |= {x.id for x in ast.walk(arg) if isinstance(x, ast.Name)}
        self.data_scalars = frozenset(i for i, (nm, sg) in enumerate(zip(self.arg_names, self.arg_sigs))
                                      if sg[0] == "S" and nm not in in_ranges)
        self.device = None
        self.sm_count = 148
        self.cell_names = self._find_cell_names()
        self.overwritten, self._range_codes = self._find_overwritten()

    def _find_cell_names(self) -> frozenset:
        """Arrays that the loop touches only as targets of its own reductions (`s[0] += ...`, what a
        shared(...) scalar becomes).  When such an array arrives as a small host array it needs no device
        mirror: the kernel is given a cell in mapped host memory (_host_cells)."""
        from ...frontend.loop_normalize import reductions_of
        targets = {}
        for text in reductions_of(self.ir.loop):
            node = ast.parse(text, mode="eval").body
            if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name) \
                    and isinstance(node.slice, ast.Constant):
                targets.setdefault(node.value.id, set()).add(text)
            elif isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name):
                targets.setdefault(node.value.id, set()).add(None)        # not a constant index: no cell
        names = set()
        for name, texts in targets.items():
            if None in texts:
                continue
            ok = True
            for st in ast.walk(self.ir.loop):
                if isinstance(st, (ast.Assign, ast.AugAssign)):
                    if not any(isinstance(x, ast.Name) and x.id == name for x in ast.walk(st)):
                        continue
                    tgt = st.targets[0] if isinstance(st, ast.Assign) else st.target
                    if ast.unparse(tgt) not in texts:
                        ok = False
                elif isinstance(st, (ast.If, ast.While, ast.For)):
                    head = st.test if not isinstance(st, ast.For) else st.iter
                    if any(isinstance(x, ast.Name) and x.id == name for x in ast.walk(head)):
                        ok = False
            if ok:
                names.add(name)
        return frozenset(names)

    def _find_overwritten(self):
        """(names, (lo code, hi code)): one-dimensional arrays that the loop never reads and whose only
        store is `name[i] = ...` with the parallel index, unconditionally, in the loop's top-level body.
        When the loop runs over the whole array, every element is written, so the host copy need not be
        uploaded first (_skip_uploads)."""
        loop = self.ir.loop
        var = loop.target.id if isinstance(loop.target, ast.Name) else None
        it = loop.iter
        if var is None or not (isinstance(it, ast.Call) and 1 <= len(it.args) <= 3):
            return frozenset(), None
        if len(it.args) == 3 and not (isinstance(it.args[2], ast.Constant) and it.args[2].value == 1):
            return frozenset(), None
        import re
        hoist = lambda node: re.sub(r"\b(\w+)\.shape\[(\d+)\]", r"\1_shape_\2", ast.unparse(node))
        lo_src = "0" if len(it.args) == 1 else hoist(it.args[0])
        hi_src = hoist(it.args[0] if len(it.args) == 1 else it.args[1])
        try:
            codes = (compile(lo_src, "<lo>", "eval"), compile(hi_src, "<hi>", "eval"))
        except SyntaxError:
            return frozenset(), None
        if any(isinstance(x, (ast.Continue, ast.Break, ast.Return)) for x in ast.walk(loop)):
            return frozenset(), None            # a top-level store may be jumped over
        stores = {}
        for st in loop.body:
            if isinstance(st, ast.Assign) and len(st.targets) == 1 and isinstance(st.targets[0], ast.Subscript):
                t = st.targets[0]
                if isinstance(t.value, ast.Name) and isinstance(t.slice, ast.Name) and t.slice.id == var:
                    stores.setdefault(t.value.id, []).append(t)
        names = set()
        for name, tgts in stores.items():
            if name not in self.stored or name in self.cell_names:
                continue
            mentions = [x for x in ast.walk(loop) if isinstance(x, ast.Name) and x.id == name]
            if len(mentions) == len(tgts):          # mentioned nowhere but as those targets
                names.add(name)
        return frozenset(names), codes

    def _skip_uploads(self, args, arrays) -> tuple:
        """Names of this call's host arrays that are written in full before anything could read them."""
        if not self.overwritten or self.options.get("distribute") or not self.options.get("_skip_uploads", True):
            return ()
        try:
            scope = self._scope(args, arrays)
            lo, hi = int(eval(self._range_codes[0], {}, scope)), int(eval(self._range_codes[1], {}, scope))
        except Exception:
            return ()
        return tuple(a.name for a in arrays if a.host and a.name in self.overwritten and a.tmp is None
                     and len(a.shape) == 1 and lo == 0 and hi == a.shape[0])

    def _host_cells(self, arrays) -> tuple:
        """Names of the host arrays of this call that become cells in mapped host memory: reduction-only
        targets (cell_names) of at most 64 bytes, at most eight per call; never in a distributed or
        cross-GPU combining loop (their cells are exchanged through device memory)."""
        if not self.cell_names or not self.options.get("_host_cells", True) or self.options.get("distribute") \
                or self.options.get("combine"):
            return ()
        picked = [a for a in arrays if a.host and a.name in self.cell_names and 0 < a.nbytes <= 64
                  and a.tmp is None]
        spans = sorted((a.hptr, a.hptr + a.nbytes) for a in arrays if a.host and a.nbytes)
        if any(spans[i][1] > spans[i + 1][0] for i in range(len(spans) - 1)):
            return ()           # two names for one host array accumulate into one mirror; two cells would not
        return tuple(a.name for a in picked[:8])

    # ------------------------------------------------------------------ specialisation
    def _resolve_arrays(self, args):
        arrays = []
        torch = sys.modules.get("torch")
        for name, sig, v in zip(self.arg_names, self.arg_sigs, args):
            if sig[0] != "A":
                continue
            a = _Array()
            a.name, a.obj, a.tmp, a.hptr, a.cell = name, v, None, 0, 0
            a.pinnable = sig[1] == "np"      # NumPy owners can be tracked by a finaliser; tensor views cannot
            if sig[1] == "cuda":
                a.host = False
                a.dptr = v.data_ptr()
                a.shape, a.itemsize = tuple(v.shape), v.element_size()
                a.strides = tuple(v.stride())
                a.nbytes = 0
            else:
                h = v if sig[1] == "np" else v.numpy()
                if not h.flags.c_contiguous:
                    a.tmp = np.ascontiguousarray(h)
                    h2 = a.tmp
                else:
                    h2 = h
                a.host = True
                a.obj = h
                a.hptr = h2.ctypes.data
                a.nbytes = h2.nbytes
                a.shape, a.itemsize = tuple(h2.shape), h2.itemsize
                a.strides = tuple(s // h2.itemsize for s in h2.strides)
                a.dptr = 0
            arrays.append(a)
        return arrays

    def _acquire_device(self, arrays, stream, slices=None, hostcells=(), skip=()):
        """Device mirrors of the host arrays, filled from the host.  `slices` (distributed loops):
        {array name: (first byte, one past last byte)} for arrays of which this rank touches only a part.
        `hostcells`: names of arrays that get a cell in the device's page of mapped host memory instead
        (the value is copied in by the CPU; the kernel reads and writes it over PCIe)."""
        window = None
        for a in arrays:
            a.cell = 0
            if not a.host:
                continue
            if a.nbytes == 0:
                a.dptr = 0
                continue
            if a.name in hostcells:
                if window is None:      # this call's 512 bytes of the page: eight calls may be in flight
                    page = _cell_pages.get(self.device)
                    if page is None:
                        page = _cell_pages[self.device] = rt.host_cells()
                    base_h, base_d = page[0], page[1]
                    _cell_turn[0] = turn = (_cell_turn[0] + 1) % 8
                    window = [base_h + 512 * turn, base_d + 512 * turn]
                C.memmove(window[0], a.hptr, a.nbytes)
                a.cell, a.dptr = window[0], window[1]
                window[0] += 64
                window[1] += 64
                transfer_stats["h2d"] += a.nbytes
                continue
            a.dptr, created = rt.mirror(a.hptr, a.nbytes)
            if a.name in skip:          # every element is written by the loop before anything reads it
                _maybe_pin(a.hptr, a.nbytes, a.obj, a.pinnable and self.options.get("pin_host", True))
                continue
            state = _resident.get(a.hptr) if (_resident and not slices and a.tmp is None) else None
            if state is not None and state[0] == a.nbytes:
                if state[1] and not created:
                    if state[2] != stream:           # the upload was queued on another stream: let it finish
                        rt.sync(state[2])
                        state[2] = stream
                    continue                         # the mirror holds what the host holds: nothing to move
                state[1], state[2] = True, stream
            b0, b1 = slices.get(a.name, (0, a.nbytes)) if slices else (0, a.nbytes)
            transfer_stats["h2d"] += max(0, b1 - b0)
            _upload(a.dptr + b0, a.hptr + b0, b1 - b0, a.hptr, a.nbytes, a.obj,
                    a.tmp is None and a.pinnable and self.options.get("pin_host", True), stream)

    def _spec_key(self, arrays, hostcells=()):
        key = []
        for a in arrays:
            nd = len(a.shape)
            unit_last = nd == 0 or a.strides[-1] == 1 or a.shape[-1] <= 1
            lead = a.strides[:-1] if nd > 1 else ()
            vec = tuple(all(s % V == 0 for s in lead) for V in (2, 4, 8, 16))
            ext = sum((n - 1) * abs(s) for n, s in zip(a.shape, a.strides)) + 1 if all(a.shape) else 0
            key.append((a.dptr % 16 == 0 if a.dptr else True, unit_last, vec, ext < 2 ** 31))
        # overlap of a stored array with any other array disables the read-only path
        noalias = True
        spans = []
        for a in arrays:
            ext = sum((n - 1) * abs(s) for n, s in zip(a.shape, a.strides)) + 1 if all(a.shape) else 0
            base = a.hptr if a.host else a.dptr
            spans.append((base, base + ext * a.itemsize, a.name))
        for (lo1, hi1, n1) in spans:
            if n1 not in self.stored:
                continue
            for (lo2, hi2, n2) in spans:
                if n2 != n1 and lo1 < hi2 and lo2 < hi1:
                    noalias = False
        shape_spec = ()
        if self.options.get("_shape_spec", True):
            shape_spec = tuple((a.name, a.shape[1]) for a in arrays if len(a.shape) == 2 and a.name in self.stored)
        return (tuple(key), noalias, shape_spec, tuple(hostcells))

    def _variant(self, arrays, key) -> Variant:
        v = self.variants.get(key)
        if v is not None:
            return v
        infos = []
        by_name = {a.name: a for a in arrays}
        flags = dict(zip([a.name for a in arrays], key[0]))
        for name, sig in zip(self.names, self.signature):
            if sig[0] == "M":
                infos.append(ArgInfo(name, "module"))
            elif sig[0] == "S":
                sty = _scalar_type(sig[1])
                if sig[1] == "pyfloat" and self.options.get("fp_contract") == "triton":
                    sty = T.F32          # a Python float reaches the reference's Triton kernel as fp32
                infos.append(ArgInfo(name, "scalar", sty))
            else:
                a = by_name[name]
                aligned, unit_last, vec, small = flags[name]
                infos.append(ArgInfo(name, "array", _elem_type(sig[2]), len(a.shape), unit_last, aligned,
                                     dict(zip((2, 4, 8, 16), vec)), a.itemsize, small))
        opts = dict(self.options)
        opts["_noalias"] = key[1]
        opts["_shape"] = {(n, 1): s for n, s in key[2]}
        if len(key) > 3 and key[3]:
            # cells in mapped host memory: one read and one write per cell at the very end of the kernel
            # (atomics on host memory would cross PCIe one by one)
            opts["ordered_reduction"] = True
        import copy as _copy
        ir = _copy.deepcopy(self.ir)
        plan = Lowering(ir, self.kernel_name, infos, opts).lower()
        if self.options.get("fp_contract", "numpy") == "numpy":
            plan.info["nvrtc"] = ["--fmad=false", "--prec-div=true", "--prec-sqrt=true", "--ftz=false"]
        else:
            # the reference backend's numerics: FMA contraction, float32 `/` as div.full.f32 (emitted
            # explicitly), float literals float64, Python floats float32 (emit.py, Env.numerics)
            plan.info["nvrtc"] = ["--fmad=true", "--prec-div=true", "--prec-sqrt=true", "--ftz=false"]
        v = Variant(plan)
        self.variants[key] = v
        self.last_source = plan.source
        return v

    # ------------------------------------------------------------------ launch
    def _scope(self, args, arrays):
        scope = {}
        for name, sig, val in zip(self.arg_names, self.arg_sigs, args):
            if sig[0] == "S":
                scope[name] = val
        for a in arrays:
            for d, n in enumerate(a.shape):
                scope.setdefault(f"{a.name}_shape_{d}", n)
        return scope

    def _pack(self, variant: Variant, args, arrays, lo, hi, stream, scratch_bytes: int = 0):
        by_name = {a.name: a for a in arrays}
        scal = dict(zip(self.arg_names, args))
        vals = []
        for p in variant.plan.params:
            if p.kind == "array":
                vals.append(C.c_void_p(by_name[p.name].dptr))
            elif p.kind == "scalar":
                ty = p.ty.strong()
                v = scal[p.name]
                vals.append(_CT[(ty.kind, ty.bits)](v.item() if isinstance(v, np.generic) else v))
            elif p.kind == "shape":
                vals.append(C.c_int64(by_name[p.array].shape[p.dim]))
            elif p.kind == "stride":
                vals.append(C.c_int64(by_name[p.array].strides[p.dim]))
            elif p.kind == "lo":
                vals.append(C.c_int64(lo))
            elif p.kind == "hi":
                vals.append(C.c_int64(hi))
            elif p.kind == "ws":
                vals.append(C.c_void_p(rt.workspace(stream)))
            elif p.kind == "scratch":
                vals.append(C.c_void_p(rt.scratch(stream, max(scratch_bytes, 1 << 20))))
            elif p.kind == "mb":
                from . import multi_gpu
                vals.append(C.c_void_p(multi_gpu.combiner().descriptor))
            elif p.kind == "seq":
                from . import multi_gpu
                vals.append(C.c_uint64(multi_gpu.combiner().next_seq()))
            elif p.kind == "pend":
                from . import multi_gpu
                vals.append(multi_gpu.Pending2())      # filled at launch time, when the grid is known
        return rt.ArgPack(vals)

    _P2P_OPS = {"+": 0, "*": 1, "max": 2, "min": 3}

    def _deferred_cells(self, args, arrays):
        """(address, operator code, type code) of every reduction cell of this loop, for the launch that will
        collect this one.  The cells must live in device memory: a host cell is read back right after the
        launch, before anyone has collected it."""
        out = []
        for view, op in self._reduction_cells(args, arrays):
            name = str(view.dtype).replace("torch.", "")
            ty = {"float32": 0, "float64": 1, "int32": 2, "int64": 3}.get(name)
            if ty is None or op not in self._P2P_OPS:
                raise NotImplementedError(f"defer=True: unsupported reduction type {view.dtype} or operator {op!r}")
            out.append((view.data_ptr(), self._P2P_OPS[op], ty))
        return out

    def _inner_trip(self, plan, scope, lo=0, hi=0):
        """Trip count of the (first) inner simd loop for this call, or None when it is not known on the
        host.  Bounds that depend on the outer index (triangular loops) are taken at the middle of the
        outer range, which is the mean row length for a linear dependence."""
        hi_n, lo_n = plan.info.get("inner_hi"), plan.info.get("inner_lo")
        if hi_n is None:
            return None
        for extra in ({}, {plan.info.get("outer_var", "_"): (lo + hi) // 2}):
            try:
                sc = dict(scope, **extra) if extra else scope
                return max(0, int(eval(compile(ast.Expression(body=hi_n), "<t>", "eval"), {}, sc)) -
                           int(eval(compile(ast.Expression(body=lo_n), "<t>", "eval"), {}, sc)))
            except Exception:
                continue
        return None

    def _shape_class(self, variant: Variant, scope, arrays, n_iter: int, stream, lo: int = 0):
        """(class, overrides): launches of one class share their tunables; the overrides are the
        defaults this class starts from.  The class is what the choice depends on beyond the code
        itself: the inner trip count for row loops, the row-length profile of the matrix for CSR
        loops, the size bucket of the outer range."""
        plan = variant.plan
        bucket = max(n_iter, 1).bit_length()
        if plan.kind in ("group", "rowdot"):
            trip = self._inner_trip(plan, scope, lo, lo + n_iter)
            if trip is None:
                return ("rows", bucket, None), {}
            ov = {}
            if plan.kind == "group":
                # a lane takes about four packs (or four elements) of the row; at least two lanes, so
                # that neighbouring rows still coalesce; from 2048 iterations on, a CTA per row
                # (512 threads once a thread would otherwise walk more than 16 packs)
                per = 4 * max(1, plan.info.get("inner_vec", 1))
                g = 2
                while g < 32 and g * per < trip:
                    g *= 2
                if trip >= 2048:
                    g = 0
                    ov["P_BLOCK"] = 512 if trip >= 16384 else 256
            else:
                per = 4 * max(1, plan.vec)
                g = 1
                while g < 32 and g * per < trip:
                    g *= 2
            ov["P_G"] = g
            if g == 0 and plan.info.get("splittable") and n_iter < 4 * self.sm_count:
                # few long rows of a perfect nest: cut every row into segments until about eight CTAs
                # per SM have work, keeping at least 2048 iterations per segment
                seg = 1
                while seg < 64 and n_iter * seg < 8 * self.sm_count and trip // (seg * 4) >= 2048:
                    seg *= 4
                ov["P_SEG"] = seg
            if plan.kind == "rowdot" and plan.vec > 1 and trip >= 256 * plan.vec:
                # Long dense rows: few, deep, contiguous streams keep DRAM pages open (thousands of
                # concurrent warp-per-row streams of two chunks each were measured 20 % slower on
                # 16384 x 16384 and 262144 x 1024 matrices).  Eight 16-byte chunks per lane and row in
                # flight, two rows at once when the body streams at most two arrays, register budget
                # open.  Rows of at least 256 x 8 chunks get a 256-thread CTA per row pair (two CTAs per
                # SM); shorter ones a warp per row pair, so that the unrolled loop still runs.
                light = plan.info.get("streams", 9) <= 2
                u = 8 if light else 4
                if trip >= 256 * u * plan.vec:
                    pair = light and n_iter >= 4 * self.sm_count        # with few rows every row gets its own CTA
                    ov.update({"P_G": 0, "P_BLOCK": 256, "P_U": u, "P_R": 2 if pair else 1, "P_MINB": 2})
                else:
                    ov.update({"P_G": 32, "P_BLOCK": 128, "P_U": u, "P_R": 2 if light else 1, "P_MINB": 1})
            return ("rows", bucket, max(trip, 1).bit_length()), ov
        if plan.kind == "csrdense" and "P_STREAM" in plan.tunables:
            # The streaming form starts one wave of CTAs and a second kernel whatever the size; below a few
            # thousand rows the row-tiled form (one CTA per 32 rows) is over before that pays.
            if n_iter < self.options.get("_stream_rows", 4096) or n_iter >= 2 ** 31:
                return ("n", bucket, "tiled"), dict(plan.info["row_tiled"], P_STREAM=0)
            return ("n", bucket, "stream"), {}
        if plan.kind == "csr" and plan.info.get("indptr"):
            row_class, ov = self._csr_profile(variant, arrays, stream)
            return ("csr", bucket, row_class), ov
        return ("n", bucket), {}

    def _csr_profile(self, variant: Variant, arrays, stream):
        """(row-length class, lanes per row) from the row-length histogram of this matrix (cached per
        indptr buffer; runs on the stream the uploads were queued on)."""
        plan = variant.plan
        ip = next((a for a in arrays if a.name == plan.info["indptr"]), None)
        if ip is None or ip.shape[0] <= 1:
            return "", {}
        ckey = (ip.dptr, ip.shape[0])
        cache = variant.__dict__.setdefault("csr_choice", {})
        if ckey not in cache:
            if len(cache) > 64:
                cache.clear()
            counts, _mx = rt.row_histogram(ip.dptr, ip.itemsize, ip.shape[0] - 1, stream)
            total = sum(counts)
            acc, med = 0, 0
            for b, c in enumerate(counts):      # median row-length bin decides the lanes per row
                acc += c
                if acc * 2 >= total:
                    med = b
                    break
            length = 1 << max(med - 1, 0)
            g = 1 if length <= 1 else 2 if length <= 4 else 4 if length <= 16 else \
                8 if length <= 64 else 16 if length <= 256 else 32
            row_class = f"med{med}max{max((b for b, c in enumerate(counts) if c), default=0)}"
            cache[ckey] = (row_class, {"P_G": g})
        return cache[ckey]

    def _want_autotune(self) -> bool:
        return bool(self.options.get("autotune", os.environ.get("APPY_AUTOTUNE", "0") == "1"))

    def _choose_tunables(self, variant: Variant, args, arrays, scope, lo, hi, stream) -> dict:
        forced = getattr(variant, "forced_tun", None)        # experiments and sweeps
        if forced is not None:
            return forced
        cls, ov = self._shape_class(variant, scope, arrays, hi - lo, stream, lo)
        tun = variant.choice.get(cls)
        if tun is None:
            tun = dict(variant.tun, **{k: v for k, v in ov.items() if k in variant.tun})
            # A kernel that exchanges its totals with other ranks in its tail is not timed: every trial
            # launch would need its own sequence number on every rank at once.  It keeps the defaults.
            fused_exchange = any(p.kind == "seq" for p in variant.plan.params)
            if self._want_autotune() and not fused_exchange and hi > lo:
                tun = self._autotune(variant, args, arrays, lo, hi, stream, tun, cls)
            if len(variant.choice) > 64:
                variant.choice.clear()
            variant.choice[cls] = tun
        variant.last_tun = tun
        return tun

    def _autotune(self, variant: Variant, args, arrays, lo, hi, stream, start: dict, cls) -> dict:
        plan = variant.plan
        n_iter = hi - lo
        store = _tune_store()
        tkey = hashlib.sha1((plan.source + "|".join(map(str, plan.info.get("nvrtc", [])))).encode()).hexdigest() \
            + ":" + ":".join(str(c) for c in cls)
        if tkey in store:
            return dict(start, **store[tkey])
        # keep the stored arrays intact: run candidates, then restore
        saved = []
        saved_cells = []        # cells in mapped host memory are saved and restored by the CPU
        for a in arrays:
            if a.host and getattr(a, "cell", 0):
                saved_cells.append((a, C.string_at(a.cell, a.nbytes)))
                continue
            if a.name in self.stored:
                ext = (sum((n - 1) * abs(s) for n, s in zip(a.shape, a.strides)) + 1) * a.itemsize if all(a.shape) else 0
                if ext:
                    tmp = rt.malloc(ext)
                    rt.check(rt.lib().appy_d2d_async(C.c_void_p(tmp), C.c_void_p(a.dptr), ext, C.c_void_p(stream)))
                    saved.append((a, tmp, ext))
        best, best_t = dict(start), float("inf")
        # coordinate descent over the tunables, starting from this class's defaults
        cur = dict(start)
        widest = {k: max(v) for k, v in plan.tunables.items()}     # the largest scratch any candidate needs
        pack = self._pack(variant, args, arrays, lo, hi, stream, plan.scratch_bytes(widest, n_iter, self.sm_count))
        for name in list(plan.tunables):
            for cand in plan.tunables[name]:
                trial = dict(cur)
                trial[name] = cand
                try:
                    h = variant.handle(trial)
                    grid, block, smem = plan.launch_config(trial, n_iter, self.sm_count)
                    t = rt.time_launches(h, grid, block, pack, smem, stream, warmup=1, iters=5)
                    post = plan.post_config(trial, n_iter, self.sm_count)
                    if post is not None:       # the second kernel of a two-kernel plan is part of the cost
                        t += rt.time_launches(variant.post_handle(trial), post[0], post[1], pack, 0, stream,
                                              warmup=1, iters=5)
                except rt.AppyRuntimeError:
                    continue
                if t < best_t:
                    best_t, best = t, dict(trial)
            cur = dict(best)
        for a, tmp, ext in saved:
            rt.check(rt.lib().appy_d2d_async(C.c_void_p(a.dptr), C.c_void_p(tmp), ext, C.c_void_p(stream)))
        rt.sync(stream)
        for _a, tmp, _e in saved:
            rt.free(tmp)
        for a, raw in saved_cells:
            C.memmove(a.cell, raw, a.nbytes)
        store[tkey] = best
        _tune_save()
        if os.environ.get("APPY_TUNE_LOG") == "1":
            sys.stderr.write(f"[appy autotune] {plan.name} ({plan.info.get('template')}) n={n_iter} {cls}: {best} "
                             f"{best_t * 1e3:.1f} us\n")
        return best

    # ------------------------------------------------------------------ distribution over ranks
    def _check_distributable(self):
        """Generic rule: arrays written by the loop must be indexed by the parallel index in their
        leading dimension (then every rank writes a disjoint slice); reduction targets are combined;
        anything else cannot be split across GPUs."""
        if getattr(self, "_dist_checked", False):
            return
        from ...frontend.loop_normalize import reductions_of
        loop = self.ir.loop
        var = loop.target.id
        red = set(reductions_of(loop))
        for n in ast.walk(loop):
            if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Store) and isinstance(n.value, ast.Name):
                if ast.unparse(n) in red:
                    continue
                first = n.slice.elts[0] if isinstance(n.slice, ast.Tuple) else n.slice
                if not (isinstance(first, ast.Name) and first.id == var):
                    raise NotImplementedError(
                        f"cannot distribute this loop over GPUs: `{ast.unparse(n)}` is not written at the "
                        f"parallel index `{var}` in its leading dimension")
        self._dist_checked = True

    def _shard_classes(self, variant) -> dict:
        """Which arrays a rank touches only in part when the outer range is split:
        "rows"  every subscript has the parallel index itself as its leading index;
        "nnz"   (CSR loops) every subscript is the index of an inner loop that runs from
                indptr[i] to indptr[i+1].  Everything else (gathered or shifted operands) is whole."""
        cached = getattr(variant, "shard_classes", None)
        if cached is not None:
            return cached
        loop = self.ir.loop
        var = loop.target.id
        indptr = variant.plan.info.get("indptr")
        nnz_vars = set()
        if indptr:
            bound = {}      # local name -> "lo" / "hi" when assigned from indptr[i] / indptr[i + 1]
            for n in ast.walk(loop):
                if isinstance(n, ast.Assign) and isinstance(n.targets[0], ast.Name) and isinstance(n.value, ast.Subscript) \
                        and isinstance(n.value.value, ast.Name) and n.value.value.id == indptr:
                    txt = ast.unparse(n.value.slice).replace(" ", "")
                    if txt == var:
                        bound[n.targets[0].id] = "lo"
                    elif txt in (f"{var}+1", f"1+{var}"):
                        bound[n.targets[0].id] = "hi"
            for n in ast.walk(loop):
                if isinstance(n, ast.For) and n is not loop and isinstance(n.iter, ast.Call) and len(n.iter.args) >= 2:
                    a0, a1 = n.iter.args[0], n.iter.args[1]
                    if isinstance(a0, ast.Name) and isinstance(a1, ast.Name) and bound.get(a0.id) == "lo" \
                            and bound.get(a1.id) == "hi":
                        nnz_vars.add(n.target.id)
        seen = {}
        for n in ast.walk(loop):
            if not (isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name)):
                continue
            name = n.value.id
            elts = n.slice.elts if isinstance(n.slice, ast.Tuple) else [n.slice]
            first = elts[0]
            if isinstance(first, ast.Name) and first.id == var:
                kind = "rows"
            elif len(elts) == 1 and isinstance(first, ast.Name) and first.id in nnz_vars:
                kind = "nnz"
            else:
                kind = None
            seen[name] = kind if seen.get(name, kind) == kind else None
        variant.shard_classes = {k: v for k, v in seen.items() if v and k != indptr}
        return variant.shard_classes

    def _rank_slices(self, variant, arrays, lo, hi) -> dict:
        """Byte ranges of the host arrays this rank needs for its sub-range [lo, hi) (see _shard_classes)."""
        out = {}
        classes = self._shard_classes(variant)
        by_name = {a.name: a for a in arrays}
        ip = by_name.get(variant.plan.info.get("indptr")) if variant.plan.info.get("indptr") else None
        for a in arrays:
            kind = classes.get(a.name)
            if not a.host or kind is None or not a.shape:
                continue
            if hi <= lo:
                out[a.name] = (0, 0)
            elif kind == "rows":
                row = (a.nbytes // a.shape[0]) if a.shape[0] else 0
                out[a.name] = (max(0, lo) * row, min(hi, a.shape[0]) * row)
            elif ip is not None:
                host = ip.obj if ip.host else None
                if host is None:
                    continue
                k0, k1 = int(host[lo]), int(host[hi])
                out[a.name] = (k0 * a.itemsize, min(k1 * a.itemsize, a.nbytes))
        return out

    def _rank_range(self, variant, arrays, lo, hi):
        from . import multi_gpu
        rank, world_size = multi_gpu.world()
        if world_size == 1 or hi <= lo:
            return lo, hi
        self._check_distributable()
        plan = variant.plan
        if plan.kind in ("csr", "csrdense") and plan.info.get("indptr"):
            ip = next(a for a in arrays if a.name == plan.info["indptr"])
            key = (ip.dptr if not ip.host else ip.hptr, ip.shape[0], lo, hi, world_size)
            cache = self.__dict__.setdefault("_row_split", {})
            if key not in cache:
                host = ip.obj if ip.host else ip.obj.detach().cpu().numpy()
                # a row costs the row-reduction kernel about as much as eight of its non-zeros (pointer loads,
                # the group's reduction, the store) and the row-times-dense kernel about one (the C row's store)
                row_cost = int(self.options.get("_row_cost", 8 if plan.kind == "csr" else 1))
                b = rt.partition_rows(np.ascontiguousarray(host[lo:hi + 1]), world_size, row_cost)
                if len(cache) > 64:
                    cache.clear()
                cache[key] = [lo + x for x in b]
            b = cache[key]
            return b[rank], b[rank + 1]
        return multi_gpu.split_range(lo, hi, world_size, rank, 32)

    def _reduction_cells(self, args, arrays):
        """(torch view of the 1-element target cell, operator) for every reduction of the loop."""
        import torch
        from ...frontend.loop_normalize import reductions_of
        cells = []
        by_name = {a.name: a for a in arrays}
        tens = dict(zip(self.arg_names, args))
        for text, op in reductions_of(self.ir.loop).items():
            node = ast.parse(text, mode="eval").body
            if not (isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name)
                    and isinstance(node.slice, ast.Constant) and node.value.id in by_name):
                raise NotImplementedError(f"distributed reduction target must be `name[<constant>]`: {text}")
            a = by_name[node.value.id]
            idx = int(node.slice.value)
            if a.host:
                dt = np.dtype(a.obj.dtype)
                view = torch.as_tensor(_DevView(a.dptr + idx * a.itemsize, 1, dt.str), device="cuda")
            else:
                view = tens[a.name].view(-1)[idx:idx + 1]
            cells.append((view, op))
        return cells

    def _memo_key(self, args):
        """Key of the launch record, computed from the values alone.  Device tensors enter with their
        address, layout and dtype, host arrays with their layout and dtype only (their device mirror is
        looked up on every call), scalars with their type and value.  None: this call cannot use a
        record (a host array that is not C-contiguous, or an argument of an unexpected kind)."""
        key = []
        tt = _TORCH_TENSOR
        data = self.data_scalars
        for i, v in enumerate(args):
            t = type(v)
            if i in data:
                if t in _SIMPLE_KINDS or isinstance(v, np.generic):
                    key.append(t)             # value patched into the record's arguments at launch
                    continue
                return None
            if t is tt or (tt is not None and isinstance(v, tt)):
                if v.is_cuda:
                    key.append((v.data_ptr(), v.shape, v.stride(), v.dtype))
                elif v.is_contiguous():
                    key.append((v.shape, v.dtype))
                else:
                    return None
            elif t is np.ndarray or isinstance(v, np.ndarray):
                if not v.flags.c_contiguous:
                    return None
                key.append((v.shape, v.dtype))
            elif tt is None and _is_torch(v):
                return None                       # first sight of a tensor: the slow path registers the class
            else:
                key.append((t, v))
        return tuple(key)

    def _host_args(self, args, slots):
        """(arrays, disjoint): the host arrays of a memoised call resolved again, and whether the
        stored ones still overlap no other host array (the record was made under that assumption)."""
        arrays = []
        for argi, name, _slot in slots:
            v = args[argi]
            a = _Array()
            a.name, a.tmp, a.cell = name, None, 0
            a.pinnable = type(v) is np.ndarray or isinstance(v, np.ndarray)
            h = v if a.pinnable else v.numpy()
            a.obj, a.host, a.hptr, a.nbytes, a.dptr = h, True, h.ctypes.data, h.nbytes, 0
            arrays.append(a)
        spans = sorted((a.hptr, a.hptr + a.nbytes) for a in arrays if a.nbytes)
        disjoint = all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1))
        return arrays, disjoint

    def fast_call(self, args) -> bool:
        """Launch from a record if this exact call (addresses, layouts, dtypes, scalar values) was seen
        before; False sends the caller down the full path."""
        if self.device is None or len(args) != len(self.arg_names):
            return False
        try:
            mkey = self._memo_key(args)
            memo = self.memo.get(mkey) if mkey is not None else None
        except TypeError:                 # an unhashable argument
            return False
        return memo is not None and self._replay(memo, args)

    def _replay(self, memo, args) -> bool:
        (handle, grid, block, smem, pack, seq_slot, memo_stream, cells, host_slots, scalar_slots, post, scratch,
         deferred, hostcells, skip) = memo
        torch = sys.modules.get("torch")
        if torch is not None and (self.has_device_args or not host_slots):
            stream = _torch_stream(torch, self.device)      # orders with the producers of the device tensors
        else:
            stream = rt.stream(0)
        harr, disjoint = self._host_args(args, host_slots) if host_slots else ((), True)
        if not disjoint or not (memo_stream is None or memo_stream == stream):     # a workspace belongs to one stream
            return False
        if host_slots:        # mirrors of the host arrays: look up, upload, patch into the arguments
            self._acquire_device(harr, stream, None, hostcells, skip)
            for a, (_argi, _name, slot) in zip(harr, host_slots):
                pack.values[slot].value = a.dptr
        for argi, slot in scalar_slots:
            v = args[argi]
            pack.values[slot].value = v.item() if isinstance(v, np.generic) else v
        if cells:
            self._pre_combine(cells)
        if grid:
            mine = None
            if seq_slot is not None:
                from . import multi_gpu
                comb = multi_gpu.combiner()
                pack.values[seq_slot].value = comb.next_seq()
                if deferred is not None:      # which launches this one serves, and where its own partials go
                    mine = comb.begin_split(pack.values[deferred[0]], deferred[2], grid)
            if scratch is not None:     # the stream's scratch buffer may have been replaced by a larger one
                pack.values[scratch[0]].value = rt.scratch(stream, scratch[1])
            rt.launch(handle, grid, block, pack, smem, stream)
            if mine is not None:
                comb.end_split(pack.values[seq_slot].value, grid, mine, deferred[1])
            if post is not None:
                rt.launch(post[0], post[1], post[2], pack, 0, stream)
        if cells:
            self._post_combine(cells)
        if host_slots:
            for a in harr:
                if a.name in self.stored and a.nbytes and not a.cell:
                    rt.d2h(a.hptr, a.dptr, a.nbytes, stream)
                    transfer_stats["d2h"] += a.nbytes
            rt.sync(stream)
            for a in harr:
                if a.cell:
                    C.memmove(a.hptr, a.cell, a.nbytes)
                    transfer_stats["d2h"] += a.nbytes
        return True

    def __call__(self, *args):
        if len(args) != len(self.arg_names):
            raise TypeError(f"{self.loop_name} expects {len(self.arg_names)} arguments, got {len(args)}")
        if self.device is None:
            if rt.device_count() < 1:
                raise RuntimeError("NVIDIA GPU not found")
            torch = sys.modules.get("torch")
            self.device = torch.cuda.current_device() if (torch is not None and torch.cuda.is_initialized()) else 0
            rt.init(self.device)
            self.sm_count = rt.device_info(self.device)["sm_count"]
        mkey = self._memo_key(args)
        memo = self.memo.get(mkey) if mkey is not None else None
        if memo is not None and self._replay(memo, args):
            return
        arrays = self._resolve_arrays(args)
        any_host = any(a.host for a in arrays)
        torch = sys.modules.get("torch")
        if torch is not None and (any(not a.host for a in arrays) or self.options.get("distribute")):
            stream = _torch_stream(torch, self.device)     # orders with torch ops and with collectives
        else:
            stream = rt.stream(0)
        from . import multi_gpu
        sharded = bool(self.options.get("distribute")) and any_host and multi_gpu.world()[1] > 1
        hostcells = self._host_cells(arrays) if any_host else ()
        skip = self._skip_uploads(args, arrays) if any_host else ()
        if not sharded:
            self._acquire_device(arrays, stream, None, hostcells, skip)
        key = self._spec_key(arrays, hostcells)     # mirrors are 16-byte aligned whether or not they exist yet
        variant = self._variant(arrays, key)
        self.last_variant = variant
        scope = self._scope(args, arrays)
        lo = int(eval(variant.lo_code, {}, scope))
        hi = int(eval(variant.hi_code, {}, scope))
        cells = []
        slices = None
        exchange_only = False
        if self.options.get("distribute"):
            full_lo, full_hi = lo, hi
            lo, hi = self._rank_range(variant, arrays, lo, hi)
            # A rank whose share of the range is empty still has to take part in an exchange fused into
            # the kernel's tail: it launches one CTA on the empty range [hi, hi), whose accumulators are
            # the identities, so that it posts its words, draws its sequence number and leaves with
            # the world's totals like every other rank.
            exchange_only = (hi <= lo and full_hi > full_lo and multi_gpu.world()[1] > 1
                             and any(p.kind == "seq" for p in variant.plan.params))
            if exchange_only:
                lo = hi = max(lo, hi)
            if sharded:      # every rank uploads only the part of the row- and nnz-indexed arrays it works on
                slices = self._rank_slices(variant, arrays, lo, hi)
                self._acquire_device(arrays, stream, slices)
            if multi_gpu.world()[1] > 1 and self.options.get("combine") != "p2p":
                cells = self._reduction_cells(args, arrays)
                self._pre_combine(cells)
        if hi > lo or exchange_only:
            tun = self._choose_tunables(variant, args, arrays, scope, lo, hi, stream)
            need = variant.plan.scratch_bytes(tun, hi - lo, self.sm_count)
            pack = self._pack(variant, args, arrays, lo, hi, stream, need)
            h = variant.handle(tun)
            grid, block, smem = variant.plan.launch_config(tun, hi - lo, self.sm_count)
            kinds_ = [p.kind for p in variant.plan.params]
            deferred = None
            if "pend" in kinds_:            # split-phase exchange: the next two launches fold, post and collect this one
                if any_host and any(a.host and a.name in self.stored for a in arrays):
                    raise NotImplementedError("defer=True needs the shared(...) cells in device memory "
                                              "(a host cell is read back before the exchange has completed)")
                deferred = (kinds_.index("pend"), tuple(self._deferred_cells(args, arrays)), rt.workspace(stream))
                comb = multi_gpu.combiner()
                mine = comb.begin_split(pack.values[deferred[0]], deferred[2], grid)
            rt.launch(h, grid, block, pack, smem, stream)
            if deferred is not None:
                comb.end_split(pack.values[kinds_.index("seq")].value, grid, mine, deferred[1])
            post = variant.plan.post_config(tun, hi - lo, self.sm_count)
            if post is not None:        # second kernel of a two-kernel plan: same arguments, same stream
                post = (variant.post_handle(tun), post[0], post[1])
                rt.launch(post[0], post[1], post[2], pack, 0, stream)
            scratch = (kinds_.index("scratch"), max(need, 1 << 20)) if "scratch" in kinds_ else None
            # Launch record.  With host arrays it is kept when they are contiguous, none of them had to
            # be copied to become so, the stored ones overlap nothing, and the loop does not distribute
            # or combine (those paths look at the arrays again).
            recordable = mkey is not None and (not any_host or (
                key[1] and not cells and not self.options.get("distribute")
                and variant.plan.kind != "csr"          # lanes per row follow the matrix, not only its shape
                and all(a.tmp is None for a in arrays)))
            if recordable:
                if len(self.memo) > 256:
                    self.memo.clear()
                kinds = [p.kind for p in variant.plan.params]
                seq_slot = kinds.index("seq") if "seq" in kinds else None
                host_slots = []
                if any_host:
                    pnames = [p.name if p.kind == "array" else None for p in variant.plan.params]
                    for argi, (name, sig) in enumerate(zip(self.arg_names, self.arg_sigs)):
                        if sig[0] == "A" and sig[1] != "cuda":
                            host_slots.append((argi, name, pnames.index(name)))
                pslot = {p.name: k for k, p in enumerate(variant.plan.params) if p.kind == "scalar"}
                scalar_slots = tuple((i, pslot[self.arg_names[i]]) for i in sorted(self.data_scalars)
                                     if self.arg_names[i] in pslot)
                self.memo[mkey] = (h, grid, block, smem, pack, seq_slot,
                                   stream if (variant.plan.uses_ws or any_host or scratch) else None, cells,
                                   tuple(host_slots), scalar_slots, post, scratch, deferred, hostcells, skip)
        elif not any_host and mkey is not None:
            self.memo[mkey] = (0, 0, 0, 0, None, None, None, cells, (), (), None, None, None, (), ())
        if cells:
            self._post_combine(cells)
        if any_host:
            for a in arrays:
                if a.host and a.name in self.stored and a.nbytes and not a.cell:
                    b0, b1 = slices.get(a.name, (0, a.nbytes)) if slices else (0, a.nbytes)
                    if b1 > b0:
                        rt.d2h(a.hptr + b0, a.dptr + b0, b1 - b0, stream)
                        transfer_stats["d2h"] += b1 - b0
            rt.sync(stream)
            for a in arrays:            # cells in mapped host memory: the kernel has written them
                if a.host and a.cell:
                    C.memmove(a.hptr, a.cell, a.nbytes)
                    transfer_stats["d2h"] += a.nbytes
            for a in arrays:
                if a.host and a.tmp is not None:
                    if a.name in self.stored:
                        a.obj[...] = a.tmp
                    rt.check(rt.lib().appy_evict(C.c_void_p(a.hptr)))    # the contiguous copy dies with this call

    def _pre_combine(self, cells):
        """Every rank starts from the same initial value b0; only rank 0 keeps it, so that the
        all-reduce after the kernel yields b0 (op) total and not world * b0 (op) total."""
        from . import multi_gpu
        if multi_gpu.world()[0] == 0:
            return
        for view, op in cells:
            if op in _IDENTITY:
                view.fill_(_IDENTITY[op])

    def _post_combine(self, cells):
        from . import multi_gpu
        for view, op in cells:
            multi_gpu.all_reduce(view, op)

    # convenience for tests and dumps
    def source_for(self, *args) -> str:
        arrays = self._resolve_arrays(args)    # host arrays: dptr 0, mirrors are always aligned
        return self._variant(arrays, self._spec_key(arrays, self._host_cells(arrays))).plan.source


def _maybe_pin(base: int, base_bytes: int, owner, may_pin: bool) -> bool:
    """Pin the host buffer [base, base + base_bytes) in place when it is at least 1 MiB and is seen for
    the second time; True if it is pinned.  Serves downloads as well as uploads: a copy into pageable
    memory is staged by the driver and blocks the caller."""
    pinned = base in _finalizers
    if base_bytes >= _PIN_MIN_BYTES and may_pin and not pinned:
        if len(_seen_host) > 4096:
            _seen_host.clear()
        seen = _seen_host.get(base, 0) + 1
        _seen_host[base] = seen
        if seen == 2:      # a buffer that comes back is worth pinning in place
            try:
                rt.check(rt.lib().appy_register_host(C.c_void_p(base), base_bytes))
                _register_finalizer(owner, base)
                pinned = base in _finalizers
            except rt.AppyRuntimeError:
                pass
    return pinned


def _upload(dst: int, src: int, nbytes: int, base: int, base_bytes: int, owner, may_pin: bool, stream: int) -> None:
    """Host-to-device copy of [src, src + nbytes), a part of the host buffer [base, base + base_bytes)
    owned by `owner`.  A buffer of at least 1 MiB that comes back a second time is pinned in place, after
    which its copies are true DMA; until then large pageable buffers go through the pinned staging
    buffers of the runtime."""
    if nbytes <= 0:
        return
    pinned = _maybe_pin(base, base_bytes, owner, may_pin)
    if pinned or base_bytes < _PIN_MIN_BYTES:
        rt.h2d(dst, src, nbytes, stream)          # true DMA, or too small to matter
    else:
        rt.h2d_staged(dst, src, nbytes, stream)   # pageable: pinned staging buffers


def to_device(array):
    """A NumPy array as a new torch CUDA tensor, uploaded with the copy path of the loops (pinned in
    place from the second time on).  Returns after the copy has completed, so the host array may be
    modified at once.  This is what `appy.to_gpu` uses for NumPy arguments."""
    import torch
    h = np.ascontiguousarray(array)
    t = torch.empty(h.shape, dtype=torch.from_numpy(h[:0] if h.ndim else h.reshape(1)[:0]).dtype, device="cuda")
    if h.nbytes:
        dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
        rt.init(dev)
        stream = _torch_stream(torch, dev)
        _upload(t.data_ptr(), h.ctypes.data, h.nbytes, h.ctypes.data, h.nbytes, h, h is array, stream)
        transfer_stats["h2d"] += h.nbytes
        rt.sync(stream)
    return t


# ---- host arrays declared resident: uploaded once, then again only after `touch`
#
# The reference's generated host code copies every NumPy argument to the device on every call
# (host_passes/gen_data_movement.py:14-96), and so does this backend by default: it cannot know whether
# the caller wrote to the array in between.  `resident(a)` is the caller's promise to say so: the
# array's device mirror is filled by the next loop that uses it and trusted from then on; `touch(a)`
# after a host-side write makes the next loop upload it again.  A loop that stores to the array copies
# it back as always, after which host and mirror agree again.
_resident: dict = {}        # host pointer -> [bytes, mirror is current, stream of the last upload]


def _host_base(a):
    if not (isinstance(a, np.ndarray) and a.flags.c_contiguous):
        raise TypeError("resident/touch/release take C-contiguous NumPy arrays")
    return a.ctypes.data


def resident(*arrays):
    import weakref
    for a in arrays:
        p = _host_base(a)
        if p not in _resident:
            _resident[p] = [a.nbytes, False, 0]
            base = a
            while getattr(base, "base", None) is not None and isinstance(base.base, np.ndarray):
                base = base.base
            try:
                weakref.finalize(base, _resident.pop, p, None)      # the address may be reused once the owner dies
            except TypeError:
                pass
        elif _resident[p][0] != a.nbytes:
            _resident[p] = [a.nbytes, False, 0]
    return arrays[0] if len(arrays) == 1 else arrays


def touch(*arrays):
    """The host copies of these arrays were written: the next loop that uses them uploads them again."""
    for a in arrays:
        st = _resident.get(_host_base(a))
        if st is not None:
            st[1] = False


def release(*arrays):
    for a in arrays:
        _resident.pop(_host_base(a), None)


_finalizers: dict = {}
transfer_stats = {"h2d": 0, "d2h": 0}      # bytes moved for host arrays (tests read this)


def _register_finalizer(obj, hptr: int) -> None:
    """Unpin and evict the device mirror when the owner of the host buffer goes away."""
    import weakref
    base = obj
    while getattr(base, "base", None) is not None and isinstance(base.base, np.ndarray):
        base = base.base
    if hptr in _finalizers:
        return

    def _drop(p=hptr):
        _finalizers.pop(p, None)
        _seen_host.pop(p, None)
        try:
            rt.lib().appy_unregister_host(C.c_void_p(p))
            rt.lib().appy_evict(C.c_void_p(p))
        except Exception:
            pass

    try:
        _finalizers[hptr] = weakref.finalize(base, _drop)
    except TypeError:
        pass


_OPTION_KEYS = ("ordered_reduction", "combine", "defer", "distribute", "fp_contract", "autotune", "pin_host", "_generic_only", "_vectorize",
                "_stream_hint", "_hoist_safe", "_shape_spec", "_neighbours", "_bulk_rows", "_group_vectorize",
                "_spmm_stream", "_stream_rows", "_row_cost", "_host_cells", "_skip_uploads")


_site_options: dict = {}       # site number -> option key; the loops of one rewritten function always pass the same options


def codegen(loop_source: str, loop_name: str, val_map: dict, options: dict):
    """Backend plugin entry (see module docstring)."""
    names = tuple(val_map)
    signature = tuple([_kind_of(v) for v in val_map.values()])
    fn = options.get("_fn")
    site = options.get("_site")             # set by the decoration-time rewrite, one per rewritten function
    opt_key = _site_options.get(site) if site is not None else None
    if opt_key is None:
        opt_key = tuple([options.get(k) for k in _OPTION_KEYS])
        if site is not None:
            if len(_site_options) > 4096:
                _site_options.clear()
            _site_options[site] = opt_key
    cache_key = (loop_source, loop_name, names, signature, opt_key, fn)
    entry = code_cache.get(cache_key)
    fresh = entry is None
    if fresh:
        entry = CompiledLoop(loop_source, loop_name, list(names), signature, options)
        code_cache[cache_key] = entry
    code_src = entry.last_source
    if code_src is None:
        args = [v for v in val_map.values() if not isinstance(v, _types.ModuleType)]
        code_src = entry.source_for(*args)
    if fresh and (options.get("dump_code") or options.get("dump_code_to_file")):
        if options.get("dump_code"):
            pretty_dump(code_src, loop_name)
        if options.get("dump_code_to_file"):
            with open(options["dump_code_to_file"], "w") as fh:
                fh.write(code_src)
    return entry, code_src
