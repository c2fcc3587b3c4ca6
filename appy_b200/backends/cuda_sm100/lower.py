"""Lowering of a normalised loop onto the CUDA C kernel templates.

Replaces the reference's device-side pipeline
(appy/backends/triton/passes/gen_device_code.py:43-81 and device_passes/*): where
that emits one Triton program per outer iteration with 256-lane masked tiles, this
chooses one of five hand-written templates (csrc/templates/*.cuh) and generates only
the loop-specific *body functor* that the template calls:

  flat      `parallel for [simd]`, no inner simd loop        -> t_flat.cuh      (T1, T2)
  rowdot    one inner simd reduction over a dense range      -> t_rowdot.cuh    (T4)
  csr       one inner simd reduction over indptr[i]..[i+1]   -> t_csr_rows.cuh  (T3)
  csrdense  row-slice accumulation over indptr[i]..[i+1]     -> t_csr_dense.cuh (T5)
  group     any other body with inner simd loops             -> t_group.cuh

Every lowering returns a ``KernelPlan``: the CUDA source (tunables left as ``P_*``
macros so the autotuner can rebuild variants from the same text), the kernel
parameter list, and a function that turns (tunables, trip count, SM count) into a
launch configuration.
"""
from __future__ import annotations

import ast
import copy
from dataclasses import dataclass, field

from ...frontend.loop_normalize import LoopIR, reductions_of
from . import dtypes as T
from .dtypes import Ty
from .emit import ArraySym, Emitter, Env, ScalarSym, cast

OPS = {"+": "appy_add", "*": "appy_mul", "max": "appy_max", "min": "appy_min"}

# Python identifiers that cannot be used as C++ identifiers in the generated kernel
CXX_RESERVED = frozenset("""alignas alignof asm auto bitand bitor bool case catch char char16_t char32_t compl const
constexpr const_cast decltype default delete do double dynamic_cast enum explicit export extern float friend goto
inline int long mutable namespace new noexcept not_eq nullptr operator or_eq private protected public register
reinterpret_cast short signed sizeof static static_assert static_cast struct switch template this thread_local throw
typedef typeid typename union unsigned using virtual void volatile wchar_t xor xor_eq and_eq
i64 u64 u32 u8 threadIdx blockIdx blockDim gridDim warpSize""".split())


@dataclass
class Param:
    name: str          # name in val_map (or implicit / internal name)
    kind: str          # 'array' | 'scalar' | 'shape' | 'stride' | 'lo' | 'hi' | 'ws'
    ty: Ty | None = None
    array: str | None = None
    dim: int = 0


@dataclass
class KernelPlan:
    kind: str
    name: str
    source: str
    params: list                     # [Param] in kernel-argument order
    tunables: dict                   # name -> list of candidate values (first = default)
    lo_expr: ast.AST = None          # outer range bounds, evaluated on the host
    hi_expr: ast.AST = None
    uses_ws: bool = False
    vec: int = 1
    info: dict = field(default_factory=dict)
    post: str | None = None          # name of a second kernel launched after the main one (same arguments)

    def post_config(self, tun: dict, n_iter: int, sm_count: int):
        """(grid, block) of the second kernel, or None when this choice of tunables has none."""
        if self.post and self.kind == "csrdense" and tun.get("P_STREAM"):
            return 4 * sm_count, 256
        return None

    def scratch_bytes(self, tun: dict, n_iter: int, sm_count: int) -> int:
        """Bytes of per-stream scratch the launch needs (pieces of rows cut by share boundaries)."""
        if self.kind == "csrdense" and tun.get("P_STREAM"):
            workers = sm_count * tun["P_MINB"] * tun["P_WARPS"]
            return (16 + 16 * workers + 255) // 256 * 256 + workers * 2 * self.info["row_bytes_padded"]
        return 0

    def launch_config(self, tun: dict, n_iter: int, sm_count: int):
        """(grid, block, dynamic shared bytes) for `n_iter` outer iterations."""
        k = self.kind
        if k == "flat":
            block, u = tun["P_BLOCK"], tun["P_U"]
            chunks = (n_iter + self.vec - 1) // self.vec + 1
            tiles = max(1, (chunks + block * u - 1) // (block * u))
            per_sm = tun.get("P_CTAS", 0)
            grid = tiles if per_sm == 0 else min(tiles, sm_count * per_sm)
            return min(grid, 2 ** 31 - 1), block, 0
        if k in ("group", "rowdot"):
            block, g = tun["P_BLOCK"], tun["P_G"]
            units = (n_iter + tun.get("P_R", 1) - 1) // tun.get("P_R", 1)      # R rows per group at once
            units *= tun.get("P_SEG", 1)                                       # column segments per row
            groups = units if g == 0 else (units * g + block - 1) // block
            per_sm = tun.get("P_CTAS", 0)
            grid = groups if per_sm == 0 else min(groups, sm_count * per_sm)
            return max(1, min(grid, 2 ** 31 - 1)), block, 0
        if k == "csr":
            rows = tun["P_ROWS"]
            return max(1, min((n_iter + rows - 1) // rows, 2 ** 31 - 1)), tun["P_BLOCK"], 0
        if k == "csrdense" and tun.get("P_STREAM"):
            # one wave of resident CTAs; every warp of the grid takes an equal share of the non-zeros
            w = tun["P_WARPS"]
            dyn = (w * tun["P_D"] * self.info["row_bytes_padded"] if tun.get("P_RING", 1) else 0) + w * 32 * 4
            return sm_count * tun["P_MINB"], 32 * w, dyn
        if k == "csrdense":
            rows = tun["P_ROWS"]
            dyn = tun["P_WARPS"] * tun["P_S"] * (self.info["row_bytes"] + 8) if "P_S" in tun else 0   # ring + barriers
            return max(1, min((n_iter + rows - 1) // rows, 2 ** 31 - 1)), 32 * tun["P_WARPS"], dyn
        raise AssertionError(k)


@dataclass
class ArgInfo:
    """What the lowering needs to know about one runtime argument."""
    name: str
    kind: str                 # 'array' | 'scalar' | 'module'
    ty: Ty | None = None
    ndim: int = 0
    unit_last: bool = True
    aligned: bool = True      # base pointer is 16-byte aligned
    strides_vec_ok: dict = field(default_factory=dict)   # V -> all leading strides % V == 0
    itemsize: int = 0
    small: bool = False       # every element offset fits in 31 bits


# P_MINB > 0 states the resident CTAs per SM a kernel is meant for (second argument of
# __launch_bounds__); 0 leaves the choice to the compiler
MINB_MACRO = "#if P_MINB > 0\n#define APPY_MINB_ARG , P_MINB\n#else\n#define APPY_MINB_ARG\n#endif"


# --------------------------------------------------------------------------- analysis helpers

def _subscripts(node):
    return [n for n in ast.walk(node) if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name)]


def stored_arrays(stmts) -> set:
    out = set()
    for st in stmts:
        for n in ast.walk(st):
            if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Store) and isinstance(n.value, ast.Name):
                out.add(n.value.id)
    return out


def loaded_arrays(stmts) -> set:
    out = set()
    for st in stmts:
        for n in ast.walk(st):
            if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Load) and isinstance(n.value, ast.Name):
                out.add(n.value.id)
    return out


def _names_in(node) -> set:
    return {n.id for n in ast.walk(node) if isinstance(n, ast.Name)}


def _is_simd(loop) -> bool:
    return isinstance(loop, ast.For) and "simd" in getattr(loop, "pragma", {})


def _has_inner_simd(stmts) -> bool:
    for st in stmts:
        for n in ast.walk(st):
            if _is_simd(n):
                return True
    return False


def conditional_loads(stmts) -> set:
    """ids of Subscript nodes that Python evaluates only under a condition: inside a nested
    if/while/for statement, in a branch of a ternary, or after the first operand of and/or."""
    out = set()

    def mark(node):
        for n in ast.walk(node):
            if isinstance(n, ast.Subscript):
                out.add(id(n))

    def expr(node):
        for n in ast.walk(node):
            if isinstance(n, ast.IfExp):
                mark(n.body)
                mark(n.orelse)
            elif isinstance(n, ast.BoolOp):
                for v in n.values[1:]:
                    mark(v)

    for st in stmts:
        if isinstance(st, (ast.If, ast.While, ast.For)):
            for fld in ("body", "orelse"):
                for inner in getattr(st, fld, []) or []:
                    mark(inner)
            if isinstance(st, (ast.If, ast.While)):
                expr(st.test)
        else:
            expr(st)
    return out


def _last_index_offset(sub: ast.Subscript, var: str):
    """If the last index of `sub` is `var`, `var + c` or `var - c` (c an int literal) and no
    other index mentions `var`, return c; else None."""
    elts = sub.slice.elts if isinstance(sub.slice, ast.Tuple) else [sub.slice]
    for e in elts[:-1]:
        if var in _names_in(e):
            return None
    last = elts[-1]
    if isinstance(last, ast.Name) and last.id == var:
        return 0
    if isinstance(last, ast.BinOp) and isinstance(last.op, (ast.Add, ast.Sub)):
        l, r = last.left, last.right
        if isinstance(l, ast.Name) and l.id == var and isinstance(r, ast.Constant) and isinstance(r.value, int):
            return r.value if isinstance(last.op, ast.Add) else -r.value
        if isinstance(last.op, ast.Add) and isinstance(r, ast.Name) and r.id == var \
                and isinstance(l, ast.Constant) and isinstance(l.value, int):
            return l.value
    return None


# --------------------------------------------------------------------------- the lowering driver

class Lowering:
    def __init__(self, ir: LoopIR, loop_name: str, args: list, options: dict):
        self.ir = ir
        self.loop = ir.loop
        self.name = loop_name
        self.args = {a.name: a for a in args}
        self.arg_order = [a.name for a in args]
        self.options = options
        body = self.loop.body
        st_arr = stored_arrays(body)
        self.env = Env()
        self.env.numerics = "triton" if options.get("fp_contract") == "triton" else "numpy"
        for a in args:
            if a.kind == "array":
                self.env.arrays[a.name] = ArraySym(a.name, a.ty, a.ndim, a.unit_last,
                                                   readonly=(a.name not in st_arr) and options.get("_noalias", True))
            elif a.kind == "scalar":
                self.env.scalars[a.name] = ScalarSym(a.name, a.ty)
            elif a.kind == "module":
                self.env.modules.add(a.name)
        self.env.modules |= {"np", "numpy", "math"}
        self.var = self.loop.target.id
        callees = {id(n.func) for n in ast.walk(self.loop) if isinstance(n, ast.Call)}
        for n in ast.walk(self.loop):
            if isinstance(n, ast.Name) and id(n) not in callees \
                    and (n.id in CXX_RESERVED or n.id.startswith("__")) and not n.id.startswith(("__s", "__r")):
                raise NotImplementedError(
                    f"the name `{n.id}` cannot be used inside a parallel loop: it is reserved in the generated "
                    f"CUDA C (rename the variable)")
        self.env.indices[self.var] = T.WEAK_INT
        self.env.indices["__i0"] = T.I64
        self.env.indices["__j0"] = T.I64
        self.em = Emitter(self.env)
        self.lo_expr, self.hi_expr = self.loop.iter.args[0], self.loop.iter.args[1]
        self.reductions = {}           # target text -> (op, Ty, member name)
        self._setup_outer_reductions()

    # ---- shared(...) / constant-index reductions on the parallel loop
    def _setup_outer_reductions(self):
        n = 0
        for text, op in reductions_of(self.loop).items():
            node = ast.parse(text, mode="eval").body
            if isinstance(node, ast.Name):
                # a plain name reduced by a parallel loop would be a by-value scalar: the reference
                # cannot return it either; treat as an error early
                raise NotImplementedError(
                    f"`{text}` is reduced by a parallel loop but is not declared shared(...)")
            if not (isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name)
                    and node.value.id in self.env.arrays):
                continue
            arr = self.env.arrays[node.value.id]
            if op not in OPS:
                raise NotImplementedError(f"Unsupported reduction operator: {op}")
            self.reductions[text] = (op, arr.ty, f"__acc{n}", node)
            n += 1
        if len(self.reductions) > 4:
            raise NotImplementedError("at most 4 reduction variables per loop are supported")

    # ---- kernel parameters
    def _params(self, uses_ws: bool) -> list:
        ps = []
        for name in self.arg_order:
            a = self.args[name]
            if a.kind == "array":
                ps.append(Param(name, "array", a.ty))
            elif a.kind == "scalar":
                ps.append(Param(name, "scalar", a.ty))
        for name in sorted(self.env.implicit):
            arr, kind, dim = self.env.implicit[name]
            if name in self.args:
                continue
            ps.append(Param(name, kind, T.I64, array=arr, dim=dim))
        ps.append(Param("__lo", "lo", T.I64))
        ps.append(Param("__hi", "hi", T.I64))
        if uses_ws:
            ps.append(Param("__ws", "ws"))
        if getattr(self, "_uses_scratch", False):
            ps.append(Param("__scratch", "scratch"))
        if uses_ws and self.options.get("combine") == "p2p":
            ps.append(Param("__mb", "mb"))
            ps.append(Param("__seq", "seq", Ty("u", 64)))
            if self.options.get("defer"):
                ps.append(Param("__pend", "pend"))       # earlier launches whose totals this kernel collects
        return ps

    def _c_param(self, p: Param) -> str:
        if p.kind == "array":
            a = self.env.arrays[p.name]
            if a.readonly:
                return f"const {a.ty.c}* __restrict__ {p.name}"
            if self.options.get("_noalias", True):
                return f"{a.ty.c}* __restrict__ {p.name}"      # no argument overlaps a stored array
            return f"{a.ty.c}* {p.name}"
        if p.kind == "ws":
            return "void* __ws"
        if p.kind == "scratch":
            return "void* __scratch"
        if p.kind == "mb":
            return "const appy_mailbox* __mb"
        if p.kind == "pend":
            return "appy_pending2 __pend"
        return f"{p.ty.strong().c} {p.name}"

    def _members(self, params) -> list[str]:
        return [self._c_param(p) + ";" for p in params if p.kind not in ("lo", "hi")]

    def _kernel_wrapper(self, params, body_struct: str, call: str, smem_decl: str, extra_init: list[str] = (),
                        launch_bounds: str = "P_BLOCK", name: str | None = None) -> list[str]:
        sig = ", ".join(self._c_param(p) for p in params)
        lines = [f'extern "C" __global__ void __launch_bounds__({launch_bounds}) {name or self.name}({sig}) {{',
                 f"  {smem_decl}",
                 f"  {body_struct} __body;"]
        for p in params:
            if p.kind not in ("lo", "hi", "seq"):
                lines.append(f"  __body.{p.name} = {p.name};")
            elif p.kind == "seq":
                lines.append(f"  __body.{p.name} = {p.name};")
        lines += ["  " + l for l in extra_init]
        if any(p.kind == "pend" for p in params):
            # split-phase exchange: one warp serves the two launches before this one beside the kernel's own
            # work.  The last CTA does it: in a grid-stride loop it never has more tiles than the others, and
            # one fewer whenever the tiles do not divide evenly, which absorbs the warp's late start.
            lines.append("  if (blockIdx.x == gridDim.x - 1 && threadIdx.x < 32) appy_split_service(__mb, __pend);")
        lines += [f"  {call}", "}"]
        return lines

    # ------------------------------------------------------------------ dispatch
    def _check_carried_scalars(self) -> None:
        """Iterations of the parallel loop and of every simd loop run concurrently.  A scalar that is
        read before it is written in an iteration carries a value from another iteration; that is only
        meaningful for the recognised reductions (+, *, max, min).  Anything else would silently give a
        lane-dependent result, so it is refused."""
        loops = [self.loop] + [n for n in ast.walk(self.loop) if isinstance(n, ast.For) and n is not self.loop and _is_simd(n)]
        for lp in loops:
            declared = set(reductions_of(lp))
            written = set()
            for st in lp.body:
                if isinstance(st, ast.Assign) and isinstance(st.targets[0], ast.Name):
                    name = st.targets[0].id
                    if name in _names_in(st.value) and name not in written and name not in declared \
                            and getattr(st, "reduce", None) is None and lp is not self.loop:
                        raise NotImplementedError(
                            f"`{ast.unparse(st)}`: `{name}` carries a value between iterations of a simd loop; "
                            "only +, *, max and min reductions of the form `x = x op (...)` can do that")
                    written.add(name)
                elif isinstance(st, (ast.If, ast.For, ast.While)):
                    written |= {n.targets[0].id for n in ast.walk(st)
                                if isinstance(n, ast.Assign) and isinstance(n.targets[0], ast.Name)}

    def lower(self) -> KernelPlan:
        self._check_carried_scalars()
        body = self.loop.body
        if not _has_inner_simd(body):
            return self.lower_flat()
        for attempt in (self.try_csrdense, self.try_rowreduce):
            if self.options.get("_generic_only"):
                break
            saved = copy.copy(self.env.implicit), dict(self.env.locals), dict(self.env.indices)
            plan = attempt()
            if plan is not None:
                return plan
            self.env.implicit, self.env.locals, self.env.indices = saved[0], saved[1], saved[2]
            self.em.load_override.clear()
            self.em.store_override.clear()
        return self.lower_group()

    # ------------------------------------------------------------------ reductions epilogue (flat)
    def _reduction_setup(self):
        """Install overrides so that `b[0]` inside the loop is a per-thread accumulator."""
        for text, (op, ty, acc, _node) in self.reductions.items():
            self.em.load_override[text] = (acc, ty)
            self.em.store_override[text] = (lambda code, t, acc=acc, ty=ty: [f"{acc} = {cast(code, t, ty)};"])

    def _reduction_members(self) -> list[str]:
        return [f"{ty.c} {acc};" for (_op, ty, acc, _n) in self.reductions.values()]

    def _reduction_init(self) -> list[str]:
        return [f"__body.{acc} = {OPS[op]}::id<{ty.c}>();" for (op, ty, acc, _n) in self.reductions.values()]

    def _reduction_finish(self, ordered: bool) -> list[str]:
        if not self.reductions:
            return []
        out = []
        items = list(self.reductions.values())
        for op, ty, acc, _n in items:
            out.append(f"{acc} = appy_block_reduce<{OPS[op]}, {ty.c}>({acc}, reinterpret_cast<{ty.c}*>(__smem));")
        em = Emitter(self.env)       # plain addresses of the targets (no overrides)
        addrs = []
        for op, ty, acc, node in items:
            off, arr = em.offset(node)
            addrs.append(f"({arr.name} + ({off}))")
        if self.options.get("combine") == "p2p" and self.options.get("defer"):
            # split phase: a CTA only stores its partials; warp 0 of CTA 0 of the next two such kernels folds,
            # posts and collects them (appy_split_service, called at the top of the kernel)
            for r, (op, ty, acc, _n) in enumerate(items):
                out.append(f"appy_split_publish<{ty.c}>(__pend.partials, {r}, {acc});")
            return out
        if not ordered:
            out.append("if (threadIdx.x == 0) {")
            for (op, ty, acc, _n), addr in zip(items, addrs):
                out.append(f"  appy_atomic({OPS[op]}(), {addr}, {acc});")
            out.append("}")
        else:
            out.append("const appy_ws __w = appy_ws_from(__ws);")
            for r, (op, ty, acc, _n) in enumerate(items):
                out.append(f"appy_ws_publish<{ty.c}>(__w, {r}, {acc});")
            out.append("if (appy_ws_arrive(__w, __smem)) {")
            if self.options.get("combine") == "p2p":
                # this GPU's totals, then the exchange with the other ranks inside the same kernel
                for r, (op, ty, acc, _n) in enumerate(items):
                    out.append(f"  {ty.c} __t{r} = appy_ws_collect<{OPS[op]}, {ty.c}>(__w, {r}, __smem);")
                # first warp: lane r exchanges with rank r, then the warp folds in rank order
                out.append("  if (threadIdx.x < 32) {")
                bits = ", ".join(f"appy_to_bits<{ty.c}>(__t{r})" for r, (op, ty, acc, _n) in enumerate(items))
                out.append(f"    u64 __x[{len(items)}] = {{{bits}}};")
                out.append(f"    const bool __ok = appy_p2p_exchange<{len(items)}>(__mb, __seq, __x);")
                for r, ((op, ty, acc, _n), addr) in enumerate(zip(items, addrs)):
                    out.append(f"    __t{r} = appy_p2p_fold<{OPS[op]}, {ty.c}>(__mb, __x[{r}]);")
                    out.append(f"    if (!__ok) __t{r} = appy_p2p_poison<{ty.c}>(__t{r});")
                    out.append(f"    if (threadIdx.x == 0) *{addr} = {OPS[op]}::op<{ty.c}>(*{addr}, __t{r});")
                out.append("  }")
            else:
                for r, ((op, ty, acc, _n), addr) in enumerate(zip(items, addrs)):
                    out.append(f"  {{ const {ty.c} __t = appy_ws_collect<{OPS[op]}, {ty.c}>(__w, {r}, __smem);")
                    out.append(f"    if (threadIdx.x == 0) *{addr} = {OPS[op]}::op<{ty.c}>(*{addr}, __t); }}")
            out.append("}")
        return out

    # ------------------------------------------------------------------ FLAT (T1 / T2)
    def _stream_accesses(self, V: int, body=None, var=None):
        """Classify subscripts for the vector path.  Returns (loads, stores):
        loads  : {text: (array, node)} hoistable 16-byte loads at index exactly `i`
        stores : {text: (array, node)} unconditional top-level stores at index exactly `i`."""
        inner = body is not None          # an inner simd loop of the group lowering: (body, var) given
        body = self.loop.body if body is None else body
        var = self.var if var is None else var
        if V == 1:
            return {}, {}
        st_arr = stored_arrays(self.loop.body)        # stored anywhere in the kernel
        ld_arr = loaded_arrays(body)
        loads, stores = {}, {}
        hoist_cond_ok = self.options.get("_hoist_safe", True) and not inner
        never = conditional_loads(body) if inner else set()

        def arr_ok(name):
            a = self.args.get(name)
            return (a is not None and a.kind == "array" and a.unit_last and a.aligned
                    and a.strides_vec_ok.get(V, False) and name not in self.reductions_arrays())

        # top-level unconditional stores
        store_stmt_index = {}
        for k, st in enumerate(body):
            if isinstance(st, ast.Assign) and isinstance(st.targets[0], ast.Subscript):
                tgt = st.targets[0]
                if isinstance(tgt.value, ast.Name) and arr_ok(tgt.value.id) and _last_index_offset(tgt, var) == 0:
                    name = tgt.value.id
                    # every other store to this array must be this same element
                    others = [n for s2 in body for n in ast.walk(s2)
                              if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Store)
                              and isinstance(n.value, ast.Name) and n.value.id == name]
                    telts = tgt.slice.elts if isinstance(tgt.slice, ast.Tuple) else [tgt.slice]
                    if any((_names_in(e) - {self.var, var}) & set(self._assigned_locals()) for e in telts[:-1]):
                        continue
                    if len(others) == 1:
                        stores[ast.unparse(tgt)] = (name, tgt)
                        store_stmt_index[name] = k
        # loads
        for k, st in enumerate(body):
            top_level = not isinstance(st, (ast.If, ast.For, ast.While))
            for n in ast.walk(st):
                if not (isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Load) and isinstance(n.value, ast.Name)):
                    continue
                name = n.value.id
                if not arr_ok(name) or _last_index_offset(n, var) != 0 or id(n) in never:
                    continue
                if name in st_arr:
                    # read-modify-write of the same element: only loads at or before the single store
                    if name not in store_stmt_index or k > store_stmt_index[name]:
                        continue
                    if ast.unparse(n) not in stores and ast.unparse(n).replace(" ", "") not in \
                            {s.replace(" ", "") for s in stores}:
                        continue
                if not top_level and not hoist_cond_ok:
                    continue
                # indices other than the last must not depend on loop-local values
                elts = n.slice.elts if isinstance(n.slice, ast.Tuple) else [n.slice]
                if any((_names_in(e) - {self.var, var}) & set(self._assigned_locals()) for e in elts[:-1]):
                    continue
                loads[ast.unparse(n)] = (name, n)
        # a stored array that is also loaded somewhere not covered above cannot use a deferred vector store
        for text, (name, _n) in list(stores.items()):
            if name in ld_arr:
                all_loads = [ast.unparse(n) for s2 in body for n in ast.walk(s2)
                             if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Load)
                             and isinstance(n.value, ast.Name) and n.value.id == name]
                if any(t not in loads for t in all_loads):
                    del stores[text]
                    for t in [t for t, (nm, _x) in loads.items() if nm == name]:
                        del loads[t]
        # Neighbour loads (stencils): `a[.., i + d]` with 0 < |d| < V on an array the loop only reads.
        # The pack of `a[.., i]` plus |d| scalar elements on the side holds every operand, so each
        # element travels from L1 to registers once instead of once per offset.
        self.neighbours = {}
        if self.options.get("_neighbours", True) and not inner:
            cond = conditional_loads(body)
            for st in body:
                if isinstance(st, (ast.If, ast.For, ast.While)):
                    continue
                for n in ast.walk(st):
                    if not (isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Load) and isinstance(n.value, ast.Name)):
                        continue
                    name = n.value.id
                    d = _last_index_offset(n, self.var)
                    if not d or abs(d) >= V or abs(d) > 2 or name in st_arr or not arr_ok(name) or id(n) in cond:
                        continue
                    elts = n.slice.elts if isinstance(n.slice, ast.Tuple) else [n.slice]
                    if any((_names_in(e) - {self.var}) & set(self._assigned_locals()) for e in elts[:-1]):
                        continue
                    base = copy.deepcopy(n)
                    if isinstance(base.slice, ast.Tuple):
                        base.slice.elts[-1] = ast.Name(id=self.var, ctx=ast.Load())
                    else:
                        base.slice = ast.Name(id=self.var, ctx=ast.Load())
                    base_text = ast.unparse(base)
                    if base_text not in loads:
                        loads[base_text] = (name, base)        # the centre pack is fetched for the sides' sake
                    self.neighbours[ast.unparse(n)] = (base_text, d)
        return loads, stores

    def reductions_arrays(self) -> set:
        return {node.value.id for (_o, _t, _a, node) in self.reductions.values()}

    def _assigned_locals(self) -> list[str]:
        out = []
        for n in ast.walk(self.loop):
            if isinstance(n, ast.Assign) and isinstance(n.targets[0], ast.Name):
                out.append(n.targets[0].id)
            if isinstance(n, ast.For) and n is not self.loop:
                out.append(n.target.id)
        return out

    def pick_vector_width(self) -> int:
        if not self.options.get("_vectorize", True):
            return 1
        body = self.loop.body
        sizes = []
        for n in [s for st in body for s in _subscripts(st)]:
            a = self.args.get(n.value.id)
            if a is not None and a.kind == "array" and _last_index_offset(n, self.var) == 0:
                sizes.append(a.itemsize)
        if not sizes:
            return 1
        V = max(1, 16 // max(sizes))
        for cand in (V, V // 2, V // 4):
            if cand >= 2:
                loads, stores = self._stream_accesses(cand)
                if loads or stores:
                    return cand
        return 1

    def lower_flat(self) -> KernelPlan:
        em, env = self.em, self.env
        body = self.loop.body
        self._reduction_setup()
        em.infer_locals(body)
        ordered = bool(self.options.get("ordered_reduction", False) or self.options.get("combine") == "p2p") \
            and bool(self.reductions)
        V = self.pick_vector_width()
        loads, stores = self._stream_accesses(V)
        local_decl = em.declare_locals()

        # ---- scalar path: one(i)
        one = [f"APPY_DEV void one(i64 {self.var}) {{"] + ["  " + l for l in local_decl] + em.block(body) + ["}"]

        # ---- vector path
        regs, load_lines, out_decl, out_store = [], [], [], []
        slot = {}
        cond = conditional_loads(body)
        cond_texts = {ast.unparse(n) for st in body for n in ast.walk(st)
                      if isinstance(n, ast.Subscript) and id(n) in cond}
        uncond_texts = {ast.unparse(n) for st in body for n in ast.walk(st)
                        if isinstance(n, ast.Subscript) and isinstance(n.ctx, ast.Load) and id(n) not in cond}
        for text, (name, node) in loads.items():
            arr = env.arrays[name]
            s = f"l{len(slot)}"
            slot[text] = s
            regs.append(f"appy_pack<{arr.ty.c}, {V}> {s};")
            off, _ = Emitter(env).offset(_replace_index(node, self.var, "__i0"))
            ld = "appy_ld_cs" if (arr.readonly and self.options.get("_stream_hint", True)) else \
                ("appy_ld_nc" if arr.readonly else "appy_ld")
            line = f"__rg.{s} = {ld}<{arr.ty.c}, {V}>({name} + ({off}));"
            if text in cond_texts and text not in uncond_texts:
                # Python would evaluate this element only under a condition, so the array may be
                # shorter than the iteration range: fetch the pack only when it lies inside the array
                shape = f"{name}_shape_{arr.ndim - 1}"
                env.implicit[shape] = (name, "shape", arr.ndim - 1)
                line = (f"if (__i0 + {V} <= {shape}) {line} else {{ for (int __k = 0; __k < {V}; ++__k) "
                        f"__rg.{s}.v[__k] = (__i0 + __k < {shape}) ? {name}[({off}) + __k] : {arr.ty.c}(0); }}")
            load_lines.append(line)
        side = {}       # centre text -> (elements needed below, elements needed above)
        for _t, (base_text, d) in getattr(self, "neighbours", {}).items():
            lo_n, hi_n = side.get(base_text, (0, 0))
            side[base_text] = (max(lo_n, -d), max(hi_n, d))
        for base_text, (lo_n, hi_n) in side.items():
            name, node = loads[base_text]
            arr = env.arrays[name]
            sl = slot[base_text]
            off, _ = Emitter(env).offset(_replace_index(node, self.var, "__i0"))
            regs.append(f"{arr.ty.c} {sl}lo[{max(lo_n, 1)}]; {arr.ty.c} {sl}hi[{max(hi_n, 1)}];")
            for k in range(lo_n):
                load_lines.append(f"__rg.{sl}lo[{k}] = appy_ldg1({name} + (({off}) - {k + 1}));")
            for k in range(hi_n):
                load_lines.append(f"__rg.{sl}hi[{k}] = appy_ldg1({name} + (({off}) + {V + k}));")
        if V > 1:
            saved_l, saved_s = dict(em.load_override), dict(em.store_override)
            for text, s in slot.items():
                arr = env.arrays[loads[text][0]]
                em.load_override[text] = (f"__rg.{s}.v[__k]", arr.ty)
            for text, (base_text, d) in getattr(self, "neighbours", {}).items():
                arr = env.arrays[loads[base_text][0]]
                sl = slot[base_text]
                em.load_override[text] = (f"appy_side(__rg.{sl}, __rg.{sl}lo, __rg.{sl}hi, __k + ({d}))", arr.ty)
            for n_out, (text, (name, node)) in enumerate(stores.items()):
                arr = env.arrays[name]
                o = f"__o{n_out}"       # generated names begin with two underscores: users' names cannot
                out_decl.append(f"appy_pack<{arr.ty.c}, {V}> {o};")
                em.store_override[text] = (lambda code, t, o=o, ty=arr.ty: [f"{o}.v[__k] = {cast(code, t, ty)};"])
                off, _ = Emitter(env).offset(_replace_index(node, self.var, "__i0"))
                stc = "appy_st_cs" if self.options.get("_stream_hint", True) and name not in loaded_arrays(body) \
                    else "appy_st"
                out_store.append(f"{stc}<{arr.ty.c}, {V}>({name} + ({off}), {o});")
            inner = [f"const i64 {self.var} = __i0 + __k;"] + local_decl + [l.strip() for l in em.block(body, "")]
            compute = ([f"APPY_DEV void compute(i64 __i0, const Regs& __rg) {{"] + ["  " + l for l in out_decl] +
                       ["#pragma unroll", f"  for (int __k = 0; __k < {V}; ++__k) {{"] + ["    " + l for l in inner] +
                       ["  }"] + ["  " + l for l in out_store] + ["}"])
            em.load_override, em.store_override = saved_l, saved_s
            load_fn = ["APPY_DEV void load(i64 __i0, Regs& __rg) const {"] + ["  " + l for l in load_lines] + ["}"]
        else:
            compute = [f"APPY_DEV void compute(i64 __i0, const Regs&) {{ one(__i0); }}"]
            load_fn = ["APPY_DEV void load(i64, Regs&) const {}"]
        finish = ["APPY_DEV void finish(void* __smem) {"] + ["  " + l for l in self._reduction_finish(ordered)] + ["}"]

        params = self._params(uses_ws=ordered)
        struct = f"{self.name}_body"
        src = ['#include "t_flat.cuh"', f"struct {struct} {{"]
        src += ["  " + m for m in self._members(params)]
        src += ["  " + m for m in self._reduction_members()]
        src += ["  struct Regs { " + " ".join(regs) + " };"]
        src += ["  " + l for l in load_fn + compute + one + finish]
        src += ["};"]
        src += self._kernel_wrapper(params, struct, f"appy_flat<{V}, P_U>(__body, __lo, __hi, __smem);",
                                    "__shared__ double __smem[33];", self._reduction_init(),
                                    launch_bounds="P_BLOCK APPY_MINB_ARG")
        src.insert(1, MINB_MACRO)
        tun = {"P_BLOCK": [256, 128, 512], "P_U": [1, 2, 4, 8] if V > 1 else [1, 2, 4], "P_MINB": [0, 1, 2]}
        if self.reductions:
            # default: 512-thread CTAs, two per SM, open register budget (measured 4-5 % faster on the
            # 2^26-element sums than 256-thread CTAs at eight per SM)
            tun = {"P_BLOCK": [512, 256], "P_U": [4, 2, 8], "P_CTAS": [2, 4, 8], "P_MINB": [1, 0, 2]}
        return KernelPlan("flat", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr,
                          uses_ws=ordered, vec=V,
                          info={"template": "T2 shared-scalar reduction" if self.reductions else "T1 elementwise",
                                "vector_width": V, "stream_loads": len(loads), "stream_stores": len(stores)})

    # ------------------------------------------------------------------ GROUP (generic)
    def _group_emitter(self, hazard_arrays: set) -> "GroupEmitter":
        ge = GroupEmitter(self.env, hazard_arrays)
        ge.load_override = self.em.load_override
        ge.store_override = self.em.store_override
        ge.lowering = self
        return ge

    def lower_group(self) -> KernelPlan:
        body = self.loop.body
        hazards = stored_arrays(body) & loaded_arrays(body)
        ge = self._group_emitter(hazards)
        ordered = False
        if self.reductions:
            # shared(...) reductions of the parallel loop (reference: one atomic per program,
            # device_passes/rewrite_par_reduce_to_atomics.py:10-88).  Every lane of a group executes
            # scalar statements redundantly, so only lane 0 of the group accumulates; the CTA's
            # accumulators are combined once at the end of the kernel, like in the flat lowering.
            ordered = bool(self.options.get("ordered_reduction", False) or self.options.get("combine") == "p2p")
            for text, (op, ty, acc, _node) in self.reductions.items():
                ge.load_override[text] = (acc, ty)
                ge.store_override[text] = (lambda code, t, acc=acc, ty=ty:
                                           [f"if (__g.lane == 0) {acc} = {cast(code, t, ty)};"])
            ge.outer_reductions = set(self.reductions)
        # perfect nest: the outer body is one simd loop without reductions -> its range may be cut
        # into segments worked on by different groups (P_SEG)
        ge.split = len(body) == 1 and _is_simd(body[0]) and not reductions_of(body[0]) and not self.reductions
        ge.infer_locals(body)
        decl = ge.declare_locals()
        lines = ge.block(body, "    ")
        params = self._params(uses_ws=ordered)
        struct = f"{self.name}_body"
        src = ['#include "t_group.cuh"', f"struct {struct} {{"]
        if self.reductions:
            src[0] = '#include "t_group.cuh"\n#include "t_flat.cuh"'
        src += ["  " + m for m in self._members(params)]
        src += ["  " + m for m in self._reduction_members()]
        src += [f"  template <class Grp> APPY_DEV void iter(i64 {self.var}, const Grp& __g) {{"]
        src += ["    " + l for l in decl] + lines + ["  }"]
        call = "appy_group_rows<P_G, P_SEG>(__body, __lo, __hi, __smem);"
        if self.reductions:
            src += ["  APPY_DEV void finish(void* __smem) {"] + \
                   ["    " + l for l in self._reduction_finish(ordered)] + ["  }"]
            call += " __syncthreads(); __body.finish(__smem);"
        src += ["};"]
        src += self._kernel_wrapper(params, struct, call, "__shared__ double __smem[33];", self._reduction_init())
        src.insert(1, "#ifndef P_SEG\n#define P_SEG 1\n#endif")
        tun = {"P_G": [8, 1, 2, 4, 16, 32, 0], "P_BLOCK": [256, 128, 512]}
        info = {"template": "generic group lowering", "splittable": ge.split,
                "inner_vec": getattr(ge, "widest_pack", 1)}
        if ge.split:
            tun["P_SEG"] = [1, 4, 16, 64]
        if self.reductions:
            tun["P_CTAS"] = [8, 4, 16]          # persistent grid: one commit per CTA
        inner = next((n for st in body for n in ast.walk(st) if isinstance(n, ast.For) and _is_simd(n)), None)
        if inner is not None and isinstance(inner.iter, ast.Call) and len(inner.iter.args) >= 2:
            info.update({"inner_lo": inner.iter.args[0], "inner_hi": inner.iter.args[1],    # lanes per row follow it
                         "outer_var": self.var})
        return KernelPlan("group", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr,
                          uses_ws=ordered, info=info)

    # ------------------------------------------------------------------ T3 / T4: single inner simd reduction
    def try_rowreduce(self):
        body = self.loop.body
        if self.reductions:
            return None
        simd = [st for st in body if _is_simd(st)]
        if len(simd) != 1 or any(_has_inner_simd(getattr(st, "body", [])) for st in body if st is not simd[0]):
            return None
        loop = simd[0]
        k = body.index(loop)
        reds = reductions_of(loop)
        if len(reds) != 1 or len(loop.body) != 1:
            return None
        (acc_name, op), = reds.items()
        st = loop.body[0]
        if not (isinstance(st, ast.Assign) and isinstance(st.targets[0], ast.Name) and st.targets[0].id == acc_name
                and getattr(st, "reduce", None) == op and op in OPS):
            return None
        jvar = loop.target.id
        # term = the non-accumulator operand
        if isinstance(st.value, ast.BinOp):
            l, r = st.value.left, st.value.right
            term = r if (isinstance(l, ast.Name) and l.id == acc_name) else l
        else:
            a0, a1 = st.value.args
            term = a1 if (isinstance(a0, ast.Name) and a0.id == acc_name) else a0
        if acc_name in _names_in(term):
            return None
        prefix, suffix = body[:k], body[k + 1:]
        # prefix: scalar assignments only (no stores, no control flow)
        init = None
        for p in prefix:
            if not (isinstance(p, ast.Assign) and isinstance(p.targets[0], ast.Name)):
                return None
            if p.targets[0].id == acc_name:
                init = p.value
        if init is None or acc_name in _names_in(ast.Module(body=[p for p in prefix if p.targets[0].id != acc_name],
                                                            type_ignores=[])):
            return None
        for s in suffix:
            if isinstance(s, (ast.For, ast.While)):
                return None
        # the term must not read anything the suffix/prefix stores (no hazards inside one row)
        if stored_arrays(body) & loaded_arrays([loop]):
            return None
        em, env = self.em, self.env
        em.infer_locals(body)
        acc_ty = env.locals[acc_name].strong()
        lo_c, hi_c = em.range_bounds(loop)
        env.indices[jvar] = T.WEAK_INT

        # CSR form: bounds are locals assigned from P[i] and P[i+1]
        lo_n, hi_n = loop.iter.args[0], loop.iter.args[1]
        csr_ptr = None
        if isinstance(lo_n, ast.Name) and isinstance(hi_n, ast.Name):
            d = {p.targets[0].id: p.value for p in prefix}
            a, b = d.get(lo_n.id), d.get(hi_n.id)
            if isinstance(a, ast.Subscript) and isinstance(b, ast.Subscript) and isinstance(a.value, ast.Name) \
                    and isinstance(b.value, ast.Name) and a.value.id == b.value.id \
                    and a.value.id in env.arrays and env.arrays[a.value.id].ndim == 1 \
                    and _last_index_offset(a, self.var) == 0 and _last_index_offset(b, self.var) == 1 \
                    and env.arrays[a.value.id].ty.is_int and env.arrays[a.value.id].readonly:
                others = [p for p in prefix if p.targets[0].id not in (lo_n.id, hi_n.id, acc_name)]
                if not others and not ({lo_n.id, hi_n.id} & _names_in(ast.Module(body=suffix, type_ignores=[]))):
                    csr_ptr = a.value.id
        if self.var in _names_in(term):
            csr_ptr = None       # the CSR template evaluates term(k) without the row; the row-dot template passes it
        term_c, term_t = em.expr(term)
        # finish(i, total): the suffix statements with acc bound to the total
        fin_em = Emitter(env)
        fin_em.load_override = dict(em.load_override)
        params_decl_suffix = [l.strip() for l in fin_em.block(suffix, "")]
        init_c = em.as_type(init, acc_ty)
        opc = OPS[op]
        struct = f"{self.name}_body"
        other_locals = [n for n in env.locals if n != acc_name]

        if csr_ptr is not None:
            ptr = env.arrays[csr_ptr]
            # everything the term needs besides k must be a kernel argument
            if (_names_in(term) - {jvar}) & set(other_locals):
                return None
            fin = [f"APPY_DEV void finish(i64 {self.var}, Acc __total) const {{",
                   f"  {acc_ty.c} {acc_name} = {opc}::op<Acc>({init_c}, __total);"] + \
                  ["  " + l for l in em.declare_locals([n for n in other_locals
                                                        if n not in (lo_n.id, hi_n.id)])] + \
                  ["  " + l for l in params_decl_suffix] + ["}"]
            params = self._params(uses_ws=False)
            src = ['#include "t_csr_rows.cuh"', f"struct {struct} {{",
                   f"  typedef {acc_ty.c} Acc; typedef {opc} Op;"]
            src += ["  " + m for m in self._members(params)]
            src += [f"  APPY_DEV Acc term(i64 {jvar}) const {{ return {cast(term_c, term_t, acc_ty)}; }}"]
            src += ["  " + l for l in fin] + ["};"]
            smem = ("__shared__ __align__(16) unsigned char __smem[32 * sizeof(" + acc_ty.c +
                    ") + (2 * P_ROWS + 2) * sizeof(int)];")
            call = (f"appy_csr_vector<P_G, P_BLOCK, P_ROWS, P_G * 16, 512, {ptr.ty.c}>"
                    f"(__body, {csr_ptr}, __lo, __hi, __smem);")
            src += self._kernel_wrapper(params, struct, call, smem)
            tun = {"P_G": [4, 2, 8, 1, 16, 32], "P_BLOCK": [128, 256], "P_ROWS": [64, 128, 256]}
            return KernelPlan("csr", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr,
                              info={"template": "T3 CSR row loop", "indptr": csr_ptr})

        # dense form (T4): vector loads for subscripts streaming on j
        V = 1
        if self.options.get("_vectorize", True):
            sizes = [self.args[n.value.id].itemsize for n in _subscripts(term)
                     if _last_index_offset(n, jvar) == 0 and n.value.id in self.args]
            if sizes:
                V = max(1, 16 // max(sizes))
        streams = {}
        if V > 1:
            lazy = conditional_loads([ast.Expr(value=term)])      # evaluated only under a condition: keep scalar
            for n in _subscripts(term):
                a = self.args.get(n.value.id)
                if a is None or a.kind != "array" or id(n) in lazy:
                    continue
                if _last_index_offset(n, jvar) == 0 and a.unit_last and a.aligned and a.strides_vec_ok.get(V, False):
                    elts = n.slice.elts if isinstance(n.slice, ast.Tuple) else [n.slice]
                    if any((_names_in(e) - {self.var}) & set(other_locals) for e in elts[:-1]):
                        continue
                    streams[ast.unparse(n)] = n
            if not streams:
                V = 1
        # lo/hi of the inner loop may use prefix locals: evaluate the prefix in bounds()
        pre_lines = [l.strip() for l in em.block([p for p in prefix if p.targets[0].id != acc_name], "")]
        pre_decl = em.declare_locals(other_locals)
        regs, load_lines = [], []
        saved = dict(em.load_override)
        for n_s, (text, node) in enumerate(streams.items()):
            arr = env.arrays[node.value.id]
            regs.append(f"appy_pack<{arr.ty.c}, {V}> l{n_s};")
            off, _ = Emitter(env).offset(_replace_index(node, jvar, "__j0"))
            big = self.args[node.value.id].ndim > 1
            ld = "appy_ld_cs" if big else "appy_ld_nc"
            load_lines.append(f"__rg.l{n_s} = {ld}<{arr.ty.c}, {V}>({node.value.id} + ({off}));")
            em.load_override[text] = (f"__rg.l{n_s}.v[__k]", arr.ty)
        vterm_c, vterm_t = em.expr(term)
        em.load_override = saved
        needs_pre = bool(pre_lines)
        pre_block = pre_decl + pre_lines if needs_pre else []
        src = ['#include "t_rowdot.cuh"', f"struct {struct} {{",
               f"  typedef {acc_ty.c} Acc; typedef {opc} Op;"]
        params = self._params(uses_ws=False)
        src += ["  " + m for m in self._members(params)]
        src += ["  struct Regs { " + " ".join(regs) + " };"]
        src += [f"  APPY_DEV void bounds(i64 {self.var}, i64& __jlo, i64& __jhi) const {{"] + \
               ["    " + l for l in pre_block] + [f"    __jlo = {lo_c}; __jhi = {hi_c};", "  }"]
        src += [f"  APPY_DEV void load(i64 {self.var}, i64 __j0, Regs& __rg) const {{"] + \
               ["    " + l for l in pre_block] + ["    " + l for l in load_lines] + ["  }"]
        src += [f"  APPY_DEV Acc fold(i64 {self.var}, i64 __j0, const Regs& __rg, Acc __a) const {{"] + \
               ["    " + l for l in pre_block] + \
               ["#pragma unroll", f"    for (int __k = 0; __k < {V}; ++__k) {{ const i64 {jvar} = __j0 + __k;",
                f"      __a = {opc}::op<Acc>(__a, {cast(vterm_c, vterm_t, acc_ty)}); }}", "    return __a;", "  }"]
        src += [f"  APPY_DEV Acc one(i64 {self.var}, i64 {jvar}, Acc __a) const {{"] + \
               ["    " + l for l in pre_block] + \
               [f"    return {opc}::op<Acc>(__a, {cast(term_c, term_t, acc_ty)});", "  }"]
        src += [f"  APPY_DEV void finish(i64 {self.var}, Acc __total) const {{"] + \
               ["    " + l for l in pre_block] + \
               [f"    {acc_ty.c} {acc_name} = {opc}::op<Acc>({init_c}, __total);"] + \
               ["    " + l for l in params_decl_suffix] + ["  }", "};"]
        src += self._kernel_wrapper(params, struct, f"appy_rowdot<P_G, {V}, P_U, P_R>(__body, __lo, __hi, __smem);",
                                    "__shared__ double __smem[33];", launch_bounds="P_BLOCK APPY_MINB_ARG")
        # P_MINB > 0 states the resident CTAs per SM the kernel is meant for, which opens the register
        # budget: the compiler then really keeps the U x R loads of a lane in flight instead of
        # interleaving them with the arithmetic to save registers (0 = no statement, compiler's default)
        src.insert(1, MINB_MACRO)
        tun = {"P_G": [32, 0, 8, 4, 16], "P_BLOCK": [128, 256, 512], "P_U": [4, 2, 8], "P_R": [1, 2, 4],
               "P_MINB": [0, 1, 2]}
        return KernelPlan("rowdot", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr, vec=V,
                          info={"template": "T4 row-dot", "vector_width": V, "inner_lo": loop.iter.args[0],
                                "inner_hi": loop.iter.args[1], "streams": len(streams), "outer_var": self.var})

    # ------------------------------------------------------------------ T5: CSR x dense
    def try_csrdense(self):
        body = self.loop.body
        if self.reductions or len(body) != 4:
            return None
        env = self.env
        a0, a1, z, kl = body
        if not (isinstance(a0, ast.Assign) and isinstance(a1, ast.Assign) and _is_simd(z)
                and isinstance(kl, ast.For) and not _is_simd(kl)):
            return None
        if not (isinstance(a0.targets[0], ast.Name) and isinstance(a1.targets[0], ast.Name)):
            return None
        lo_n, hi_n = kl.iter.args[0], kl.iter.args[1]
        if not (isinstance(lo_n, ast.Name) and isinstance(hi_n, ast.Name)
                and lo_n.id == a0.targets[0].id and hi_n.id == a1.targets[0].id):
            return None
        pa, pb = a0.value, a1.value
        if not (isinstance(pa, ast.Subscript) and isinstance(pb, ast.Subscript) and isinstance(pa.value, ast.Name)
                and isinstance(pb.value, ast.Name) and pa.value.id == pb.value.id and pa.value.id in env.arrays
                and env.arrays[pa.value.id].ndim == 1 and env.arrays[pa.value.id].ty.is_int
                and _last_index_offset(pa, self.var) == 0 and _last_index_offset(pb, self.var) == 1):
            return None
        indptr = pa.value.id
        # z: C[i, s] = const over the full row
        if len(z.body) != 1 or not isinstance(z.body[0], ast.Assign):
            return None
        zt = z.body[0].targets[0]
        svar = z.target.id
        if not (isinstance(zt, ast.Subscript) and isinstance(zt.value, ast.Name) and zt.value.id in env.arrays
                and env.arrays[zt.value.id].ndim == 2 and isinstance(z.body[0].value, ast.Constant)):
            return None
        cname = zt.value.id
        zelts = zt.slice.elts
        if not (isinstance(zelts[0], ast.Name) and zelts[0].id == self.var and isinstance(zelts[1], ast.Name)
                and zelts[1].id == svar):
            return None
        zext = z.iter.args
        if not (isinstance(zext[0], ast.Constant) and zext[0].value == 0 and isinstance(zext[1], ast.Name)
                and zext[1].id == f"{cname}_shape_1"):
            return None
        # kl: for k: [simd s2: C[i,s2] = C[i,s2] + coef * B[row, s2]]
        if len(kl.body) != 1 or not _is_simd(kl.body[0]) or len(kl.body[0].body) != 1:
            return None
        il = kl.body[0]
        s2 = il.target.id
        kvar = kl.target.id
        st = il.body[0]
        if not (isinstance(st, ast.Assign) and isinstance(st.targets[0], ast.Subscript)):
            return None
        tgt = st.targets[0]
        if ast.unparse(tgt) != f"{cname}[{self.var}, {s2}]":
            return None
        iext = il.iter.args
        if not (isinstance(iext[0], ast.Constant) and iext[0].value == 0 and isinstance(iext[1], ast.Name)
                and iext[1].id == f"{cname}_shape_1"):
            return None
        v = st.value
        if not (isinstance(v, ast.BinOp) and isinstance(v.op, ast.Add) and ast.unparse(v.left) == ast.unparse(tgt)
                and isinstance(v.right, ast.BinOp) and isinstance(v.right.op, ast.Mult)):
            return None
        m1, m2 = v.right.left, v.right.right
        bsub, coef = (m2, m1) if isinstance(m2, ast.Subscript) and s2 in _names_in(m2) else (m1, m2)
        if not (isinstance(bsub, ast.Subscript) and isinstance(bsub.value, ast.Name) and bsub.value.id in env.arrays
                and env.arrays[bsub.value.id].ndim == 2 and s2 not in _names_in(coef)):
            return None
        bname = bsub.value.id
        belts = bsub.slice.elts
        if not (isinstance(belts[1], ast.Name) and belts[1].id == s2 and s2 not in _names_in(belts[0])):
            return None
        if bname == cname or env.arrays[bname].ty != env.arrays[cname].ty or not env.arrays[cname].ty.is_float:
            return None
        if not (env.arrays[bname].unit_last and env.arrays[cname].unit_last):
            return None
        if (_names_in(coef) | _names_in(belts[0])) & {lo_n.id, hi_n.id}:
            return None
        ncols = self.options.get("_shape", {}).get((cname, 1))
        if ncols is None or ncols > 2048:
            return None
        elt = env.arrays[cname].ty
        em = self.em
        env.indices[kvar] = T.WEAK_INT
        coef_c = em.as_type(coef, elt)
        row_c, row_t = em.expr(belts[0])
        a_b, a_c = self.args[bname], self.args[cname]
        V = 16 // (elt.bits // 8)              # elements per 16-byte pack
        vec_ok = (a_b.aligned and a_c.aligned and a_b.strides_vec_ok.get(V, False)
                  and a_c.strides_vec_ok.get(V, False) and ncols % V == 0 and self.options.get("_vectorize", True))
        if not vec_ok:
            V = 1
        Tn = (ncols + 32 * V - 1) // (32 * V)
        if Tn > 16:
            return None
        env.implicit[f"{bname}_stride_0"] = (bname, "stride", 0)
        env.implicit[f"{cname}_stride_0"] = (cname, "stride", 0)
        off_ty = "unsigned int" if a_b.small else "i64"
        nc = ncols if ncols == 32 * V * Tn else 0
        init_c = cast(*em.expr(z.body[0].value), elt)
        struct = f"{self.name}_body"
        bulk = bool(self.options.get("_bulk_rows")) and nc > 0 and V > 1
        # the streaming form (non-zeros dealt out to the warps, t_csr_dense_stream.cuh) keeps the pieces of
        # rows cut by share boundaries in a scratch buffer between its two kernels
        stream = not bulk and self.options.get("_spmm_stream", True)
        self._uses_scratch = stream
        params = self._params(uses_ws=bulk)           # the bulk variant reports a wait that ran out at ws+8
        ptr = env.arrays[indptr]
        src = ['#include "t_csr_dense.cuh"', f"struct {struct} {{",
               f"  typedef {elt.c} Elt; typedef {off_ty} Off;"]
        src += ["  " + m for m in self._members(params)]
        src += [f"  APPY_DEV Elt coef(i64 {kvar}) const {{ return {coef_c}; }}",
                f"  APPY_DEV Off brow_off(i64 {kvar}) const {{ return (Off)({row_c}) * (Off){bname}_stride_0; }}",
                f"  APPY_DEV const Elt* bbase() const {{ return {bname}; }}",
                f"  APPY_DEV Elt* crow_ptr(i64 {self.var}) const {{ return {cname} + {self.var} * {cname}_stride_0; }}",
                f"  APPY_DEV Elt init() const {{ return {init_c}; }}", "};"]
        smem = (f"__shared__ __align__(16) unsigned char __smem[appy_csr_dense_smem<{V}, {Tn}, P_WARPS, P_ROWS, "
                f"{elt.c}>::bytes];")
        call = (f"appy_csr_dense<{V}, {Tn}, P_D, P_WARPS, P_ROWS, {nc}, P_ROLL, {ptr.ty.c}>"
                f"(__body, {indptr}, __lo, __hi, {ncols}, __smem);")
        if bulk:
            # B rows travel by asynchronous bulk copies into a per-warp ring in shared memory
            # (t_csr_dense_bulk.cuh); measured slower than register gathers for 512-byte rows, kept as an option
            src[0] = '#include "t_csr_dense_bulk.cuh"'
            smem += "\n  extern __shared__ __align__(128) unsigned char __dyn[];"
            call = (f"appy_csr_dense_bulk<{V}, {Tn}, P_S, P_WARPS, P_ROWS, {nc}, {ptr.ty.c}>(__body, {indptr}, __lo, "
                    f"__hi, __smem, __dyn, reinterpret_cast<unsigned*>(reinterpret_cast<char*>(__ws) + 8), 1u << 22);")
        row_bytes_padded = 32 * V * Tn * (elt.bits // 8)
        if stream:
            src[0] = '#include "t_csr_dense_stream.cuh"'
            src += ["#if P_STREAM"]
            src += self._kernel_wrapper(
                params, struct,
                f"appy_csr_dense_stream<{V}, {Tn}, P_D, P_WARPS, {nc}, (P_RING != 0), {ptr.ty.c}>(__body, {indptr}, __lo, __hi, {ncols}, "
                f"__scratch, __dyn);",
                "extern __shared__ __align__(16) unsigned char __dyn[];", launch_bounds="32 * P_WARPS, P_MINB")
            src += self._kernel_wrapper(
                params, struct,
                f"appy_csr_dense_fixup<{V}, {Tn}, {nc}, {ptr.ty.c}>(__body, {indptr}, __lo, __hi, {ncols}, __scratch);",
                "", launch_bounds="256", name=f"{self.name}_fixup")
            src += ["#else"]
        src += self._kernel_wrapper(params, struct, call, smem, launch_bounds="32 * P_WARPS, P_MINB")
        if stream:
            src += ["#endif"]
        if bulk:
            tun = {"P_WARPS": [8, 4, 16], "P_ROWS": [32, 16, 64], "P_S": [4, 8, 16], "P_MINB": [2, 1]}
            return KernelPlan("csrdense", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr,
                              uses_ws=True, vec=V,
                              info={"template": "T5 CSR x dense (bulk-copy rows)", "ncols": ncols, "vector_width": V,
                                    "indptr": indptr, "row_bytes": ncols * (elt.bits // 8)})
        small = V * Tn <= 4
        # a row that is one 16-byte pack per lane: 16 warps x 3 CTAs per SM, four gathers in flight per
        # warp, no rolling ring (634 us against 673 us for 8 warps x 4 CTAs with a ring of 8 on the
        # 2^18-row, 128-column case); wider rows keep 8 warps and fewer, larger gathers
        one_pack = V == 4 and Tn == 1
        tun = {"P_WARPS": [16, 8, 4] if one_pack else [8, 4], "P_ROWS": [32, 16, 64],
               "P_D": ([4, 8, 2] if one_pack else [8, 4, 2]) if small else [2, 4],
               "P_MINB": ([3, 4, 2] if one_pack else [4, 3, 5, 2]) if small else [2, 1],
               "P_ROLL": [0, 1] if one_pack else [1, 0]}
        info = {"template": "T5 CSR x dense", "ncols": ncols, "vector_width": V, "indptr": indptr,
                "row_bytes_padded": row_bytes_padded}
        if not stream:
            return KernelPlan("csrdense", self.name, "\n".join(src), params, tun, self.lo_expr, self.hi_expr, vec=V,
                              info=info)
        # Streaming form: rows in flight per warp (P_D, a ring in shared memory) and warps per SM sized so that
        # about 192 KB of B rows are in flight per SM; the accumulators (V*T per lane) bound the CTAs per SM.
        warps = 16 if row_bytes_padded <= 512 else 8
        d = 8 if row_bytes_padded <= 1024 else 16
        while d > 1 and warps * d * row_bytes_padded > 64 * 1024:
            d //= 2
        while warps > 2 and warps * d * row_bytes_padded > 64 * 1024:
            warps //= 2
        minb = 2 if (row_bytes_padded <= 512 or V * Tn > 8) else 3      # 128-192 KB of rings per SM
        if V * Tn > 16:
            minb = 1
        info["row_tiled"] = {k: v[0] for k, v in tun.items()}       # defaults of the row-tiled form (small inputs)
        info["template"] = "T5 CSR x dense (streaming: non-zeros dealt out to the warps)"
        stun = {"P_STREAM": [1, 0],
                "P_WARPS": [warps] + [w for w in (16, 8, 4) if w != warps],
                "P_D": [d] + [x for x in (16, 8, 4, 2) if x != d],
                "P_MINB": [minb] + [x for x in (4, 3, 2, 1) if x != minb],
                # where the rows in flight wait: 1 = ring in shared memory (cp.async; more rows in flight, best
                # when most gathers miss L2), 0 = ring in registers (less traffic through the L1/shared-memory
                # pipe, best when the gathered rows are L2-resident)
                "P_RING": [1, 0],
                "P_ROWS": tun["P_ROWS"], "P_ROLL": tun["P_ROLL"]}
        return KernelPlan("csrdense", self.name, "\n".join(src), params, stun, self.lo_expr, self.hi_expr, vec=V,
                          info=info, post=f"{self.name}_fixup")


def _replace_index(sub: ast.Subscript, var: str, new: str) -> ast.Subscript:
    sub = copy.deepcopy(sub)

    class R(ast.NodeTransformer):
        def visit_Name(self, node):
            if node.id == var:
                return ast.Name(id=new, ctx=ast.Load())
            return node

    sub.slice = R().visit(sub.slice)
    return sub


class GroupEmitter(Emitter):
    """Statement emitter for the body of an outer iteration executed by a group of lanes."""

    def __init__(self, env, hazard_arrays: set):
        super().__init__(env)
        self.hazards = hazard_arrays
        self.in_simd = False
        self.store_guard = "__g.lane == 0"
        self.env.indices.setdefault("__i0", T.I64)

    def s_Assign(self, st):
        lines = super().s_Assign(st)
        tgt = st.targets[0]
        if not self.in_simd and isinstance(tgt, ast.Subscript) and isinstance(tgt.value, ast.Name) \
                and tgt.value.id in self.hazards:
            lines = lines + ["__g.barrier();"]
        return lines

    def _vector_plan(self, st, v):
        """(V, loads, stores) when the simd loop `st` over `v` can move 16-byte packs, else None."""
        low = getattr(self, "lowering", None)
        if low is None or not low.options.get("_vectorize", True) or not low.options.get("_group_vectorize", True):
            return None
        sizes = [low.args[n.value.id].itemsize for b in st.body for n in _subscripts(b)
                 if n.value.id in low.args and low.args[n.value.id].kind == "array" and _last_index_offset(n, v) == 0]
        if not sizes:
            return None
        V0 = max(1, 16 // max(sizes))
        for V in (V0, V0 // 2):
            if V >= 2:
                loads, stores = low._stream_accesses(V, st.body, v)
                if loads or stores:
                    return V, loads, stores
        return None

    def _vector_loop(self, st, v, lo, hi, V, loads, stores):
        """The simd loop as a loop over chunks of V consecutive iterations, aligned to multiples of V in
        absolute index space: chunks wholly inside [lo, hi) move packs, the ragged ones run element-wise."""
        env = self.env
        out = [f"  const i64 __vlo = ({lo}), __vhi = ({hi});",
               f"  const i64 __c_lo = appy_floor_div_i64(__vlo, {V}), __c_hi = (__vhi > __vlo) ? appy_floor_div_i64(__vhi - 1, {V}) + 1 : __c_lo;",
               f"  const i64 __cf_lo = appy_floor_div_i64(__vlo + {V - 1}, {V}), __cf_hi = appy_floor_div_i64(__vhi, {V});",
               "#pragma unroll 2",
               "  for (i64 __c = __c_lo + __g.lane; __c < __c_hi; __c += __g.size()) {",
               f"    const i64 __j0 = __c * {V};",
               "    if (__c >= __cf_lo && __c < __cf_hi) {"]
        saved_l, saved_s = dict(self.load_override), dict(self.store_override)
        tail = []
        for n_l, (text, (name, node)) in enumerate(loads.items()):
            arr = env.arrays[name]
            off, _ = Emitter(env).offset(_replace_index(node, v, "__j0"))
            ld = "appy_ld_nc" if arr.readonly else "appy_ld"
            out.append(f"      const appy_pack<{arr.ty.c}, {V}> __v{n_l} = {ld}<{arr.ty.c}, {V}>({name} + ({off}));")
            self.load_override[text] = (f"__v{n_l}.v[__k]", arr.ty)
        for n_o, (text, (name, node)) in enumerate(stores.items()):
            arr = env.arrays[name]
            off, _ = Emitter(env).offset(_replace_index(node, v, "__j0"))
            out.append(f"      appy_pack<{arr.ty.c}, {V}> __o{n_o};")
            self.store_override[text] = (lambda code, t, o=f"__o{n_o}", ty=arr.ty: [f"{o}.v[__k] = {cast(code, t, ty)};"])
            tail.append(f"      appy_st<{arr.ty.c}, {V}>({name} + ({off}), __o{n_o});")
        out += ["#pragma unroll", f"      for (int __k = 0; __k < {V}; ++__k) {{", f"        const i64 {v} = __j0 + __k;"]
        out += self.block(st.body, "        ")
        out += ["      }"] + tail + ["    } else {"]
        for text in list(loads) + list(stores):          # the ragged chunks use plain element accesses
            for table, saved in ((self.load_override, saved_l), (self.store_override, saved_s)):
                if text in saved:
                    table[text] = saved[text]
                else:
                    table.pop(text, None)
        out += [f"      for (int __k = 0; __k < {V}; ++__k) {{", f"        const i64 {v} = __j0 + __k;",
                f"        if ({v} >= __vlo && {v} < __vhi) {{"]
        out += self.block(st.body, "          ")
        out += ["        }", "      }", "    }", "  }"]
        return out

    def s_For(self, st):
        if self.in_simd or not _is_simd(st):
            return super().s_For(st)
        lo, hi = self.range_bounds(st)
        v = st.target.id
        self.env.indices[v] = T.WEAK_INT
        reds = reductions_of(st)
        out = ["{"]
        saved_l, saved_s = dict(self.load_override), dict(self.store_override)
        post = []
        for n, (text, op) in enumerate(reds.items()):
            outer = text in getattr(self, "outer_reductions", ())
            if text not in self.env.locals and not outer:
                raise NotImplementedError(f"simd reduction target `{text}` must be a loop-local scalar")
            if outer:        # a shared(...) target of the parallel loop reduced directly inside the simd loop
                tgt, ty = self.load_override[text]
                p = f"__p{n}_r"
            else:
                tgt, ty = text, self.env.locals[text].strong()
                p = f"__p{n}_{text}"
            out.append(f"  {ty.c} {p} = {OPS[op]}::id<{ty.c}>();")
            self.load_override[text] = (p, ty)
            self.store_override[text] = (lambda code, t, p=p, ty=ty: [f"{p} = {cast(code, t, ty)};"])
            if outer:
                post.append(f"  {{ const {ty.c} __r = __g.template reduce<{OPS[op]}, {ty.c}>({p}); "
                            f"if (__g.lane == 0) {tgt} = {OPS[op]}::op<{ty.c}>({tgt}, __r); }}")
            else:
                post.append(f"  {text} = {OPS[op]}::op<{ty.c}>({text}, __g.template reduce<{OPS[op]}, {ty.c}>({p}));")
        self.in_simd = True
        guard, self.store_guard = self.store_guard, None
        if getattr(self, "split", False):          # this group's segment of [lo, hi)
            out.append(f"  const i64 __l0 = ({lo}), __len = ({hi}) - __l0;")
            out.append("  const i64 __slo = __l0 + (__len > 0 ? __len * __g.seg / P_SEG : 0);")
            out.append("  const i64 __shi = __l0 + (__len > 0 ? __len * (__g.seg + 1) / P_SEG : 0);")
            lo, hi = "__slo", "__shi"
        vec = self._vector_plan(st, v)
        if vec is not None:
            self.widest_pack = max(getattr(self, "widest_pack", 1), vec[0])
            out += self._vector_loop(st, v, lo, hi, *vec)
        else:
            # iterations of a simd loop are independent: unrolled, a lane has several of them in flight
            out.append("#pragma unroll 4")
            out.append(f"  for (i64 {v} = ({lo}) + __g.lane; {v} < {hi}; {v} += __g.size()) {{")
            out += self.block(st.body, "    ")
            out.append("  }")
        self.store_guard = guard
        self.in_simd = False
        self.load_override, self.store_override = saved_l, saved_s
        out += post
        if stored_arrays([st]) & self.hazards:
            out.append("  __g.barrier();")
        out.append("}")
        return out
