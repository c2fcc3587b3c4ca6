"""Loop-level normalisation, run the first time an annotated loop executes.

Input: the loop source string handed to ``_kernel_launch`` (pragma line + ``for``).
Output: a ``LoopIR`` whose ``loop`` is a Python ``ast.For`` in normal form:

* the loop source holds exactly one top-level loop and starts with its pragma
  (appy/frontend/sanity_check.py:4-18);
* ``a, b = x, y`` is split into two assignments
  (appy/frontend/rewrite_tuple_assign.py:3-19) and ``x += e`` becomes ``x = x + e``
  (appy/frontend/rewrite_aug_assign.py:4-21);
* every ``range`` has three arguments and a step other than the literal 1 raises
  ``Exception("Only step 1 is supported in range, got: ...")``
  (appy/frontend/rewrite_range.py:20-24);
* a ``#pragma`` line is parsed (appy/utils.py:97-150) and attached as ``.pragma`` to the
  next ``for`` — or swallowed by the next assignment, as in the reference, where a
  ``#pragma simd`` placed before ``s = 0.0`` does not reach the loop after it
  (appy/frontend/attach_pragma.py:4-28);
* 1-D slice statements (``y[i, :] = 0``, ``y[i, :] += a * B[r, :]``,
  ``C[i, :i+1] *= beta``, ``np.sum(<slices>)``, 1-D ``u @ v``) become explicit simd
  loops, the job the reference hands to ``astpass.vector_op_to_loop``
  (appy/backends/triton/passes/lower_array_op_to_loop.py:5-22,
  appy/backends/triton/passes/rewrite_vector_dot.py:4-34);
* reductions are detected with the reference's rule: within a pragma'd loop a scalar
  name or constant-index subscript is a reduction iff *all* its assignments there have
  the same operator among ``+ * max min`` with the target as an operand
  (appy/frontend/reduction_detection.py:12-107).
"""
from __future__ import annotations

import ast
import copy
from dataclasses import dataclass, field

from ..utils import parse_pragma
from . import pragma_ast


@dataclass
class LoopIR:
    loop: ast.For
    pragma: dict
    source: str
    used_names: list = field(default_factory=list)     # first-use order (kernel argument order)
    extra_names: list = field(default_factory=list)    # X_shape_d names introduced by slice lowering


# --------------------------------------------------------------------------- helpers

def _is_name_or_const_index(node) -> bool:
    return isinstance(node, ast.Name) or (isinstance(node, ast.Subscript) and isinstance(node.slice, ast.Constant))


def _s(node) -> str:
    return ast.unparse(node)


def used_names(tree) -> list[str]:
    """Names loaded or stored in the loop source, in order of first appearance; names that
    only occur as the callee of a call (``range``, ``max``) are left out.  The order of
    this list is the order of the kernel's arguments (appy/dispatcher.py:13-17)."""
    callees = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name):
            callees.add(id(node.func))
    order: list[str] = []
    seen = set()

    class V(ast.NodeVisitor):
        def visit_Name(self, node):
            if id(node) not in callees and node.id not in seen:
                seen.add(node.id)
                order.append(node.id)

        def visit_Assign(self, node):       # value is evaluated before the target is bound
            self.visit(node.value)
            for t in node.targets:
                self.visit(t)

        def visit_AugAssign(self, node):
            self.visit(node.target)
            self.visit(node.value)

    V().visit(tree)
    return order


# --------------------------------------------------------------------------- simple rewrites

class _Simple(ast.NodeTransformer):
    def visit_Assign(self, node):
        self.generic_visit(node)
        if isinstance(node.value, ast.Tuple) and isinstance(node.targets[0], ast.Tuple):
            tgt, val = node.targets[0].elts, node.value.elts
            if len(tgt) != len(val):
                raise ValueError(f"tuple assignment arity mismatch: {_s(node)}")
            return [ast.copy_location(ast.Assign(targets=[t], value=v), node) for t, v in zip(tgt, val)]
        return node

    def visit_AugAssign(self, node):
        self.generic_visit(node)
        left = copy.deepcopy(node.target)
        for n in ast.walk(left):
            if hasattr(n, "ctx"):
                n.ctx = ast.Load()
        return ast.copy_location(
            ast.Assign(targets=[node.target], value=ast.BinOp(left=left, op=node.op, right=node.value)), node)

    def visit_Call(self, node):
        self.generic_visit(node)
        f = node.func
        is_range = isinstance(f, ast.Name) and f.id in ("range", "prange")
        is_range = is_range or (isinstance(f, ast.Attribute) and f.attr in ("range", "prange")
                                and isinstance(f.value, ast.Name) and f.value.id in ("appy", "appy_b200"))
        if is_range:
            node.func = ast.Name(id="range", ctx=ast.Load())
            node.keywords = []
            if len(node.args) == 1:
                node.args = [ast.Constant(0), node.args[0], ast.Constant(1)]
            elif len(node.args) == 2:
                node.args = [node.args[0], node.args[1], ast.Constant(1)]
            elif len(node.args) == 3:
                step = node.args[2]
                if not (isinstance(step, ast.Constant) and step.value == 1):
                    raise Exception(f"Only step 1 is supported in range, got: {_s(node)}")
            else:
                raise Exception(f"range expects 1 to 3 arguments, got: {_s(node)}")
        return node


def _attach_pragmas(stmts: list) -> list:
    """Drop pragma marker statements, attaching each to the statement that follows."""
    out = []
    pending = None
    for st in stmts:
        text = pragma_ast.pragma_text(st)
        if text is not None:
            pending = text
            continue
        if pending is not None and isinstance(st, (ast.For, ast.Assign)):
            st.pragma = parse_pragma(pending)   # an Assign swallows it, like the reference
            pending = None
        for fld in ("body", "orelse"):
            block = getattr(st, fld, None)
            if isinstance(block, list) and block and isinstance(block[0], ast.stmt):
                new = _attach_pragmas(block)
                setattr(st, fld, new if (new or fld == "orelse") else [ast.Pass()])
        out.append(st)
    return out


# --------------------------------------------------------------------------- slice lowering

class _SliceInfo:
    def __init__(self):
        self.extent = None      # ast expr: number of elements of the 1-D slices in this statement
        self.count = 0


class SliceLowering:
    """Turns statements that use 1-D slices into simd loops.  `ndim_of(name)` gives the rank
    of an array argument (None for non-arrays)."""

    def __init__(self, ndim_of):
        self.ndim_of = ndim_of
        self.counter = 0
        self.extra_names: list[str] = []

    # ---- queries
    def _has_slice(self, node) -> bool:
        for n in ast.walk(node):
            if isinstance(n, ast.Subscript):
                elts = n.slice.elts if isinstance(n.slice, ast.Tuple) else [n.slice]
                if any(isinstance(e, ast.Slice) for e in elts):
                    return True
            if isinstance(n, ast.BinOp) and isinstance(n.op, ast.MatMult):
                return True
        return False

    def _shape_name(self, arr: str, dim: int) -> ast.Name:
        name = f"{arr}_shape_{dim}"
        if name not in self.extra_names:
            self.extra_names.append(name)
        return ast.Name(id=name, ctx=ast.Load())

    def _slice_bounds(self, sub: ast.Subscript):
        """(dim, lo, hi) of the single slice in `sub`, with defaults filled in."""
        if not isinstance(sub.value, ast.Name):
            raise RuntimeError(f"Unsupported sliced expression: {_s(sub)}")
        elts = sub.slice.elts if isinstance(sub.slice, ast.Tuple) else [sub.slice]
        dims = [d for d, e in enumerate(elts) if isinstance(e, ast.Slice)]
        if len(dims) != 1:
            raise RuntimeError(f"Only 1-D slices are supported, got: {_s(sub)}")
        d = dims[0]
        sl = elts[d]
        if sl.step is not None and not (isinstance(sl.step, ast.Constant) and sl.step.value == 1):
            raise RuntimeError(f"Only unit-step slices are supported, got: {_s(sub)}")
        lo = sl.lower if sl.lower is not None else ast.Constant(0)
        if sl.upper is None:
            hi = self._shape_name(sub.value.id, d)
        elif isinstance(sl.upper, ast.UnaryOp) and isinstance(sl.upper.op, ast.USub) \
                and isinstance(sl.upper.operand, ast.Constant):
            hi = ast.BinOp(left=self._shape_name(sub.value.id, d), op=ast.Sub(), right=sl.upper.operand)
        else:
            hi = sl.upper
        if isinstance(lo, ast.UnaryOp) and isinstance(lo.op, ast.USub) and isinstance(lo.operand, ast.Constant):
            lo = ast.BinOp(left=self._shape_name(sub.value.id, d), op=ast.Sub(), right=lo.operand)
        return d, lo, hi

    # ---- element-wise rewrite of one expression for loop variable `var`
    def _elementwise(self, expr, var: str, info: _SliceInfo):
        low = self

        class R(ast.NodeTransformer):
            def visit_Subscript(self, node):
                elts = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
                if not any(isinstance(e, ast.Slice) for e in elts):
                    self.generic_visit(node)
                    return node
                d, lo, hi = low._slice_bounds(node)
                if info.extent is None:
                    if isinstance(lo, ast.Constant) and lo.value == 0:
                        info.extent = copy.deepcopy(hi)
                    else:
                        info.extent = ast.BinOp(left=copy.deepcopy(hi), op=ast.Sub(), right=copy.deepcopy(lo))
                info.count += 1
                idx = ast.Name(id=var, ctx=ast.Load())
                if not (isinstance(lo, ast.Constant) and lo.value == 0):
                    idx = ast.BinOp(left=copy.deepcopy(lo), op=ast.Add(), right=idx)
                new_elts = [self.visit(e) if k != d else idx for k, e in enumerate(elts)]
                node.slice = ast.Tuple(elts=new_elts, ctx=ast.Load()) if len(new_elts) > 1 else new_elts[0]
                return node

            def visit_Call(self, node):
                if low._reduction_call(node) is not None:
                    raise RuntimeError(f"Nested array reductions are not supported: {_s(node)}")
                self.generic_visit(node)
                return node

        return R().visit(expr)

    def _reduction_call(self, node):
        """('+'|'max'|'min', arg) if node is np.sum/np.max/np.min/sum(...) over a sliced expression."""
        if not isinstance(node, ast.Call) or len(node.args) != 1 or node.keywords:
            return None
        f = node.func
        name = f.attr if isinstance(f, ast.Attribute) else (f.id if isinstance(f, ast.Name) else None)
        if isinstance(f, ast.Attribute) and not (isinstance(f.value, ast.Name) and f.value.id in ("np", "numpy")):
            return None
        op = {"sum": "+", "max": "max", "min": "min", "amax": "max", "amin": "min"}.get(name)
        if op is None or not self._has_slice(node.args[0]):
            return None
        return op, node.args[0]

    def _rewrite_matmul(self, expr):
        """1-D ``u @ v`` -> ``np.sum(u * v)``; anything else raises like the reference."""
        low = self

        class M(ast.NodeTransformer):
            def visit_BinOp(self, node):
                self.generic_visit(node)
                if isinstance(node.op, ast.MatMult):
                    if low._vector_rank(node.left) == 1 and low._vector_rank(node.right) == 1:
                        return ast.Call(func=ast.Attribute(value=ast.Name(id="np", ctx=ast.Load()), attr="sum",
                                                           ctx=ast.Load()),
                                        args=[ast.BinOp(left=low._as_vector(node.left), op=ast.Mult(),
                                                        right=low._as_vector(node.right))], keywords=[])
                    raise RuntimeError(f"Unsupported matmul expression: {_s(node)}")
                return node

        return M().visit(expr)

    def _vector_rank(self, node):
        if isinstance(node, ast.Name):
            return self.ndim_of(node.id)
        if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name):
            elts = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
            return sum(isinstance(e, ast.Slice) for e in elts)
        return None

    def _as_vector(self, node):
        if isinstance(node, ast.Name):     # a whole 1-D array used as a vector
            return ast.Subscript(value=node, slice=ast.Slice(lower=None, upper=None, step=None), ctx=ast.Load())
        return node

    # ---- statements
    def _new_var(self, prefix):
        self.counter += 1
        return f"__{prefix}{self.counter}"

    def _simd_loop(self, var, extent, body, reduction=None):
        loop = ast.For(target=ast.Name(id=var, ctx=ast.Store()),
                       iter=ast.Call(func=ast.Name(id="range", ctx=ast.Load()),
                                     args=[ast.Constant(0), extent, ast.Constant(1)], keywords=[]),
                       body=body, orelse=[])
        loop.pragma = {"simd": True}
        if reduction:
            loop.pragma["reduction"] = reduction
        loop._from_slice = True
        return loop

    def lower_stmt(self, st):
        if not isinstance(st, ast.Assign) or not self._has_slice(st):
            return [st]
        st.value = self._rewrite_matmul(st.value)
        pre = []
        # hoist array reductions out of the expression into scalar temporaries
        low = self

        class H(ast.NodeTransformer):
            def visit_Call(self, node):
                red = low._reduction_call(node)
                if red is None:
                    self.generic_visit(node)
                    return node
                op, arg = red
                tmp = low._new_var("r")
                var = low._new_var("s")
                info = _SliceInfo()
                elem = low._elementwise(copy.deepcopy(arg), var, info)
                if op == "+":
                    init = ast.Constant(0.0)
                    upd = ast.BinOp(left=ast.Name(id=tmp, ctx=ast.Load()), op=ast.Add(), right=elem)
                else:
                    init = ast.Call(func=ast.Name(id="float", ctx=ast.Load()),
                                    args=[ast.Constant("-inf" if op == "max" else "inf")], keywords=[])
                    upd = ast.Call(func=ast.Name(id=op, ctx=ast.Load()),
                                   args=[ast.Name(id=tmp, ctx=ast.Load()), elem], keywords=[])
                pre.append(ast.Assign(targets=[ast.Name(id=tmp, ctx=ast.Store())], value=init))
                body = ast.Assign(targets=[ast.Name(id=tmp, ctx=ast.Store())], value=upd)
                pre.append(low._simd_loop(var, info.extent, [body], reduction=f"{op}:{tmp}"))
                return ast.Name(id=tmp, ctx=ast.Load())

        st.value = H().visit(st.value)
        target = st.targets[0]
        if not self._has_slice(target) and not self._has_slice(st.value):
            return pre + [st]
        if not self._has_slice(target):
            raise RuntimeError(f">1-D array expression or array-valued scalar assignment is not supported: {_s(st)}")
        var = self._new_var("s")
        info = _SliceInfo()
        tname = target.value.id if isinstance(target.value, ast.Name) else None
        new_target = self._elementwise(target, var, info)
        new_target.ctx = ast.Store()
        tgt_index = _s(new_target)
        new_value = self._elementwise(st.value, var, info)
        # reading the target array at a different offset than it is written needs a temporary
        for n in ast.walk(new_value):
            if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name) and n.value.id == tname:
                if _s(n) != tgt_index and var in {x.id for x in ast.walk(n) if isinstance(x, ast.Name)}:
                    raise NotImplementedError(
                        f"Slice statement reads `{tname}` at an offset from where it writes it; "
                        f"this needs a temporary and is not supported: {_s(st)}")
        body = ast.Assign(targets=[new_target], value=new_value)
        return pre + [self._simd_loop(var, info.extent, [body])]

    def lower_block(self, stmts):
        out = []
        for st in stmts:
            for fld in ("body", "orelse"):
                block = getattr(st, fld, None)
                if isinstance(block, list) and block and isinstance(block[0], ast.stmt):
                    setattr(st, fld, self.lower_block(block))
            out.extend(self.lower_stmt(st))
        return out


# --------------------------------------------------------------------------- reduction detection

def _reduction_op(node: ast.Assign):
    target, value = node.targets[0], node.value
    if not _is_name_or_const_index(target):
        return None
    t = _s(target)
    if isinstance(value, ast.BinOp) and isinstance(value.op, (ast.Add, ast.Mult)):
        op = "+" if isinstance(value.op, ast.Add) else "*"
        for side in (value.left, value.right):
            if _is_name_or_const_index(side) and _s(side) == t:
                return op
    elif isinstance(value, ast.Call) and isinstance(value.func, ast.Name) and value.func.id in ("max", "min") \
            and len(value.args) == 2:
        for side in value.args:
            if _is_name_or_const_index(side) and _s(side) == t:
                return value.func.id
    return None


def _chain_reduction(node: ast.Assign):
    """`t = t + a - b + c` or `t = t * a * b` written as one left-associated chain whose leftmost
    operand is the target: returns (op, value in the canonical form `t op (rest)`), else None.
    (`t -= e` arrives here as `t = t - e` and becomes `t = t + (-e)`.)  The rewrite re-associates, which
    a reduction does anyway; it is applied only to statements that then qualify as reductions."""
    target, value = node.targets[0], node.value
    if not _is_name_or_const_index(target) or not isinstance(value, ast.BinOp):
        return None
    t = _s(target)
    spine = []          # (operator, right operand) from the outermost to the innermost
    cur = value
    while isinstance(cur, ast.BinOp) and isinstance(cur.op, (ast.Add, ast.Sub, ast.Mult)):
        spine.append((cur.op, cur.right))
        cur = cur.left
    if not (_is_name_or_const_index(cur) and _s(cur) == t) or not spine:
        return None
    spine.reverse()
    if all(isinstance(op, ast.Mult) for op, _ in spine):
        kind = "*"
    elif all(isinstance(op, (ast.Add, ast.Sub)) for op, _ in spine):
        kind = "+"
    else:
        return None
    if len(spine) == 1 and not isinstance(spine[0][0], ast.Sub):
        return None     # already canonical
    if any(t in {_s(x) for x in ast.walk(operand) if _is_name_or_const_index(x)} for _, operand in spine):
        return None     # the target also appears inside an operand
    op0, rest = spine[0]
    if isinstance(op0, ast.Sub):
        rest = ast.UnaryOp(op=ast.USub(), operand=rest)
    for op, operand in spine[1:]:
        rest = ast.BinOp(left=rest, op=op, right=operand)
    new_value = ast.BinOp(left=cur, op=ast.Mult() if kind == "*" else ast.Add(), right=rest)
    return kind, ast.fix_missing_locations(ast.copy_location(new_value, value))


def detect_reductions(loop: ast.For) -> None:
    """Innermost loops first; marks ``Assign.reduce`` and extends ``For.pragma['reduction']``."""
    for child in ast.walk(loop):
        if child is not loop and isinstance(child, ast.For) and not getattr(child, "_red_done", False):
            detect_reductions(child)
    loop._red_done = True
    pragma = getattr(loop, "pragma", None)
    if pragma is None:
        return
    ops: dict[str, set] = {}
    assigns = [n for n in ast.walk(loop) if isinstance(n, ast.Assign)]
    chains = {}
    for a in assigns:
        if _is_name_or_const_index(a.targets[0]):
            kind = _reduction_op(a)
            if kind is None:
                ch = _chain_reduction(a)
                if ch is not None:
                    kind, chains[id(a)] = ch[0], ch[1]
            ops.setdefault(_s(a.targets[0]), set()).add(kind)
    for a in assigns:       # chains become `t = t op (rest)` where that makes the variable a reduction
        if id(a) in chains:
            kinds = ops.get(_s(a.targets[0]), set())
            if len(kinds) == 1 and None not in kinds:
                a.value = chains[id(a)]
    found: dict[str, str] = {}
    for a in assigns:
        key = _s(a.targets[0])
        kinds = ops.get(key, set())
        if len(kinds) == 1 and None not in kinds:
            found[key] = next(iter(kinds))
            a.reduce = found[key]
    if found and ("parallel_for" in pragma or "simd" in pragma):
        entries = [e for e in str(pragma.get("reduction", "")).split(",") if e]
        for var, op in found.items():
            if f"{op}:{var}" not in entries:
                entries.append(f"{op}:{var}")
        pragma["reduction"] = ",".join(entries)


def reductions_of(loop: ast.For) -> dict[str, str]:
    """{variable text: op} declared on a loop's pragma."""
    out = {}
    for e in str(getattr(loop, "pragma", {}).get("reduction", "")).split(","):
        if e:
            op, var = e.split(":", 1)
            out[var] = op
    return out


# --------------------------------------------------------------------------- driver

def normalize(loop_source: str, ndim_of=lambda name: None) -> LoopIR:
    tree = pragma_ast.parse(loop_source)
    loops = [n for n in tree.body if isinstance(n, ast.For)]
    if len(loops) > 1:
        raise Exception(f"Input AST should only contain a single for loop while {len(loops)} found.")
    if not tree.body or pragma_ast.pragma_text(tree.body[0]) is None:
        raise AssertionError("Input AST should start with a pragma")
    names = used_names(tree)
    tree = _Simple().visit(tree)
    tree.body = _attach_pragmas(tree.body)
    if len(tree.body) != 1 or not isinstance(tree.body[0], ast.For):
        raise Exception("Loop source must consist of a pragma followed by one for loop.")
    loop = tree.body[0]
    if not hasattr(loop, "pragma"):
        loop.pragma = parse_pragma("#pragma parallel for")
    lowering = SliceLowering(ndim_of)
    loop.body = lowering.lower_block(loop.body)
    ast.fix_missing_locations(tree)
    detect_reductions(loop)
    return LoopIR(loop=loop, pragma=loop.pragma, source=loop_source, used_names=names,
                  extra_names=lowering.extra_names)
