"""Decoration-time rewrite of a ``@jit`` function (runs once per function).

Same observable behaviour as the reference's four static passes:

* shape hoisting — ``X.shape[k]`` inside an outermost ``for`` becomes the name
  ``X_shape_k``, assigned just before that loop
  (appy/frontend/hoist_shape_attr.py:4-48);
* shared scalars — for ``shared(s)`` the loop is bracketed by
  ``s = numpy.array([s])`` / ``s = s.item()`` and every ``s`` in the loop becomes
  ``s[0]`` (appy/frontend/process_shared.py:4-75), which is how a scalar survives the
  by-value snapshot of ``locals()``;
* stub replacement — an annotated loop (``#pragma parallel for ...`` or a
  ``prange`` iterator) is replaced by a call
  ``<rt>._kernel_launch(loop_source, "kernel_loop_<n>", locals(), globals(), options)``
  (appy/frontend/replace_pfor_with_stub.py:3-81);
* the decorator list of the function is dropped so that executing the rewritten
  source does not recurse.

Everything outside annotated loops stays ordinary interpreted Python.
"""
from __future__ import annotations

import ast
import copy
import re

from . import pragma_ast

RUNTIME_NAME = "__appy_rt__"


class _ShapeRewriter(ast.NodeTransformer):
    def __init__(self):
        self.found: list[tuple[str, int]] = []

    def visit_Subscript(self, node):
        self.generic_visit(node)
        v = node.value
        if isinstance(v, ast.Attribute) and v.attr == "shape" and isinstance(v.value, ast.Name) \
                and isinstance(node.slice, ast.Constant) and isinstance(node.slice.value, int):
            self.found.append((v.value.id, node.slice.value))
            return ast.copy_location(ast.Name(id=f"{v.value.id}_shape_{node.slice.value}", ctx=ast.Load()), node)
        return node


class _HoistShapes(ast.NodeTransformer):
    """Applies to every outermost ``for`` (nested loops are covered by the inner walk)."""

    def visit_For(self, node):
        rw = _ShapeRewriter()
        rw.visit(node)
        assigns, seen = [], set()
        for name, dim in rw.found:
            if (name, dim) in seen:
                continue
            seen.add((name, dim))
            assigns.append(ast.Assign(
                targets=[ast.Name(id=f"{name}_shape_{dim}", ctx=ast.Store())],
                value=ast.Subscript(value=ast.Attribute(value=ast.Name(id=name, ctx=ast.Load()), attr="shape",
                                                        ctx=ast.Load()),
                                    slice=ast.Constant(value=dim), ctx=ast.Load()),
                lineno=node.lineno))
        return assigns + [node]


class _SharedToSubscript(ast.NodeTransformer):
    def __init__(self, names):
        self.names = set(names)

    def visit_Name(self, node):
        if node.id in self.names:
            return ast.Subscript(value=ast.Name(id=node.id, ctx=ast.Load()), slice=ast.Constant(value=0),
                                 ctx=node.ctx)
        return node


def _is_prange_loop(node: ast.For) -> bool:
    it = node.iter
    if not isinstance(it, ast.Call):
        return False
    f = it.func
    if isinstance(f, ast.Name) and f.id == "prange":
        return True
    return isinstance(f, ast.Attribute) and f.attr == "prange" and isinstance(f.value, ast.Name) \
        and f.value.id in ("appy", "appy_b200")


def _shared_names(pragma: str) -> list[str]:
    names: list[str] = []
    for group in re.findall(r"shared\(([^)]*)\)", pragma):
        names.extend(v.strip() for v in group.split(",") if v.strip())
    return names


import itertools as _itertools

_site_ids = _itertools.count(1)


class _Rewriter:
    def __init__(self, options: dict, fn_name: str = ""):
        self.options = dict(options)
        self.options["_site"] = next(_site_ids)  # one number per rewritten function: its loops' options never change
        if fn_name:
            self.options["_fn"] = fn_name      # names the CUDA kernel after the function (profilers)
        self.counter = 0

    def _stub(self, loop_source: str, loop_name: str) -> ast.Expr:
        call = ast.Call(
            func=ast.Attribute(value=ast.Name(id=RUNTIME_NAME, ctx=ast.Load()), attr="_kernel_launch",
                               ctx=ast.Load()),
            args=[ast.Constant(value=loop_source), ast.Constant(value=loop_name),
                  ast.Call(func=ast.Name(id="locals", ctx=ast.Load()), args=[], keywords=[]),
                  ast.Call(func=ast.Name(id="globals", ctx=ast.Load()), args=[], keywords=[]),
                  ast.Dict(keys=[ast.Constant(value=k) for k in self.options],
                           values=[ast.Constant(value=v) for v in self.options.values()])],
            keywords=[])
        return ast.Expr(value=call)

    def rewrite_block(self, stmts: list) -> list:
        out: list = []
        pending: str | None = None          # a "#pragma parallel for ..." waiting for its loop
        for st in stmts:
            text = pragma_ast.pragma_text(st)
            if text is not None and text.startswith("#pragma parallel for"):
                pending = text
                continue
            if isinstance(st, ast.For) and (pending is not None or _is_prange_loop(st)):
                pragma = pending if pending is not None else "#pragma parallel for"
                pending = None
                out.extend(self._launch(st, pragma))
                continue
            self._recurse(st)
            out.append(st)
        return out

    def _recurse(self, st) -> None:
        for field in ("body", "orelse", "finalbody"):
            block = getattr(st, field, None)
            if isinstance(block, list) and block and isinstance(block[0], ast.stmt):
                setattr(st, field, self.rewrite_block(block) or [ast.Pass()])
        for h in getattr(st, "handlers", []) or []:
            h.body = self.rewrite_block(h.body) or [ast.Pass()]
        for case in getattr(st, "cases", []) or []:
            case.body = self.rewrite_block(case.body) or [ast.Pass()]

    def _launch(self, loop: ast.For, pragma: str) -> list:
        self.counter += 1
        loop_name = f"kernel_loop_{self.counter}"
        shared = _shared_names(pragma)
        loop = copy.deepcopy(loop)
        if _is_prange_loop(loop):          # prange(...) is range(...) inside the kernel source
            loop.iter.func = ast.Name(id="range", ctx=ast.Load())
            loop.iter.keywords = []
        if shared:
            loop = _SharedToSubscript(shared).visit(loop)
        ast.fix_missing_locations(loop)
        loop_source = pragma + "\n" + pragma_ast.unparse(loop)
        pre = [ast.parse(f"{v} = numpy.array([{v}])").body[0] for v in shared]
        post = [ast.parse(f"{v} = {v}.item()").body[0] for v in shared]
        return pre + [self._stub(loop_source, loop_name)] + post


def rewrite_function_source(source: str, options: dict) -> str:
    """Return the rewritten source of the (single) function defined in `source`."""
    tree = pragma_ast.parse(source)
    tree = _HoistShapes().visit(tree)
    for node in ast.walk(tree):
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)):
            node.decorator_list = []
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)):
            rw = _Rewriter(options, node.name)
            node.body = rw.rewrite_block(node.body) or [ast.Pass()]
    ast.fix_missing_locations(tree)
    return pragma_ast.unparse(tree)
