"""Seeded random element-wise expressions: the generated kernel against NumPy, bit for bit.

Every loop is ``[t = <expr>; [u = <expr>;]] out[i] = <expr>`` over arrays of mixed dtypes (float32, float64, int32, int64, bool)
and Python scalars.  The expression text is evaluated twice: by NumPy on whole arrays (``a[i]``
replaced by the array ``a``), which is the oracle, and by the CUDA kernel generated for the loop.
Operators are those with one correctly rounded result per operation (+ - * / // % abs min max sqrt,
comparisons, and/or/not, ternary), so with the default ``fp_contract="numpy"`` flags (no FMA
contraction, IEEE division and square root) and NEP-50 promotion the two must agree exactly,
NaN for NaN.  Integer division and modulo get non-zero divisors by construction.
"""
import math
import os
import tempfile
import importlib.util

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

N = 2053
ARRAYS = {"f": np.float32, "d": np.float64, "k": np.int32, "l": np.int64, "m": np.bool_}


_LOCALS: list = []      # names of the loop-local scalars an expression may use (set by the test)


def _rand_expr(rng, depth, want):
    """An expression string of kind `want` ('num' or 'bool') over a[i]-style operands."""
    if want == "bool":
        r = rng.integers(0, 5 if depth > 0 else 2)
        if r == 0:
            return "m[i]"
        if r == 1 or depth == 0:
            op = rng.choice(["<", "<=", ">", ">=", "==", "!="])
            return f"({_rand_expr(rng, max(depth - 1, 0), 'num')} {op} {_rand_expr(rng, max(depth - 1, 0), 'num')})"
        if r == 2:
            return f"(not {_rand_expr(rng, depth - 1, 'bool')})"
        op = "and" if r == 3 else "or"
        return f"({_rand_expr(rng, depth - 1, 'bool')} {op} {_rand_expr(rng, depth - 1, 'bool')})"
    if depth == 0:
        r = rng.integers(0, 7)
        if r < 4:
            return f"{'fdkl'[r]}[i]"
        if r == 4:
            return repr(float(rng.choice([0.5, 2.0, 3.25, -1.75, 10.0])))
        if r == 5:
            return repr(int(rng.integers(-7, 8)))
        return rng.choice(["alpha", "n2"] + list(_LOCALS))
    r = rng.integers(0, 12)
    a = _rand_expr(rng, depth - 1, "num")
    b = _rand_expr(rng, depth - 1, "num")
    if r < 5:
        return f"({a} {'+-*'[r % 3]} {b})"
    if r == 5:
        return f"({a} / (abs({b}) + 1))"
    if r == 6:
        return f"(k[i] // (abs(l[i]) + 1))" if rng.integers(0, 2) else f"(l[i] % (abs(k[i]) + 2))"
    if r == 7:
        return f"abs({a})"
    if r == 8:
        return f"{'min' if rng.integers(0, 2) else 'max'}({a}, {b})"
    if r == 9:
        return f"np.sqrt(abs({a}))"
    if r == 10:
        if "[i]" not in a and "[i]" not in b:
            # two Python scalars: the scalar loop yields a weak Python value chosen per element, which
            # whole-array NumPy cannot express; give one branch an array operand
            b = f"({b} * d[i])"
        return f"({a} if {_rand_expr(rng, depth - 1, 'bool')} else {b})"
    return f"(-{a})"


def _vectorised(expr):
    """The same expression on whole arrays: NumPy functions for the Python builtins that are not
    element-wise (min, max, abs are fine as ufunc-backed operators; and/or/not and the ternary are not)."""
    import ast

    class V(ast.NodeTransformer):
        def visit_Subscript(self, node):
            return ast.Name(id=node.value.id, ctx=ast.Load())

        def visit_IfExp(self, node):
            self.generic_visit(node)
            return ast.Call(func=ast.Name(id="_where", ctx=ast.Load()), args=[node.test, node.body, node.orelse], keywords=[])

        def visit_BoolOp(self, node):
            self.generic_visit(node)
            fn = "_and" if isinstance(node.op, ast.And) else "_or"
            out = node.values[0]
            for v in node.values[1:]:
                out = ast.Call(func=ast.Name(id=fn, ctx=ast.Load()), args=[out, v], keywords=[])
            return out

        def visit_UnaryOp(self, node):
            self.generic_visit(node)
            if isinstance(node.op, ast.Not):
                return ast.Call(func=ast.Name(id="_not", ctx=ast.Load()), args=[node.operand], keywords=[])
            return node

        def visit_Call(self, node):
            self.generic_visit(node)
            if isinstance(node.func, ast.Name) and node.func.id in ("min", "max"):
                node.func = ast.Name(id="_" + node.func.id, ctx=ast.Load())
            return node

    tree = V().visit(ast.parse(expr, mode="eval"))
    return compile(ast.fix_missing_locations(tree), "<vec>", "eval")


def _py_minmax(fn):
    # Python's min(a, b) returns a unless b < a (max: unless b > a); for floats that differs from
    # np.minimum on NaN and signed zeros, and the generated code follows Python.  Python scalars stay
    # Python scalars (weak types under NEP 50), as in the scalar loop.
    def f(a, b):
        if not isinstance(a, np.ndarray) and not isinstance(b, np.ndarray):
            return min(a, b) if fn == "min" else max(a, b)
        rt_ = np.result_type(a, b)
        a, b = np.broadcast_arrays(np.asarray(a), np.asarray(b))
        pick_b = (b < a) if fn == "min" else (b > a)
        return np.where(pick_b, b.astype(rt_), a.astype(rt_))
    return f


def _py_abs(a):
    return np.abs(a) if isinstance(a, np.ndarray) else abs(a)


def _promote_like_python(test, x, y):
    if not any(isinstance(v, np.ndarray) for v in (test, x, y)):
        return x if test else y
    rt_ = np.result_type(x, y)                 # Python scalars enter as weak types
    return np.where(test, np.asarray(x).astype(rt_), np.asarray(y).astype(rt_))


@pytest.mark.parametrize("seed", range(int(os.environ.get("APPY_RANDOM_EXPR_SEEDS", "12"))))
def test_random_elementwise_expressions(seed):
    rng = np.random.default_rng(1000 + seed)
    data = {
        "f": rng.uniform(-4, 4, N).astype(np.float32),
        "d": rng.uniform(-4, 4, N),
        "k": rng.integers(-50, 50, N).astype(np.int32),
        "l": rng.integers(-1000, 1000, N).astype(np.int64),
        "m": rng.random(N) < 0.5,
    }
    alpha, n2 = 1.5, 3
    # every loop: up to two loop-local scalars, each assigned once, then the stored expression
    loops = []
    for _ in range(10):
        del _LOCALS[:]
        pre = []
        for name in ("t", "u")[:int(rng.integers(0, 3))]:
            pre.append((name, _rand_expr(rng, int(rng.integers(0, 3)), "num")))
            _LOCALS.append(name)
        loops.append((pre, _rand_expr(rng, int(rng.integers(1, 4)), "num")))
    del _LOCALS[:]
    exprs = [e for _pre, e in loops]
    src = ["import math", "import numpy as np", "import appy_b200 as appy", ""]
    for j, (pre, e) in enumerate(loops):
        src += ["@appy.jit", f"def loop{j}(f, d, k, l, m, alpha, n2, out):", "    #pragma parallel for simd",
                "    for i in range(out.shape[0]):"] + [f"        {nm} = {ex}" for nm, ex in pre] + [f"        out[i] = {e}", ""]
    path = os.path.join(tempfile.gettempdir(), f"appy_random_expr_{os.getpid()}_{seed}.py")
    with open(path, "w") as fh:
        fh.write("\n".join(src))
    spec = importlib.util.spec_from_file_location(f"appy_random_expr_{seed}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dev = {k: torch.from_numpy(v).cuda() for k, v in data.items()}
    env = dict(data, alpha=alpha, n2=n2, np=np, math=math, abs=_py_abs, _where=_promote_like_python,
               _and=np.logical_and, _or=np.logical_or, _not=np.logical_not,
               _min=_py_minmax("min"), _max=_py_minmax("max"))
    for j, (pre, e) in enumerate(loops):
        env.pop("t", None), env.pop("u", None)
        with np.errstate(all="ignore"):
            for nm, ex in pre:
                env[nm] = eval(_vectorised(ex), env)
            ref = np.asarray(eval(_vectorised(e), env))
        ref = np.broadcast_to(ref, (N,)).copy()
        if ref.dtype == np.bool_:
            continue                                   # a purely boolean value has no array to land in here
        out = torch.empty(N, dtype=torch.from_numpy(ref[:0]).dtype, device="cuda")
        getattr(mod, f"loop{j}")(dev["f"], dev["d"], dev["k"], dev["l"], dev["m"], alpha, n2, out)
        got = out.cpu().numpy()
        same = (got == ref) | (np.isnan(got.astype(np.float64)) & np.isnan(ref.astype(np.float64)))
        assert same.all(), (pre, e, ref.dtype, got[~same][:4], ref[~same][:4])
