"""Seeded random row loops: ``for i: acc = init; simd for j: acc = acc (op) term(i, j); out[i] = f(acc)``.

One reduction per row goes to the row-dot template (T4), two to the generic group lowering; the
terms mix row-indexed matrices (float32 and float64), vectors indexed by the inner index, vectors
indexed by the row, Python scalars, ternaries and abs/min/max.  The oracle is the same term evaluated by
NumPy on whole arrays and reduced along the row in float64; sums within 1e-5 of sum|term| per row
(float32 accumulation in a different order), maxima and minima exactly.
"""
import ast as ast_mod
import importlib.util
import os
import tempfile

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

LEAVES = ["A[i, j]", "B[i, j]", "D[i, j]", "x[j]", "w[i]", "alpha", "2.0", "0.5", "-1.25"]


def _term(rng, depth):
    if depth == 0:
        return LEAVES[int(rng.integers(0, len(LEAVES)))]
    r = int(rng.integers(0, 8))
    a, b = _term(rng, depth - 1), _term(rng, depth - 1)
    if r < 4:
        return f"({a} {'+-**'[r]} {b})"
    if r == 4:
        return f"abs({a})"
    if r == 5:
        return f"{'min' if rng.integers(0, 2) else 'max'}({a}, {b})"
    if r == 6:
        return f"({a} if {a} > {b} else {b} * 0.5)"
    return f"(-{a})"


def _vec(expr):
    """Whole-array form: A[i, j] -> A, x[j] -> x (row vector), w[i] -> w (column)."""
    import ast

    class V(ast.NodeTransformer):
        def visit_Subscript(self, node):
            return ast.Name(id="_" + node.value.id, ctx=ast.Load())

        def visit_IfExp(self, node):
            self.generic_visit(node)
            return ast.Call(func=ast.Name(id="_where", ctx=ast.Load()), args=[node.test, node.body, node.orelse], keywords=[])

        def visit_Call(self, node):
            self.generic_visit(node)
            if isinstance(node.func, ast.Name) and node.func.id in ("min", "max", "abs"):
                node.func = ast.Name(id="_" + node.func.id, ctx=ast.Load())
            return node

    return compile(ast.fix_missing_locations(V().visit(ast.parse(expr, mode="eval"))), "<vec>", "eval")


def _where(t, a, b):
    return np.where(t, a, b)


def _pymin(a, b):
    return np.where(np.asarray(b) < np.asarray(a), b, a)


def _pymax(a, b):
    return np.where(np.asarray(b) > np.asarray(a), b, a)


@pytest.mark.parametrize("seed", range(int(os.environ.get("APPY_RANDOM_ROW_SEEDS", "8"))))
@pytest.mark.parametrize("shape,lo,hi", [((37, 100), 0, 100), ((5, 5000), 3, 4999), ((300, 8), 0, 8)])
def test_random_row_reductions(seed, shape, lo, hi):
    rng = np.random.default_rng(500 + seed)
    M, N = shape
    data = {"A": rng.uniform(-1, 1, shape).astype(np.float32), "B": rng.uniform(-1, 1, shape).astype(np.float32),
            "D": rng.uniform(-1, 1, shape), "x": rng.uniform(-1, 1, N).astype(np.float32),
            "w": rng.uniform(-1, 1, M).astype(np.float32)}
    alpha = 0.75
    cases = []
    for _ in range(4):
        t1, t2 = _term(rng, int(rng.integers(1, 3))), _term(rng, int(rng.integers(1, 3)))
        op = ["+", "max", "min"][int(rng.integers(0, 3))]
        two = bool(rng.integers(0, 2))
        if "j]" not in t1:
            t1 = f"({t1} + A[i, j])"
        cases.append((op, t1, t2 if two else None))
    src = ["import numpy as np", "import appy_b200 as appy", ""]
    for c, (op, t1, t2) in enumerate(cases):
        init = {"+": "0.0", "max": "float('-inf')", "min": "float('inf')"}[op]
        upd = (lambda acc, t: f"{acc} + {t}") if op == "+" else (lambda acc, t: f"{op}({acc}, {t})")
        body = ["@appy.jit", f"def rows{c}(A, B, D, x, w, alpha, lo, hi, out, out2):", "    #pragma parallel for",
                "    for i in range(A.shape[0]):", f"        s = {init}"]
        if t2 is not None:
            body.append("        q = 0.0")
        body += ["        #pragma simd", "        for j in range(lo, hi):", f"            s = {upd('s', t1)}"]
        if t2 is not None:
            body.append(f"            q = q + {t2}")
        body.append("        out[i] = s")
        if t2 is not None:
            body.append("        out2[i] = q * w[i]")
        src += body + [""]
    path = os.path.join(tempfile.gettempdir(), f"appy_random_rows_{os.getpid()}_{seed}_{M}.py")
    with open(path, "w") as fh:
        fh.write("\n".join(src))
    spec = importlib.util.spec_from_file_location(f"appy_random_rows_{seed}_{M}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dev = {k: torch.from_numpy(v).cuda() for k, v in data.items()}
    sl = slice(lo, hi)
    env = {"_A": data["A"][:, sl].astype(np.float64), "_B": data["B"][:, sl].astype(np.float64), "_D": data["D"][:, sl],
           "_x": data["x"][None, sl].astype(np.float64), "_w": data["w"][:, None].astype(np.float64), "alpha": alpha,
           "_where": _where, "_min": _pymin, "_max": _pymax, "_abs": np.abs}
    for c, (op, t1, t2) in enumerate(cases):
        v1 = np.broadcast_to(eval(_vec(t1), env), (M, hi - lo))
        out = torch.full((M,), 7.0, dtype=torch.float64, device="cuda")
        out2 = torch.full((M,), 7.0, dtype=torch.float64, device="cuda")
        getattr(mod, f"rows{c}")(dev["A"], dev["B"], dev["D"], dev["x"], dev["w"], alpha, lo, hi, out, out2)
        got = out.cpu().numpy()
        if op == "+":
            ref, scale = v1.sum(1), np.abs(v1).sum(1)
            assert np.all(np.abs(got - ref) <= 2e-5 * scale + 1e-6), (op, t1, np.abs(got - ref).max())
        else:
            # terms are evaluated in the promoted type of their operands (float32 unless D takes part)
            ref = v1.max(1) if op == "max" else v1.min(1)
            assert np.all(np.abs(got - ref) <= 1e-5 * np.abs(ref) + 1e-6), (op, t1, np.abs(got - ref).max())
        if t2 is not None:
            v2 = np.broadcast_to(eval(_vec(t2), env), (M, hi - lo))
            ref2, scale2 = v2.sum(1) * data["w"], np.abs(v2).sum(1) * np.abs(data["w"])
            assert np.all(np.abs(out2.cpu().numpy() - ref2) <= 2e-5 * scale2 + 1e-6), (t2,)


FLAT_LEAVES = ["a[i]", "b[i]", "d[i]", "alpha", "2.0", "0.5", "-1.25"]


def _flat_term(rng, depth):
    if depth == 0:
        return FLAT_LEAVES[int(rng.integers(0, len(FLAT_LEAVES)))]
    r = int(rng.integers(0, 8))
    a, b = _flat_term(rng, depth - 1), _flat_term(rng, depth - 1)
    if r < 4:
        return f"({a} {'+-**'[r]} {b})"
    if r == 4:
        return f"abs({a})"
    if r == 5:
        return f"{'min' if rng.integers(0, 2) else 'max'}({a}, {b})"
    if r == 6:
        return f"({a} if mask[i] else {b})"
    return f"(-{a})"


@pytest.mark.parametrize("seed", range(int(os.environ.get("APPY_RANDOM_ROW_SEEDS", "8"))))
def test_random_shared_scalar_reductions(seed):
    """One to three shared(...) scalars per loop (+, max, min), written the way the reference's examples
    are (`s = 0.0 ... shared(s) ... return s`): rtol 1e-5 of sum|term| for sums (float64 accumulation of
    float32 terms), exact up to term rounding for the extrema."""
    rng = np.random.default_rng(900 + seed)
    n = int(rng.choice([1, 31, 4099, 262147]))
    data = {"a": rng.uniform(-1, 1, n).astype(np.float32), "b": rng.uniform(-1, 1, n).astype(np.float32),
            "d": rng.uniform(-1, 1, n), "mask": rng.random(n) < 0.5}
    alpha = 0.75
    src = ["import numpy as np", "import appy_b200 as appy", ""]
    cases = []
    for c in range(5):
        k = int(rng.integers(1, 4))
        ops = [["+", "max", "min"][int(rng.integers(0, 3))] for _ in range(k)]
        terms = [_flat_term(rng, int(rng.integers(1, 3))) for _ in range(k)]
        terms = [t if "[i]" in t else f"({t} * a[i])" for t in terms]
        names = ["r0", "r1", "r2"][:k]
        init = {"+": "0.0", "max": "-1.0e30", "min": "1.0e30"}
        body = ["@appy.jit", f"def red{c}(a, b, d, mask, alpha):"] + [f"    {nm} = {init[op]}" for nm, op in zip(names, ops)]
        body += [f"    #pragma parallel for simd shared({', '.join(names)})", "    for i in range(a.shape[0]):"]
        for nm, op, t in zip(names, ops, terms):
            body.append(f"        {nm} = {nm} + {t}" if op == "+" else f"        {nm} = {op}({nm}, {t})")
        body.append(f"    return {', '.join(names)}" + ("," if k == 1 else ""))
        src += body + [""]
        cases.append((ops, terms))
    path = os.path.join(tempfile.gettempdir(), f"appy_random_red_{os.getpid()}_{seed}.py")
    with open(path, "w") as fh:
        fh.write("\n".join(src))
    spec = importlib.util.spec_from_file_location(f"appy_random_red_{seed}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dev = {k: torch.from_numpy(v).cuda() for k, v in data.items()}
    env = {"_a": data["a"].astype(np.float64), "_b": data["b"].astype(np.float64), "_d": data["d"], "_mask": data["mask"],
           "alpha": alpha, "_where": _where, "_min": _pymin, "_max": _pymax, "_abs": np.abs}
    for c, (ops, terms) in enumerate(cases):
        got = getattr(mod, f"red{c}")(dev["a"], dev["b"], dev["d"], dev["mask"], alpha)
        for op, t, g in zip(ops, terms, got):
            v = np.broadcast_to(eval(_vec(t), env), (n,))
            if op == "+":
                assert abs(g - v.sum()) <= 1e-5 * np.abs(v).sum() + 1e-6, (op, t, g, v.sum())
            else:
                ref = v.max() if op == "max" else v.min()
                assert abs(g - ref) <= 1e-5 * abs(ref) + 1e-6, (op, t, g, ref)


CSR_TERMS = ["D[j] * x[J[j]]", "D[j] * x[J[j]] * w[i]", "abs(D[j]) + x[J[j]]", "D[j] * (x[J[j]] - z[J[j]])",
             "(D[j] if x[J[j]] > 0.0 else -D[j])", "D[j] * D[j]", "x[J[j]] * z[J[j]] + alpha",
             "min(D[j], x[J[j]]) * 2.0"]


@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("val_dtype", [np.float32, np.float64])
def test_csr_row_loops_with_varied_terms(idx_dtype, val_dtype):
    """CSR row loops whose inner term is not the plain SpMV product: per-row factors, two gathered
    vectors, ternaries, max/min reductions; int32 and int64 index arrays, float32 and float64 values."""
    from appy_b200 import workloads as W
    A, x = W.spmv(2500, 12, kind="zipf", cap=700, seed=31)
    rng = np.random.default_rng(32)
    D = A.data.astype(val_dtype)
    P, J = A.indptr.astype(idx_dtype), A.indices.astype(idx_dtype)
    xv = x.astype(val_dtype)
    zv = rng.uniform(-1, 1, x.size).astype(val_dtype)
    wv = rng.uniform(-1, 1, A.shape[0]).astype(val_dtype)
    alpha = 0.25
    src = ["import numpy as np", "import appy_b200 as appy", ""]
    cases = [(t, op) for t in CSR_TERMS for op in ("+",)] + [(CSR_TERMS[0], "max"), (CSR_TERMS[3], "min")]
    for c, (t, op) in enumerate(cases):
        init = {"+": "0.0", "max": "-1.0e30", "min": "1.0e30"}[op]
        upd = f"s = s + {t}" if op == "+" else f"s = {op}(s, {t})"
        src += ["@appy.jit", f"def csr{c}(D, P, J, x, z, w, alpha, y, M):", "    #pragma parallel for",
                "    for i in range(M):", "        start, end = P[i], P[i+1]", f"        s = {init}", "        #pragma simd",
                "        for j in range(start, end):", f"            {upd}", "        y[i] = s", ""]
    path = os.path.join(tempfile.gettempdir(), f"appy_random_csr_{os.getpid()}_{np.dtype(idx_dtype).name}_{np.dtype(val_dtype).name}.py")
    with open(path, "w") as fh:
        fh.write("\n".join(src))
    spec = importlib.util.spec_from_file_location("appy_random_csr_" + np.dtype(idx_dtype).name + np.dtype(val_dtype).name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dev = [torch.from_numpy(v).cuda() for v in (D, P, J, xv, zv, wv)]
    M = A.shape[0]
    rows = np.repeat(np.arange(M), np.diff(A.indptr))
    env = {"_D": D.astype(np.float64), "_x": xv.astype(np.float64)[A.indices], "_z": zv.astype(np.float64)[A.indices],
           "_w": wv.astype(np.float64)[rows], "_J": None, "alpha": alpha, "_where": _where, "_min": _pymin, "_max": _pymax,
           "_abs": np.abs}

    class GatherVec(ast_mod.NodeTransformer):
        def visit_Subscript(self, node):      # x[J[j]] -> _x (already gathered), D[j] -> _D, w[i] -> _w
            return ast_mod.Name(id="_" + node.value.id, ctx=ast_mod.Load())

        def visit_IfExp(self, node):
            self.generic_visit(node)
            return ast_mod.Call(func=ast_mod.Name(id="_where", ctx=ast_mod.Load()), args=[node.test, node.body, node.orelse], keywords=[])

        def visit_Call(self, node):
            self.generic_visit(node)
            if isinstance(node.func, ast_mod.Name) and node.func.id in ("min", "max", "abs"):
                node.func = ast_mod.Name(id="_" + node.func.id, ctx=ast_mod.Load())
            return node

    for c, (t, op) in enumerate(cases):
        tree = GatherVec().visit(ast_mod.parse(t, mode="eval"))
        v = np.broadcast_to(eval(compile(ast_mod.fix_missing_locations(tree), "<csr>", "eval"), env), (A.nnz,))
        y = torch.full((M,), 7.0, dtype=torch.float64, device="cuda")
        getattr(mod, f"csr{c}")(*dev, alpha, y, M)
        got = y.cpu().numpy()
        if op == "+":
            ref = np.zeros(M); np.add.at(ref, rows, v)
            scale = np.zeros(M); np.add.at(scale, rows, np.abs(v))
            assert np.all(np.abs(got - ref) <= 2e-5 * scale + 1e-6), (t, np.abs(got - ref).max())
        else:
            ref = np.full(M, -1.0e30 if op == "max" else 1.0e30)
            (np.maximum if op == "max" else np.minimum).at(ref, rows, v)
            assert np.all(np.abs(got - ref) <= 1e-5 * np.abs(ref) + 1e-6), (t, op)
