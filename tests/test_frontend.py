"""Front-end behaviour that must match the reference (CPU only).

Each case cites the reference behaviour it pins."""
import ast

import numpy as np
import pytest

import appy_b200 as appy
from appy_b200.frontend import pragma_ast
from appy_b200.frontend.loop_normalize import normalize, reductions_of, used_names
from appy_b200.frontend.static_rewrite import rewrite_function_source
from appy_b200.utils import dict_to_pragma, parse_pragma


# ---- appy/utils.py:97-172
def test_parse_pragma_clauses():
    p = parse_pragma("#pragma parallel for simd shared(a, b) reduction(+:x)")
    assert list(p.items()) == [("parallel_for", True), ("simd", True), ("shared", ["a", "b"]), ("reduction", "+:x")]
    assert parse_pragma("#pragma simd") == {"simd": True}
    assert parse_pragma("#pragma parallel for block(8, 16)")["block"] == ("8", "16")
    assert dict_to_pragma(parse_pragma("#pragma parallel for simd")) == "#pragma parallel for simd"


def test_unknown_clause_names_the_clause():
    # tests/unit/general/pragma/test_invalid_pragma.py
    with pytest.raises(ValueError) as e:
        parse_pragma("#pragma parallel for simd my_directive")
    assert "my_directive" in str(e.value)


# ---- comment-preserving parse (the role of ast_comments in appy/__init__.py:40-41)
def test_pragma_lines_survive_parse_and_unparse():
    src = "def f(a):\n    x = '#pragma not a comment'\n    #pragma parallel for\n\n    for i in range(3):\n        #pragma simd\n        for j in range(2):\n            a[i, j] = 0  # trailing #pragma ignored\n"
    tree = pragma_ast.parse(src)
    texts = [pragma_ast.pragma_text(n) for n in ast.walk(tree) if pragma_ast.pragma_text(n)]
    assert "#pragma parallel for" in texts and "#pragma simd" in texts
    out = pragma_ast.unparse(tree)
    assert "    #pragma parallel for" in out and "        #pragma simd" in out


# ---- static rewrite: appy/frontend/{hoist_shape_attr,process_shared,replace_pfor_with_stub}.py
def test_static_rewrite_shapes_shared_and_stub():
    src = '''
@appy.jit
def f(a, n):
    s = 0.0
    #pragma parallel for simd shared(s)
    for i in range(a.shape[0]):
        s += a[i]
    for t in range(n):
        #pragma parallel for
        for i in range(1, a.shape[0] - 1):
            a[i] = t
    return s
'''
    out = rewrite_function_source(src, {"backend": None})
    assert "'_fn': 'f'" in out
    assert "@appy.jit" not in out
    assert "a_shape_0 = a.shape[0]" in out
    assert "s = numpy.array([s])" in out and "s = s.item()" in out
    assert "s[0] += a[i]" in out
    assert out.count("_kernel_launch(") == 2
    assert "'kernel_loop_1'" in out and "'kernel_loop_2'" in out
    assert "locals(), globals()" in out
    # the second loop sits inside a plain Python loop, which stays interpreted
    assert "for t in range(n):" in out


def test_prange_loops_are_replaced():
    src = "def f(a, n):\n    for i in appy.prange(n):\n        a[i] = 1\n    for i in prange(n):\n        a[i] = 2\n"
    out = rewrite_function_source(src, {})
    assert out.count("_kernel_launch(") == 2 and "for i in range(n)" in out


# ---- tests/unit/general/pragma/test_no_pragma.py: undecorated behaviour is preserved
def test_no_pragma_functions_run_unchanged():
    @appy.jit
    def foo(x):
        return x

    assert foo([1, 2, 3]) == [1, 2, 3]

    @appy.jit
    def bar(x):
        for i in range(x.shape[0]):
            x[i] += 1
        return x

    assert all(bar(np.zeros(10)) == np.ones(10))

    @appy.jit
    def baz(x):
        s = 0
        for i in range(x.shape[0]):
            s += x[i]
        return s

    assert baz(np.arange(10)) == 45


def test_jit_accepts_options():
    @appy.jit(dump_code=False, dry_run=True)
    def foo(x):
        return x + 1

    assert foo(1) == 2


# ---- loop normalisation
SPMV = '''#pragma parallel for
for i in range(M):
    start, end = A_indptr[i], A_indptr[i+1]
    s = 0.0
    #pragma simd
    for j in range(start, end):
        s += A_data[j] * x[A_indices[j]]
    y[i] = s'''


def test_normalize_spmv():
    ir = normalize(SPMV)
    # kernel-argument order = first use in the loop source (appy/dispatcher.py:13-17)
    assert ir.used_names == ["i", "M", "A_indptr", "start", "end", "s", "j", "A_data", "x", "A_indices", "y"]
    text = ast.unparse(ir.loop)
    assert "start = A_indptr[i]" in text and "end = A_indptr[i + 1]" in text      # tuple assign split
    assert "s = s + A_data[j] * x[A_indices[j]]" in text                           # aug assign expanded
    assert "range(0, M, 1)" in text and "range(start, end, 1)" in text             # 3-argument ranges
    inner = [n for n in ast.walk(ir.loop) if isinstance(n, ast.For) and n is not ir.loop][0]
    assert inner.pragma["simd"] is True and reductions_of(inner) == {"s": "+"}
    # `s = 0.0` in the outer body makes s a per-iteration local, not an outer reduction
    assert reductions_of(ir.loop) == {}


def test_step_other_than_one_raises():
    # tests/unit/general/loop_range/test_irregular_range.py
    with pytest.raises(Exception) as e:
        normalize("#pragma parallel for simd\nfor i in range(0, n, 2):\n    c[i] = a[i]")
    assert "range" in str(e.value) and "step" in str(e.value)


def test_loop_source_must_start_with_pragma():
    with pytest.raises(AssertionError):
        normalize("for i in range(n):\n    c[i] = 1")


def test_simd_pragma_before_assignment_binds_to_the_assignment():
    # tests/integration/triton/tutorial/test_rowwise_reduction.py:8-10
    ir = normalize("#pragma parallel for\nfor i in range(n):\n    #pragma simd\n    s = 0.0\n    for j in range(m):\n        s += a[i, j]\n    b[i] = s")
    inner = [n for n in ast.walk(ir.loop) if isinstance(n, ast.For) and n is not ir.loop][0]
    assert not hasattr(inner, "pragma")


def test_shared_reduction_detection_under_if():
    ir = normalize("#pragma parallel for shared(b)\nfor i in range(n):\n    if mask[i]:\n        b[0] += a[i]")
    assert reductions_of(ir.loop) == {"b[0]": "+"}
    ir = normalize("#pragma parallel for simd shared(m)\nfor i in range(n):\n    m[0] = max(m[0], a[i])")
    assert reductions_of(ir.loop) == {"m[0]": "max"}
    # a plain store is not a reduction (tests/integration/triton/tutorial/test_var_write.py)
    ir = normalize("#pragma parallel for shared(a)\nfor i in range(10):\n    if i == 3:\n        a[0] = 1")
    assert reductions_of(ir.loop) == {}


def test_slice_statements_become_simd_loops():
    src = '''#pragma parallel for
for i in range(M):
    start, end = P[i], P[i+1]
    y[i, :] = 0
    for k in range(start, end):
        y[i, :] += D[k] * B[J[k], :]'''
    ir = normalize(src, {"y": 2, "B": 2}.get)
    loops = [n for n in ast.walk(ir.loop) if isinstance(n, ast.For) and n is not ir.loop]
    simd = [l for l in loops if getattr(l, "pragma", {}).get("simd")]
    assert len(simd) == 2
    text = ast.unparse(ir.loop)
    assert "y[i, __s1] = 0" in text and "y[i, __s2] = y[i, __s2] + D[k] * B[J[k], __s2]" in text
    assert "y_shape_1" in ir.extra_names


def test_np_sum_and_vector_dot_are_lowered_to_reductions():
    src = "#pragma parallel for\nfor i in range(n):\n    y[i] = np.sum(alpha * A[i, :] * x[:])\n    z[i] = A[i, :] @ x\n    C[i, :i + 1] *= beta"
    ir = normalize(src, {"A": 2, "x": 1, "C": 2}.get)
    text = ast.unparse(ir.loop)
    assert "__r1 = __r1 + alpha * A[i, __s2] * x[__s2]" in text
    assert "A[i, __s4] * x[__s4]" in text
    assert "range(0, i + 1, 1)" in text and "C[i, __s5] = C[i, __s5] * beta" in text
    with pytest.raises(RuntimeError) as e:
        normalize("#pragma parallel for\nfor i in range(n):\n    y[i, :] = A @ B[:, i]", {"A": 2, "B": 2, "y": 2}.get)
    assert "matmul" in str(e.value)


def test_offset_slice_update_is_refused():
    # docs/metal_simd_memory_hazards.md: `A[i, 1:] = A[i, :-1]` would need a temporary
    with pytest.raises(NotImplementedError):
        normalize("#pragma parallel for\nfor i in range(n):\n    A[i, 1:] = A[i, :-1] + 1", {"A": 2}.get)


SLICE_CASES = {
    "row_times_gathered_rows": (
        "#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    y[i, :] = 0\n"
        "    for k in range(start, end):\n        y[i, :] += D[k] * B[J[k], :]", ["y"]),
    "sums_dots_and_extrema": (
        "#pragma parallel for\nfor i in range(M):\n    y1[i] = np.sum(alpha * A[i, :] * x[:])\n    y2[i] = A[i, :] @ x\n"
        "    y3[i] = np.max(A[i, 1:N-1]) - np.min(A[i, :])", ["y1", "y2", "y3"]),
    "triangular_rank_k_update": (
        "#pragma parallel for\nfor i in range(M):\n    S[i, :i + 1] *= beta\n    for k in range(N):\n"
        "        S[i, :i + 1] += alpha * A[i, k] * A[:i + 1, k]", ["S"]),
    "windows_with_negative_bounds": (
        "#pragma parallel for\nfor i in range(M):\n    W[i, 1:-1] = 2.0 * A[i, 1:-1] - A[i, 2:] + A[i, :-2]\n"
        "    W[i, 0:1] = A[i, 0:1]", ["W"]),
}


@pytest.mark.parametrize("name", sorted(SLICE_CASES))
def test_slice_lowering_preserves_numpy_semantics(name):
    """P1/P2: the slice front end (the role of the absent astpass.vector_op_to_loop).  The loop with
    its slice statements runs in NumPy as written; the normalised loop (explicit inner loops, hoisted
    shapes) runs as plain Python; stored arrays must agree (sums to 1e-12: NumPy adds pairwise)."""
    src, stored = SLICE_CASES[name]
    rng = np.random.default_rng(5)
    M, N = 7, 9

    def fresh():
        r = np.random.default_rng(6)
        P = np.array([0, 2, 2, 5, 9, 9, 12, 14])
        return dict(M=M, N=N, alpha=1.5, beta=0.25, np=np, P=P, D=r.standard_normal(14),
                    J=r.integers(0, M, 14), B=r.standard_normal((M, N)), A=r.standard_normal((M, N)),
                    x=r.standard_normal(N), y=np.ones((M, N)), y1=np.zeros(M), y2=np.zeros(M), y3=np.zeros(M),
                    S=r.standard_normal((M, M)), W=np.ones((M, N)))

    ndims = {k: v.ndim for k, v in fresh().items() if isinstance(v, np.ndarray)}
    ir = normalize(src, ndims.get)
    direct, lowered = fresh(), fresh()
    exec(compile(src.split("\n", 1)[1], "<direct>", "exec"), direct)
    for nm in ir.extra_names:
        arr, _shape, dim = nm.rpartition("_shape_")
        lowered[nm] = lowered[arr].shape[int(dim)]
    exec(compile(ast.unparse(ir.loop), "<lowered>", "exec"), lowered)
    for nm in stored:
        assert np.allclose(lowered[nm], direct[nm], rtol=1e-12, atol=1e-13), nm
        assert not np.array_equal(direct[nm], fresh()[nm]), "the case must change the array"


def test_chained_and_subtractive_updates_are_reductions():
    """`s = s + a - b + c`, `s -= a` and `p = p * a * b` are sums / products of a re-associated rest; an
    element update `c[i] = c[i] + a[i] + b[i]` is left exactly as written."""
    ir = normalize("#pragma parallel for simd shared(s)\nfor i in range(n):\n    s[0] = s[0] + a[i] - b[i] + 2.0")
    assert reductions_of(ir.loop) == {"s[0]": "+"} and "s[0] = s[0] + (a[i] - b[i] + 2.0)" in ast.unparse(ir.loop)
    ir = normalize("#pragma parallel for simd shared(s)\nfor i in range(n):\n    s[0] -= a[i]")
    assert reductions_of(ir.loop) == {"s[0]": "+"} and "s[0] = s[0] + -a[i]" in ast.unparse(ir.loop)
    ir = normalize("#pragma parallel for simd shared(p)\nfor i in range(n):\n    p[0] = p[0] * a[i] * b[i]")
    assert reductions_of(ir.loop) == {"p[0]": "*"}
    ir = normalize("#pragma parallel for simd\nfor i in range(n):\n    c[i] = c[i] + a[i] + b[i]")
    assert reductions_of(ir.loop) == {} and "c[i] = c[i] + a[i] + b[i]" in ast.unparse(ir.loop)
    ir = normalize("#pragma parallel for\nfor i in range(n):\n    t = 0.0\n    #pragma simd\n    for j in range(m):\n"
                   "        t = t + abs(A[i, j]) + x[j]\n    y[i] = t", {"A": 2}.get)
    inner = [n for n in ast.walk(ir.loop) if isinstance(n, ast.For) and n is not ir.loop][0]
    assert reductions_of(inner) == {"t": "+"}
