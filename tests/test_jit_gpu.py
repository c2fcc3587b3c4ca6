"""End-to-end parity of ``@appy.jit`` loops on the GPU against NumPy/SciPy.

The first block restates the reference's own result tests for this path
(tests/integration/triton/tutorial/*.py and tests/unit/general/**: float64 NumPy
inputs, ``np.allclose`` defaults or atol=1e-6).  The second block runs the five
benchmark loops as written in examples/01..06 at float32 on seeded inputs against the
oracle with the tolerances stated per kernel:
  vec_add: bit-exact; reductions: rtol 1e-5 vs float64;
  SpMV / GEMV / SpMM: |y - y64| <= 1e-5 * sum|a*x| per element.
"""
import numpy as np
import pytest

import appy_b200 as appy
from appy_b200 import workloads as W
from oracle import numpy_oracle as O
from oracle import python_loops as PL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(rt):
    return rt


# =========================================================================== reference tutorial tests

@appy.jit(backend="triton", dump_code=True)
def t_vec_add(a, b):
    c = np.empty_like(a)
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]
    return c


def test_vec_add():
    a = np.ones(100)
    b = np.ones(100)
    assert np.allclose(t_vec_add(a, b), a + b)


@appy.jit(backend="triton", dump_code=True)
def t_mat_add(a, b):
    c = np.empty_like(a)
    #pragma parallel for
    for i in range(a.shape[0]):
        #pragma simd
        for j in range(a.shape[1]):
            c[i, j] = a[i, j] + b[i, j]
    return c


def test_mat_add():
    a = np.random.default_rng(0).random((100, 100))
    b = np.ones((100, 100))
    assert np.allclose(t_mat_add(a, b), a + b)


@appy.jit(backend="triton")
def t_sum(a):
    sum = 0.0
    #pragma parallel for simd shared(sum)
    for i in range(a.shape[0]):
        sum += a[i]
    return sum


@appy.jit(backend="triton")
def t_max(a):
    m = -np.inf
    #pragma parallel for simd shared(m)
    for i in range(a.shape[0]):
        m = max(m, a[i])
    return m


@appy.jit(backend="triton")
def t_min(a):
    m = np.inf
    #pragma parallel for simd shared(m)
    for i in range(a.shape[0]):
        m = min(m, a[i])
    return m


def test_global_reductions():
    a = np.random.default_rng(1).random(1000)
    assert np.allclose(t_sum(a), a.sum())
    assert np.allclose(t_max(a), a.max())
    assert np.allclose(t_min(a), a.min())


@appy.jit(backend="triton")
def t_rowwise_sum(a, b):
    #pragma parallel for
    for i in range(a.shape[0]):
        #pragma simd
        s = 0.0
        for j in range(a.shape[1]):
            s += a[i, j]
        b[i] = s


@appy.jit(backend="triton")
def t_rowwise_max(a, b):
    #pragma parallel for
    for i in range(a.shape[0]):

        s = -1e308
        #pragma simd
        for j in range(a.shape[1]):
            s = max(s, a[i, j])
        b[i] = s


@appy.jit(backend="triton")
def t_rowwise_min(a, b):
    #pragma parallel for
    for i in range(a.shape[0]):

        s = 1e308
        #pragma simd
        for j in range(a.shape[1]):
            s = min(s, a[i, j])
        b[i] = s


def test_rowwise_reductions():
    a = np.random.default_rng(2).random((100, 100))
    b = np.empty(100)
    t_rowwise_sum(a, b)
    assert np.allclose(b, a.sum(axis=1))
    t_rowwise_max(a, b)
    assert np.allclose(b, a.max(axis=1))
    t_rowwise_min(a, b)
    assert np.allclose(b, a.min(axis=1))


@appy.jit(backend="triton", dump_code=True)
def t_spmv(A_data, A_indptr, A_indices, x, M, N):
    y = np.empty(M, dtype=x.dtype)
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s
    return y


def test_spmv_csr_scipy():
    import scipy.sparse as sp
    N = 1000
    A = sp.rand(N, N, density=0.01, format="csr", random_state=3)
    x = np.random.default_rng(3).random(N)
    y = t_spmv(A.data, A.indptr, A.indices, x, N, N)
    assert np.allclose(y, A @ x, atol=1e-6)


@appy.jit(dump_code=True)
def t_pi(num_steps, step):
    sum = 0.0
    #pragma parallel for simd shared(sum,step)
    for i in range(1, num_steps + 1):
        x = (i - 0.5) * step
        sum += 4.0 / (1.0 + x * x)
    return step * sum


def test_pi():
    n = 1_000_000
    got = t_pi(n, 1.0 / n)
    assert np.isclose(got, np.pi, rtol=1e-6, atol=1e-8)


@appy.jit
def t_var_write():
    a = 0
    #pragma parallel for shared(a)
    for i in range(10):
        if i == 3:
            a = 1
    return a


def test_var_write():
    assert t_var_write() == 1


@appy.jit(backend="triton")
def t_irregular(a, b):
    c = np.empty_like(a)
    #pragma parallel for simd
    for i in range(0, a.shape[0], 2):
        c[i] = a[i] + b[i]
    return c


def test_irregular_range_raises_at_first_execution():
    with pytest.raises(Exception) as e:
        t_irregular(np.ones(100), np.ones(100))
    assert "range" in str(e.value) and "step" in str(e.value)


@appy.jit(backend="triton")
def t_bad_pragma(a, b):
    c = np.empty_like(a)
    #pragma parallel for simd my_directive
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]
    return c


@appy.jit(backend="triton")
def t_blank_line_pragma(a, b):
    c = np.empty_like(a)
    #pragma parallel for simd

    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]
    return c


def test_invalid_pragma():
    a, b = np.ones(10), np.ones(10)
    assert np.allclose(t_blank_line_pragma(a, b), a + b)
    with pytest.raises(Exception) as e:
        t_bad_pragma(a, b)
    assert "my_directive" in str(e.value)


def test_unknown_backend_raises():
    @appy.jit(backend="metal")
    def f(a):
        #pragma parallel for simd
        for i in range(a.shape[0]):
            a[i] = 1
        return a

    with pytest.raises(NotImplementedError):
        f(np.zeros(4))


# =========================================================================== semantics of the front end

@appy.jit
def scalars_by_value(a, k):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        a[i] = a[i] + k
        k2 = k + 1
    return k


def test_scalars_are_by_value_and_arrays_in_place():
    a = np.zeros(33)
    assert scalars_by_value(a, 5) == 5
    assert np.all(a == 5)


@appy.jit(dry_run=True)
def dry(a):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        a[i] = a[i] * 2
    return a


def test_dry_run_executes_the_plain_loop():
    assert np.all(dry(np.ones(7)) == 2)


@appy.jit
def jacobi_like(T, A, B):
    for t in range(1, T):
        #pragma parallel for simd
        for i in range(1, A.shape[0] - 1):
            B[i] = 0.33333 * (A[i-1] + A[i] + A[i+1])
        #pragma parallel for simd
        for i in range(1, B.shape[0] - 1):
            A[i] = 0.33333 * (B[i-1] + B[i] + B[i+1])
    return A, B


def test_stencil_inside_a_python_time_loop():
    n = 1000
    A = (np.arange(n) + 2.0) / n
    B = (np.arange(n) + 3.0) / n
    A1, B1 = A.copy(), B.copy()
    for t in range(1, 10):
        B1[1:-1] = 0.33333 * (A1[:-2] + A1[1:-1] + A1[2:])
        A1[1:-1] = 0.33333 * (B1[:-2] + B1[1:-1] + B1[2:])
    A2, B2 = jacobi_like(10, A.copy(), B.copy())
    assert np.allclose(A1, A2, atol=1e-6) and np.allclose(B1, B2, atol=1e-6)


@appy.jit
def slices_np_sum(alpha, beta, A, B, x):
    y = np.empty((A.shape[0],), dtype=x.dtype)
    #pragma parallel for
    for i in range(A.shape[0]):
        y[i] = np.sum(alpha * A[i, :] * x[:] + beta * B[i, :] * x[:])
    return y


@appy.jit
def triangular_update(alpha, beta, C, A):
    #pragma parallel for
    for i in range(A.shape[0]):
        C[i, :i + 1] *= beta
        for k in range(A.shape[1]):
            C[i, :i + 1] += alpha * A[i, k] * A[:i + 1, k]
    return C


def test_slice_expressions():
    rng = np.random.default_rng(4)
    n = 100
    A, B, x = rng.random((n, n)), rng.random((n, n)), rng.random(n)
    assert np.allclose(slices_np_sum(1.5, 1.2, A, B, x), 1.5 * A @ x + 1.2 * B @ x)
    C = rng.random((n, n))
    ref = C.copy()
    for i in range(n):
        ref[i, :i + 1] *= 1.2
        for k in range(n):
            ref[i, :i + 1] += 1.5 * A[i, k] * A[:i + 1, k]
    assert np.allclose(triangular_update(1.5, 1.2, C.copy(), A), ref)


@appy.jit
def trace_tanh(a):
    trace = 0.0
    #pragma parallel for simd shared(trace)
    for i in range(a.shape[0]):
        trace += np.tanh(a[i, i])
    return a + trace


def test_math_functions_and_diagonal_access():
    x = np.random.default_rng(42).random((100, 100))
    assert np.allclose(trace_tanh(x), x + np.tanh(np.diag(x)).sum(), atol=1e-6)


@appy.jit
def int_histogram_total(idx, n):
    total = 0
    #pragma parallel for simd shared(total)
    for i in range(n):
        total += idx[i] % 3
    return total


def test_integer_shared_reduction():
    idx = np.arange(1000, dtype=np.int32)
    assert int_histogram_total(idx, 1000) == int((idx % 3).sum())


@appy.jit
def strided_rows(src, dst):
    #pragma parallel for simd
    for i in range(src.shape[1]):
        dst[1, i] = 2.0 * src[0, i]


def test_noncontiguous_numpy_views_round_trip():
    big = np.arange(60, dtype=np.float64).reshape(6, 10)
    src = big[::2, :7]           # non-contiguous view
    dst_big = np.zeros((4, 9))
    dst = dst_big[:, 1:8]
    strided_rows(src, dst)
    assert np.all(dst[1] == 2.0 * src[0]) and np.all(dst_big[:, 0] == 0) and np.all(dst[0] == 0)


# =========================================================================== the five benchmark loops (float32)

@appy.jit
def k_vec_add(a, b, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]


@appy.jit
def k_sum(a):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i]
    return b


@appy.jit(ordered_reduction=True)
def k_sum_ordered(a):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i]
    return b


@appy.jit
def k_masked_if(a, mask):
    b = 0.0
    #pragma parallel for shared(b)
    for i in range(a.shape[0]):
        if mask[i]:
            b += a[i]
    return b


@appy.jit
def k_masked_ternary(a, mask):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i] if mask[i] else 0.0
    return b


@appy.jit
def k_spmv(A_data, A_indptr, A_indices, x, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s


@appy.jit
def k_gemv(alpha, A, x, y):
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi


@appy.jit
def k_spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


@appy.jit(_generic_only=True)
def k_spmm_generic(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


@appy.jit(_generic_only=True)
def k_spmv_generic(A_data, A_indptr, A_indices, x, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s


@pytest.mark.parametrize("n", [1, 5, 1023, 4096, (1 << 20) + 3])
def test_c1_vec_add_bit_exact_numpy_and_torch(n):
    import torch
    a, b = W.vec_add(n, seed=n)
    c = np.empty_like(a)
    k_vec_add(a, b, c)
    assert np.array_equal(c, a + b)
    if n <= 1023:
        assert np.array_equal(c, PL.vec_add(a, b))      # the reference's CPU semantics: the plain loop
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dc = torch.empty_like(da)
    k_vec_add(da, db, dc)
    assert np.array_equal(dc.cpu().numpy(), a + b)
    # an element offset of 1 leaves the pointer 4-byte aligned: scalar variant
    dc.zero_()
    k_vec_add(da[1:], db[1:], dc[1:])
    assert np.array_equal(dc.cpu().numpy()[1:], (a + b)[1:])


@pytest.mark.parametrize("n", [1, 1000, (1 << 21) + 5])
def test_c2_reductions(n):
    import torch
    a, m = W.masked_sum(n, seed=n)
    assert np.isclose(k_sum(a), O.vec_sum(a), rtol=1e-5, atol=0)
    assert np.isclose(k_sum_ordered(a), O.vec_sum(a), rtol=1e-5, atol=0)
    ref = O.masked_sum(a, m)
    assert np.isclose(k_masked_if(a, m), ref, rtol=1e-5, atol=1e-12)
    assert np.isclose(k_masked_ternary(a, m), ref, rtol=1e-5, atol=1e-12)
    da, dm = torch.from_numpy(a).cuda(), torch.from_numpy(m).cuda()
    assert np.isclose(k_masked_ternary(da, dm), ref, rtol=1e-5, atol=1e-12)
    assert np.isclose(k_sum(da), O.vec_sum(a), rtol=1e-5, atol=0)


def test_c2_ordered_reduction_is_reproducible():
    a = W.vec_sum(1 << 20, seed=9)
    vals = {k_sum_ordered(a) for _ in range(4)}
    assert len(vals) == 1


@pytest.mark.parametrize("kind", ["poisson", "zipf"])
@pytest.mark.parametrize("fn", [k_spmv, k_spmv_generic])
def test_c3_spmv(kind, fn):
    import torch
    A, x = W.spmv(1 << 14, 16, kind=kind, cap=4096, seed=7)
    ref = O.spmv(A.data, A.indptr, A.indices, x)
    scale = O.spmv_abs(A.data, A.indptr, A.indices, x)
    y = np.full(A.shape[0], np.nan, np.float32)
    fn(A.data, A.indptr, A.indices, x, y, A.shape[0])
    assert np.all(np.abs(y - ref) <= 1e-5 * scale + 1e-30)
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, x)]
    dy = torch.empty(A.shape[0], device="cuda")
    fn(d[0], d[1], d[2], d[3], dy, A.shape[0])
    assert np.all(np.abs(dy.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30)


@pytest.mark.parametrize("m,n", [(257, 1027), (512, 4096)])
def test_c4_gemv(m, n):
    rng = np.random.default_rng(m)
    A = rng.standard_normal((m, n), dtype=np.float32)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    y = np.empty(m, np.float32)
    k_gemv(1.0, A, x, y)
    assert np.all(np.abs(y - O.gemv(1.0, A, x)) <= 1e-5 * O.gemv_abs(1.0, A, x) + 1e-30)
    k_gemv(np.float32(0.5), A, x, y)
    assert np.all(np.abs(y - O.gemv(0.5, A, x)) <= 1e-5 * O.gemv_abs(0.5, A, x) + 1e-30)


@pytest.mark.parametrize("fn,nrows,ncols", [(k_spmm, 3000, 128), (k_spmm, 500, 200), (k_spmm, 300, 33),
                                            (k_spmm_generic, 500, 128)])
def test_c5_spmm(fn, nrows, ncols):
    A, B = W.spmm(nrows, 32, 8192, ncols, seed=nrows)
    ref = O.spmm(A.data, A.indptr, A.indices, B)
    scale = O.spmm_abs(A.data, A.indptr, A.indices, B)
    y = np.full((nrows, ncols), np.nan, np.float32)
    fn(A.data, A.indptr, A.indices, B, y, nrows)
    assert np.all(np.abs(y - ref) <= 1e-5 * scale + 1e-30)


@appy.jit(_stream_rows=0)
def k_spmm_streamed(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


@pytest.mark.parametrize("nrows,ncols,dtype,itype", [(3000, 128, np.float32, np.int32), (700, 200, np.float64, np.int64),
                                                    (300, 33, np.float32, np.int32), (40, 64, np.float32, np.int64),
                                                    (5000, 512, np.float32, np.int32)])
def test_c5_spmm_streaming_form_on_small_and_ragged_inputs(nrows, ncols, dtype, itype):
    """The form used from 4096 rows on (non-zeros dealt out to the warps, second kernel for cut and empty
    rows), forced here on inputs of any size: more warps than non-zeros, rows cut by many share
    boundaries, empty rows, column counts that fill no whole 16-byte pack, float64 with int64 indices."""
    A, B = W.spmm(nrows, 24, 4000, ncols, seed=nrows)
    rng = np.random.default_rng(nrows)
    lens = np.diff(A.indptr).astype(np.int64)
    lens[rng.random(nrows) < 0.3] = 0
    A = W.csr_from_lengths(lens, nrows, rng)
    data, B = A.data.astype(dtype), B.astype(dtype)
    ref = O.spmm(data, A.indptr, A.indices, B)
    scale = O.spmm_abs(data, A.indptr, A.indices, B)
    y = np.full((nrows, ncols), np.nan, dtype)
    k_spmm_streamed(data, A.indptr.astype(itype), A.indices.astype(itype), B, y, nrows)
    tol = 1e-5 if dtype == np.float32 else 1e-13
    assert np.all(np.abs(y - ref) <= tol * scale + 1e-30)
    from appy_b200.backends.cuda_sm100 import codegen as cg
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("k_spmm_streamed_")][-1]
    assert entry.last_variant.last_tun["P_STREAM"] == 1 and entry.last_variant.plan.post


@pytest.mark.parametrize("density", [0.0001, 0.001, 0.01, 0.1])
def test_c5_spmm_as_the_reference_example_checks_it(density):
    """The one check the reference holds for this loop (examples/06-spmm.py:30-48): float64
    values, the parts of a torch CSR tensor as arguments (``values()``, ``crow_indices()``,
    ``col_indices()``: int64 indices on the device), a dense operand with 200 columns,
    densities 1e-4 .. 1e-1, ``assert_close(rtol=1e-6, atol=1e-6)`` against ``A @ B``.  The
    matrix side is 2000 here instead of 10000 so that the four cases run in seconds."""
    import torch
    n = 2000
    g = torch.Generator(device="cuda").manual_seed(int(density * 1e6))
    A = torch.randn(n, n, device="cuda", dtype=torch.float64, generator=g)
    mask = torch.rand(n, n, device="cuda", generator=g) < density
    A = (A * mask).to_sparse_csr()
    B = torch.randn(n, 200, device="cuda", dtype=torch.float64, generator=g)
    y_ref = A @ B
    y = torch.full((n, 200), float("nan"), device="cuda", dtype=torch.float64)
    assert A.crow_indices().dtype == torch.int64 and A.col_indices().dtype == torch.int64
    k_spmm(A.values(), A.crow_indices(), A.col_indices(), B, y, n)
    torch.cuda.synchronize()
    torch.testing.assert_close(y, y_ref, rtol=1e-6, atol=1e-6)
    # and against the dense product, so that the check does not rest on one library routine
    torch.testing.assert_close(y, A.to_dense() @ B, rtol=1e-6, atol=1e-6)


def test_small_loops_match_the_plain_python_loops():
    """The reference's CPU execution of the same functions (decorator removed)."""
    A, x = W.spmv(200, 8, seed=1)
    y = np.empty(200, np.float32)
    k_spmv(A.data, A.indptr, A.indices, x, y, 200)
    assert np.allclose(y, PL.spmv(A.data, A.indptr, A.indices, x, 200), rtol=1e-5, atol=1e-6)
    a, m = W.masked_sum(500, seed=2)
    assert np.isclose(k_masked_if(a, m), PL.masked_sum_if(a, m), rtol=1e-5)
    As, B = W.spmm(50, 4, 64, 16, seed=3)
    y2 = np.empty((50, 16), np.float32)
    k_spmm(As.data, As.indptr, As.indices, B, y2, 50)
    assert np.allclose(y2, PL.spmm(As.data, As.indptr, As.indices, B, np.empty((50, 16), np.float32), 50),
                       rtol=1e-5, atol=1e-6)


def test_autotuner_preserves_results():
    @appy.jit(autotune=True)
    def saxpy_inplace(alpha, x, y):
        #pragma parallel for simd
        for i in range(x.shape[0]):
            y[i] = y[i] + alpha * x[i]

    n = 1 << 18
    x = np.ones(n, np.float32)
    y = np.full(n, 2.0, np.float32)
    saxpy_inplace(3.0, x, y)          # tuning runs the kernel repeatedly; y must be updated exactly once
    assert np.all(y == 5.0)
    saxpy_inplace(3.0, x, y)
    assert np.all(y == 8.0)


def test_fp_contract_modes():
    """`fp_contract="numpy"` (default) reproduces NumPy's two roundings of a*x+y bit for bit;
    `fp_contract="triton"` may fuse them (one rounding), as the reference's Triton code does."""
    @appy.jit
    def axpy_np(alpha, x, y, out):
        #pragma parallel for simd
        for i in range(x.shape[0]):
            out[i] = alpha * x[i] + y[i]

    @appy.jit(fp_contract="triton")
    def axpy_fused(alpha, x, y, out):
        #pragma parallel for simd
        for i in range(x.shape[0]):
            out[i] = alpha * x[i] + y[i]

    rng = np.random.default_rng(0)
    x = rng.standard_normal(100000).astype(np.float32)
    y = rng.standard_normal(100000).astype(np.float32)
    alpha = np.float32(1.2345678)
    o1, o2 = np.empty_like(x), np.empty_like(x)
    axpy_np(alpha, x, y, o1)
    axpy_fused(alpha, x, y, o2)
    assert np.array_equal(o1, alpha * x + y)
    fused = (alpha.astype(np.float64) * x.astype(np.float64) + y.astype(np.float64)).astype(np.float32)
    assert np.array_equal(o2, fused)
    assert not np.array_equal(o1, o2)       # the two contracts really differ on this input


def test_kernel_cache_is_reused():
    from appy_b200.backends.cuda_sm100 import codegen as cg
    a, b = W.vec_add(1000)
    c = np.empty_like(a)
    k_vec_add(a, b, c)
    n_entries = len(cg.code_cache)
    k_vec_add(a, b, c)
    assert len(cg.code_cache) == n_entries


def test_conditionally_read_array_may_be_shorter_than_the_range():
    """`a[i] if i < m else 0` must not touch a[] beyond m, also on the 16-byte vector path."""
    @appy.jit
    def guarded(a, m, out):
        #pragma parallel for simd
        for i in range(out.shape[0]):
            out[i] = a[i] * 2.0 if i < m else -1.0

    @appy.jit
    def guarded_sum(a, m, n):
        s = 0.0
        #pragma parallel for simd shared(s)
        for i in range(n):
            if i < m:
                s += a[i]
        return s

    import torch
    for m in (6, 1023, 4096):
        a = torch.arange(m, dtype=torch.float32, device="cuda")
        out = torch.empty(m + 37, dtype=torch.float32, device="cuda")
        guarded(a, m, out)
        exp = np.concatenate([np.arange(m, dtype=np.float32) * 2, -np.ones(37, np.float32)])
        assert np.array_equal(out.cpu().numpy(), exp)
        assert guarded_sum(a, m, m + 37) == float(np.arange(m, dtype=np.float64).sum())


@appy.jit
def few_long_rows_axpy(alpha, x, y):
    #pragma parallel for
    for i in range(x.shape[0]):
        #pragma simd
        for j in range(1, x.shape[1] - 1):
            y[i, j] = alpha * x[i, j] + y[i, j]


def test_perfect_nest_with_few_long_rows_is_cut_into_segments():
    """3 rows of 100003 elements: the row range [1, N-1) is split over many CTAs; every element is
    written exactly once and the two border columns stay untouched."""
    import torch
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (3, 100003)).astype(np.float32)
    y = rng.uniform(-1, 1, (3, 100003)).astype(np.float32)
    ref = y.copy()
    ref[:, 1:-1] = np.float32(0.5) * x[:, 1:-1] + y[:, 1:-1]
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    few_long_rows_axpy(0.5, dx, dy)
    assert np.array_equal(dy.cpu().numpy(), ref)
    from appy_b200.backends.cuda_sm100 import codegen as cg
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("few_long_rows_axpy_")][0]
    assert entry.last_variant.last_tun["P_SEG"] > 1 and entry.last_variant.last_tun["P_G"] == 0


@appy.jit
def weighted_total_and_max(A, w):
    s = 0.0
    m = -1.0e30
    #pragma parallel for shared(s, m)
    for i in range(A.shape[0]):
        t = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            t += A[i, j]
            m = max(m, A[i, j])
        s += t * w[i]
    return s, m


@appy.jit(ordered_reduction=True)
def weighted_total_ordered(A, w):
    s = 0.0
    #pragma parallel for shared(s)
    for i in range(A.shape[0]):
        t = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            t += A[i, j]
        s += t * w[i]
    return s


@pytest.mark.parametrize("shape", [(1000, 37), (37, 5000), (513, 256)])
def test_shared_reduction_on_a_parallel_loop_with_inner_simd_loops(shape):
    """The reference lowers this to one atomic per program
    (device_passes/rewrite_par_reduce_to_atomics.py:10-88); rtol 1e-5 against float64."""
    rng = np.random.default_rng(shape[0])
    A = rng.uniform(0, 1, shape).astype(np.float32)
    w = rng.uniform(0, 1, shape[0]).astype(np.float32)
    ref = float(np.sum(A.astype(np.float64).sum(1) * w.astype(np.float64)))
    s, m = weighted_total_and_max(A, w)
    assert np.isclose(s, ref, rtol=1e-5, atol=0) and m == float(A.max())
    assert np.isclose(weighted_total_ordered(A, w), ref, rtol=1e-5, atol=0)
    assert weighted_total_ordered(A, w) == weighted_total_ordered(A, w)      # scheduling-independent commit


@appy.jit
def five_point_1d(a, b, lo, hi):
    #pragma parallel for simd
    for i in range(lo, hi):
        b[i] = a[i - 2] - 2.0 * a[i - 1] + 4.0 * a[i] - 2.0 * a[i + 1] + a[i + 2]


@appy.jit
def row_of_matrix_stencil(A, b, r):
    #pragma parallel for simd
    for i in range(1, A.shape[1] - 1):
        b[i] = A[r, i + 1] - A[r, i - 1]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("lo,hi", [(2, 100001), (3, 4099), (5, 9)])
def test_neighbour_loads_equal_numpy_bit_for_bit(dtype, lo, hi):
    """Offsets of one and two elements around the vectorised centre pack (float64 packs hold two
    elements, so there only the +-1 offsets ride on the pack); one rounding per operation, so the
    result equals the same NumPy expression exactly."""
    import torch
    rng = np.random.default_rng(lo + hi)
    a = rng.uniform(-1, 1, hi + 2).astype(dtype)
    b = np.full(hi + 2, 7, dtype)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    five_point_1d(da, db, lo, hi)
    ref = b.copy()
    c = np.arange(lo, hi)
    two, four = dtype(2.0), dtype(4.0)
    ref[c] = a[c - 2] - two * a[c - 1] + four * a[c] - two * a[c + 1] + a[c + 2]
    assert np.array_equal(db.cpu().numpy(), ref)
    A = rng.uniform(-1, 1, (3, 1001)).astype(dtype)
    out = np.zeros(1001, dtype)
    dA, dout = torch.from_numpy(A).cuda(), torch.from_numpy(out).cuda()
    row_of_matrix_stencil(dA, dout, 2)
    ref2 = out.copy()
    ref2[1:-1] = A[2, 2:] - A[2, :-2]
    assert np.array_equal(dout.cpu().numpy(), ref2)


@appy.jit(_bulk_rows=True)
def spmm_bulk_rows(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


def test_spmm_with_rows_fetched_by_bulk_copies(rt):
    """The opt-in variant of the CSR x dense template whose B rows arrive through `cp.async.bulk`
    and mbarriers: same result bound as the default kernel, and no wait ran out."""
    import ctypes as C
    import torch
    A, B = W.spmm(3000, 24, cap=2000, seed=5)
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, B)]
    y = torch.full((A.shape[0], B.shape[1]), 7.0, device="cuda")
    spmm_bulk_rows(d[0], d[1], d[2], d[3], y, A.shape[0])
    ref, scale = O.spmm(A.data, A.indptr, A.indices, B), O.spmm_abs(A.data, A.indptr, A.indices, B)
    assert np.all(np.abs(y.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30)
    from appy_b200.backends.cuda_sm100 import codegen as cg
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("spmm_bulk_rows_")][0]
    assert entry.last_variant.plan.info["template"].endswith("(bulk-copy rows)")
    status = np.zeros(1, np.uint32)
    stream = torch.cuda.current_stream().cuda_stream
    rt.d2h(status.ctypes.data, rt.workspace(stream) + 8, 4, stream)
    rt.sync(stream)
    assert status[0] == 0


@appy.jit
def host_axpy(alpha, x, y):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        y[i] = alpha * x[i] + y[i]


@appy.jit
def host_shift(src, dst):
    #pragma parallel for simd
    for i in range(dst.shape[0]):
        dst[i] = src[i] + 1.0


def test_repeated_calls_with_host_arrays_reuse_the_launch_record_safely():
    """Calls with NumPy arguments are memoised by layout; what the record assumed is checked again on
    every call: other arrays of the same shape, the same array passed twice (overlap), a strided view."""
    rng = np.random.default_rng(21)
    for trial in range(4):                                   # same shapes, different buffers and values
        x = rng.uniform(-1, 1, 5001).astype(np.float32)
        y = rng.uniform(-1, 1, 5001).astype(np.float32)
        ref = np.float32(0.5) * x + y
        host_axpy(0.5, x, y)
        assert np.array_equal(y, ref)
    z = rng.uniform(-1, 1, 5001).astype(np.float32)
    ref = np.float32(0.5) * z + z
    host_axpy(0.5, z, z)                                     # x and y are the same buffer
    assert np.array_equal(z, ref)
    big = rng.uniform(-1, 1, 10002).astype(np.float32)
    xv, yv = big[0::2], big[1::2].copy()                     # a strided host view takes the copying path
    ref = np.float32(0.5) * xv + yv
    host_axpy(0.5, xv, yv)
    assert np.array_equal(yv, ref)
    buf = rng.uniform(-1, 1, 6000).astype(np.float32)        # overlapping, shifted views of one buffer
    a, b = buf[:5001].copy(), np.empty(5001, np.float32)
    host_shift(a, b)
    host_shift(a, b)
    assert np.array_equal(b, a + np.float32(1.0))
    src, dst = buf[0:5001], buf[500:5501]
    expect = src.copy() + np.float32(1.0)
    host_shift(src, dst)                                     # a record exists for this layout; the overlap is seen
    assert np.array_equal(dst, expect)


@appy.jit
def rows_window_update(a, b, c, lo, hi):
    #pragma parallel for
    for i in range(a.shape[0]):
        #pragma simd
        for j in range(lo, hi):
            c[i, j] = 2.0 * a[i, j] - b[i, j] + c[i, j]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape,lo,hi", [((7, 40), 0, 40), ((7, 40), 1, 39), ((5, 64), 3, 10), ((5, 64), 9, 9),
                                         ((3, 100004), 1, 100003), ((300, 36), 2, 35), ((4, 37), 0, 37)])
def test_inner_simd_loops_with_packs_and_ragged_ends(dtype, shape, lo, hi):
    """Inner simd loops of the group lowering move 16-byte packs where whole aligned chunks lie inside
    [lo, hi) and run element-wise at the ragged ends (and everywhere when rows are not 16-byte
    aligned, as for 37 columns); elements outside the window stay untouched.  Bit-exact vs NumPy."""
    import torch
    rng = np.random.default_rng(shape[1] + lo)
    a = rng.uniform(-1, 1, shape).astype(dtype)
    b = rng.uniform(-1, 1, shape).astype(dtype)
    c = rng.uniform(-1, 1, shape).astype(dtype)
    ref = c.copy()
    ref[:, lo:hi] = dtype(2.0) * a[:, lo:hi] - b[:, lo:hi] + c[:, lo:hi]
    da, db, dc = (torch.from_numpy(v).cuda() for v in (a, b, c))
    rows_window_update(da, db, dc, lo, hi)
    assert np.array_equal(dc.cpu().numpy(), ref)


def test_to_gpu_uploads_numpy_arrays_with_the_runtime_copy_path():
    """appy.to_gpu (appy/__init__.py: to_gpu) returns torch CUDA tensors; NumPy inputs go through the
    runtime's pinned path and the host array may be changed right after the call returns."""
    import torch
    rng = np.random.default_rng(9)
    for trial in range(3):                            # the third upload of the same buffer is pinned DMA
        a = rng.standard_normal(1 << 19).astype(np.float32) if trial == 0 else a
        expect = a.copy()
        d = appy.to_gpu(a)
        a += 1.0                                      # the copy has completed
        assert d.is_cuda and d.dtype == torch.float32 and np.array_equal(d.cpu().numpy(), expect)
    m = rng.random((7, 5)) < 0.5
    strided = rng.standard_normal((64, 10))[:, ::2]
    dm, ds, k = appy.to_gpu(m, strided, 3)
    assert dm.dtype == torch.bool and np.array_equal(dm.cpu().numpy(), m)
    assert np.array_equal(ds.cpu().numpy(), strided) and k == 3
    assert appy.to_gpu(np.zeros((0, 4), np.float64)).shape == (0, 4)
    back = appy.to_cpu(ds)
    assert isinstance(back, np.ndarray) and np.array_equal(back, strided)


@appy.jit
def relax_through(path, k):
    #pragma parallel for
    for i in range(path.shape[0]):
        #pragma simd
        for j in range(path.shape[1]):
            path[i, j] = min(path[i, j], path[i, k] + path[k, j])


@appy.jit
def scale_prefix(x, alpha, m):
    #pragma parallel for simd
    for i in range(m):
        x[i] = alpha * x[i]


def test_scalars_that_only_feed_the_arithmetic_share_one_launch_record():
    """`k` changes on every call of a Floyd-Warshall sweep and `alpha` on every scaling, but neither
    shapes the launch: one record serves all values (the value is patched into the arguments); `m`
    bounds the range, so every value of `m` has its own record."""
    import torch
    from appy_b200.backends.cuda_sm100 import codegen as cg
    rng = np.random.default_rng(17)
    n = 48
    d = rng.uniform(1, 10, (n, n))
    np.fill_diagonal(d, 0.0)
    ref = d.copy()
    for k in range(n):
        ref = np.minimum(ref, ref[:, k:k + 1] + ref[k:k + 1, :])
    dp = torch.from_numpy(d).cuda()
    for k in range(n):
        relax_through(dp, k)
    assert np.allclose(dp.cpu().numpy(), ref, rtol=1e-12, atol=0)
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("relax_through_")][0]
    assert len(entry.memo) == 1

    x = torch.ones(1000, dtype=torch.float64, device="cuda")
    expect = np.ones(1000)
    for alpha, m in ((2.0, 1000), (0.5, 1000), (3.0, 10), (1.5, 10), (-1.0, 1000)):
        scale_prefix(x, alpha, m)
        expect[:m] *= alpha
    assert np.array_equal(x.cpu().numpy(), expect)
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("scale_prefix_")][0]
    assert len(entry.memo) == 2                      # m = 1000 and m = 10


@appy.jit
def k_axpy_host(alpha, x, y):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        y[i] = alpha * x[i] + y[i]


def test_resident_host_arrays_are_uploaded_once_and_again_after_touch():
    """`appy.resident(a)`: the array's device mirror is trusted until `appy.touch(a)`; without it every call
    uploads every NumPy argument (what the reference's generated host code does on every call)."""
    import ctypes as C
    from appy_b200.backends.cuda_sm100 import codegen as cg, runtime as rtm
    n = 1 << 16
    x = np.arange(n, dtype=np.float32)
    y = np.ones(n, np.float32)
    cg.transfer_stats.update(h2d=0, d2h=0)
    k_axpy_host(2.0, x, y)
    k_axpy_host(2.0, x, y)
    assert cg.transfer_stats == {"h2d": 4 * 4 * n, "d2h": 2 * 4 * n}          # both arrays, both calls
    assert np.array_equal(y, 1 + 4 * x)
    appy.resident(x, y)
    cg.transfer_stats.update(h2d=0, d2h=0)
    k_axpy_host(1.0, x, y)                      # first use after the declaration: uploaded, then trusted
    k_axpy_host(1.0, x, y)
    k_axpy_host(1.0, x, y)
    assert cg.transfer_stats == {"h2d": 2 * 4 * n, "d2h": 3 * 4 * n}          # y still comes back every time
    assert np.array_equal(y, 1 + 7 * x)
    x[:] = 1.0                                  # a host write ...
    appy.touch(x)                               # ... that the caller reports
    cg.transfer_stats.update(h2d=0, d2h=0)
    k_axpy_host(1.0, x, y)
    assert cg.transfer_stats["h2d"] == 4 * n and np.array_equal(y, 2 + 7 * np.arange(n, dtype=np.float32))
    # a mirror that was dropped in between is filled again without being asked
    rtm.check(rtm.lib().appy_evict(C.c_void_p(x.ctypes.data)))
    cg.transfer_stats.update(h2d=0, d2h=0)
    k_axpy_host(1.0, x, y)
    assert cg.transfer_stats["h2d"] == 4 * n and np.array_equal(y, 3 + 7 * np.arange(n, dtype=np.float32))
    appy.release(x, y)
    cg.transfer_stats.update(h2d=0, d2h=0)
    k_axpy_host(1.0, x, y)
    assert cg.transfer_stats["h2d"] == 2 * 4 * n


@appy.jit
def k_cells_three(a, n):
    s = 0.0
    hi = -1.0e30
    cnt = 0
    #pragma parallel for simd shared(s, hi, cnt)
    for i in range(n):
        s += a[i]
        hi = max(hi, a[i])
        cnt += 1
    return s, hi, cnt


@appy.jit
def k_cell_and_stored_array(a, b, n):
    s = 1.5
    #pragma parallel for simd shared(s)
    for i in range(n):
        b[i] = a[i] * 2.0
        s += a[i]
    return s


@appy.jit(_host_cells=False)
def k_cells_mirrored(a, n):
    s = 0.0
    #pragma parallel for simd shared(s)
    for i in range(n):
        s += a[i]
    return s


@appy.jit
def k_two_cells_into(a, o1, o2):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        o1[0] += a[i]
        o2[0] += 2.0 * a[i]


def test_shared_scalars_live_in_mapped_host_memory():
    """shared(...) scalars reach the kernel as cells in the device's page of mapped host memory: no mirror, no
    copy call; the kernel reads the initial value and writes the result itself (ordered commit).  Same values
    as with mirrored cells; several cells per loop, float and integer, next to an ordinary stored NumPy array,
    from the launch record as well as on first sight."""
    import torch
    from appy_b200.backends.cuda_sm100 import codegen as cg
    rng = np.random.default_rng(5)
    for n in (1, 1000, 100_000, 3_000_001):
        a = rng.standard_normal(n).astype(np.float32)
        da = torch.from_numpy(a).cuda()
        for _rep in range(3):                       # first sight, then the launch record
            s, hi, cnt = k_cells_three(da, n)
            assert cnt == n and hi == a.max()
            assert abs(s - float(a.sum(dtype=np.float64))) <= 1e-6 * float(np.abs(a).sum(dtype=np.float64)) + 1e-12
        assert abs(k_cells_mirrored(da, n) - s) <= 1e-6 * float(np.abs(a).sum(dtype=np.float64)) + 1e-12
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith("k_cells_three_")][0]
    assert entry.cell_names == {"s", "hi", "cnt"}
    assert "appy_ws_arrive" in entry.last_variant.plan.source and "appy_atomic" not in entry.last_variant.plan.source
    mirrored = [e for e in cg.code_cache.values() if e.kernel_name.startswith("k_cells_mirrored_")][0]
    assert "appy_atomic" in mirrored.last_variant.plan.source
    a_last = da.cpu().numpy()
    a_dev_sum = a_last.sum(dtype=np.float64)
    # NumPy inputs: the array is mirrored and comes back by a copy, the cell does not
    a = rng.standard_normal(5000).astype(np.float32)
    b = np.zeros(5000, np.float32)
    cg.transfer_stats.update(h2d=0, d2h=0)
    for _rep in range(2):
        s = k_cell_and_stored_array(a, b, 5000)
        assert np.array_equal(b, a * 2) and abs(s - 1.5 - float(a.sum(dtype=np.float64))) < 1e-3
    assert cg.transfer_stats == {"h2d": 2 * (4 * 5000 + 8), "d2h": 2 * (4 * 5000 + 8)}     # b is only written
    # an empty range leaves the cells as they were
    assert k_cells_three(da, 0) == (0.0, -1.0e30, 0)
    # one host array under two names: both reductions land in the same cell, as with a mirror
    o = np.zeros(1)
    k_two_cells_into(da, o, o)
    assert abs(o[0] - 3.0 * float(a_dev_sum)) <= 1e-6 * float(np.abs(a_last).sum(dtype=np.float64))


@appy.jit
def k_overwrite_all(a, b, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]


@appy.jit
def k_overwrite_part(a, c, n):
    #pragma parallel for simd
    for i in range(n):
        c[i] = a[i] * 2.0


@appy.jit
def k_overwrite_some(a, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        if a[i] > 0.0:
            c[i] = a[i]


def test_an_array_that_is_overwritten_in_full_is_not_uploaded():
    """A NumPy array that the loop never reads and stores in every element (`c[i] = ...` at the top level, over
    the whole array) is not uploaded first; a partial range or a conditional store still uploads it, so the
    elements the loop leaves alone come back unchanged."""
    from appy_b200.backends.cuda_sm100 import codegen as cg
    n = 10_000
    rng = np.random.default_rng(11)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    for _rep in range(2):                           # full path, then the launch record
        c = np.full(n, 7.0, np.float32)
        cg.transfer_stats.update(h2d=0, d2h=0)
        k_overwrite_all(a, b, c)
        assert np.array_equal(c, a + b)
        assert cg.transfer_stats == {"h2d": 2 * 4 * n, "d2h": 4 * n}
    for m in (n, n // 2, 0):
        c = np.full(n, 7.0, np.float32)
        cg.transfer_stats.update(h2d=0, d2h=0)
        k_overwrite_part(a, c, m)
        assert np.array_equal(c[:m], a[:m] * 2) and np.all(c[m:] == 7.0)
        assert cg.transfer_stats["h2d"] == (4 * n if m == n else 2 * 4 * n)
    c = np.full(n, 7.0, np.float32)
    k_overwrite_some(a, c)
    assert np.array_equal(c, np.where(a > 0, a, np.float32(7.0)))
