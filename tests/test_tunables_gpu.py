"""Every value the autotuner may choose yields the right result.

The autotuner times candidates but does not check them, so each candidate of each tunable of the
five templates and of the group lowering is forced in turn (coordinate-wise around the defaults,
the way the tuner walks) on a small case and compared with the oracle: bit-exact for the
element-wise loop, rtol 1e-5 for the reduction, |y - y64| <= 1e-5 * sum|a*x| for the row kernels.
"""
import numpy as np
import pytest

import appy_b200 as appy
from appy_b200 import workloads as W
from appy_b200.backends.cuda_sm100 import codegen as cg
from oracle import numpy_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@appy.jit
def tn_axpy(alpha, x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = alpha * x[i] + y[i]


@appy.jit
def tn_sum_into(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]


@appy.jit
def tn_gemv(alpha, A, x, y):
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi


@appy.jit
def tn_mat_add(a, b, c):
    #pragma parallel for
    for i in range(a.shape[0]):
        #pragma simd
        for j in range(a.shape[1]):
            c[i, j] = a[i, j] + b[i, j]


@appy.jit
def tn_spmv(A_data, A_indptr, A_indices, x, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s


@appy.jit
def tn_spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


def _walk_candidates(prefix, run, check):
    """Run once to create the variant, then force every candidate of every tunable."""
    run()
    entry = [e for e in cg.code_cache.values() if e.kernel_name.startswith(prefix + "_kernel")][0]
    variant = entry.last_variant
    base = dict(variant.last_tun)
    tried = 0
    try:
        for name, cands in variant.plan.tunables.items():
            for cand in cands:
                variant.forced_tun = dict(base, **{name: cand})
                entry.memo.clear()
                run()
                check(f"{name}={cand}")
                tried += 1
    finally:
        variant.forced_tun = None
        entry.memo.clear()
    assert tried >= sum(len(c) for c in variant.plan.tunables.values())


def test_flat_elementwise_candidates():
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal(70001).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.standard_normal(70001).astype(np.float32)).cuda()
    out = torch.empty_like(x)
    ref = np.float32(1.5) * x.cpu().numpy() + y.cpu().numpy()

    def check(what):
        assert np.array_equal(out.cpu().numpy(), ref), what

    _walk_candidates("tn_axpy", lambda: (out.fill_(-1), tn_axpy(1.5, x, y, out)), check)


def test_flat_reduction_candidates():
    a = W.vec_sum((1 << 18) + 7, seed=2)
    da = torch.from_numpy(a).cuda()
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    ref = float(np.sum(a, dtype=np.float64))

    def check(what):
        assert np.isclose(out.item(), ref, rtol=1e-5, atol=0), what

    _walk_candidates("tn_sum_into", lambda: (out.zero_(), tn_sum_into(da, out)), check)


@pytest.mark.parametrize("shape", [(301, 96), (37, 8192)])          # short rows; long rows (CTA per row pair)
def test_row_dot_candidates(shape):
    rng = np.random.default_rng(shape[0])
    A = rng.standard_normal(shape).astype(np.float32)
    x = rng.uniform(-1, 1, shape[1]).astype(np.float32)
    dA, dx, dy = torch.from_numpy(A).cuda(), torch.from_numpy(x).cuda(), torch.empty(shape[0], device="cuda")
    ref, scale = O.gemv(0.75, A, x), O.gemv_abs(0.75, A, x)

    def check(what):
        assert np.all(np.abs(dy.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30), what

    _walk_candidates("tn_gemv", lambda: (dy.fill_(-1), tn_gemv(0.75, dA, dx, dy)), check)


@pytest.mark.parametrize("shape", [(300, 36), (5, 40004)])          # sub-warp groups; segments of long rows
def test_group_candidates(shape):
    rng = np.random.default_rng(shape[1])
    a = rng.standard_normal(shape).astype(np.float32)
    b = rng.standard_normal(shape).astype(np.float32)
    da, db, dc = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.empty(shape, device="cuda")

    def check(what):
        assert np.array_equal(dc.cpu().numpy(), a + b), what

    _walk_candidates("tn_mat_add", lambda: (dc.fill_(-1), tn_mat_add(da, db, dc)), check)


def test_csr_row_candidates():
    A, x = W.spmv(3000, 20, kind="zipf", cap=1500, seed=4)
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, x)]
    y = torch.empty(A.shape[0], device="cuda")
    ref, scale = O.spmv(A.data, A.indptr, A.indices, x), O.spmv_abs(A.data, A.indptr, A.indices, x)

    def check(what):
        assert np.all(np.abs(y.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30), what

    _walk_candidates("tn_spmv", lambda: (y.fill_(-1), tn_spmv(d[0], d[1], d[2], d[3], y, A.shape[0])), check)


@pytest.mark.parametrize("ncols", [128, 256, 48])                   # one pack per lane; two; ragged columns
def test_csr_dense_candidates(ncols):
    A, B = W.spmm(1500, 24, cap=1200, ncols_b=ncols, seed=6)
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, B)]
    y = torch.empty((A.shape[0], ncols), device="cuda")
    ref, scale = O.spmm(A.data, A.indptr, A.indices, B), O.spmm_abs(A.data, A.indptr, A.indices, B)

    def check(what):
        assert np.all(np.abs(y.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30), what

    _walk_candidates("tn_spmm", lambda: (y.fill_(-1), tn_spmm(d[0], d[1], d[2], d[3], y, A.shape[0])), check)
