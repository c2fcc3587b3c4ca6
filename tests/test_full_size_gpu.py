"""Parity at the full benchmark sizes (GPU).  The CPU side is the oracle's C port with
OpenMP, which finishes each configuration in about a second; inputs are the seeded
generators of appy_b200/workloads.py.  Tolerances as everywhere else: C1 bit-exact,
C2 rtol 1e-5 against float64, C3/C4/C5 |y - y_ref| <= 1e-5 * sum|a*x| per element, where the
reference rows are accumulated in float64 by NumPy/SciPy for a sample of rows and in float32
by the C port for all rows (the C port's own rounding is covered by the same bound)."""
import numpy as np
import pytest

from appy_b200 import workloads as W
from oracle import c_loops, numpy_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def J(rt):
    import test_jit_gpu
    return test_jit_gpu


def test_c1_full_size_bit_exact(J):
    a, b = W.vec_add()
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dc = torch.empty_like(da)
    J.k_vec_add(da, db, dc)
    got = dc.cpu().numpy()
    assert np.array_equal(got, a + b)
    assert np.array_equal(got, c_loops.vec_add(a, b))


def test_c2_full_size(J):
    a, m = W.masked_sum()
    da, dm = torch.from_numpy(a).cuda(), torch.from_numpy(m).cuda()
    assert np.isclose(J.k_sum(da), O.vec_sum(a), rtol=1e-5, atol=0)
    assert np.isclose(J.k_sum_ordered(da), O.vec_sum(a), rtol=1e-5, atol=0)
    assert np.isclose(J.k_masked_ternary(da, dm), O.masked_sum(a, m), rtol=1e-5, atol=0)
    assert np.isclose(J.k_masked_if(da, dm), O.masked_sum(a, m), rtol=1e-5, atol=0)
    # a checksum identity that needs no oracle: sum(a) == sum(a[mask]) + sum(a[~mask])
    dn = torch.from_numpy(~m).cuda()
    assert np.isclose(J.k_sum(da), J.k_masked_ternary(da, dm) + J.k_masked_ternary(da, dn), rtol=1e-9, atol=0)


@pytest.mark.parametrize("kind", ["poisson", "zipf"])
def test_c3_full_size(J, kind):
    A, x = W.spmv(kind=kind)
    M = A.shape[0]
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, x)]
    dy = torch.full((M,), float("nan"), device="cuda")
    J.k_spmv(d[0], d[1], d[2], d[3], dy, M)
    y = dy.cpu().numpy()
    scale = c_loops.spmv(np.abs(A.data), A.indptr, A.indices, np.abs(x)).astype(np.float64)
    ref32 = c_loops.spmv(A.data, A.indptr, A.indices, x)
    assert np.all(np.abs(y - ref32) <= 2e-5 * scale + 1e-30)          # both sides carry float32 rounding
    ref64 = O.spmv(A.data, A.indptr, A.indices, x)
    assert np.all(np.abs(y - ref64) <= 1e-5 * scale + 1e-30)
    # linearity, a size-independent property: A @ (2x) == 2 (A @ x) exactly in binary floating point
    dy2 = torch.empty(M, device="cuda")
    J.k_spmv(d[0], d[1], d[2], d[3] * 2, dy2, M)
    assert torch.equal(dy2, dy * 2)


def test_c4_full_size(J):
    _al, A, x = W.gemv()
    dA, dx = torch.from_numpy(A).cuda(), torch.from_numpy(x).cuda()
    dy = torch.empty(A.shape[0], device="cuda")
    J.k_gemv(1.0, dA, dx, dy)
    y = dy.cpu().numpy()
    scale = c_loops.gemv(1.0, np.abs(A), np.abs(x)).astype(np.float64)
    assert np.all(np.abs(y - c_loops.gemv(1.0, A, x)) <= 2e-5 * scale + 1e-30)
    x64 = x.astype(np.float64)          # every row against float64, in row blocks (the float64 copy of A is 2 GiB)
    for r0 in range(0, A.shape[0], 2048):
        ref64 = A[r0:r0 + 2048].astype(np.float64) @ x64
        assert np.all(np.abs(y[r0:r0 + 2048] - ref64) <= 1e-5 * scale[r0:r0 + 2048] + 1e-30)
    J.k_gemv(-0.5, dA, dx, dy)
    assert np.allclose(dy.cpu().numpy(), -0.5 * y, rtol=1e-6, atol=1e-6)


def test_c5_full_size(J):
    A, B = W.spmm()
    M = A.shape[0]
    d = [torch.from_numpy(v).cuda() for v in (A.data, A.indptr, A.indices, B)]
    dC = torch.full((M, B.shape[1]), float("nan"), device="cuda")
    J.k_spmm(d[0], d[1], d[2], d[3], dC, M)
    Cg = dC.cpu().numpy()
    scale = c_loops.spmm(np.abs(A.data), A.indptr, A.indices, np.abs(B)).astype(np.float64)
    ref32 = c_loops.spmm(A.data, A.indptr, A.indices, B)
    assert np.all(np.abs(Cg - ref32) <= 2e-5 * scale + 1e-30)
    ref64 = O.spmm(A.data, A.indptr, A.indices, B)
    assert np.all(np.abs(Cg - ref64) <= 1e-5 * scale + 1e-30)
    # column-block independence: the first 64 columns computed alone give the same bits
    dB64 = d[3][:, :64].contiguous()
    dC64 = torch.empty((M, 64), device="cuda")
    J.k_spmm(d[0], d[1], d[2], dB64, dC64, M)
    assert torch.equal(dC64, dC[:, :64])
