"""float64 NumPy/SciPy statements of the five workloads (oracle; test infrastructure).

Each function cites the reference loop it restates.  Inputs may be any dtype; the
arithmetic is carried out in float64 so the result serves as ground truth for the
stated tolerances.
"""
from __future__ import annotations

import numpy as np


def vec_add(a, b):
    """c[i] = a[i] + b[i] in the operands' own dtype — examples/01-vec_add.py:7-13.
    A single IEEE addition per element: NumPy's result is the bit-exact target."""
    return a + b


def vec_sum(a, init=0.0):
    """b += a[i], b a Python float (float64) — examples/02-vec_sum.py:5-11."""
    return float(init) + float(np.sum(a, dtype=np.float64))


def masked_sum(a, mask, init=0.0):
    """b += a[i] where mask[i] — examples/04-masked_sum.py:7-23 (both forms)."""
    return float(init) + float(np.sum(a[mask.astype(bool)], dtype=np.float64))


def spmv(data, indptr, indices, x, nrows=None):
    """y[i] = sum_k data[k] * x[indices[k]] over k in [indptr[i], indptr[i+1]) —
    examples/03-spmv.py:5-16, tests/integration/triton/tutorial/test_spmv.py:10-21."""
    nrows = len(indptr) - 1 if nrows is None else nrows
    prod = data.astype(np.float64) * x.astype(np.float64)[indices]
    y = np.zeros(nrows, dtype=np.float64)
    lens = np.diff(indptr[: nrows + 1]).astype(np.int64)
    rows = np.repeat(np.arange(nrows), lens)
    lo = int(indptr[0])
    if len(rows):
        y = np.bincount(rows, weights=prod[lo: lo + len(rows)], minlength=nrows).astype(np.float64)
    return y


def spmv_abs(data, indptr, indices, x, nrows=None):
    """Row-wise sum of |data[k] * x[indices[k]]|: the scale of the stated tolerance."""
    return spmv(np.abs(data), indptr, indices, np.abs(x), nrows)


def gemv(alpha, A, x):
    """y[i] = sum_j alpha * A[i, j] * x[j] — examples/05-gemv.py:7-17."""
    return float(alpha) * (A.astype(np.float64) @ x.astype(np.float64))


def gemv_abs(alpha, A, x):
    return abs(float(alpha)) * (np.abs(A).astype(np.float64) @ np.abs(x).astype(np.float64))


def spmm(data, indptr, indices, B, nrows=None):
    """C[i, :] = sum_k data[k] * B[indices[k], :] — examples/06-spmm.py:4-11."""
    import scipy.sparse as sp
    nrows = len(indptr) - 1 if nrows is None else nrows
    A = sp.csr_matrix((data.astype(np.float64), indices, indptr[: nrows + 1]), shape=(nrows, B.shape[0]))
    return np.asarray(A @ B.astype(np.float64))


def spmm_abs(data, indptr, indices, B, nrows=None):
    return spmm(np.abs(data), indptr, indices, np.abs(B), nrows)
