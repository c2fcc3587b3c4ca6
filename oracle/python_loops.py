"""The annotated loops as the reference executes them on the CPU (oracle; test
infrastructure).  These are the example kernels with the decorator removed — the
reference's documented debug mode ("Comment this line to run the function in the
Python interpreter", examples/02-vec_sum.py:5) and what ``dry_run`` executes
(appy/dispatcher.py:46-53).  Interpreted Python: use small sizes.
"""
from __future__ import annotations

import numpy as np


def vec_add(a, b):
    """examples/01-vec_add.py:7-13"""
    c = np.empty_like(a)
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]
    return c


def vec_sum(a):
    """examples/02-vec_sum.py:5-11"""
    b = 0.0
    for i in range(a.shape[0]):
        b += a[i]
    return b


def masked_sum_if(a, mask):
    """examples/04-masked_sum.py:7-14 (control-flow form)"""
    b = 0.0
    for i in range(a.shape[0]):
        if mask[i]:
            b += a[i]
    return b


def masked_sum_ternary(a, mask):
    """examples/04-masked_sum.py:17-23 (ternary form)"""
    b = 0.0
    for i in range(a.shape[0]):
        b += a[i] if mask[i] else 0.0
    return b


def spmv(A_data, A_indptr, A_indices, x, M):
    """examples/03-spmv.py:5-16"""
    y = np.empty(M, dtype=x.dtype)
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i + 1]
        s = 0.0
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s
    return y


def gemv(alpha, A, x):
    """examples/05-gemv.py:7-17"""
    y = np.empty(A.shape[0], dtype=x.dtype)
    for i in range(A.shape[0]):
        yi = 0.0
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi
    return y


def spmm(A_data, A_indptr, A_indices, B, y, M):
    """examples/06-spmm.py:4-11"""
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i + 1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]
    return y
