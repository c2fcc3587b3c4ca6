"""A collection of annotated loops of the shapes the reference's integration tests exercise
(elementwise math, 2-D stencils, triangular inner ranges, running minima over a pivot,
normalisations with rowwise reductions, masked accumulation, slice expressions, integer
work, pivot loops on the host around column-strided reductions and updates, stores inside a
reduction loop, diagonal reductions, two reductions of different types per bin, staggered
neighbour updates in a time loop).  The formulas are this repository's own.  Each entry: (function, make_args(rng),
numpy_reference, tolerance)."""
import numpy as np

import appy_b200 as appy  # noqa: F401  (the decorators are applied by the tests)


def option_pricing_like(s, k, t, r, v, call, put):
    #pragma parallel for simd
    for i in range(s.shape[0]):
        d1 = (np.log(s[i] / k[i]) + (r + 0.5 * v * v) * t[i]) / (v * np.sqrt(t[i]))
        d2 = d1 - v * np.sqrt(t[i])
        nd1 = 0.5 + 0.5 * math.erf(d1 / 1.4142135623730951)
        nd2 = 0.5 + 0.5 * math.erf(d2 / 1.4142135623730951)
        disc = np.exp(-r * t[i])
        call[i] = s[i] * nd1 - k[i] * disc * nd2
        put[i] = k[i] * disc * (1.0 - nd2) - s[i] * (1.0 - nd1)


def option_pricing_ref(s, k, t, r, v, call, put):
    from scipy.special import erf
    d1 = (np.log(s / k) + (r + 0.5 * v * v) * t) / (v * np.sqrt(t))
    d2 = d1 - v * np.sqrt(t)
    nd1, nd2 = 0.5 + 0.5 * erf(d1 / np.sqrt(2)), 0.5 + 0.5 * erf(d2 / np.sqrt(2))
    disc = np.exp(-r * t)
    call[:] = s * nd1 - k * disc * nd2
    put[:] = k * disc * (1 - nd2) - s * (1 - nd1)


def stencil2d(T, A, B):
    for t in range(T):
        #pragma parallel for
        for i in range(1, A.shape[0] - 1):
            #pragma simd
            for j in range(1, A.shape[1] - 1):
                B[i, j] = 0.2 * (A[i, j] + A[i, j-1] + A[i, j+1] + A[i+1, j] + A[i-1, j])
        #pragma parallel for
        for i in range(1, A.shape[0] - 1):
            #pragma simd
            for j in range(1, A.shape[1] - 1):
                A[i, j] = 0.2 * (B[i, j] + B[i, j-1] + B[i, j+1] + B[i+1, j] + B[i-1, j])


def stencil2d_ref(T, A, B):
    for t in range(T):
        B[1:-1, 1:-1] = 0.2 * (A[1:-1, 1:-1] + A[1:-1, :-2] + A[1:-1, 2:] + A[2:, 1:-1] + A[:-2, 1:-1])
        A[1:-1, 1:-1] = 0.2 * (B[1:-1, 1:-1] + B[1:-1, :-2] + B[1:-1, 2:] + B[2:, 1:-1] + B[:-2, 1:-1])


def pivot_minimum(D):
    for k in range(D.shape[0]):
        #pragma parallel for
        for i in range(D.shape[0]):
            #pragma simd
            for j in range(D.shape[1]):
                D[i, j] = min(D[i, j], D[i, k] + D[k, j])


def pivot_minimum_ref(D):
    for k in range(D.shape[0]):
        D[:] = np.minimum(D, D[:, k:k + 1] + D[k:k + 1, :])


def triangular_scale_add(alpha, B, A):
    #pragma parallel for
    for j in range(B.shape[1]):
        for i in range(B.shape[0]):
            acc = 0.0
            for k in range(i + 1, B.shape[0]):
                acc += A[k, i] * B[k, j]
            B[i, j] = alpha * (B[i, j] + acc)


def triangular_scale_add_ref(alpha, B, A):
    m = B.shape[0]
    for i in range(m):
        B[i, :] = alpha * (B[i, :] + A[i + 1:, i] @ B[i + 1:, :])


def row_normalise(A, out):
    #pragma parallel for
    for i in range(A.shape[0]):
        nrm = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            nrm += A[i, j] * A[i, j]
        nrm = np.sqrt(nrm)
        #pragma simd
        for j in range(A.shape[1]):
            out[i, j] = A[i, j] / nrm


def row_normalise_ref(A, out):
    out[:] = A / np.sqrt((A * A).sum(axis=1, keepdims=True))


def rank2_update(alpha, beta, C, A, B):
    #pragma parallel for
    for i in range(A.shape[0]):
        C[i, :i + 1] *= beta
        for k in range(A.shape[1]):
            C[i, :i + 1] += A[:i + 1, k] * alpha * B[i, k] + B[:i + 1, k] * alpha * A[i, k]


def rank2_update_ref(alpha, beta, C, A, B):
    for i in range(A.shape[0]):
        C[i, :i + 1] *= beta
        for k in range(A.shape[1]):
            C[i, :i + 1] += A[:i + 1, k] * alpha * B[i, k] + B[:i + 1, k] * alpha * A[i, k]


def masked_bin_mean(data, radius, lo, hi):
    total = 0.0
    count = 0
    #pragma parallel for simd shared(total, count)
    for i in range(data.shape[0]):
        inside = (radius[i] >= lo) and (radius[i] < hi)
        total += data[i] if inside else 0.0
        count += 1 if inside else 0
    return total / max(count, 1)


def masked_bin_mean_ref(data, radius, lo, hi):
    sel = (radius >= lo) & (radius < hi)
    return data[sel].sum() / max(int(sel.sum()), 1)


def axpy_rows_then_matvec(alpha, beta, A, u1, v1, x, y, z):
    #pragma parallel for
    for i in range(A.shape[0]):
        A[i, :] += u1[i] * v1[:]
    #pragma parallel for
    for i in range(A.shape[0]):
        x[i] = x[i] + beta * np.sum(A[:, i] * y[:]) + z[i]


def axpy_rows_then_matvec_ref(alpha, beta, A, u1, v1, x, y, z):
    A += np.outer(u1, v1)
    x += beta * (A.T @ y) + z


def integer_work(idx, out, n):
    #pragma parallel for simd
    for i in range(n):
        q = idx[i] // 7
        r = idx[i] % 7
        out[i] = q * 7 + r + (idx[i] >> 1) - (-idx[i]) // 3 + (-idx[i]) % 5


def integer_work_ref(idx, out, n):
    out[:n] = (idx // 7) * 7 + idx % 7 + (idx >> 1) - (-idx) // 3 + (-idx) % 5


def running_max_abs(a):
    m = 0.0
    lo = 1e300
    #pragma parallel for simd shared(m, lo)
    for i in range(a.shape[0]):
        m = max(m, abs(a[i]))
        lo = min(lo, a[i] * a[i])
    return m, lo


def running_max_abs_ref(a):
    return np.abs(a).max(), (a * a).min()


def orthogonalise_columns(A, w):
    """Host loop over pivots with NumPy statements between the parallel loops; inside, a parallel loop over
    the remaining columns with a column-strided reduction followed by a column-strided update."""
    Q = np.zeros_like(A)
    R = np.zeros((A.shape[1], A.shape[1]), dtype=A.dtype)
    for k in range(A.shape[1]):
        R[k, k] = np.sqrt(np.dot(w * A[:, k], A[:, k]))
        Q[:, k] = A[:, k] / R[k, k]
        #pragma parallel for
        for j in range(k + 1, A.shape[1]):
            s = 0.0
            #pragma simd
            for i in range(A.shape[0]):
                s += w[i] * Q[i, k] * A[i, j]
            #pragma simd
            for i in range(A.shape[0]):
                A[i, j] -= Q[i, k] * s
            R[k, j] = s
    return Q, R


def orthogonalise_columns_ref(A, w):
    Q = np.zeros_like(A)
    R = np.zeros((A.shape[1], A.shape[1]), dtype=A.dtype)
    for k in range(A.shape[1]):
        R[k, k] = np.sqrt(np.dot(w * A[:, k], A[:, k]))
        Q[:, k] = A[:, k] / R[k, k]
        for j in range(k + 1, A.shape[1]):
            s = np.dot(w * Q[:, k], A[:, j])
            A[:, j] -= Q[:, k] * s
            R[k, j] = s
    return Q, R


def symmetric_accumulate(alpha, C, A, B, tmp):
    """Host loop over rows; a parallel loop over columns whose inner simd loop both updates a column of C
    (a store inside the reduction loop) and accumulates a scalar; a host-side slice statement after it."""
    for i in range(C.shape[0]):
        #pragma parallel for
        for j in range(C.shape[1]):
            s = 0.0
            #pragma simd
            for k in range(i):
                C[k, j] += alpha * B[i, j] * A[i, k] - 0.25 * A[k, i]
                s += B[k, j] * A[i, k]
            tmp[j] = s
        C[i, :] += alpha * (B[i, :] * A[i, i] + tmp)


def symmetric_accumulate_ref(alpha, C, A, B, tmp):
    for i in range(C.shape[0]):
        C[:i, :] += alpha * np.outer(A[i, :i], B[i, :]) - 0.25 * A[:i, i:i + 1]
        tmp[:] = A[i, :i] @ B[:i, :]
        C[i, :] += alpha * (B[i, :] * A[i, i] + tmp)


def diagonal_sum_shift(a):
    """A shared reduction over the diagonal of a matrix (stride ncols + 1), then a NumPy expression."""
    acc = 0.0
    #pragma parallel for simd shared(acc)
    for i in range(a.shape[0]):
        acc += np.arctan(a[i, i]) * 0.5
    return a - acc


def diagonal_sum_shift_ref(a):
    return a - 0.5 * np.arctan(np.diag(a)).sum()


def binned_mean(data, radius, nbins, out):
    """A parallel loop over bins; the inner simd loop carries two reductions of different types under a mask."""
    top = radius.max() * 1.0000001
    #pragma parallel for
    for i in range(nbins):
        lo = top * i / nbins
        hi = top * (i + 1) / nbins
        s, cnt = 0.0, 0
        #pragma simd
        for j in range(radius.shape[0]):
            inside = (lo <= radius[j]) & (radius[j] < hi)
            s += data[j] * data[j] if inside else 0.0
            cnt += 1 if inside else 0
        out[i] = s / max(cnt, 1)


def binned_mean_ref(data, radius, nbins, out):
    top = radius.max() * 1.0000001
    for i in range(nbins):
        sel = (top * i / nbins <= radius) & (radius < top * (i + 1) / nbins)
        out[i] = (data[sel] ** 2).sum() / max(int(sel.sum()), 1)


def staggered_fields(T, ex, ey, hz, src):
    """A time loop with a host-side slice statement and three 2-D loops that read neighbours at -1 and +1."""
    for t in range(T):
        ey[0, :] = src[t]
        #pragma parallel for
        for i in range(1, ey.shape[0]):
            #pragma simd
            for j in range(ey.shape[1]):
                ey[i, j] -= 0.4 * (hz[i, j] - hz[i - 1, j])
        #pragma parallel for
        for i in range(ex.shape[0]):
            #pragma simd
            for j in range(1, ex.shape[1]):
                ex[i, j] -= 0.4 * (hz[i, j] - hz[i, j - 1])
        #pragma parallel for
        for i in range(hz.shape[0] - 1):
            #pragma simd
            for j in range(hz.shape[1] - 1):
                hz[i, j] -= 0.6 * (ex[i, j + 1] - ex[i, j] + ey[i + 1, j] - ey[i, j])


def staggered_fields_ref(T, ex, ey, hz, src):
    for t in range(T):
        ey[0, :] = src[t]
        ey[1:, :] -= 0.4 * (hz[1:, :] - hz[:-1, :])
        ex[:, 1:] -= 0.4 * (hz[:, 1:] - hz[:, :-1])
        hz[:-1, :-1] -= 0.6 * (ex[:-1, 1:] - ex[:-1, :-1] + ey[1:, :-1] - ey[:-1, :-1])


def _f(x):
    return np.ascontiguousarray(x)


def cases():
    out = []

    def mk_opt(rng):
        n = 5000
        return (rng.uniform(10, 50, n), rng.uniform(10, 50, n), rng.uniform(1, 2, n), 0.1, 0.2, np.empty(n), np.empty(n))
    out.append(("option_pricing_like", option_pricing_like, option_pricing_ref, mk_opt, (5, 6), 1e-9))

    def mk_st(rng):
        return (3, rng.random((40, 50)), rng.random((40, 50)))
    out.append(("stencil2d", stencil2d, stencil2d_ref, mk_st, (1, 2), 1e-12))

    def mk_piv(rng):
        return (rng.integers(1, 100, (30, 30)).astype(np.float64),)
    out.append(("pivot_minimum", pivot_minimum, pivot_minimum_ref, mk_piv, (0,), 0.0))

    def mk_tri(rng):
        return (1.5, rng.random((24, 17)), rng.random((24, 24)))
    out.append(("triangular_scale_add", triangular_scale_add, triangular_scale_add_ref, mk_tri, (1,), 1e-9))

    def mk_rn(rng):
        return (rng.random((33, 70)) + 0.1, np.empty((33, 70)))
    out.append(("row_normalise", row_normalise, row_normalise_ref, mk_rn, (1,), 1e-12))

    def mk_r2(rng):
        return (1.5, 1.2, rng.random((20, 20)), rng.random((20, 15)), rng.random((20, 15)))
    out.append(("rank2_update", rank2_update, rank2_update_ref, mk_r2, (2,), 1e-12))

    def mk_ax(rng):
        n = 37
        return (1.5, 1.2, rng.random((n, n)), rng.random(n), rng.random(n), np.zeros(n), rng.random(n), rng.random(n))
    out.append(("axpy_rows_then_matvec", axpy_rows_then_matvec, axpy_rows_then_matvec_ref, mk_ax, (2, 5), 1e-12))

    def mk_sym(rng):
        m, n = 19, 23
        return (1.5, rng.random((m, n)), rng.random((m, m)), rng.random((m, n)), np.zeros(n))
    out.append(("symmetric_accumulate", symmetric_accumulate, symmetric_accumulate_ref, mk_sym, (1, 4), 1e-12))

    def mk_bin(rng):
        n = 3000
        return (rng.random(n), rng.random(n) * 7.0, 40, np.zeros(40))
    out.append(("binned_mean", binned_mean, binned_mean_ref, mk_bin, (3,), 1e-12))

    def mk_stag(rng):
        nx, ny, T = 31, 45, 4
        return (T, rng.random((nx, ny)), rng.random((nx, ny)), rng.random((nx, ny)), rng.random(T))
    out.append(("staggered_fields", staggered_fields, staggered_fields_ref, mk_stag, (1, 2, 3), 1e-12))

    def mk_int(rng):
        n = 1000
        return (rng.integers(-500, 500, n).astype(np.int64), np.zeros(n, np.int64), n)
    out.append(("integer_work", integer_work, integer_work_ref, mk_int, (1,), 0.0))
    return out
