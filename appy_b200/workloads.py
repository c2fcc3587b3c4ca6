"""Seeded synthetic inputs for the five benchmark workloads.

The reference's example programs (examples/01-vec_add.py .. examples/06-spmm.py)
draw unseeded ``torch.randn`` data at small sizes; the benchmark configurations fix
sizes, dtypes and distributions instead, and these generators realise them with
``numpy.random.default_rng(seed)``.  Every generator takes a ``scale`` so that tests
can run the same distribution at a fraction of the full size.

    C1  vec_add      a, b ~ U(-1,1) float32, n = 2**24
    C2a sum          A ~ U(0,1) float32, n = 2**26
    C2b masked sum   same A, M ~ Bernoulli(0.5) bool
    C3  SpMV         M = N = 2**20, 16 nnz/row; row lengths Poisson(16) or
                     Zipf(2.0) capped at 4096 with the same total; sorted unique
                     uniform-random columns; int32 indptr/indices; values ~ N(0,1)
                     float32; x ~ U(-1,1) float32
    C4  GEMV         A ~ N(0,1) float32 16384 x 16384 row-major, x ~ U(-1,1)
    C5  SpMM         M = N = 2**18, 32 nnz/row, Zipf(2.0) capped at 8192;
                     B ~ U(-1,1) float32 [N x 128] row-major
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def vec_add(n: int = 1 << 24, seed: int = 0):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, n).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, n).astype(np.float32)
    return a, b


def vec_sum(n: int = 1 << 26, seed: int = 0):
    rng = np.random.default_rng(seed)
    return rng.random(n, dtype=np.float32)


def masked_sum(n: int = 1 << 26, seed: int = 0):
    rng = np.random.default_rng(seed)
    a = rng.random(n, dtype=np.float32)
    m = rng.random(n, dtype=np.float32) < 0.5
    return a, m


@dataclass
class Csr:
    data: np.ndarray      # float32 [nnz]
    indptr: np.ndarray    # int32 [nrows+1]
    indices: np.ndarray   # int32 [nnz]
    shape: tuple

    @property
    def nnz(self) -> int:
        return int(self.indptr[-1])


def poisson_lengths(nrows: int, mean: float, rng) -> np.ndarray:
    return rng.poisson(mean, nrows).astype(np.int64)


def zipf_lengths(nrows: int, total: int, cap: int, rng, a: float = 2.0) -> np.ndarray:
    """Row lengths min(Zipf(a), cap) rescaled by one common factor so that they sum to
    `total`; the rounding residual is spread one unit at a time over random rows that
    have room (below the cap, above zero)."""
    z = np.minimum(rng.zipf(a, nrows).astype(np.float64), float(cap))
    cap = min(cap, max(1, total))
    f = total / z.sum()
    lens = np.minimum(np.floor(z * f), cap)
    for _ in range(60):  # the cap clips, so the factor is refined until the sum settles
        s = lens.sum()
        if abs(s - total) <= nrows:
            break
        f *= total / s
        lens = np.minimum(np.floor(z * f), cap)
    lens = lens.astype(np.int64)
    resid = int(total - lens.sum())
    while resid != 0:
        step = 1 if resid > 0 else -1
        room = np.flatnonzero(lens < cap) if step > 0 else np.flatnonzero(lens > 0)
        take = min(abs(resid), len(room))
        pick = rng.choice(room, size=take, replace=False)
        lens[pick] += step
        resid -= step * take
    return lens


def csr_from_lengths(lens: np.ndarray, ncols: int, rng) -> Csr:
    """Sorted, unique, uniform-random column indices per row; values ~ N(0,1) float32."""
    nrows = len(lens)
    lens = np.minimum(lens, ncols)
    indptr = np.zeros(nrows + 1, dtype=np.int64)
    np.cumsum(lens, out=indptr[1:])
    nnz = int(indptr[-1])
    rows = np.repeat(np.arange(nrows, dtype=np.int64), lens)
    cols = rng.integers(0, ncols, nnz, dtype=np.int64)
    # rows that take a large share of the columns: rejection would not converge, so
    # draw them without replacement one row at a time (there are few of them)
    for r in np.flatnonzero(lens * 8 > ncols):
        cols[indptr[r]:indptr[r + 1]] = rng.choice(ncols, size=int(lens[r]), replace=False)
    key = rows * ncols + cols
    key.sort()
    # duplicates inside a row: redraw them (rare for short rows) until every key is unique
    for _ in range(200):
        dup = np.flatnonzero(key[1:] == key[:-1]) + 1
        if len(dup) == 0:
            break
        r = key[dup] // ncols
        key[dup] = r * ncols + rng.integers(0, ncols, len(dup), dtype=np.int64)
        key.sort(kind="stable")   # nearly sorted already: timsort makes this pass cheap
    else:
        raise RuntimeError("could not make column indices unique")
    indices = (key % ncols).astype(np.int32)
    data = rng.standard_normal(nnz, dtype=np.float32)
    assert indptr[-1] < 2**31
    return Csr(data, indptr.astype(np.int32), indices, (nrows, ncols))


def spmv(nrows: int = 1 << 20, avg: int = 16, kind: str = "poisson", cap: int = 4096, seed: int = 0):
    """Returns (Csr A [nrows x nrows], x).  `kind` is 'poisson' or 'zipf'; the zipf variant
    has the same total non-zero count as the poisson one drawn from the same seed."""
    rng = np.random.default_rng(seed)
    lens = poisson_lengths(nrows, avg, rng)
    if kind == "zipf":
        total = int(lens.sum())
        lens = zipf_lengths(nrows, total, cap, np.random.default_rng(seed + 1))
    elif kind != "poisson":
        raise ValueError(kind)
    A = csr_from_lengths(lens, nrows, rng)
    x = rng.uniform(-1.0, 1.0, nrows).astype(np.float32)
    return A, x


def gemv(n: int = 16384, seed: int = 0):
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((n, n), dtype=np.float32)
    x = rng.uniform(-1.0, 1.0, n).astype(np.float32)
    return np.float32(1.0), A, x


def spmm(nrows: int = 1 << 18, avg: int = 32, cap: int = 8192, ncols_b: int = 128, seed: int = 0):
    """Returns (Csr A [nrows x nrows], B [nrows x ncols_b])."""
    rng = np.random.default_rng(seed)
    lens = zipf_lengths(nrows, nrows * avg, cap, rng)
    A = csr_from_lengths(lens, nrows, rng)
    B = rng.uniform(-1.0, 1.0, (nrows, ncols_b)).astype(np.float32)
    return A, B


# --------------------------------------------------------------------------- byte counts

def bytes_vec_add(n: int) -> int:
    return 3 * 4 * n


def bytes_sum(n: int) -> int:
    return 4 * n


def bytes_masked_sum(n: int) -> int:
    return 5 * n


def bytes_spmv(nrows: int, ncols: int, nnz: int) -> int:
    return 8 * nnz + 4 * (nrows + 1) + 4 * nrows + 4 * ncols


def bytes_gemv(m: int, n: int) -> int:
    return 4 * (m * n + m + n)


def bytes_spmm(nrows: int, nrows_b: int, nnz: int, ncols_b: int) -> tuple[int, int]:
    """(compulsory bytes with an ideal cache, bytes when every B-row gather goes to memory)"""
    primary = 8 * nnz + 4 * (nrows + 1) + 4 * nrows_b * ncols_b + 4 * nrows * ncols_b
    secondary = nnz * (8 + 4 * ncols_b) + 4 * (nrows + 1) + 4 * nrows * ncols_b
    return primary, secondary
