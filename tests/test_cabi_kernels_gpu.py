"""Parity of the prebuilt C-ABI kernels with the CPU oracle (GPU).

Every call goes through libappy_sm100's extern "C" entry points with plain device
pointers; torch only provides device memory.  Tolerances:
  vec_add                 bit-exact (one IEEE float32 addition per element)
  sum / masked sum        rtol 1e-5 against the float64 NumPy sum
  SpMV / GEMV / SpMM      |y - y64| <= 1e-5 * sum_k |a_k * x_k| (+1e-30) per output element
"""
import ctypes as C

import numpy as np
import pytest

from appy_b200 import workloads as W
from oracle import c_loops, numpy_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


def ok(rt, status):
    rt.check(status)


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 255, 1024, 4099, 1 << 20, (1 << 22) + 7])
def test_vec_add_bit_exact(rt, n):
    a, b = W.vec_add(max(n, 1), seed=n)
    a, b = a[:n], b[:n]
    da, db = dev(a), dev(b)
    dc = torch.empty_like(da)
    ok(rt, rt.lib().appy_vec_add_f32(ptr(da), ptr(db), ptr(dc), n, None))
    torch.cuda.synchronize()
    assert np.array_equal(dc.cpu().numpy(), O.vec_add(a, b))
    if 0 < n <= 4099:
        assert np.array_equal(dc.cpu().numpy(), c_loops.vec_add(a, b))


def test_vec_add_unaligned_pointers(rt):
    a, b = W.vec_add(10001, seed=5)
    da, db = dev(a), dev(b)
    dc = torch.zeros(10001, dtype=torch.float32, device="cuda")
    # element offset 1: 4-byte aligned only, exercises the scalar path
    n = 10000
    ok(rt, rt.lib().appy_vec_add_f32(C.c_void_p(da.data_ptr() + 4), C.c_void_p(db.data_ptr() + 4),
                                     C.c_void_p(dc.data_ptr() + 4), n, None))
    torch.cuda.synchronize()
    got = dc.cpu().numpy()
    assert got[0] == 0.0
    assert np.array_equal(got[1:], a[1:] + b[1:])


@pytest.mark.parametrize("ordered", [0, 1])
@pytest.mark.parametrize("n", [0, 1, 7, 1000, 4097, 1 << 20, (1 << 23) + 3])
def test_sum(rt, n, ordered):
    a = W.vec_sum(max(n, 1), seed=n)[:n]
    da = dev(a)
    res = torch.full((1,), 2.5, dtype=torch.float64, device="cuda")
    ok(rt, rt.lib().appy_sum_f32(ptr(da), n, ptr(res), ordered, None))
    torch.cuda.synchronize()
    ref = O.vec_sum(a, init=2.5)
    assert np.isclose(res.item(), ref, rtol=1e-5, atol=0.0)


def test_sum_ordered_is_reproducible(rt):
    a = W.vec_sum(1 << 22, seed=3)
    da = dev(a)
    vals = []
    for _ in range(5):
        res = torch.zeros(1, dtype=torch.float64, device="cuda")
        ok(rt, rt.lib().appy_sum_f32(ptr(da), a.size, ptr(res), 1, None))
        torch.cuda.synchronize()
        vals.append(res.item())
    assert len(set(vals)) == 1


@pytest.mark.parametrize("ordered", [0, 1])
@pytest.mark.parametrize("n", [1, 6, 1000, 4097, (1 << 22) + 1])
def test_masked_sum(rt, n, ordered):
    a, m = W.masked_sum(n, seed=n)
    da, dm = dev(a), dev(m.view(np.uint8))
    res = torch.zeros(1, dtype=torch.float64, device="cuda")
    ok(rt, rt.lib().appy_masked_sum_f32(ptr(da), ptr(dm), n, ptr(res), ordered, None))
    torch.cuda.synchronize()
    assert np.isclose(res.item(), O.masked_sum(a, m), rtol=1e-5, atol=0.0)


def _run_spmv(rt, A, x, strategy, lo=0, hi=None):
    nrows = A.shape[0]
    hi = nrows if hi is None else hi
    d = [dev(A.data), dev(A.indptr), dev(A.indices), dev(x)]
    y = torch.full((nrows,), 777.0, dtype=torch.float32, device="cuda")
    ok(rt, rt.lib().appy_spmv_csr_f32(ptr(d[0]), ptr(d[1]), ptr(d[2]), ptr(d[3]), ptr(y), lo, hi, strategy, None))
    torch.cuda.synchronize()
    return y.cpu().numpy()


def _check_spmv(A, x, y, lo=0, hi=None):
    hi = A.shape[0] if hi is None else hi
    ref = O.spmv(A.data, A.indptr, A.indices, x)
    scale = O.spmv_abs(A.data, A.indptr, A.indices, x)
    err = np.abs(y[lo:hi] - ref[lo:hi])
    assert np.all(err <= 1e-5 * scale[lo:hi] + 1e-30), float((err / (scale[lo:hi] + 1e-30)).max())
    assert np.all(y[:lo] == 777.0) and np.all(y[hi:] == 777.0)


@pytest.mark.parametrize("strategy", [0, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("kind,nrows", [("poisson", 1), ("poisson", 300), ("poisson", 5000),
                                        ("zipf", 5000), ("poisson", 1 << 16), ("zipf", 1 << 16)])
def test_spmv(rt, kind, nrows, strategy):
    A, x = W.spmv(nrows, 16, kind=kind, cap=4096, seed=nrows)
    y = _run_spmv(rt, A, x, strategy)
    _check_spmv(A, x, y)


@pytest.mark.parametrize("strategy", [0, 8])
def test_spmv_empty_and_giant_rows(rt, strategy):
    rng = np.random.default_rng(11)
    nrows = 700
    lens = np.zeros(nrows, dtype=np.int64)
    lens[5] = 20000          # longer than one shared-memory chunk
    lens[6] = 1
    lens[300:310] = 70       # just above the warp-fold threshold
    lens[699] = 9000
    A = W.csr_from_lengths(lens, 40000, rng)
    x = rng.uniform(-1, 1, 40000).astype(np.float32)
    y = _run_spmv(rt, A, x, strategy)
    _check_spmv(A, x, y)
    assert np.all(y[[0, 1, 7, 698]] == 0.0)


@pytest.mark.parametrize("strategy", [0, 4])
def test_spmv_row_range(rt, strategy):
    A, x = W.spmv(3000, 16, seed=9)
    y = _run_spmv(rt, A, x, strategy, lo=1001, hi=2503)
    _check_spmv(A, x, y, lo=1001, hi=2503)


@pytest.mark.parametrize("lanes", [32, 0])
@pytest.mark.parametrize("m,n", [(1, 1), (3, 5), (64, 100), (100, 4096), (257, 1027), (1024, 8192)])
def test_gemv(rt, m, n, lanes):
    rng = np.random.default_rng(m * 131 + n)
    A = rng.standard_normal((m, n), dtype=np.float32)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    alpha = 1.5
    dA, dx = dev(A), dev(x)
    y = torch.empty(m, dtype=torch.float32, device="cuda")
    ok(rt, rt.lib().appy_gemv_f32(C.c_float(alpha), ptr(dA), n, ptr(dx), ptr(y), 0, m, n, lanes, None))
    torch.cuda.synchronize()
    ref, scale = O.gemv(alpha, A, x), O.gemv_abs(alpha, A, x)
    assert np.all(np.abs(y.cpu().numpy() - ref) <= 1e-5 * scale + 1e-30)


def test_gemv_strided_rows_and_range(rt):
    rng = np.random.default_rng(2)
    big = rng.standard_normal((300, 1000), dtype=np.float32)
    A = big[:, :997]                       # lda = 1000, ncols = 997
    x = rng.uniform(-1, 1, 997).astype(np.float32)
    dbig, dx = dev(big), dev(x)
    y = torch.full((300,), -3.0, dtype=torch.float32, device="cuda")
    ok(rt, rt.lib().appy_gemv_f32(C.c_float(1.0), ptr(dbig), 1000, ptr(dx), ptr(y), 10, 290, 997, 32, None))
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    ref, scale = O.gemv(1.0, A, x), O.gemv_abs(1.0, A, x)
    assert np.all(np.abs(got[10:290] - ref[10:290]) <= 1e-5 * scale[10:290] + 1e-30)
    assert np.all(got[:10] == -3.0) and np.all(got[290:] == -3.0)


@pytest.mark.parametrize("nrows,ncols_b,avg,cap", [(1, 128, 4, 8), (200, 128, 8, 64), (3000, 128, 32, 8192),
                                                  (3000, 64, 16, 600), (500, 200, 8, 300), (400, 33, 8, 100),
                                                  (1 << 14, 128, 32, 8192)])
def test_spmm(rt, nrows, ncols_b, avg, cap):
    A, B = W.spmm(nrows, avg, cap, ncols_b, seed=nrows + ncols_b)
    d = [dev(A.data), dev(A.indptr), dev(A.indices), dev(B)]
    Cm = torch.full((nrows, ncols_b), 9.0, dtype=torch.float32, device="cuda")
    ok(rt, rt.lib().appy_spmm_csr_f32(ptr(d[0]), ptr(d[1]), ptr(d[2]), ptr(d[3]), ncols_b, ptr(Cm), ncols_b,
                                      0, nrows, ncols_b, None))
    torch.cuda.synchronize()
    ref = O.spmm(A.data, A.indptr, A.indices, B)
    scale = O.spmm_abs(A.data, A.indptr, A.indices, B)
    err = np.abs(Cm.cpu().numpy() - ref)
    assert np.all(err <= 1e-5 * scale + 1e-30), float((err / (scale + 1e-30)).max())


def _ragged_csr(nrows, ncols, lens, seed):
    rng = np.random.default_rng(seed)
    return W.csr_from_lengths(np.asarray(lens, np.int64), ncols, rng)


@pytest.mark.parametrize("case", ["zipf", "empty_rows", "one_giant_row", "all_empty", "few_nonzeros", "sub_range"])
@pytest.mark.parametrize("ncols_b", [128, 96, 256])
def test_spmm_streaming_form(rt, case, ncols_b):
    """From 4096 rows on appy_spmm_csr_f32 deals the non-zeros out to the warps of one wave of CTAs and
    mends the rows cut by share boundaries in a second kernel: rows without non-zeros, a row that spans
    hundreds of shares, a matrix with fewer non-zeros than warps, and a sub-range of rows."""
    nrows, ncols_a = 6000, 50000
    rng = np.random.default_rng(len(case) + ncols_b)
    if case == "zipf":
        lens = W.zipf_lengths(nrows, nrows * 24, 5000, rng)
    elif case == "empty_rows":
        lens = W.zipf_lengths(nrows, nrows * 8, 2000, rng)
        lens[rng.random(nrows) < 0.6] = 0
        lens[:70] = 0                       # a long run of empty rows at the start, and one at the end
        lens[-45:] = 0
    elif case == "one_giant_row":
        lens = np.full(nrows, 3)
        lens[1234] = 45000                  # spans many warps' shares
        lens[1235] = 0
    elif case == "all_empty":
        lens = np.zeros(nrows, np.int64)
    elif case == "few_nonzeros":
        lens = np.zeros(nrows, np.int64)
        lens[rng.integers(0, nrows, 40)] = 1
    else:
        lens = W.zipf_lengths(nrows + 3000, (nrows + 3000) * 12, 3000, rng)
    A = _ragged_csr(len(lens), ncols_a, lens, 7)
    B = rng.uniform(-1, 1, (ncols_a, ncols_b)).astype(np.float32)
    lo, hi = (1500, 1500 + nrows) if case == "sub_range" else (0, len(lens))
    d = [dev(A.data), dev(A.indptr), dev(A.indices), dev(B)]
    Cm = torch.full((len(lens), ncols_b), 9.0, dtype=torch.float32, device="cuda")
    for _ in range(2):                      # the scratch buffer is reused by the second call
        ok(rt, rt.lib().appy_spmm_csr_f32(ptr(d[0]), ptr(d[1]), ptr(d[2]), ptr(d[3]), ncols_b, ptr(Cm), ncols_b,
                                          lo, hi, ncols_b, None))
    torch.cuda.synchronize()
    got = Cm.cpu().numpy()
    ref = O.spmm(A.data, A.indptr, A.indices, B)
    scale = O.spmm_abs(A.data, A.indptr, A.indices, B)
    err = np.abs(got[lo:hi] - ref[lo:hi])
    assert np.all(err <= 1e-5 * scale[lo:hi] + 1e-30), float((err / (scale[lo:hi] + 1e-30)).max())
    assert np.all(got[:lo] == 9.0) and np.all(got[hi:] == 9.0)        # rows outside the range are not touched


def test_free_of_a_free_or_mirrored_block_is_refused(rt):
    p = rt.malloc(4096)
    rt.free(p)
    with pytest.raises(rt.AppyRuntimeError, match="already free"):
        rt.free(p)
    host = np.ones(1 << 16, np.float32)
    m, _created = rt.mirror(host.ctypes.data, host.nbytes)
    with pytest.raises(rt.AppyRuntimeError, match="mirror of a host range"):
        rt.free(m)
    rt.check(rt.lib().appy_evict(C.c_void_p(host.ctypes.data)))
    q = rt.malloc(4096)                       # the cached block comes back, once
    r = rt.malloc(4096)
    assert q != r
    rt.free(q)
    rt.free(r)


def test_scratch_grows_and_is_kept_per_stream(rt):
    a = rt.scratch(0, 1000)
    assert rt.scratch(0, 500) == a and rt.scratch(0, 1 << 20) == a      # at least 1 MiB from the start
    b = rt.scratch(0, 3 << 20)
    assert rt.scratch(0, 1 << 20) == b
    s1 = rt.stream(1)
    assert rt.scratch(s1, 1000) != b


def test_row_histogram(rt):
    A, _ = W.spmv(10000, 16, kind="zipf", cap=512, seed=4)
    dptr = dev(A.indptr)
    counts, mx = rt.row_histogram(dptr.data_ptr(), 4, A.shape[0])
    lens = np.diff(A.indptr)
    assert mx == lens.max()
    exp = np.zeros(32, dtype=np.int64)
    for L in lens:
        exp[0 if L == 0 else int(L).bit_length()] += 1
    assert counts == exp.tolist()


def test_launch_counter_counts(rt):
    before = rt.launch_count()
    a = torch.ones(1000, device="cuda")
    c = torch.empty_like(a)
    ok(rt, rt.lib().appy_vec_add_f32(ptr(a), ptr(a), ptr(c), 1000, None))
    torch.cuda.synchronize()
    assert rt.launch_count() == before + 1
    assert float(c.sum()) == 2000.0


def test_staged_upload_from_pageable_memory(rt):
    """appy_h2d_staged: chunked upload through the pinned staging buffers (sizes around the 8 MiB chunk)."""
    for nbytes in (1, 4097, (8 << 20) - 1, 8 << 20, (8 << 20) + 5, (20 << 20) + 3):
        h = np.random.default_rng(nbytes % 97).integers(0, 256, nbytes, dtype=np.uint8)
        d = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        rt.h2d_staged(d.data_ptr(), h.ctypes.data, nbytes, 0)
        torch.cuda.synchronize()
        assert np.array_equal(d.cpu().numpy(), h)


def test_mirror_is_reused_and_evicted(rt):
    h = np.arange(1000, dtype=np.float32)
    p1, created1 = rt.mirror(h.ctypes.data, h.nbytes)
    p2, created2 = rt.mirror(h.ctypes.data, h.nbytes)
    assert created1 and not created2 and p1 == p2
    rt.check(rt.lib().appy_evict(C.c_void_p(h.ctypes.data)))
    _p3, created3 = rt.mirror(h.ctypes.data, h.nbytes)
    assert created3
    rt.check(rt.lib().appy_evict(C.c_void_p(h.ctypes.data)))


def test_mirror_cache_is_bounded(rt):
    """More distinct host buffers than the cache holds: old mirrors are dropped, recent ones survive."""
    keep = [np.zeros(16, np.float32) for _ in range(1500)]
    ptrs = []
    for h in keep:
        p, created = rt.mirror(h.ctypes.data, h.nbytes)
        assert created
        ptrs.append(p)
    _p, created_recent = rt.mirror(keep[-1].ctypes.data, keep[-1].nbytes)
    assert not created_recent                       # the newest is still cached
    _p, created_old = rt.mirror(keep[0].ctypes.data, keep[0].nbytes)
    assert created_old                              # the oldest was dropped and is rebuilt
    for h in keep:
        rt.check(rt.lib().appy_evict(C.c_void_p(h.ctypes.data)))
