"""The kernels the reference's Triton backend generates for the five benchmark loops,
restated by hand so they can be timed on the same GPU (the reference package itself cannot
be imported in this image: ``ast_comments`` and ``astpass`` are missing).

Not part of the product: only ``bench.py`` imports this module, to print the reference's
kernel time beside ours.  Each kernel follows what the reference's passes emit
(appy/backends/triton/passes/): one program per outer iteration, or per 256-element tile
when the parallel loop is also ``simd`` (block_loop.py:77-159); ``num_warps=4``
(host_passes/gen_kernel_launch.py:65); every float literal is a float64 scalar
(device_passes/lower_constants.py:22-38); a shared-scalar reduction is one ``tl.sum`` per
tile followed by ``tl.atomic_add`` on the 1-element float64 array
(device_passes/rewrite_par_reduce_to_atomics.py:10-88); reductions in inner simd loops are
``tl.sum`` of a masked 256-wide tile added to the scalar accumulator
(device_passes/apply_mask_to_reduction.py:3-57); slice statements become 256-wide masked
loads and stores of the row (lower_array_op_to_loop.py:5-22).
"""
import triton
import triton.language as tl

TILE = 256
NUM_WARPS = 4


@triton.jit
def _vec_add(a_shape_0, a, b, c):
    idx = 0 + tl.program_id(0) * 256
    i = idx + tl.arange(0, 256)
    m = idx + tl.arange(0, 256) < a_shape_0
    tl.store(c + i, tl.load(a + i, mask=m) + tl.load(b + i, mask=m), mask=m)


@triton.jit
def _vec_sum(a_shape_0, b, a):
    idx = 0 + tl.program_id(0) * 256
    i = idx + tl.arange(0, 256)
    m = idx + tl.arange(0, 256) < a_shape_0
    tl.atomic_add(b + 0, tl.sum(tl.where(m, tl.load(a + i, mask=m), 0)))


@triton.jit
def _masked_sum_ternary(a_shape_0, b, mask, a):
    idx = 0 + tl.program_id(0) * 256
    i = idx + tl.arange(0, 256)
    m = idx + tl.arange(0, 256) < a_shape_0
    v = tl.where(tl.load(mask + i, mask=m), tl.load(a + i, mask=m), tl.full((), 0.0, dtype=tl.float64))
    tl.atomic_add(b + 0, tl.sum(tl.where(m, v, 0)))


@triton.jit
def _masked_sum_if(a_shape_0, mask, b, a):
    i = 0 + tl.program_id(0) * 1
    if tl.load(mask + i):
        tl.atomic_add(b + 0, tl.load(a + i))


@triton.jit
def _spmv(M, A_indptr, A_data, x, A_indices, y):
    i = 0 + tl.program_id(0) * 1
    start = tl.load(A_indptr + i)
    end = tl.load(A_indptr + (i + 1))
    s = tl.full((), 0.0, dtype=tl.float64)
    for jb in range(start, end, 256):
        j = jb + tl.arange(0, 256)
        m = jb + tl.arange(0, 256) < end
        s = s + tl.sum(tl.where(m, tl.load(A_data + j, mask=m) * tl.load(x + tl.load(A_indices + j, mask=m), mask=m), 0))
    tl.store(y + i, s)


@triton.jit
def _gemv(A_shape_0, A_shape_1, alpha, A, x, y, A_stride_0):
    i = 0 + tl.program_id(0) * 1
    yi = tl.full((), 0.0, dtype=tl.float64)
    for jb in range(0, A_shape_1, 256):
        j = jb + tl.arange(0, 256)
        m = jb + tl.arange(0, 256) < A_shape_1
        yi = yi + tl.sum(tl.where(m, alpha * tl.load(A + (i * A_stride_0 + j), mask=m) * tl.load(x + j, mask=m), 0))
    tl.store(y + i, yi)


@triton.jit
def _spmm(M, A_indptr, y, A_data, B, A_indices, y_shape_1, y_stride_0, B_stride_0):
    i = 0 + tl.program_id(0) * 1
    start = tl.load(A_indptr + i)
    end = tl.load(A_indptr + (i + 1))
    for sb in range(0, y_shape_1, 256):
        s1 = sb + tl.arange(0, 256)
        m1 = sb + tl.arange(0, 256) < y_shape_1
        tl.store(y + (i * y_stride_0 + s1), 0, mask=m1)
    for k in range(start, end, 1):
        for sb in range(0, y_shape_1, 256):
            s2 = sb + tl.arange(0, 256)
            m2 = sb + tl.arange(0, 256) < y_shape_1
            tl.store(y + (i * y_stride_0 + s2),
                     tl.load(y + (i * y_stride_0 + s2), mask=m2)
                     + tl.load(A_data + k) * tl.load(B + (tl.load(A_indices + k) * B_stride_0 + s2), mask=m2),
                     mask=m2)


def vec_add(a, b, c):
    n = a.shape[0]
    _vec_add[((n - 0 + 255) // 256,)](n, a, b, c, num_warps=NUM_WARPS)


def vec_sum(a, b):
    n = a.shape[0]
    _vec_sum[((n - 0 + 255) // 256,)](n, b, a, num_warps=NUM_WARPS)


def masked_sum_ternary(a, mask, b):
    n = a.shape[0]
    _masked_sum_ternary[((n - 0 + 255) // 256,)](n, b, mask, a, num_warps=NUM_WARPS)


def masked_sum_if(a, mask, b):
    n = a.shape[0]
    _masked_sum_if[(n,)](n, mask, b, a, num_warps=NUM_WARPS)


def spmv(A_data, A_indptr, A_indices, x, y, M):
    _spmv[(M,)](M, A_indptr, A_data, x, A_indices, y, num_warps=NUM_WARPS)


def gemv(alpha, A, x, y):
    _gemv[(A.shape[0],)](A.shape[0], A.shape[1], alpha, A, x, y, A.stride(0), num_warps=NUM_WARPS)


def spmm(A_data, A_indptr, A_indices, B, y, M):
    _spmm[(M,)](M, A_indptr, y, A_data, B, A_indices, y.shape[1], y.stride(0), B.stride(0), num_warps=NUM_WARPS)
