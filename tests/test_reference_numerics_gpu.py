"""`@jit(fp_contract="triton")`: the numerics of the reference's Triton backend, bit for bit, on loops of
more than one operation.  The kernels on the other side are written here the way the reference generates
them (256-lane programs, masked loads and stores, appy/backends/triton/passes/block_loop.py:77-159,
device_passes/lower_subscripts.py:3-87): a Python float argument arrives as fp32, a float literal is a
float64 scalar tensor (device_passes/lower_constants.py:22-38), `/` on float32 is Triton's own division,
and the compiler may contract a*x+y to one FMA.  The default mode (NumPy's rules) is checked beside it."""
import numpy as np
import pytest

import appy_b200 as appy

torch = pytest.importorskip("torch")
triton = pytest.importorskip("triton")
import triton.language as tl  # noqa: E402

pytestmark = pytest.mark.gpu


@triton.jit
def _t_axpy(alpha, x, y, out, n):
    i = tl.program_id(0) * 256 + tl.arange(0, 256)
    m = i < n
    tl.store(out + i, alpha * tl.load(x + i, mask=m) + tl.load(y + i, mask=m), mask=m)


@triton.jit
def _t_literal_axpy(x, y, out, n):
    i = tl.program_id(0) * 256 + tl.arange(0, 256)
    m = i < n
    tl.store(out + i, tl.full((), 2.5, tl.float64) * tl.load(x + i, mask=m) + tl.load(y + i, mask=m), mask=m)


@triton.jit
def _t_div(x, y, out, n):
    i = tl.program_id(0) * 256 + tl.arange(0, 256)
    m = i < n
    tl.store(out + i, tl.load(x + i, mask=m) / tl.load(y + i, mask=m), mask=m)


@appy.jit(fp_contract="triton")
def r_axpy(alpha, x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = alpha * x[i] + y[i]


@appy.jit(fp_contract="triton")
def r_literal_axpy(x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = 2.5 * x[i] + y[i]


@appy.jit(fp_contract="triton")
def r_div(x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = x[i] / y[i]


@appy.jit
def n_axpy(alpha, x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = alpha * x[i] + y[i]


@appy.jit
def n_div(x, y, out):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        out[i] = x[i] / y[i]


def _inputs(n=100003, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, device="cuda", generator=g) * 37.0
    y = torch.randn(n, device="cuda", generator=g) * 0.01 + 1e-3
    return x, y


def _bits(t):
    return t.view(torch.int32)


def test_reference_mode_matches_the_triton_kernels_bit_for_bit(rt):
    x, y = _inputs()
    n = x.numel()
    grid = ((n + 255) // 256,)
    a, b = torch.empty_like(x), torch.empty_like(x)
    alpha = 1.0 / 3.0
    _t_axpy[grid](alpha, x, y, a, n)
    r_axpy(alpha, x, y, b)
    assert torch.equal(_bits(a), _bits(b))
    _t_literal_axpy[grid](x, y, a, n)
    r_literal_axpy(x, y, b)
    assert torch.equal(_bits(a), _bits(b))
    _t_div[grid](x, y, a, n)
    r_div(x, y, b)
    assert torch.equal(_bits(a), _bits(b))


def test_default_mode_matches_numpy_bit_for_bit_and_differs_from_the_reference_mode(rt):
    x, y = _inputs(seed=1)
    xh, yh = x.cpu().numpy(), y.cpu().numpy()
    out = torch.empty_like(x)
    alpha = 1.0 / 3.0
    n_axpy(alpha, x, y, out)
    assert np.array_equal(out.cpu().numpy(), np.float32(alpha) * xh + yh)      # two roundings, no FMA
    n_div(x, y, out)
    assert np.array_equal(out.cpu().numpy(), xh / yh)                          # IEEE division
    ref = torch.empty_like(x)
    r_axpy(alpha, x, y, ref)
    n_axpy(alpha, x, y, out)
    assert not torch.equal(_bits(ref), _bits(out))       # the FMA rounds once: some elements differ in the last bit
    bound = 1e-6 * ((alpha * x).abs() + y.abs())         # one rounding of the product apart
    assert bool(((ref - out).abs() <= bound).all())
