"""A sample of the device-function table evaluated on the GPU against NumPy / Python integers
(every name's compilation is covered on the CPU by test_device_functions.py)."""
import math

import numpy as np
import pytest

import appy_b200 as appy

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(rt):
    return rt


@appy.jit
def k_float_funcs(a, b, o1, o2, o3, o4, o5, o6):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        o1[i] = np.fma_rn(a[i], b[i], a[i])
        o2[i] = np.ldexp(a[i], 3) + np.hypot(a[i], b[i])
        o3[i] = np.fast_expf(a[i])
        o4[i] = np.ilogb(b[i])
        o5[i] = np.llrint(a[i] * 10.0)
        o6[i] = np.norm3d(a[i], b[i], a[i])


@appy.jit
def k_int_funcs(u, v, o1, o2, o3, o4, o5):
    #pragma parallel for simd
    for i in range(u.shape[0]):
        o1[i] = np.popc(u[i])
        o2[i] = np.clz(v[i])
        o3[i] = np.brev(u[i])
        o4[i] = np.mulhi(v[i], v[i])
        o5[i] = np.float_as_int(np.int_as_float(v[i]))


def test_float_functions():
    rng = np.random.default_rng(0)
    a = rng.uniform(-2, 2, 1000).astype(np.float32)
    b = rng.uniform(0.5, 9, 1000).astype(np.float32)
    o = [np.zeros(1000, np.float32) for _ in range(3)] + [np.zeros(1000, np.int32), np.zeros(1000, np.int64),
                                                          np.zeros(1000, np.float32)]
    k_float_funcs(a, b, *o)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    assert np.array_equal(o[0], (a64 * b64 + a64).astype(np.float32))            # one rounding
    assert np.allclose(o[1], a * 8 + np.hypot(a, b), rtol=1e-6, atol=1e-5)       # the sum can cancel
    assert np.allclose(o[2], np.exp(a), rtol=2e-5)                               # the fast form: a few ulp
    assert np.array_equal(o[3], np.floor(np.log2(b)).astype(np.int32))
    assert np.array_equal(o[4], np.rint((a * np.float32(10.0)).astype(np.float32)).astype(np.int64))
    assert np.allclose(o[5], np.sqrt(2 * a64 * a64 + b64 * b64), rtol=1e-6)


def test_integer_functions():
    rng = np.random.default_rng(1)
    u = rng.integers(0, 2 ** 32, 1000, dtype=np.uint32)
    v = rng.integers(1, 2 ** 31 - 1, 1000, dtype=np.int32)
    o = [np.zeros(1000, np.int32), np.zeros(1000, np.int32), np.zeros(1000, np.uint32), np.zeros(1000, np.int32),
         np.zeros(1000, np.int32)]
    k_int_funcs(u, v, *o)
    assert np.array_equal(o[0], [bin(int(x)).count("1") for x in u])
    assert np.array_equal(o[1], [32 - int(x).bit_length() for x in v])
    assert np.array_equal(o[2], [int(f"{int(x):032b}"[::-1], 2) for x in u])
    assert np.array_equal(o[3], [(int(x) * int(x)) >> 32 for x in v])
    assert np.array_equal(o[4], v)
