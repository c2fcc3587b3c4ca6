"""Generic lowering on a zoo of loop shapes.

CPU part (`dry_run=True`): the decoration-time rewrite and the code generator run, the
generated CUDA C compiles with NVRTC for sm_100a, and the plain loop (executed by dry_run)
reproduces the NumPy reference — which validates the references used by the GPU part.
GPU part: the same functions jitted for real agree with NumPy.
"""
import copy
import math
import types

import numpy as np
import pytest

import appy_b200 as appy
import loop_zoo as Z
from appy_b200.backends.cuda_sm100 import codegen as cg
from appy_b200.backends.cuda_sm100 import runtime as rt

Z.math = math
CASES = Z.cases()


def _clone(args):
    return tuple(a.copy() if isinstance(a, np.ndarray) else a for a in args)


def _check(name, fn, ref, mk, outs, tol):
    rng = np.random.default_rng(hash(name) % 1000)
    args = mk(rng)
    a1, a2 = _clone(args), _clone(args)
    fn(*a1)
    ref(*a2)
    for k in outs:
        if tol == 0.0:
            assert np.array_equal(a1[k], a2[k]), (name, k)
        else:
            assert np.allclose(a1[k], a2[k], rtol=tol, atol=tol), (name, k, np.abs(a1[k] - a2[k]).max())


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_zoo_codegen_and_reference_cpu(case):
    name, fn, ref, mk, outs, tol = case
    before = set(cg.code_cache)
    jitted = appy.jit(dry_run=True)(fn)
    _check(name, jitted, ref, mk, outs, max(tol, 1e-9) if tol else 0.0)
    new = [cg.code_cache[k] for k in cg.code_cache if k not in before]
    assert new, "code generation did not run"
    for entry in new:
        for variant in entry.variants.values():
            plan = variant.plan
            tun = {k: v[0] for k, v in plan.tunables.items()}
            rt.compile_check(plan.source, plan.name, [f"-D{k}={v}" for k, v in tun.items()] + plan.info["nvrtc"])


def test_zoo_scalar_results_cpu():
    rng = np.random.default_rng(5)
    data, radius = rng.random(3000), rng.random(3000) * 10
    assert np.isclose(appy.jit(dry_run=True)(Z.masked_bin_mean)(data, radius, 2.0, 5.0),
                      Z.masked_bin_mean_ref(data, radius, 2.0, 5.0))
    a = rng.standard_normal(2000)
    m, lo = appy.jit(dry_run=True)(Z.running_max_abs)(a)
    assert (m, lo) == Z.running_max_abs_ref(a)
    _returned_results(lambda f: appy.jit(dry_run=True)(f), 1e-12)


def _returned_results(jit, tol):
    """Zoo functions that return new arrays instead of writing into their arguments."""
    rng = np.random.default_rng(11)
    A, w = rng.random((30, 12)) + 0.5, rng.random(30) + 0.5
    Q1, R1 = jit(Z.orthogonalise_columns)(A.copy(), w)
    Q2, R2 = Z.orthogonalise_columns_ref(A.copy(), w)
    assert np.allclose(Q1, Q2, rtol=tol, atol=tol) and np.allclose(R1, R2, rtol=tol, atol=tol)
    assert np.allclose((Q1 * w[:, None]).T @ Q1, np.eye(12), atol=1e-9)      # columns orthonormal in the weighted product
    a = rng.standard_normal((50, 50))
    assert np.allclose(jit(Z.diagonal_sum_shift)(a), Z.diagonal_sum_shift_ref(a), rtol=tol, atol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_zoo_gpu(rt_fixture_unused, case):
    name, fn, ref, mk, outs, tol = case
    _check(name, appy.jit(fn), ref, mk, outs, max(tol, 1e-9) if tol else 0.0)


@pytest.fixture
def rt_fixture_unused(rt):
    return rt


@pytest.mark.gpu
def test_zoo_scalar_results_gpu(rt):
    rng = np.random.default_rng(5)
    data, radius = rng.random(300000), rng.random(300000) * 10
    assert np.isclose(appy.jit(Z.masked_bin_mean)(data, radius, 2.0, 5.0),
                      Z.masked_bin_mean_ref(data, radius, 2.0, 5.0), rtol=1e-10)
    a = rng.standard_normal(200000)
    m, lo = appy.jit(Z.running_max_abs)(a)
    assert (m, lo) == Z.running_max_abs_ref(a)
    _returned_results(appy.jit, 1e-10)
