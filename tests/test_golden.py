"""Parity against outputs of the reference itself (tests/golden/reference_outputs.npz,
produced by tests/golden/make_golden.py: the reference's own Triton kernels run in
interpreter mode on seeded inputs).

CPU part: the oracle agrees with the reference, which is what makes the oracle a valid
checker at sizes the reference cannot reach.  GPU part: the CUDA path agrees with the
reference directly.  Tolerances: vec_add bit-exact; reductions rtol 1e-5; SpMV / GEMV
|y - ref| <= 1e-5 * sum|a*x| per element; float64 stencil rtol 1e-12.
"""
import json
import os

import numpy as np
import pytest

from appy_b200 import workloads as W
from oracle import c_loops, numpy_oracle as O, python_loops as PL

HERE = os.path.dirname(os.path.abspath(__file__))
G = np.load(os.path.join(HERE, "golden", "reference_outputs.npz"))
FACTS = json.load(open(os.path.join(HERE, "golden", "reference_facts.json")))


def inputs():
    d = {}
    d["a"], d["b"] = W.vec_add(1000, seed=0)
    d["a2"], d["m2"] = W.masked_sum(5000, seed=1)
    d["A"], d["x"] = W.spmv(300, 16, kind="poisson", seed=2)
    d["Az"], d["xz"] = W.spmv(200, 16, kind="zipf", cap=64, seed=3)
    _al, d["G"], d["gx"] = W.gemv(96, seed=4)
    d["As"], d["Bs"] = W.spmm(40, 6, 32, 16, seed=5)
    d["S"] = (np.arange(500, dtype=np.float64) + 2.0) / 500
    return d


D = inputs()


def within(y, ref, scale):
    return np.all(np.abs(np.asarray(y, np.float64) - np.asarray(ref, np.float64)) <= 1e-5 * scale + 1e-30)


# ------------------------------------------------------------------ oracle vs reference (CPU)

def test_oracle_vec_add_is_bit_identical_to_the_reference():
    for ours in (O.vec_add(D["a"], D["b"]), c_loops.vec_add(D["a"], D["b"]), PL.vec_add(D["a"], D["b"])):
        assert np.array_equal(ours, G["vec_add"])
    a64, b64 = D["a"].astype(np.float64), D["b"].astype(np.float64)
    assert np.array_equal(O.vec_add(a64, b64), G["vec_add_f64"])


def test_oracle_reductions_match_the_reference():
    a, m = D["a2"], D["m2"]
    assert np.isclose(O.vec_sum(a), G["vec_sum"], rtol=1e-5, atol=0)
    assert np.isclose(c_loops.vec_sum(a), G["vec_sum"], rtol=1e-5, atol=0)
    assert np.isclose(O.masked_sum(a, m), G["masked_ternary"], rtol=1e-5, atol=0)
    assert np.isclose(c_loops.masked_sum(a, m), G["masked_ternary"], rtol=1e-5, atol=0)
    assert np.isclose(O.masked_sum(a[:600], m[:600]), G["masked_if"], rtol=1e-5, atol=0)
    assert np.isclose(PL.masked_sum_if(a[:600], m[:600]), G["masked_if"], rtol=1e-5, atol=0)
    assert float(a.max()) == float(G["vec_max"])


def test_oracle_spmv_and_gemv_match_the_reference():
    for key, A, x in (("spmv", D["A"], D["x"]), ("spmv_zipf", D["Az"], D["xz"])):
        scale = O.spmv_abs(A.data, A.indptr, A.indices, x)
        assert within(O.spmv(A.data, A.indptr, A.indices, x), G[key], scale)
        assert within(c_loops.spmv(A.data, A.indptr, A.indices, x), G[key], scale)
    scale = O.gemv_abs(1.0, D["G"], D["gx"])
    assert within(O.gemv(1.0, D["G"], D["gx"]), G["gemv"], scale)
    assert within(c_loops.gemv(1.0, D["G"], D["gx"]), G["gemv"], scale)
    assert within(PL.gemv(1.0, D["G"][:8], D["gx"]), G["gemv"][:8], scale[:8])


def test_oracle_stencil_matches_the_reference():
    S = D["S"]
    ref = np.zeros_like(S)
    ref[1:-1] = 0.33333 * (S[:-2] + S[1:-1] + S[2:])
    assert np.allclose(ref, G["stencil"], rtol=1e-12, atol=0)


def test_spmm_fixture_is_consistent_but_not_a_pin():
    As, Bs = D["As"], D["Bs"]
    assert "spmm" not in FACTS["pinned"]
    assert within(O.spmm(As.data, As.indptr, As.indices, Bs), G["spmm"], O.spmm_abs(As.data, As.indptr, As.indices, Bs))


def test_reference_grid_facts():
    # one program per 256-element tile for simd loops, one per iteration otherwise
    assert "(256 - 1)) // 256" in FACTS["grid"]["vec_add"][0]
    assert "(1 - 1)) // 1" in FACTS["grid"]["spmv"][0]
    assert FACTS["host_signature"]["spmv"].startswith("def kernel_loop_1(M, A_indptr, A_data, x, A_indices, y")


# ------------------------------------------------------------------ CUDA path vs reference (GPU)

@pytest.mark.gpu
def test_cuda_path_matches_the_reference_outputs(rt):
    import test_jit_gpu as J
    a, b = D["a"], D["b"]
    c = np.empty_like(a)
    J.k_vec_add(a, b, c)
    assert np.array_equal(c, G["vec_add"])
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    c64 = np.empty_like(a64)
    J.k_vec_add(a64, b64, c64)
    assert np.array_equal(c64, G["vec_add_f64"])
    a2, m2 = D["a2"], D["m2"]
    assert np.isclose(J.k_sum(a2), G["vec_sum"], rtol=1e-5, atol=0)
    assert np.isclose(J.k_masked_ternary(a2, m2), G["masked_ternary"], rtol=1e-5, atol=0)
    assert np.isclose(J.k_masked_if(a2[:600].copy(), m2[:600].copy()), G["masked_if"], rtol=1e-5, atol=0)
    assert J.t_max(a2) == float(G["vec_max"])
    for key, A, x in (("spmv", D["A"], D["x"]), ("spmv_zipf", D["Az"], D["xz"])):
        y = np.empty(A.shape[0], np.float32)
        J.k_spmv(A.data, A.indptr, A.indices, x, y, A.shape[0])
        assert within(y, G[key], O.spmv_abs(A.data, A.indptr, A.indices, x))
    y = np.empty(96, np.float32)
    J.k_gemv(1.0, D["G"], D["gx"], y)
    assert within(y, G["gemv"], O.gemv_abs(1.0, D["G"], D["gx"]))
    S = D["S"]
    A2, B2 = J.jacobi_like(2, S.copy(), np.zeros_like(S))
    assert np.allclose(B2, G["stencil"], rtol=1e-12, atol=0)
