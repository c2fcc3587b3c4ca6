"""Generates tests/golden/reference_outputs.npz and reference_facts.json by running the
REFERENCE's own code on CPU.

How: the reference checkout (first command-line argument, or the APPY_REFERENCE_TREE
environment variable) is put on sys.path, the two packages it needs but that are not
installed here (``ast_comments``, ``astpass``) are provided by the stand-ins under
tests/golden/standins/, and Triton runs in interpreter mode (TRITON_INTERPRET=1), so the
reference's decorator, dispatcher, front-end passes, Triton code generator and the generated
Triton kernels all execute unmodified.  Inputs are seeded; outputs are stored as fixtures.

Run from the repository root where the reference checkout exists:
    python tests/golden/make_golden.py <path to the reference checkout>
The tests only read the committed fixtures and never need the checkout.
"""
import hashlib
import json
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(HERE, "standins"))
REFERENCE_TREE = os.path.abspath(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("APPY_REFERENCE_TREE", ""))
if not os.path.isdir(os.path.join(REFERENCE_TREE, "appy")):
    raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
sys.path.insert(0, REFERENCE_TREE)
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import appy  # noqa: E402  (the reference package)
import appy.backends.triton.passes.block_loop as _bl  # noqa: E402
from appy_b200 import workloads as W  # noqa: E402

assert appy.__file__.startswith(REFERENCE_TREE), appy.__file__
_bl.BlockLoop.__init__ = lambda self: setattr(self, "verbose", 0)   # silence the per-compile print

dumps = {}


def jit(name):
    """dump_code=True prints the generated module on the first call; the wrapper captures it.
    (dump_code_to_file cannot be used: on a cache miss the reference rebinds the generated
    function's variable to the dump file object, appy/backends/triton/codegen.py:70-73.)"""
    import contextlib
    import io

    def deco(fn):
        jitted = appy.jit(backend="triton", dump_code=True)(fn)

        def call(*args):
            buf = io.StringIO()
            with contextlib.redirect_stdout(buf):
                res = jitted(*args)
            text = buf.getvalue()
            if "--- Dumped code for loop" in text and name not in dumps:
                body = text.split("--- Dumped code for loop kernel_loop_1 ---", 1)[1]
                dumps[name] = body.split("--- End of dumped code", 1)[0].strip() + "\n"
            return res

        return call

    return deco


@jit("vec_add")
def vec_add(a, b):
    c = np.empty_like(a)
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]
    return c


@jit("vec_sum")
def vec_sum(a):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i]
    return b


@jit("masked_if")
def masked_if(a, mask):
    b = 0.0
    #pragma parallel for shared(b)
    for i in range(a.shape[0]):
        if mask[i]:
            b += a[i]
    return b


@jit("masked_ternary")
def masked_ternary(a, mask):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i] if mask[i] else 0.0
    return b


@jit("spmv")
def spmv(A_data, A_indptr, A_indices, x, M, N):
    y = np.empty(M, dtype=x.dtype)
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s
    return y


@jit("gemv")
def gemv(alpha, A, x):
    y = np.empty(A.shape[0], dtype=x.dtype)
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi
    return y


@jit("spmm")
def spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


@jit("vec_max")
def vec_max(a):
    m = -np.inf
    #pragma parallel for simd shared(m)
    for i in range(a.shape[0]):
        m = max(m, a[i])
    return m


@jit("stencil")
def stencil(A, B):
    #pragma parallel for simd
    for i in range(1, A.shape[0] - 1):
        B[i] = 0.33333 * (A[i-1] + A[i] + A[i+1])
    return B


def main():
    out = {}
    facts = {"generator": "habanero-lab/APPy (the reference checkout), Triton interpreter mode, stand-ins for "
                          "ast_comments and astpass (tests/golden/standins)",
             "pinned": [], "not_pinned": ["spmm (its slice lowering comes from the stand-in, not the reference)"]}
    a, b = W.vec_add(1000, seed=0)
    out["vec_add"] = vec_add(a, b)
    a2, m2 = W.masked_sum(5000, seed=1)
    out["vec_sum"] = np.float64(vec_sum(a2))
    out["masked_if"] = np.float64(masked_if(a2[:600], m2[:600]))
    out["masked_ternary"] = np.float64(masked_ternary(a2, m2))
    out["vec_max"] = np.float64(vec_max(a2))
    A, x = W.spmv(300, 16, kind="poisson", seed=2)
    out["spmv"] = spmv(A.data, A.indptr, A.indices, x, 300, 300)
    Az, xz = W.spmv(200, 16, kind="zipf", cap=64, seed=3)
    out["spmv_zipf"] = spmv(Az.data, Az.indptr, Az.indices, xz, 200, 200)
    al, G, gx = W.gemv(96, seed=4)
    out["gemv"] = gemv(1.0, G, gx)
    As, Bs = W.spmm(40, 6, 32, 16, seed=5)
    ys = np.empty((40, 16), np.float32)
    spmm(As.data, As.indptr, As.indices, Bs, ys, 40)
    out["spmm"] = ys
    S = (np.arange(500, dtype=np.float64) + 2.0) / 500
    out["stencil"] = stencil(S, np.zeros_like(S))
    out["vec_add_f64"] = vec_add(a.astype(np.float64), b.astype(np.float64))
    np.savez_compressed(os.path.join(HERE, "reference_outputs.npz"), **out)
    for name, text in dumps.items():
        facts.setdefault("generated_triton_sha256", {})[name] = hashlib.sha256(text.encode()).hexdigest()
        sig = [l for l in text.splitlines() if l.startswith(f"def kernel_loop_1(")]
        facts.setdefault("host_signature", {})[name] = sig[0] if sig else None
        facts.setdefault("grid", {})[name] = [l.strip() for l in text.splitlines() if l.strip().startswith("grid =")]
        if name != "spmm":
            facts["pinned"].append(name)
    facts["inputs"] = {
        "vec_add": "workloads.vec_add(1000, seed=0)", "vec_sum/masked_ternary/vec_max": "workloads.masked_sum(5000, seed=1)",
        "masked_if": "first 600 elements of workloads.masked_sum(5000, seed=1)",
        "spmv": "workloads.spmv(300, 16, 'poisson', seed=2)", "spmv_zipf": "workloads.spmv(200, 16, 'zipf', cap=64, seed=3)",
        "gemv": "workloads.gemv(96, seed=4), alpha=1.0", "spmm": "workloads.spmm(40, 6, 32, 16, seed=5)",
        "stencil": "(arange(500)+2)/500 float64", "vec_add_f64": "vec_add inputs cast to float64"}
    with open(os.path.join(HERE, "reference_facts.json"), "w") as fh:
        json.dump(facts, fh, indent=1, sort_keys=True)
    print("wrote", sorted(out))


if __name__ == "__main__":
    main()
