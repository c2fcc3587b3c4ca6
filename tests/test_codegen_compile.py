"""Generated CUDA C compiles with NVRTC for sm_100a (no GPU needed), and the right
template is chosen for each loop shape."""
import math
import types

import numpy as np
import pytest

from appy_b200 import dispatcher
from appy_b200.backends.cuda_sm100 import codegen as cg
from appy_b200.backends.cuda_sm100 import runtime as rt

f32 = np.float32


def build(src, scope, **opts):
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    entry = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), opts)
    args = [v for v in vm.values() if not isinstance(v, types.ModuleType)]
    code = entry.source_for(*args)
    variant = list(entry.variants.values())[0]
    plan = variant.plan
    for trial in range(2):   # default tunables and the last candidate of each
        tun = {k: (v[0] if trial == 0 else v[-1]) for k, v in plan.tunables.items()}
        rt.compile_check(code, "kernel_loop_1", [f"-D{k}={v}" for k, v in tun.items()] + plan.info["nvrtc"])
    return plan, code


A1 = np.ones(1000, f32)
CASES = {
    "vec_add": ("#pragma parallel for simd\nfor i in range(n):\n    c[i] = a[i] + b[i]",
                dict(a=A1, b=A1.copy(), c=A1.copy(), n=1000), "flat", 4),
    "vec_add_f64": ("#pragma parallel for simd\nfor i in range(n):\n    c[i] = a[i] + b[i]",
                    dict(a=np.ones(10), b=np.ones(10), c=np.ones(10), n=10), "flat", 2),
    "sum": ("#pragma parallel for simd shared(b)\nfor i in range(n):\n    b[0] += a[i]",
            dict(a=A1, b=np.array([0.0]), n=1000), "flat", 4),
    "masked_if": ("#pragma parallel for shared(b)\nfor i in range(n):\n    if m[i]:\n        b[0] += a[i]",
                  dict(a=A1, m=np.ones(1000, bool), b=np.array([0.0]), n=1000), "flat", 4),
    "masked_ternary": ("#pragma parallel for simd shared(b)\nfor i in range(n):\n    b[0] += a[i] if m[i] else 0.0",
                       dict(a=A1, m=np.ones(1000, bool), b=np.array([0.0]), n=1000), "flat", 4),
    "max": ("#pragma parallel for simd shared(m)\nfor i in range(n):\n    m[0] = max(m[0], a[i])",
            dict(a=np.ones(10), m=np.array([-np.inf]), n=10), "flat", 2),
    "stencil": ("#pragma parallel for simd\nfor i in range(1, n - 1):\n    B[i] = 0.33333 * (A[i-1] + A[i] + A[i+1])",
                dict(A=np.ones(100), B=np.ones(100), n=100), "flat", 2),
    "pi": ("#pragma parallel for simd shared(sum,step)\nfor i in range(1, num_steps + 1):\n    x = (i - 0.5) * step[0]\n    sum[0] += 4.0 / (1.0 + x * x)",
           dict(sum=np.array([0.0]), step=np.array([1e-6]), num_steps=1000), "flat", 1),
    "var_write": ("#pragma parallel for shared(a)\nfor i in range(10):\n    if i == 3:\n        a[0] = 1",
                  dict(a=np.array([0])), "flat", 1),
    "math": ("#pragma parallel for simd\nfor i in range(n):\n    c[i] = np.exp(a[i]) + math.sqrt(abs(a[i])) + np.tanh(a[i]) ** 2 + min(a[i], 2.0) + a[i] // 3 + a[i] % 2",
             dict(a=A1, c=A1.copy(), n=1000), "flat", 4),
    "mat_add": ("#pragma parallel for\nfor i in range(n):\n    #pragma simd\n    for j in range(m):\n        c[i, j] = a[i, j] + b[i, j]",
                dict(a=np.ones((8, 8)), b=np.ones((8, 8)), c=np.ones((8, 8)), n=8, m=8), "group", 1),
    "rowsum": ("#pragma parallel for\nfor i in range(n):\n    s = 0.0\n    #pragma simd\n    for j in range(m):\n        s += a[i, j]\n    b[i] = s",
               dict(a=np.ones((8, 8)), b=np.ones(8), n=8, m=8), "rowdot", 2),
    "rowmax_seq": ("#pragma parallel for\nfor i in range(n):\n    s = -1e308\n    for j in range(m):\n        s = max(s, a[i, j])\n    b[i] = s",
                   dict(a=np.ones((8, 8)), b=np.ones(8), n=8, m=8), "flat", 2),
    "gemv": ("#pragma parallel for\nfor i in range(n):\n    yi = 0.0\n    #pragma simd\n    for j in range(m):\n        yi += alpha * A[i, j] * x[j]\n    y[i] = yi",
             dict(A=np.ones((64, 64), f32), x=np.ones(64, f32), y=np.ones(64, f32), alpha=1.0, n=64, m=64),
             "rowdot", 4),
    "spmv": ("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    s = 0.0\n    #pragma simd\n    for j in range(start, end):\n        s += D[j] * x[J[j]]\n    y[i] = s",
             dict(D=A1, P=np.zeros(11, np.int32), J=np.zeros(1000, np.int32), x=A1, y=A1.copy(), M=10), "csr", 1),
    "spmm": ("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    y[i, :] = 0\n    for k in range(start, end):\n        y[i, :] += D[k] * B[J[k], :]",
             dict(D=A1, P=np.zeros(11, np.int32), J=np.zeros(1000, np.int32), B=np.ones((10, 128), f32),
                  y=np.ones((10, 128), f32), M=10), "csrdense", 4),
    "spmm_odd": ("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    y[i, :] = 0\n    for k in range(start, end):\n        y[i, :] += D[k] * B[J[k], :]",
                 dict(D=np.ones(10), P=np.zeros(11, np.int64), J=np.zeros(10, np.int64), B=np.ones((10, 37)),
                      y=np.ones((10, 37)), M=10), "csrdense", 1),
    "triangular": ("#pragma parallel for\nfor i in range(n):\n    C[i, :i + 1] *= beta\n    for k in range(m):\n        C[i, :i + 1] += alpha * A[i, k] * A[:i + 1, k]",
                   dict(C=np.ones((8, 8)), A=np.ones((8, 8)), alpha=1.5, beta=1.2, n=8, m=8), "group", 1),
    "np_sum": ("#pragma parallel for\nfor i in range(n):\n    y[i] = np.sum(alpha * A[i, :] * x[:] + beta * B[i, :] * x[:])",
               dict(A=np.ones((8, 8)), B=np.ones((8, 8)), x=np.ones(8), y=np.ones(8), alpha=1.5, beta=1.2, n=8),
               "rowdot", 2),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_generated_cuda_compiles(name):
    src, scope, kind, vec = CASES[name]
    plan, code = build(src, scope)
    assert plan.kind == kind, (plan.kind, code)
    assert plan.vec == vec, (plan.vec, code)
    assert f'extern "C" __global__' in code and "kernel_loop_1" in code


def test_generic_group_lowering_is_available_for_every_template_case():
    for name in ("gemv", "spmv", "spmm", "rowsum"):
        src, scope, _k, _v = CASES[name]
        plan, _code = build(src, scope, _generic_only=True)
        assert plan.kind == "group"


def test_ordered_reduction_uses_the_workspace():
    src, scope, _k, _v = CASES["sum"]
    plan, code = build(src, scope, ordered_reduction=True)
    assert plan.uses_ws and "appy_ws_arrive" in code and "appy_atomic" not in code
    assert plan.params[-1].kind == "ws"


def test_peer_mailbox_combine_compiles_and_is_fused_into_the_reduction_kernel():
    src = ("#pragma parallel for simd shared(b, c)\nfor i in range(n):\n"
           "    b[0] += a[i]\n    c[0] = max(c[0], a[i])")
    plan, code = build(src, dict(a=A1, b=np.array([0.0]), c=np.array([0.0], f32), n=1000), combine="p2p")
    assert plan.uses_ws and [p.kind for p in plan.params][-2:] == ["mb", "seq"]
    assert "appy_p2p_exchange<2>" in code and "appy_p2p_fold<appy_add, double>" in code
    assert "appy_p2p_fold<appy_max, float>" in code


def test_unaligned_or_strided_arrays_fall_back_to_scalar_accesses():
    a = np.ones(1001, f32)[1:]          # 4-byte aligned only: host arrays are mirrored, so still aligned
    t = pytest.importorskip("torch")
    src = "#pragma parallel for simd\nfor i in range(n):\n    c[i] = a[i] + b[i]"
    big = np.ones((10, 7), f32)
    plan, _ = build("#pragma parallel for simd\nfor i in range(n):\n    c[2, i] = a[1, i]",
                    dict(a=big, c=big.copy(), n=7))
    assert plan.vec == 1                 # row stride 7 is not a multiple of the vector width


def test_unknown_function_raises_value_error():
    with pytest.raises(ValueError) as e:
        build("#pragma parallel for simd\nfor i in range(n):\n    c[i] = frobnicate(a[i])", dict(a=A1, c=A1.copy(), n=4))
    assert "Unknown function" in str(e.value)


def test_argument_order_follows_first_use():
    src, scope, _k, _v = CASES["spmv"]
    plan, _ = build(src, scope)
    names = [p.name for p in plan.params]
    assert names[:6] == ["M", "P", "D", "x", "J", "y"] and names[-2:] == ["__lo", "__hi"]


def test_reserved_identifiers_and_builtin_casts():
    build("#pragma parallel for simd\nfor i in range(n):\n    c[i] = float(int(a[i])) + float('inf') * 0.0 if bool(a[i]) else 1.0",
          dict(a=A1, c=A1.copy(), n=4))
    with pytest.raises(NotImplementedError) as e:
        build("#pragma parallel for simd\nfor i in range(n):\n    register = a[i]\n    c[i] = register", dict(a=A1, c=A1.copy(), n=4))
    assert "register" in str(e.value)


def test_row_max_via_slice_reduction():
    plan, code = build("#pragma parallel for\nfor i in range(n):\n    y[i] = np.max(A[i, :]) - np.min(A[i, :])",
                       dict(A=np.ones((8, 8)), y=np.ones(8), n=8))
    assert plan.kind == "group" and "appy_max" in code and "appy_min" in code


def test_row_loop_tunables_follow_the_inner_trip_count_of_each_call():
    """One compiled variant serves short and long rows; the lanes per row must not stick to the first call."""
    A = np.ones((64, 64), f32)
    src = ("#pragma parallel for\nfor i in range(M):\n    s = 0.0\n    #pragma simd\n    for j in range(N):\n"
           "        s += A[i, j] * x[j]\n    y[i] = s")
    scope = dict(A=A, x=np.ones(64, f32), y=np.ones(64, f32), M=64, N=64)
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    entry = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), {})
    entry.source_for(*[v for v in vm.values() if not isinstance(v, types.ModuleType)])
    variant = list(entry.variants.values())[0]
    assert variant.plan.kind == "rowdot"
    short_cls, short = entry._shape_class(variant, dict(scope, N=64), [], 64, 0)
    long_cls, long_ = entry._shape_class(variant, dict(scope, N=16384), [], 16384, 0)
    assert short_cls != long_cls
    assert short["P_G"] in (4, 8, 16) and "P_R" not in short
    assert long_["P_G"] == 0 and long_["P_R"] == 2 and long_["P_MINB"] == 2     # CTA per pair of long rows
    few = entry._shape_class(variant, dict(scope, N=16384), [], 64, 0)[1]
    assert few["P_G"] == 0 and few["P_R"] == 1                                   # few rows: a CTA each
    mid = entry._shape_class(variant, dict(scope, N=2048), [], 100000, 0)[1]
    assert (mid["P_G"], mid["P_BLOCK"], mid["P_U"], mid["P_R"], mid["P_MINB"]) == (32, 128, 8, 2, 1)   # warp per row pair
    # the generic group lowering also sizes its groups from the inner trip
    src2 = "#pragma parallel for\nfor i in range(M):\n    #pragma simd\n    for j in range(N):\n        c[i, j] = A[i, j] + 1.0"
    scope2 = dict(A=A, c=A.copy(), M=64, N=64)
    vm2 = dispatcher.build_val_map(src2, scope2, {"np": np, "math": math})
    e2 = cg.CompiledLoop(src2, "kernel_loop_1", list(vm2), tuple(cg._kind_of(v) for v in vm2.values()), {})
    e2.source_for(*[v for v in vm2.values() if not isinstance(v, types.ModuleType)])
    v2 = list(e2.variants.values())[0]
    assert v2.plan.kind == "group"
    assert e2._shape_class(v2, dict(scope2, N=16), [], 64, 0)[1]["P_G"] == 2      # four packs: two lanes
    assert e2._shape_class(v2, dict(scope2, N=256), [], 64, 0)[1]["P_G"] == 16
    assert e2._shape_class(v2, dict(scope2, N=100000), [], 64, 0)[1]["P_G"] == 0
    # a few very long rows of a perfect nest are cut into column segments; many rows are not
    e2.sm_count = 148
    assert v2.plan.info["splittable"]
    assert e2._shape_class(v2, dict(scope2, N=1 << 20), [], 64, 0)[1]["P_SEG"] == 64
    assert e2._shape_class(v2, dict(scope2, N=1 << 20), [], 8192, 0)[1].get("P_SEG", 1) == 1


def test_shared_reduction_with_inner_simd_loops_uses_the_group_lowering():
    A = np.ones((64, 64), f32)
    src = ("#pragma parallel for shared(s, m)\nfor i in range(M):\n    t = 0.0\n    #pragma simd\n"
           "    for j in range(N):\n        t += A[i, j]\n        m[0] = max(m[0], A[i, j])\n    s[0] += t * w[i]")
    scope = dict(A=A, w=np.ones(64, f32), s=np.array([0.0]), m=np.array([0.0], f32), M=64, N=64)
    plan, code = build(src, scope, _host_cells=False)     # cells mirrored on the device: atomic commit
    assert plan.kind == "group" and "appy_atomic(appy_add()" in code and "appy_atomic(appy_max()" in code
    assert "if (__g.lane == 0) __acc0" in code            # one lane of the group accumulates
    plan, code = build(src, scope, ordered_reduction=True)
    assert plan.uses_ws and "appy_ws_arrive" in code


def test_split_phase_exchange_compiles():
    src = "#pragma parallel for simd\nfor i in range(n):\n    s[0] += a[i]\n    m[0] = max(m[0], a[i])"
    scope = dict(a=A1, s=np.array([0.0]), m=np.array([0.0], f32), n=1000)
    plan, code = build(src, scope, combine="p2p", defer=True)
    assert [p.kind for p in plan.params][-3:] == ["mb", "seq", "pend"]
    # the tail of a CTA is two stores; the exchange is served by one warp at the top of the kernel
    assert "appy_split_publish<double>(__pend.partials, 0," in code and "appy_split_publish<float>(__pend.partials, 1," in code
    body = code.split("struct kernel_loop_1_body")[1]
    assert "appy_ws_arrive" not in body and "appy_p2p_exchange" not in body
    assert body.index("blockIdx.x == gridDim.x - 1 && threadIdx.x < 32) appy_split_service(__mb, __pend);") < body.index("appy_flat<")
    plan, code = build(src, scope, combine="p2p")
    assert "appy_p2p_exchange<2>" in code and "pend" not in [p.kind for p in plan.params]


def test_bulk_copy_variant_of_the_csr_dense_template_compiles():
    spmm = CASES["spmm"] if "spmm" in CASES else None
    assert spmm is not None
    src, scope = spmm[0], spmm[1]
    plan, code = build(src, scope, _bulk_rows=True)
    assert plan.info["template"].endswith("(bulk-copy rows)")
    assert "appy_csr_dense_bulk<" in code and plan.uses_ws and "P_S" in plan.tunables
    grid, block, dyn = plan.launch_config({k: v[0] for k, v in plan.tunables.items()}, 1000, 148)
    assert dyn == 8 * 4 * (plan.info["row_bytes"] + 8) and block == 256


def test_streaming_form_of_the_csr_dense_template_is_a_two_kernel_plan():
    src, scope = CASES["spmm"][0], CASES["spmm"][1]
    plan, code = build(src, scope)
    assert plan.post == "kernel_loop_1_fixup" and "appy_csr_dense_stream<4, 1, P_D, P_WARPS, 128" in code
    assert 'extern "C" __global__ void __launch_bounds__(256) kernel_loop_1_fixup(' in code
    assert [p.kind for p in plan.params].count("scratch") == 1
    tun = {k: v[0] for k, v in plan.tunables.items()}
    assert (tun["P_STREAM"], tun["P_WARPS"], tun["P_D"], tun["P_MINB"]) == (1, 16, 8, 2)
    grid, block, dyn = plan.launch_config(tun, 1 << 18, 148)
    assert (grid, block, dyn) == (148 * 2, 512, 16 * 8 * 512 + 16 * 32 * 4)       # one wave; ring + row tables
    assert plan.post_config(tun, 1 << 18, 148) == (4 * 148, 256)
    workers = 148 * 2 * 16
    assert plan.scratch_bytes(tun, 1 << 18, 148) == (16 + 16 * workers + 255) // 256 * 256 + workers * 2 * 512
    regs = dict(tun, P_RING=0)                  # the ring of rows in flight in registers instead of shared memory
    rt.compile_check(code, "kernel_loop_1", [f"-D{k}={v}" for k, v in regs.items()] + plan.info["nvrtc"])
    assert plan.launch_config(regs, 1 << 18, 148)[2] == 16 * 32 * 4
    tiled = dict(tun, **plan.info["row_tiled"], P_STREAM=0)
    assert plan.post_config(tiled, 100, 148) is None and plan.scratch_bytes(tiled, 100, 148) == 0
    assert plan.launch_config(tiled, 100, 148)[0] == 4                            # a CTA per 32 rows
    # wide float64 rows: fewer rows in flight per warp, fewer CTAs per SM, same shared-memory budget
    wide = dict(scope, B=np.ones((10, 200)), y=np.ones((10, 200)), D=np.ones(1000))
    plan2, _code = build(src, wide)
    t2 = {k: v[0] for k, v in plan2.tunables.items()}
    assert plan2.info["row_bytes_padded"] == 2048 and t2["P_WARPS"] * t2["P_D"] * 2048 <= 64 * 1024
    # small problems keep the row-tiled form
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    e = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), {})
    e.source_for(*[v for v in vm.values() if not isinstance(v, types.ModuleType)])
    v = list(e.variants.values())[0]
    assert e._shape_class(v, {}, [], 1000, 0)[1]["P_STREAM"] == 0
    assert e._shape_class(v, {}, [], 1 << 18, 0)[1] == {}


def test_triangular_inner_ranges_are_sized_by_their_mean_length():
    A = np.ones((64, 64), f32)
    src = "#pragma parallel for\nfor i in range(n):\n    #pragma simd\n    for j in range(0, i + 1):\n        C[i, j] = C[i, j] * 2.0"
    scope = dict(C=A, n=64)
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    e = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), {})
    e.source_for(*[v for v in vm.values() if not isinstance(v, types.ModuleType)])
    v = list(e.variants.values())[0]
    assert e._inner_trip(v.plan, dict(n=8192), 0, 8192) == 4097          # taken at the middle row
    assert e._shape_class(v, dict(n=8192), [], 8192, 0)[1]["P_G"] == 0   # long rows on average: a CTA each
    assert e._shape_class(v, dict(n=40), [], 40, 0)[1]["P_G"] in (2, 4)


def test_csr_row_loop_whose_term_uses_the_row_index():
    """`s += D[j] * x[J[j]] * w[i]`: the CSR template has no row in term(k); the loop takes the row-dot
    template with the row bounds read from indptr."""
    src = ("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    s = 0.0\n    #pragma simd\n"
           "    for j in range(start, end):\n        s = s + D[j] * x[J[j]] * w[i]\n    y[i] = s")
    scope = dict(D=np.ones(9, f32), P=np.array([0, 2, 2, 5, 9], np.int32), J=np.zeros(9, np.int32), x=np.ones(4, f32),
                 w=np.ones(4, f32), y=np.ones(4), M=4)
    plan, code = build(src, scope)
    assert plan.kind == "rowdot" and "w + (i)" in code


def test_scalar_carried_through_a_simd_loop_without_a_reduction_is_refused():
    A = np.ones((8, 8), f32)
    src = ("#pragma parallel for\nfor i in range(M):\n    t = 1.0\n    #pragma simd\n    for j in range(N):\n"
           "        t = t * 0.5 + A[i, j]\n    y[i] = t")          # a recurrence, not a reduction
    with pytest.raises(NotImplementedError) as e:
        build(src, dict(A=A, y=np.ones(8, f32), M=8, N=8))
    assert "carries a value between iterations" in str(e.value)
    ok = ("#pragma parallel for\nfor i in range(M):\n    #pragma simd\n    for j in range(N):\n"
          "        t = A[i, j]\n        t = t * 2.0\n        B[i, j] = t")     # written first in every iteration
    plan, _code = build(ok, dict(A=A, B=A.copy(), M=8, N=8))
    assert plan.kind == "group"


def test_shared_scalar_in_a_host_array_gets_a_cell_in_mapped_host_memory():
    """A reduction-only 1-element NumPy array (what shared(s) becomes) needs no device mirror: the variant uses
    the ordered commit (one read and one write of the cell at the end of the kernel), so the cell can live in
    mapped host memory.  A loop that also reads the array elsewhere, or the option switched off, keeps the
    atomic commit on a mirrored cell."""
    src = "#pragma parallel for simd shared(s)\nfor i in range(n):\n    s[0] += a[i]"
    scope = dict(a=np.ones(100, f32), n=100, s=np.zeros(1))

    def loop(text, sc, **opts):
        vm = dispatcher.build_val_map(text, sc, {"np": np, "math": math})
        e = cg.CompiledLoop(text, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), opts)
        args = [v for v in vm.values() if not isinstance(v, types.ModuleType)]
        return e, e._resolve_arrays(args), e.source_for(*args)

    e, arrays, code = loop(src, scope)
    assert e.cell_names == {"s"} and e._host_cells(arrays) == ("s",)
    assert "appy_ws_arrive" in code and "appy_atomic" not in code
    rt.compile_check(code, "kernel_loop_1", [f"-D{k}={v}" for k, v in list(e.variants.values())[0].tun.items()])
    e, arrays, code = loop(src, scope, _host_cells=False)
    assert e._host_cells(arrays) == () and "appy_atomic" in code
    e, arrays, code = loop(src, scope, distribute=True)
    assert e._host_cells(arrays) == ()
    e, arrays, code = loop(src + "\n    b[i] = s[0]", dict(scope, b=np.ones(100, f32)))
    assert e.cell_names == frozenset() and e._host_cells(arrays) == ()
    big = dict(scope, s=np.zeros(100))          # 800 bytes: an array, not a cell
    e, arrays, code = loop(src, big)
    assert e._host_cells(arrays) == ()
