"""The device-function table of the code generator (emit.py: MATH1, MATH2, PREDICATES, DEVICE_FUNCS)
against NVRTC: every name compiles for every overload it declares (float32 and float64 where both
exist), without a GPU.  Where a checkout of the reference exists, its table of 198 names
(appy/backends/triton/passes/device_passes/tl_libdevice.py) is read in place and compared: all but
`rcp64h`, which has no CUDA C counterpart, must be known here."""
import math
import os
import re
import types

import numpy as np
import pytest

from appy_b200 import dispatcher
from appy_b200.backends.cuda_sm100 import codegen as cg
from appy_b200.backends.cuda_sm100 import emit
from appy_b200.backends.cuda_sm100 import runtime as rt

NP = {("f", 32): np.float32, ("f", 64): np.float64, ("i", 32): np.int32, ("i", 64): np.int64,
      ("u", 32): np.uint32, ("u", 64): np.uint64}


def _compile(call: str, arrays: dict, out_dtype, **opts):
    src = f"#pragma parallel for simd\nfor i in range(n):\n    out[i] = {call}"
    scope = dict(arrays, out=np.zeros(8, out_dtype), n=8)
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    entry = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()), opts)
    code = entry.source_for(*[v for v in vm.values() if not isinstance(v, types.ModuleType)])
    plan = list(entry.variants.values())[0].plan
    tun = {k: v[0] for k, v in plan.tunables.items()}
    rt.compile_check(code, "kernel_loop_1", [f"-D{k}={v}" for k, v in tun.items()] + plan.info["nvrtc"])
    return code


def _cases():
    for name, over in sorted(emit.DEVICE_FUNCS.items()):
        for args, cuda, res in over:
            yield name, args, cuda, res
    for table, n in ((emit.MATH1, 1), (emit.MATH2, 2)):
        for name, (dname, fname) in sorted(table.items()):
            yield name, (emit.T.F64,) * n, dname, emit.T.F64
            yield name, (emit.T.F32,) * n, fname, emit.T.F32


@pytest.mark.parametrize("name,args,cuda,res", list(_cases()),
                         ids=[f"{n}-{'-'.join(a.c.replace(' ', '_') for a in ar)}" for n, ar, _c, _r in _cases()])
def test_every_overload_compiles(name, args, cuda, res):
    arrays = {f"a{k}": np.ones(8, NP[(t.kind, t.bits)]) for k, t in enumerate(args)}
    call = f"np.{name}(" + ", ".join(f"a{k}[i]" for k in range(len(args))) + ")"
    code = _compile(call, arrays, NP[(res.kind, res.bits)])
    assert cuda + "(" in code, (cuda, code[-600:])


@pytest.mark.parametrize("name", sorted(emit.PREDICATES))
def test_predicates_compile(name):
    for dt in (np.float32, np.float64):
        _compile(f"np.{name}(a0[i])", {"a0": np.ones(8, dt)}, np.bool_)


def test_unknown_function_raises_as_in_the_reference():
    with pytest.raises(ValueError, match="Unknown function: np.rcp64h"):
        _compile("np.rcp64h(a0[i])", {"a0": np.ones(8)}, np.float64)
    with pytest.raises(ValueError, match="Unknown function"):
        _compile("frobnicate(a0[i])", {"a0": np.ones(8)}, np.float64)


def test_reference_numerics_mode_types_and_division():
    """fp_contract="triton": float literals are float64 (device_passes/lower_constants.py:22-38), a Python
    float argument is float32, float32 `/` is div.full.f32, and contraction to FMA is allowed."""
    x = np.ones(8, np.float32)
    code = _compile("2.5 * a0[i] + a1[i]", {"a0": x, "a1": x.copy()}, np.float32, fp_contract="triton")
    assert "(double)" in code                                   # the literal pulls the expression to float64
    code = _compile("2.5 * a0[i] + a1[i]", {"a0": x, "a1": x.copy()}, np.float32)
    assert "(double)" not in code                               # NumPy rules: the literal adopts float32
    code = _compile("a0[i] / a1[i]", {"a0": x, "a1": x.copy()}, np.float32, fp_contract="triton")
    assert "appy_div_full(" in code
    code = _compile("a0[i] / a1[i]", {"a0": np.ones(8), "a1": np.ones(8)}, np.float64, fp_contract="triton")
    assert "appy_div_full(" not in code                         # float64 division stays IEEE
    src = "#pragma parallel for simd\nfor i in range(n):\n    out[i] = alpha * a0[i]"
    scope = dict(a0=x, out=np.zeros(8, np.float32), alpha=1.5, n=8)
    vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
    for mode, want in (("triton", "float alpha"), ("numpy", "double alpha")):
        e = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()),
                            {"fp_contract": mode})
        code = e.source_for(*[v for v in vm.values() if not isinstance(v, types.ModuleType)])
        assert want in code, code[-400:]
        plan = list(e.variants.values())[0].plan
        assert ("--fmad=true" in plan.info["nvrtc"]) == (mode == "triton")


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(os.environ.get("APPY_REFERENCE_TREE") or os.path.join(os.path.dirname(ROOT), "reference"),
                   "appy", "backends", "triton", "passes", "device_passes", "tl_libdevice.py")


@pytest.mark.skipif(not os.path.exists(REF), reason="no checkout of the reference on this machine")
def test_names_of_the_reference_table_are_known():
    names = re.findall(r"^def (\w+)\(", open(REF).read(), re.M)
    assert len(names) == 198
    known = set(emit.DEVICE_FUNCS) | set(emit.MATH1) | set(emit.MATH2) | set(emit.PREDICATES) | {"abs", "fma", "pow"}
    assert [n for n in names if n not in known] == ["rcp64h"]
