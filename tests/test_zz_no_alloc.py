"""appy_sum_f32_noalloc: the float32 sum for callers that may not allocate device memory.

Some users of the library reduce in places where a device allocation is off limits — a
plug-in living inside a memory budget its host application fixed up front, code between
the synchronisation points of a pool allocator, a latency-critical loop that cannot absorb
the device-wide sync of a first-use cudaMalloc.  For them the library keeps the scratch of
the scheduling-independent sum in a fixed array of its own.  This test calls that entry
point through the C ABI twice in a row (the second call finds the array as the first left
it) and checks each result against the regular entry point, appy_sum_f32 with the ordered
commit, to the tolerance used for reductions everywhere else in the suite (rtol 1e-5).

The file name sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from appy_b200 import workloads as W

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

MAX_ALIGNED = 16384 * 8192


def _ptr(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("n", [1, 4097, (1 << 22) + 3, 1 << 24])
def test_no_alloc_sum_matches_regular_entry_point_twice(rt, n):
    lib = rt.lib()
    a = W.vec_sum(n, seed=n)
    da = torch.from_numpy(a).cuda()
    ref = torch.full((1,), 1.25, dtype=torch.float64, device="cuda")
    rt.check(lib.appy_sum_f32(_ptr(da), n, _ptr(ref), 1, None))
    torch.cuda.synchronize()
    expect = ref.item()
    assert np.isclose(expect, 1.25 + float(np.sum(a, dtype=np.float64)), rtol=1e-5, atol=0.0)
    for _call in range(2):                       # second call reuses the scratch left by the first
        out = torch.full((1,), 1.25, dtype=torch.float64, device="cuda")
        rt.check(lib.appy_sum_f32_noalloc(_ptr(da), n, _ptr(out), None))
        torch.cuda.synchronize()
        assert np.isclose(out.item(), expect, rtol=1e-5, atol=0.0), (out.item(), expect)


def test_no_alloc_sum_unaligned_input(rt):
    lib = rt.lib()
    n = 100001
    a = W.vec_sum(n + 1, seed=3)
    da = torch.from_numpy(a).cuda()
    ref = torch.zeros(1, dtype=torch.float64, device="cuda")
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    p = C.c_void_p(da.data_ptr() + 4)            # 4-byte aligned only
    rt.check(lib.appy_sum_f32(p, n, _ptr(ref), 1, None))
    rt.check(lib.appy_sum_f32_noalloc(p, n, _ptr(out), None))
    torch.cuda.synchronize()
    assert np.isclose(out.item(), ref.item(), rtol=1e-5, atol=0.0)


def test_no_alloc_sum_rejects_inputs_beyond_its_scratch(rt):
    lib = rt.lib()
    small = torch.zeros(16, device="cuda")
    out = torch.full((1,), 7.0, dtype=torch.float64, device="cuda")
    before = rt.launch_count()
    status = lib.appy_sum_f32_noalloc(_ptr(small), MAX_ALIGNED + 1, _ptr(out), None)
    assert status != 0
    msg = lib.appy_last_error().decode()
    assert "too long" in msg and "appy_sum_f32" in msg
    torch.cuda.synchronize()
    assert rt.launch_count() == before and out.item() == 7.0      # nothing was launched
    assert lib.appy_sum_f32_noalloc(_ptr(small), 0, _ptr(out), None) == 0
