"""Generated loops on device-resident tensors are plain kernel launches on torch's current
stream, so a sequence of them can be captured into a CUDA graph and replayed.

The loops are warmed up on the capture stream first: compilation, the workspace of an ordered
reduction and the memoised launch record are created then, and the captured region contains
kernel launches only.  (Loops with ``combine="p2p"`` carry a launch sequence number as a
kernel argument and are not meant for replay.)
"""
import numpy as np
import pytest

import appy_b200 as appy
from appy_b200 import workloads as W

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@appy.jit
def g_axpy(alpha, x, y):
    #pragma parallel for simd
    for i in range(x.shape[0]):
        y[i] = alpha * x[i] + y[i]


@appy.jit
def g_sum_into(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]


@appy.jit(ordered_reduction=True)
def g_sum_into_ordered(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]


@appy.jit
def g_gemv(A, x, y):
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += A[i, j] * x[j]
        y[i] = yi


def test_captured_sequence_replays_with_new_input_values(rt):
    n, m = (1 << 18) + 5, 300
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda()
    y = torch.zeros(n, device="cuda")
    A = torch.from_numpy(rng.standard_normal((m, n), dtype=np.float32)).cuda()
    z = torch.empty(m, device="cuda")
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    out_a, out_b = out[0:1], out[1:2]

    def sequence():
        g_axpy(2.0, x, y)                  # y = 2x + y
        g_sum_into(y, out_a)               # atomic commit
        g_sum_into_ordered(y, out_b)       # ordered commit through the stream's workspace
        g_gemv(A, y, z)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):                 # compile, create the workspace, memoise the launches
            sequence()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    launches0 = rt.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sequence()
    assert rt.launch_count() - launches0 == 4     # four kernels were recorded, nothing else ran

    for trial in range(3):
        xv = rng.uniform(-1, 1, n).astype(np.float32)
        yv = rng.uniform(-1, 1, n).astype(np.float32)
        x.copy_(torch.from_numpy(xv))
        y.copy_(torch.from_numpy(yv))
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        y_ref = np.float32(2.0) * xv + yv                         # one rounding per operation, as NumPy
        assert np.array_equal(y.cpu().numpy(), y_ref)
        total = float(np.sum(y_ref, dtype=np.float64))
        scale = float(np.sum(np.abs(y_ref), dtype=np.float64))
        got = out.cpu().numpy()
        assert abs(got[0] - total) <= 1e-5 * scale and abs(got[1] - total) <= 1e-5 * scale
        A64 = A.cpu().numpy().astype(np.float64)
        ref = A64 @ y_ref.astype(np.float64)
        bound = 1e-5 * (np.abs(A64) @ np.abs(y_ref).astype(np.float64))
        assert np.all(np.abs(z.cpu().numpy() - ref) <= bound)
