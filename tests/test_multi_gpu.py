"""Multi-rank host logic on CPU (gloo, world_size 2): range and nnz-balanced row partitions
cover the iteration space exactly once, per-rank results assemble to the single-rank result,
and the shared-scalar combine is an all-reduce."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from appy_b200 import workloads as W  # noqa: E402
from appy_b200.backends.cuda_sm100 import multi_gpu as mg  # noqa: E402
from oracle import c_loops, numpy_oracle as O  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert mg.world() == (rank, world)
        # --- dense range split + shared-scalar combine
        a, m = W.masked_sum(100003, seed=5)
        lo, hi = mg.split_range(0, a.size, world, rank)
        part = torch.tensor([c_loops.vec_sum(a[lo:hi]), c_loops.masked_sum(a[lo:hi], m[lo:hi])], dtype=torch.float64)
        mg.all_reduce(part, "+")
        assert np.allclose(part.numpy(), [O.vec_sum(a), O.masked_sum(a, m)], rtol=1e-12)
        mx = torch.tensor([float(a[lo:hi].max())], dtype=torch.float64)
        mg.all_reduce(mx, "max")
        assert mx.item() == float(a.max())
        # --- CSR row split balanced by nnz; y assembled from the ranks' pieces
        A, x = W.spmv(5000, 16, kind="zipf", cap=1024, seed=6)
        data_r, indptr_r, indices_r, r0, r1 = mg.shard_csr(A.data, A.indptr, A.indices, world, rank)
        assert indptr_r[0] == 0 and len(indptr_r) == r1 - r0 + 1 and len(data_r) == indptr_r[-1]
        y_r = c_loops.spmv(np.ascontiguousarray(data_r), np.ascontiguousarray(indptr_r),
                           np.ascontiguousarray(indices_r), x)
        pieces = [None] * world
        dist.all_gather_object(pieces, (r0, r1, y_r))
        pieces.sort(key=lambda p: p[0])
        assert pieces[0][0] == 0 and pieces[-1][1] == A.shape[0]
        assert all(p[1] == q[0] for p, q in zip(pieces, pieces[1:]))
        y = np.concatenate([p[2] for p in pieces])
        assert np.array_equal(y, c_loops.spmv(A.data, A.indptr, A.indices, x))
        nnz = [int(A.indptr[p[1]] - A.indptr[p[0]]) for p in pieces]
        assert max(nnz) - min(nnz) <= 2 * 1024
        # --- CSR x dense: the same row split, the dense operand whole on every rank, each rank
        # computes its rows of the result with the rebased row pointers of its shard
        As, Bs = W.spmm(3000, 24, cap=1500, ncols_b=64, seed=7)
        d_r, p_r, i_r, s0, s1 = mg.shard_csr(As.data, As.indptr, As.indices, world, rank)
        C_r = c_loops.spmm(np.ascontiguousarray(d_r), np.ascontiguousarray(p_r), np.ascontiguousarray(i_r), Bs)
        assert C_r.shape == (s1 - s0, 64)
        parts = [None] * world
        dist.all_gather_object(parts, (s0, s1, C_r))
        parts.sort(key=lambda p: p[0])
        assert parts[0][0] == 0 and parts[-1][1] == As.shape[0]
        assert all(p[1] == q[0] for p, q in zip(parts, parts[1:]))
        assert np.array_equal(np.concatenate([p[2] for p in parts]), c_loops.spmm(As.data, As.indptr, As.indices, Bs))
        share = [int(As.indptr[p[1]] - As.indptr[p[0]]) for p in parts]
        assert max(share) - min(share) <= 2 * 1500
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_split_range_is_aligned_and_exact():
    for n, w in ((1 << 20, 8), (1000003, 4), (17, 8), (0, 2)):
        cuts = [mg.split_range(0, n, w, r) for r in range(w)]
        assert cuts[0][0] == 0 and cuts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
        assert all(c[0] % 32 == 0 for c in cuts[1:] if c[0] < n)


def test_arrays_a_rank_touches_only_in_part():
    """Host transfers of a distributed loop: arrays indexed by the parallel index (rows) or by the inner
    index of a CSR row loop (non-zeros) travel in slices, gathered and shifted operands travel whole."""
    import math
    import types
    from appy_b200 import dispatcher
    from appy_b200.backends.cuda_sm100 import codegen as cg

    def compiled(src, scope):
        vm = dispatcher.build_val_map(src, scope, {"np": np, "math": math})
        e = cg.CompiledLoop(src, "kernel_loop_1", list(vm), tuple(cg._kind_of(v) for v in vm.values()),
                            {"distribute": True})
        args = [v for v in vm.values() if not isinstance(v, types.ModuleType)]
        e.source_for(*args)
        return e, list(e.variants.values())[0], e._resolve_arrays(args)

    f32 = np.float32
    a = np.ones(1000, f32)
    e, v, arrs = compiled("#pragma parallel for simd\nfor i in range(1, n - 1):\n    c[i] = a[i] + b[i - 1]",
                          dict(a=a, b=a.copy(), c=a.copy(), n=1000))
    assert e._shard_classes(v) == {"c": "rows", "a": "rows"}            # b is read at a shifted index: whole
    assert e._rank_slices(v, arrs, 250, 500) == {"c": (1000, 2000), "a": (1000, 2000)}
    assert e._rank_slices(v, arrs, 7, 7) == {"c": (0, 0), "a": (0, 0)}

    A = np.ones((64, 32), f32)
    e, v, arrs = compiled("#pragma parallel for\nfor i in range(M):\n    s = 0.0\n    #pragma simd\n"
                          "    for j in range(N):\n        s += A[i, j] * x[j]\n    y[i] = s",
                          dict(A=A, x=np.ones(32, f32), y=np.ones(64, f32), M=64, N=32))
    assert e._shard_classes(v) == {"A": "rows", "y": "rows"}
    assert e._rank_slices(v, arrs, 16, 32) == {"A": (16 * 128, 32 * 128), "y": (64, 128)}

    P = np.array([0, 2, 2, 5, 9], np.int32)
    e, v, arrs = compiled("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    s = 0.0\n"
                          "    #pragma simd\n    for j in range(start, end):\n        s += D[j] * x[J[j]]\n    y[i] = s",
                          dict(P=P, D=np.ones(9, f32), J=np.zeros(9, np.int32), x=np.ones(4, f32),
                               y=np.ones(4, f32), M=4))
    assert e._shard_classes(v) == {"D": "nnz", "J": "nnz", "y": "rows"}
    assert e._rank_slices(v, arrs, 2, 4) == {"D": (8, 36), "J": (8, 36), "y": (8, 16)}

    Bd = np.ones((4, 8), f32)
    e, v, arrs = compiled("#pragma parallel for\nfor i in range(M):\n    start, end = P[i], P[i+1]\n    y2[i, :] = 0\n"
                          "    for k in range(start, end):\n        y2[i, :] += D[k] * Bd[J[k], :]",
                          dict(P=P, y2=np.ones((4, 8), f32), D=np.ones(9, f32), Bd=Bd, J=np.zeros(9, np.int32), M=4))
    assert v.plan.kind == "csrdense"
    assert e._shard_classes(v) == {"y2": "rows", "D": "nnz", "J": "nnz"}        # the dense operand travels whole
    assert e._rank_slices(v, arrs, 2, 4) == {"y2": (64, 128), "D": (8, 36), "J": (8, 36)}
