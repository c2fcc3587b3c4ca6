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
