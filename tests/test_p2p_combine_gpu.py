"""The in-kernel combine of shared(...) scalars over peer mailboxes (`@jit(combine="p2p")`).

* one rank: the kernel exchanges with its own mailbox — exercises the whole tail on one GPU;
* time-out: a loop-back context of world 2 whose second rank does not exist, with a short
  wait limit: the kernel returns, the status word reports the time-out, the context stays
  usable.  No GPU is hung or faulted: the wait is a bounded poll;
* two ranks on two GPUs (skipped on a one-GPU box): every rank ends with the global total.
"""
import os
import socket

import numpy as np
import pytest

import appy_b200 as appy
from appy_b200 import workloads as W
from appy_b200.backends.cuda_sm100 import multi_gpu as mg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@appy.jit(combine="p2p")
def sum_and_max(a):
    s = 0.0
    m = -1.0
    #pragma parallel for simd shared(s, m)
    for i in range(a.shape[0]):
        s += a[i]
        m = max(m, a[i])
    return s, m


def test_one_rank_combines_with_itself(rt):
    mg.set_combiner(None)
    c = mg.enable_p2p()
    try:
        a = W.vec_sum((1 << 20) + 11, seed=4)
        da = torch.from_numpy(a).cuda()
        for _ in range(3):                      # both slot parities
            s, m = sum_and_max(da)
            assert np.isclose(s, float(np.sum(a, dtype=np.float64)), rtol=1e-5, atol=0) and m == float(a.max())
        assert not c.timed_out()
    finally:
        c.close()
        mg.set_combiner(None)


def test_missing_rank_times_out_with_a_status_not_a_hang(rt):
    c = mg.P2PCombiner(spin_limit=200_000, loopback_world=2)      # roughly 0.2 s
    mg.set_combiner(c)
    try:
        a = W.vec_sum(1 << 16, seed=5)
        da = torch.from_numpy(a).cuda()
        s, m = sum_and_max(da)                  # returns: the wait for rank 1 runs out
        torch.cuda.synchronize()
        assert np.isnan(s) and np.isnan(m)      # a combine that timed out does not look like a result
        assert c.timed_out()
        assert not c.timed_out()                # reading the status clears it
        out = torch.ones(8, device="cuda") * 2  # the context is still usable
        assert float(out.sum()) == 16.0
    finally:
        c.close()
        mg.set_combiner(None)


def test_standalone_combine_of_prebuilt_kernel_results_one_rank(rt):
    """appy_p2p_combine on one rank is the identity fold; the sequence numbers interleave with a
    combine="p2p" loop on the same context."""
    mg.set_combiner(None)
    c = mg.enable_p2p()
    try:
        v = torch.tensor([1.5, -2.0, 7.25], dtype=torch.float64, device="cuda")
        c.combine(v, "+")
        a = W.vec_sum(1 << 16, seed=6)
        s, _m = sum_and_max(torch.from_numpy(a).cuda())
        w = torch.tensor([3, 9], dtype=torch.int32, device="cuda")
        c.combine(w, "max")
        torch.cuda.synchronize()
        assert v.tolist() == [1.5, -2.0, 7.25] and w.tolist() == [3, 9]
        assert np.isclose(s, float(np.sum(a, dtype=np.float64)), rtol=1e-5, atol=0)
        assert not c.timed_out()
        with pytest.raises(ValueError):
            c.combine(torch.zeros(5, device="cuda"))
    finally:
        c.close()
        mg.set_combiner(None)


@appy.jit(combine="p2p", defer=True)
def sum_and_max_into(a, out_s, out_m):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out_s[0] += a[i]
        out_m[0] = max(out_m[0], a[i])


@appy.jit(combine="p2p", defer=True)
def count_into(a, out_n):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out_n[0] += 1 if a[i] > 0.5 else 0


def test_split_phase_exchange_on_one_rank(rt):
    """defer=True: a kernel only stores its CTAs' partials; the first warp of the next such kernel folds and
    posts them, the one after that collects the ranks' totals into the cells (or flush() does both)."""
    mg.set_combiner(None)
    c = mg.enable_p2p()
    try:
        a = W.vec_sum((1 << 20) + 5, seed=9)
        da = torch.from_numpy(a).cuda()
        s = torch.full((1,), 2.0, dtype=torch.float64, device="cuda")
        m = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
        n = torch.zeros(1, dtype=torch.int64, device="cuda")
        total, big, cnt = float(np.sum(a, dtype=np.float64)), float(a.max()), int((a > 0.5).sum())
        sum_and_max_into(da, s, m)              # launch 1: partials stored
        count_into(da, n)                       # launch 2: folds and posts launch 1
        torch.cuda.synchronize()
        assert s.item() == 2.0 and m.item() == -1.0 and n.item() == 0 and len(c.pending) == 2
        count_into(da, n)                       # launch 3: collects launch 1, folds and posts launch 2
        torch.cuda.synchronize()
        assert np.isclose(s.item(), 2.0 + total, rtol=1e-5) and m.item() == big and n.item() == 0
        c.flush()
        torch.cuda.synchronize()
        assert n.item() == 2 * cnt and c.pending == []
        for _ in range(12):                     # more launches than the ring has slots
            sum_and_max_into(da, s, m)
            count_into(da, n)
        c.flush()
        torch.cuda.synchronize()
        assert np.isclose(s.item(), 2.0 + 13 * total, rtol=1e-5) and m.item() == big
        assert n.item() == 14 * cnt and not c.timed_out()
        sum_and_max_into(da, s, m)              # a single launch, completed by the flush alone
        c.flush()
        torch.cuda.synchronize()
        assert np.isclose(s.item(), 2.0 + 14 * total, rtol=1e-5)
        with pytest.raises(NotImplementedError, match="device memory"):
            sum_and_max_into(a, np.zeros(1), np.zeros(1, np.float32))      # host cells cannot be deferred
    finally:
        c.close()
        mg.set_combiner(None)


@pytest.mark.parametrize("world", [2, 8])
def test_split_phase_exchange_with_all_ranks_on_one_gpu(rt, world):
    """The device side of the split-phase exchange for a world of 8 without 8 GPUs: the ranks live in this
    process (mg.local_group: mailboxes wired by address), each with its own stream, data and cells.  Every
    rank's launch k has completed before any rank's launch k+1 is queued, so no kernel ever waits for
    another one: the words a launch collects were posted by launches that are over.  All ranks must end
    with the same bits, equal to the sum over ranks and steps."""
    mg.set_combiner(None)
    group = mg.local_group(world)
    streams = [torch.cuda.Stream() for _ in range(world)]
    try:
        n = (1 << 18) + 3
        data = [torch.from_numpy(W.vec_sum(n, seed=20 + r)).cuda() for r in range(world)]
        s = [torch.full((1,), 2.0, dtype=torch.float64, device="cuda") for _ in range(world)]
        m = [torch.full((1,), -1.0, dtype=torch.float32, device="cuda") for _ in range(world)]
        cnt = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
        torch.cuda.synchronize()

        def step(fn):
            for r in range(world):
                mg.set_combiner(group[r])
                with torch.cuda.stream(streams[r]):
                    fn(r)
            torch.cuda.synchronize()

        steps = 11                                    # more than the ring's 8 slots
        for _k in range(steps):
            step(lambda r: sum_and_max_into(data[r], s[r], m[r]))
            step(lambda r: count_into(data[r], cnt[r]))
        for _ in range(2):
            step(lambda r: group[r].flush(streams[r].cuda_stream))
        host = [d.cpu().numpy() for d in data]
        total = sum(float(np.sum(h, dtype=np.float64)) for h in host)
        for r in range(world):
            assert not group[r].timed_out() and group[r].pending == []
            assert np.isclose(s[r].item(), 2.0 + steps * total, rtol=1e-5)
            assert m[r].item() == max(float(h.max()) for h in host)
            assert cnt[r].item() == steps * sum(int((h > 0.5).sum()) for h in host)
            assert s[r].item() == s[0].item()         # the same bits on every rank
    finally:
        mg.set_combiner(None)
        for c in group:
            c.close()


def test_split_phase_collect_times_out_with_a_status(rt):
    c = mg.P2PCombiner(spin_limit=100_000, loopback_world=2)
    mg.set_combiner(c)
    try:
        da = torch.from_numpy(W.vec_sum(1 << 16, seed=5)).cuda()
        s = torch.zeros(1, dtype=torch.float64, device="cuda")
        m = torch.zeros(1, dtype=torch.float32, device="cuda")
        sum_and_max_into(da, s, m)              # stores its partials: nothing to wait for
        torch.cuda.synchronize()
        assert not c.timed_out()
        c.flush()                               # folds, posts, then collects: rank 1 never posts, the bounded wait runs out
        torch.cuda.synchronize()
        assert np.isnan(s.item()) and np.isnan(m.item()) and c.timed_out()
        assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0            # the context is still usable
    finally:
        c.close()
        mg.set_combiner(None)


@appy.jit(distribute=True)
def d_vec_add(a, b, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]


@appy.jit(distribute=True)
def d_sum(a):
    s = 1.5
    #pragma parallel for simd shared(s)
    for i in range(a.shape[0]):
        s += a[i]
    return s


@appy.jit(distribute=True, combine="p2p")
def d_sum_p2p(a):
    s = 1.5
    #pragma parallel for simd shared(s)
    for i in range(a.shape[0]):
        s += a[i]
    return s


@appy.jit(distribute=True)
def d_spmv(A_data, A_indptr, A_indices, x, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s


@appy.jit(distribute=True)
def d_spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]


@appy.jit(distribute=True)
def d_scatter(idx, out):
    #pragma parallel for simd
    for i in range(idx.shape[0]):
        out[idx[i]] = 1.0


def test_distribute_on_one_rank_is_the_plain_loop(rt):
    a, b = W.vec_add(10001, seed=1)
    c = np.empty_like(a)
    d_vec_add(a, b, c)
    assert np.array_equal(c, a + b)
    assert np.isclose(d_sum(a), 1.5 + float(np.sum(a, dtype=np.float64)), rtol=1e-6)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from appy_b200.backends.cuda_sm100 import runtime as rt
        rt.init(rank)
        comb = mg.enable_p2p()
        a = W.vec_sum(1 << 20, seed=100 + rank)
        da = torch.from_numpy(a).cuda()
        total = sum(float(np.sum(W.vec_sum(1 << 20, seed=100 + r), dtype=np.float64)) for r in range(world))
        big = max(float(W.vec_sum(1 << 20, seed=100 + r).max()) for r in range(world))
        for _ in range(5):
            s, m = sum_and_max(da)
            assert np.isclose(s, total, rtol=1e-5, atol=0), (rank, s, total)
            assert m == big
        # ---- a per-GPU result of a prebuilt C-ABI kernel combined with the standalone call
        part = torch.zeros(2, dtype=torch.float64, device="cuda")
        rt.check(rt.lib().appy_sum_f32(da.data_ptr(), da.numel(), part.data_ptr(), 1, None))
        part[1] = float(rank + 1)
        comb.combine(part[0:1], "+")
        comb.combine(part[1:2], "max")
        torch.cuda.synchronize()
        assert np.isclose(part[0].item(), total, rtol=1e-5, atol=0) and part[1].item() == float(world)
        assert not comb.timed_out()
        # ---- split-phase exchange: every rank ends with the world's totals after the collecting launch
        sd = torch.zeros(1, dtype=torch.float64, device="cuda")
        md = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
        nd = torch.zeros(1, dtype=torch.int64, device="cuda")
        for _ in range(5):
            sum_and_max_into(da, sd, md)
            count_into(da, nd)
        comb.flush()
        torch.cuda.synchronize()
        cnt = sum(int((W.vec_sum(1 << 20, seed=100 + r) > 0.5).sum()) for r in range(world))
        assert np.isclose(sd.item(), 5 * total, rtol=1e-5, atol=0) and md.item() == big and nd.item() == 5 * cnt
        assert not comb.timed_out()
        # ---- the iteration space split over the ranks (`distribute=True`), replicated inputs
        x, y = W.vec_add(100003, seed=7)
        z = np.full_like(x, np.nan)
        from appy_b200.backends.cuda_sm100 import codegen as cg
        cg.transfer_stats.update(h2d=0, d2h=0)
        d_vec_add(x, y, z)                                   # every rank fills only its range
        lo, hi = mg.split_range(0, x.size, world, rank)
        assert np.array_equal(z[lo:hi], (x + y)[lo:hi]) and np.all(np.isnan(np.delete(z, np.s_[lo:hi])))
        # ... and moves only its range of the three row-indexed host arrays
        assert cg.transfer_stats == {"h2d": 3 * 4 * (hi - lo), "d2h": 4 * (hi - lo)}
        ref = 1.5 + float(np.sum(x, dtype=np.float64))
        assert np.isclose(d_sum(x), ref, rtol=1e-6)          # NCCL/gloo combine of the shared scalar
        assert np.isclose(d_sum(torch.from_numpy(x).cuda()), ref, rtol=1e-6)
        assert np.isclose(d_sum_p2p(torch.from_numpy(x).cuda()), ref, rtol=1e-6)   # mailbox combine
        A, xv = W.spmv(20000, 16, kind="zipf", cap=2048, seed=8)
        yv = np.full(A.shape[0], np.nan, np.float32)
        cg.transfer_stats.update(h2d=0, d2h=0)
        d_spmv(A.data, A.indptr, A.indices, xv, yv, A.shape[0])
        r0, r1 = mg.split_rows(A.indptr, world, rank, 8)     # rows balanced by non-zeros + 8 per row
        nnz_r = int(A.indptr[r1] - A.indptr[r0])             # data and indices in part, indptr and x whole
        assert cg.transfer_stats["h2d"] == 8 * nnz_r + A.indptr.nbytes + xv.nbytes + 4 * (r1 - r0)
        assert cg.transfer_stats["d2h"] == 4 * (r1 - r0)
        from oracle import numpy_oracle as O
        full = O.spmv(A.data, A.indptr, A.indices, xv)
        scale = O.spmv_abs(A.data, A.indptr, A.indices, xv)
        assert np.all(np.abs(yv[r0:r1] - full[r0:r1]) <= 1e-5 * scale[r0:r1] + 1e-30)
        assert np.all(np.isnan(yv[:r0])) and np.all(np.isnan(yv[r1:]))
        pieces = [None] * world
        dist.all_gather_object(pieces, (r0, r1))
        assert sorted(pieces)[0][0] == 0 and sorted(pieces)[-1][1] == A.shape[0]
        # ---- distributed SpMM: rows split by non-zeros, the dense operand whole on every rank,
        # rows of the result outside this rank's range untouched
        As, Bs = W.spmm(6000, 24, cap=3000, ncols_b=128, seed=9)
        ys = np.full((As.shape[0], 128), np.nan, np.float32)
        cg.transfer_stats.update(h2d=0, d2h=0)
        d_spmm(As.data, As.indptr, As.indices, Bs, ys, As.shape[0])
        r0, r1 = mg.split_rows(As.indptr, world, rank, 1)
        nnz_r = int(As.indptr[r1] - As.indptr[r0])
        assert cg.transfer_stats["h2d"] == 8 * nnz_r + As.indptr.nbytes + Bs.nbytes + 4 * 128 * (r1 - r0)
        assert cg.transfer_stats["d2h"] == 4 * 128 * (r1 - r0)
        full, scale = O.spmm(As.data, As.indptr, As.indices, Bs), O.spmm_abs(As.data, As.indptr, As.indices, Bs)
        assert np.all(np.abs(ys[r0:r1] - full[r0:r1]) <= 1e-5 * scale[r0:r1] + 1e-30)
        assert np.all(np.isnan(ys[:r0])) and np.all(np.isnan(ys[r1:]))
        # ... and on device tensors held in full by every rank
        dev = [torch.from_numpy(v).cuda() for v in (As.data, As.indptr, As.indices, Bs)]
        yd = torch.full((As.shape[0], 128), float("nan"), device="cuda")
        d_spmm(dev[0], dev[1], dev[2], dev[3], yd, As.shape[0])
        yh = yd.cpu().numpy()
        assert np.all(np.abs(yh[r0:r1] - full[r0:r1]) <= 1e-5 * scale[r0:r1] + 1e-30)
        assert np.all(np.isnan(yh[:r0])) and np.all(np.isnan(yh[r1:]))
        # ---- ranks whose share of a short range is empty still take part in the fused exchange:
        # 20 iterations cut at multiples of 32 leave one rank without work
        tiny = W.vec_sum(20, seed=3)
        dt = torch.from_numpy(tiny).cuda()
        shares = [mg.split_range(0, 20, world, r) for r in range(world)]
        assert any(hi_ <= lo_ for lo_, hi_ in shares)
        for _ in range(3):
            assert np.isclose(d_sum_p2p(dt), 1.5 + float(np.sum(tiny, dtype=np.float64)), rtol=1e-6)
        assert np.isclose(d_sum_p2p(torch.from_numpy(x).cuda()), ref, rtol=1e-6)     # sequence numbers still agree
        assert not comb.timed_out()
        try:
            d_scatter(np.arange(10, dtype=np.int64), np.zeros(10))
            raise AssertionError("a scattered store must not be distributable")
        except NotImplementedError:
            pass
        dist.barrier()
        comb.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
