"""Splitting an annotated loop across the GPUs of one box (one process per GPU).

The reference is single-GPU.  Here the outermost parallel-for range is cut into
contiguous pieces, one per rank: by iteration count for dense loops and by non-zero
count for CSR row loops.  Arrays indexed by the outer index are sharded along it, gathered
operands are replicated, and only ``shared(...)`` scalars are combined across ranks, with
an all-reduce over ``torch.distributed`` (NCCL for CUDA tensors, gloo for CPU tensors).
No kernel reads a peer's memory.
"""
from __future__ import annotations

import ctypes as _C

import numpy as np

from . import runtime as rt


def world():
    """(rank, world_size) of the current process; (0, 1) when torch.distributed is not initialised."""
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except ImportError:
        pass
    return 0, 1


def split_range(lo: int, hi: int, world_size: int, rank: int, align: int = 32):
    """This rank's contiguous piece [lo_r, hi_r) of [lo, hi); inner cut points are multiples of
    `align` so that 16-byte vector accesses stay aligned on every rank."""
    b = rt.partition_range(lo, hi, world_size, align)
    return b[rank], b[rank + 1]


def split_rows(indptr, world_size: int, rank: int, row_cost: int = 0):
    """This rank's contiguous row range of a CSR matrix, balanced by non-zero count plus `row_cost` per row
    (`@jit(distribute=True)` uses 8 for row reductions such as SpMV and 1 for row-times-dense loops)."""
    b = rt.partition_rows(np.asarray(indptr), world_size, row_cost)
    return b[rank], b[rank + 1]


def shard_csr(data, indptr, indices, world_size: int, rank: int):
    """Local CSR pieces for this rank: (data_r, indptr_r rebased to 0, indices_r, row_lo, row_hi).
    Works on NumPy arrays and on torch tensors (indptr must be readable on the host)."""
    ip = indptr.cpu().numpy() if hasattr(indptr, "cpu") else np.asarray(indptr)
    r0, r1 = split_rows(ip, world_size, rank)
    k0, k1 = int(ip[r0]), int(ip[r1])
    indptr_r = indptr[r0:r1 + 1] - indptr[r0]
    return data[k0:k1], indptr_r, indices[k0:k1], r0, r1


def all_reduce(values, op: str = "+"):
    """Combine per-rank partial results of ``shared`` scalars in place (tensor of any length).
    `op` is one of + * max min, the reduction operators the front end detects."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return values
    rop = {"+": dist.ReduceOp.SUM, "*": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
    t = values if isinstance(values, torch.Tensor) else torch.from_numpy(np.asarray(values))
    dist.all_reduce(t, op=rop)
    return values


class Pending(_C.Structure):
    """One split-phase launch that is still to be folded or collected (struct appy_pending of t_flat.cuh)."""
    _fields_ = [("seq", _C.c_uint64), ("nv", _C.c_int32), ("grid", _C.c_int32), ("slot", _C.c_int32),
                ("pad", _C.c_int32), ("partials", _C.c_void_p), ("cell", _C.c_void_p * 4), ("op", _C.c_int32 * 4),
                ("ty", _C.c_int32 * 4)]


class Pending2(_C.Structure):
    """What a split-phase kernel (or the flush kernel) is given: the launch to fold and post, the launch to
    collect, and where this launch's own partials go (struct appy_pending2)."""
    _fields_ = [("fold", Pending), ("coll", Pending), ("partials", _C.c_void_p)]


WS_SPLIT_OFFSET = 256 + 8 * 4 * 65536      # the split-phase partials inside the reduction workspace ...
WS_SPLIT_PARITY_BYTES = 8 * 4 * 4096       # ... per launch parity: 4 variables x 4096 CTAs
SPLIT_MAX_GRID = 4096
MB_RING = 8


class P2PCombiner:
    """Peer mailboxes for the in-kernel combine of ``shared(...)`` scalars
    (``@jit(combine="p2p")``).  Collective to create: every rank of the process group calls
    ``enable_p2p()`` once, after ``torch.cuda.set_device``.  Without a process group it is a
    one-rank combiner (the kernel then exchanges with itself), which is what single-GPU tests use.

    Every rank must execute the same sequence of combining loops on one stream: launch number
    ``seq`` of one rank pairs with launch number ``seq`` of the others.
    """

    def __init__(self, spin_limit: int = 0, loopback_world: int = 0):
        """`spin_limit`: polls (about 1 us each) a kernel waits for each rank before it gives up
        and raises the time-out flag (0 = library default, about 8 s).  `loopback_world` > 1
        builds a context whose other ranks do not exist, for exercising the time-out path."""
        import ctypes as C
        rank, world_size = world()
        if loopback_world:
            rank, world_size = 0, loopback_world
        self.rank, self.world = rank, world_size
        self._ctx = C.c_void_p()
        handle = (C.c_char * 64)()
        rt.check(rt.lib().appy_p2p_create(world_size, rank, C.byref(self._ctx), handle))
        handles = [bytes(handle)]
        if world_size > 1 and not loopback_world:
            import torch.distributed as dist
            gathered = [None] * world_size
            dist.all_gather_object(gathered, bytes(handle))
            handles = gathered
        blob = None if loopback_world else b"".join(handles)
        desc = C.c_void_p()
        rt.check(rt.lib().appy_p2p_open(self._ctx, blob, spin_limit, C.byref(desc)))
        self.descriptor = desc.value
        self._seq = 0
        self.pending = []           # split-phase launches whose cells are not final yet (to_collect, to_fold)
        self.to_fold = None
        self.to_collect = None
        self.split_count = 0
        if world_size > 1 and not loopback_world:
            import torch.distributed as dist
            dist.barrier()          # every rank has mapped every mailbox before the first launch

    def next_seq(self) -> int:
        self._seq += 1
        return self._seq

    _OPS = {"+": 0, "*": 1, "max": 2, "min": 3}
    _DTYPES = {"float32": 0, "float64": 1, "int32": 2, "int64": 3}

    def combine(self, values, op: str = "+", stream: int | None = None) -> None:
        """Fold a 1-D CUDA tensor of one to four scalars over all ranks, in place (every rank ends with
        the same bits).  For results of kernels that do not combine in their own tail, e.g. the prebuilt
        C-ABI kernels; collective like a `combine="p2p"` loop: every rank calls it at the same point."""
        import ctypes as C
        import torch
        if values.dim() != 1 or not 1 <= values.numel() <= 4 or not values.is_contiguous():
            raise ValueError("combine() takes a contiguous 1-D tensor of one to four elements")
        dt = self._DTYPES.get(str(values.dtype).replace("torch.", ""))
        if dt is None or op not in self._OPS:
            raise ValueError(f"combine(): unsupported dtype {values.dtype} or operator {op!r}")
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        rt.check(rt.lib().appy_p2p_combine(self._ctx, self.next_seq(), self._OPS[op], dt,
                                           C.c_void_p(values.data_ptr()), values.numel(), C.c_void_p(stream)))

    # ---- split-phase exchange (`@jit(combine="p2p", defer=True)`)
    # A split-phase launch goes through two stages after it has been queued: `to_fold` (its partials wait
    # in the workspace for the next launch's first warp) and `to_collect` (its totals are posted; the launch
    # after that applies the world's totals to its cells).  Each is (seq, slot, grid, partials, cells).
    def begin_split(self, pend: "Pending2", workspace: int, grid: int) -> int:
        """Fill `pend` for a split-phase kernel about to be queued with `grid` CTAs on the stream that owns
        `workspace`; returns the address where that kernel's CTAs store their partials."""
        if grid > SPLIT_MAX_GRID:
            raise RuntimeError(f"defer=True: the kernel's grid ({grid} CTAs) exceeds {SPLIT_MAX_GRID}")
        self._fill(pend.fold, self.to_fold)
        self._fill(pend.coll, self.to_collect)
        mine = workspace + WS_SPLIT_OFFSET + (self.split_count & 1) * WS_SPLIT_PARITY_BYTES
        pend.partials = mine
        return mine

    def end_split(self, seq: int, grid: int, partials: int, cells) -> None:
        """The kernel prepared by begin_split has been queued: its predecessors move one stage on."""
        self.to_collect = self.to_fold
        self.to_fold = (seq, self.split_count % MB_RING, grid, partials, list(cells))
        self.split_count += 1
        self.pending = [x for x in (self.to_collect, self.to_fold) if x]

    @staticmethod
    def _fill(e: "Pending", rec) -> None:
        if rec is None:
            e.seq, e.nv = 0, 0
            return
        seq, slot, grid, partials, cells = rec
        e.seq, e.nv, e.grid, e.slot, e.partials = seq, len(cells), grid, slot, partials
        for v, (ptr, op, ty) in enumerate(cells):
            e.cell[v], e.op[v], e.ty[v] = ptr, op, ty

    def flush(self, stream: int | None = None) -> None:
        """Complete the split-phase launches that no later kernel serves: a one-warp kernel folds and posts
        the last launch and collects the one before it, a second one collects the last launch.  Afterwards
        (once the stream has run) the shared(...) cells of every loop launched so far hold their final
        values.  Collective: every rank calls it at the same point of its launch sequence."""
        if stream is None:
            import torch
            stream = torch.cuda.current_stream().cuda_stream
        while self.to_fold or self.to_collect:
            p = Pending2()
            self._fill(p.fold, self.to_fold)
            self._fill(p.coll, self.to_collect)
            rt.check(rt.lib().appy_p2p_flush(self._ctx, _C.byref(p), _C.c_void_p(stream)))
            self.to_collect, self.to_fold = self.to_fold, None
        self.pending = []

    def timed_out(self) -> bool:
        import ctypes as C
        flag = C.c_int()
        rt.check(rt.lib().appy_p2p_status(self._ctx, C.byref(flag)))
        return bool(flag.value)

    def close(self):
        if self._ctx:
            rt.lib().appy_p2p_destroy(self._ctx)
            self._ctx = None


def local_group(world_size: int, spin_limit: int = 0) -> list:
    """`world_size` combiners, one per rank, for ranks that live in this process on the current device
    (appy_p2p_open_local: mailboxes wired by address).  A rank's loops are called with its combiner
    installed (set_combiner) and on a stream of its own (the partials of a split-phase launch wait in the
    stream's workspace); kernels of different ranks on one GPU must not wait for one another, so only
    `defer=True` loops fit, with every rank's launch k complete before any rank's launch k+1 starts."""
    import ctypes as C
    group = []
    for r in range(world_size):
        c = P2PCombiner.__new__(P2PCombiner)
        c.rank, c.world = r, world_size
        c._ctx = C.c_void_p()
        handle = (C.c_char * 64)()
        rt.check(rt.lib().appy_p2p_create(world_size, r, C.byref(c._ctx), handle))
        c._seq, c.pending, c.to_fold, c.to_collect, c.split_count = 0, [], None, None, 0
        group.append(c)
    ctxs = (C.c_void_p * world_size)(*[c._ctx.value for c in group])
    for c in group:
        desc = C.c_void_p()
        rt.check(rt.lib().appy_p2p_open_local(c._ctx, ctxs, spin_limit, C.byref(desc)))
        c.descriptor = desc.value
    return group


_COMBINER = None


def enable_p2p(spin_limit: int = 0) -> P2PCombiner:
    global _COMBINER
    if _COMBINER is None:
        _COMBINER = P2PCombiner(spin_limit)
    return _COMBINER


def set_combiner(c) -> None:
    """Install (or with None remove) the combiner used by combine="p2p" loops."""
    global _COMBINER
    _COMBINER = c


def combiner() -> P2PCombiner:
    if _COMBINER is None:
        raise RuntimeError('combine="p2p" needs multi_gpu.enable_p2p() to be called on every rank first')
    return _COMBINER
