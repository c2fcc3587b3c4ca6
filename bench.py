"""Benchmark of the generated-kernel path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-table]

Headline workload (config C2): the two shared-scalar reductions over n = 2**26 float32
elements — (a) ``b += a[i]`` and (b) ``b += a[i] if mask[i] else 0.0`` with a
Bernoulli(0.5) bool mask — run through ``@appy_b200.jit``.  A step is one pass of (a)
and one of (b).  ``value`` is effective HBM GB/s: algorithmic bytes (4n + 5n per step
and GPU) divided by the device time of K steps, inputs resident in HBM, all GPUs
summed (weak scaling: every rank owns a full-size shard; for N > 1 the two result
scalars are combined inside the timed region, by default through peer mailboxes
written by the reduction kernels themselves, with ``--combine nccl`` by an all-reduce).  ``e2e`` is the
same metric through the public API with NumPy host buffers: every step uploads its
inputs (``appy.to_gpu``), runs both loops and reads the two results back, all inside
the timed region; ``numpy_args_value`` beside it is the form in which each loop call
gets the NumPy arrays themselves and re-uploads them.
``kernels`` adds one line per benchmark configuration (C1..C5) with the kernel's own
duration, GB/s and fraction of the measured copy bandwidth.

With ``--impl reference`` the same loops are timed on the host cores with the CPU
port of the oracle (OpenMP, all cores) on a bounded sample; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_HEADLINE = 1 << 26


def ncu_traffic() -> dict:
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of every benchmark kernel, from
    one ncu capture each of the full-size workload; the file names the capture each figure comes from."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as fh:
            return json.load(fh)["kernels"]
    except Exception:
        return {}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock and throttle reasons of one GPU, read (never set) every few milliseconds by a thread of
    this process through NVML while the benchmark runs; every sample carries its time, so the samples
    that fall inside the timed region can be told from those of the per-kernel table.  Falls back to an
    `nvidia-smi -lms 100` child process when the NVML binding is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None
        self.samples = []          # (time, sm MHz, reasons bit mask)
        self.sm_max = None
        self.thread = None
        self.stop_flag = False
        self.marks = {}

    def mark(self, name: str):
        self.marks[name] = time.perf_counter()

    def _nvml_loop(self, nv, handle):
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((time.perf_counter(), float(mhz), int(bits)))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            # NVML counts physical GPUs; honour CUDA_VISIBLE_DEVICES when it is a list of indices
            phys = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    phys = int(ids[self.index])
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def _summary(self, rows):
        out = {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": len(rows)}
        if rows:
            out["sm_mhz"] = statistics.median(r[1] for r in rows)
            out["sm_mhz_min"] = min(r[1] for r in rows)
            bits = 0
            for r in rows:
                bits |= r[2]
            out["reasons"] = sorted(name for name, bit in self.REASONS if bits & bit)
        return out

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            out = self._summary(self.samples)
            out["source"] = "NVML, one reading every ~2 ms"
            t0, t1 = self.marks.get("timed_start"), self.marks.get("timed_end")
            if t0 is not None and t1 is not None:
                # the timed region is short: readings from 50 ms before it to its end count as "during"
                out["timed_region"] = self._summary([r for r in self.samples if t0 - 0.05 <= r[0] <= t1])
            return out
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        out["source"] = "nvidia-smi -lms 100"
        return out


# --------------------------------------------------------------------------- jitted loops (the product path)
def define_loops():
    src = '''
@appy.jit
def sum_into(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

@appy.jit
def masked_sum_into(a, mask, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i] if mask[i] else 0.0

@appy.jit(combine="p2p")
def sum_into_p2p(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

@appy.jit(combine="p2p")
def masked_sum_into_p2p(a, mask, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i] if mask[i] else 0.0

@appy.jit(combine="p2p", defer=True)
def sum_into_split(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

@appy.jit(combine="p2p", defer=True)
def masked_sum_into_split(a, mask, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i] if mask[i] else 0.0

@appy.jit(distribute=True)
def d_vec_add(a, b, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]

@appy.jit(distribute=True, combine="p2p")
def d_sum_into_p2p(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

@appy.jit(distribute=True, combine="p2p", defer=True)
def d_sum_into_split(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

@appy.jit(distribute=True)
def d_sum_into(a, out):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        out[0] += a[i]

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
def d_gemv(alpha, A, x, y):
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi

@appy.jit(distribute=True)
def d_spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]

@appy.jit
def vec_sum(a):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i]
    return b

@appy.jit
def masked_sum(a, mask):
    b = 0.0
    #pragma parallel for simd shared(b)
    for i in range(a.shape[0]):
        b += a[i] if mask[i] else 0.0
    return b

@appy.jit
def vec_add(a, b, c):
    #pragma parallel for simd
    for i in range(a.shape[0]):
        c[i] = a[i] + b[i]

@appy.jit
def spmv(A_data, A_indptr, A_indices, x, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        s = 0.0
        #pragma simd
        for j in range(start, end):
            s += A_data[j] * x[A_indices[j]]
        y[i] = s

@appy.jit
def gemv(alpha, A, x, y):
    #pragma parallel for
    for i in range(A.shape[0]):
        yi = 0.0
        #pragma simd
        for j in range(A.shape[1]):
            yi += alpha * A[i, j] * x[j]
        y[i] = yi

@appy.jit
def spmm(A_data, A_indptr, A_indices, B, y, M):
    #pragma parallel for
    for i in range(M):
        start, end = A_indptr[i], A_indptr[i+1]
        y[i, :] = 0
        for k in range(start, end):
            y[i, :] += A_data[k] * B[A_indices[k], :]
'''
    # the decorator reads the function source with inspect, so the text has to live in a file
    path = os.path.join(tempfile.gettempdir(), f"appy_bench_loops_{os.getpid()}.py")
    with open(path, "w") as fh:
        fh.write("import numpy as np\nimport appy_b200 as appy\n" + src)
    import importlib.util
    spec = importlib.util.spec_from_file_location("appy_bench_loops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def time_kernel(torch, fn, rot: int, iters: int, warm: int = 3, after=None):
    """Average device time (us) of one call of fn(i), with CUDA events on the current stream.
    Every one of the `rot` rotating input sets is used at least once before the timed calls, so that
    no first call of a set (launch record, row-length profile, row partition) falls inside them."""
    for i in range(max(warm, rot)):
        fn(i % rot)
    if after is not None:
        after()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i % rot)
    if after is not None:       # work that completes the timed calls (the flush of a split-phase exchange)
        after()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def _wall(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def _scipy_csr(Am):
    try:
        import scipy.sparse as sp
        return sp.csr_matrix((Am.data, Am.indices, Am.indptr), shape=Am.shape)
    except Exception as e:
        sys.stderr.write(f"[bench] SciPy unavailable for the host rows: {e!r}\n")
        return None


def _triton_arm():
    """The reference's generated Triton kernels, restated in baseline/triton_kernels.py."""
    try:
        from baseline import triton_kernels as TK
        return TK
    except Exception as e:      # Triton missing or unable to compile here: the column is left out
        sys.stderr.write(f"[bench] Triton reference arm unavailable: {e!r}\n")
        return None


def kernel_table(torch, L, peak, rank, quick=False, with_triton=True, world=1):
    """Per-configuration device timings through the jit path (device-resident inputs).
    With several ranks every rank runs its own full-size shard (weak scaling): the time is the
    maximum over ranks and GB/s is the sum over ranks; `frac` stays per GPU."""
    from appy_b200 import workloads as W
    from appy_b200.backends.cuda_sm100 import runtime as _rt
    rows = {}
    dev = "cuda"
    TK = _triton_arm() if with_triton else None
    rt_lib, rt_check = _rt.lib(), _rt.check

    def stream_of(t):
        return t.cuda.current_stream().cuda_stream

    def tri(name, byts, fn, rot, iters):
        if TK is None:
            return
        try:
            us = time_kernel(torch, fn, rot, iters, warm=2)
            rows[name]["triton_us"] = round(us, 2)
            rows[name]["triton_gbs"] = round(byts / us / 1e3, 1)
            rows[name]["speedup_vs_triton"] = round(us / rows[name]["us"], 2)
        except Exception as e:
            rows[name]["triton_us"] = None
            sys.stderr.write(f"[bench] Triton kernel for {name} failed: {e!r}\n")

    def host(name, fn, reps=2):
        """The vectorised NumPy/SciPy statement of the same loop on the host cores (one GPU runs only)."""
        if world > 1:
            return
        fn()
        best = min(_wall(fn) for _ in range(reps))
        rows[name]["numpy_ms"] = round(best * 1e3, 2)
        rows[name]["numpy_threads"] = os.cpu_count()
        rows[name]["speedup_vs_numpy"] = round(best * 1e6 / rows[name]["us"], 1)

    def add(name, byts, us, extra=None):
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([us], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        rows[name] = {"us": round(us, 2), "gbs": round(world * byts / us / 1e3, 1),
                      "frac": round(byts / us / 1e3 / peak, 4), "bytes": int(byts)}
        if extra:
            rows[name].update(extra)

    # C1: 201 MB working set is close to the L2 size -> rotate 4 buffer sets
    n = 1 << 24
    a, b = W.vec_add(n, seed=rank)
    sets = [(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev), torch.empty(n, device=dev)) for _ in range(4)]
    add("C1 vec_add f32 n=2^24", W.bytes_vec_add(n),
        time_kernel(torch, lambda i: L.vec_add(*sets[i]), 4, 40), {"l2": "4 rotating buffer sets"})
    assert np.array_equal(sets[0][2].cpu().numpy(), a + b)
    tri("C1 vec_add f32 n=2^24", W.bytes_vec_add(n), lambda i: TK.vec_add(*sets[i]), 4, 40)
    host("C1 vec_add f32 n=2^24", lambda: np.add(a, b))
    del sets
    # C4
    al, A, x = W.gemv(16384, seed=rank)
    dA, dx, dy = torch.from_numpy(A).to(dev), torch.from_numpy(x).to(dev), torch.empty(16384, device=dev)
    add("C4 gemv f32 16384x16384", W.bytes_gemv(16384, 16384),
        time_kernel(torch, lambda i: L.gemv(1.0, dA, dx, dy), 1, 20), {"l2": "1 GiB input"})
    tri("C4 gemv f32 16384x16384", W.bytes_gemv(16384, 16384), lambda i: TK.gemv(1.0, dA, dx, dy), 1, 5)
    host("C4 gemv f32 16384x16384", lambda: A @ x)
    del dA
    if quick:
        return rows
    # C3 (two row-length distributions); 147 MB working set -> rotate y only is not enough: rotate 2 full copies
    for kind in ("poisson", "zipf"):
        Am, xv = W.spmv(kind=kind, seed=rank)
        sets = []
        for _ in range(2):
            sets.append([torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, xv)] +
                        [torch.empty(Am.shape[0], device=dev)])
        byts = W.bytes_spmv(Am.shape[0], Am.shape[1], Am.nnz)
        M = Am.shape[0]
        add(f"C3 spmv {kind} M=2^20 nnz={Am.nnz}", byts,
            time_kernel(torch, lambda i: L.spmv(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M), 2, 40),
            {"l2": "2 rotating copies"})
        tri(f"C3 spmv {kind} M=2^20 nnz={Am.nnz}", byts,
            lambda i: TK.spmv(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M), 2, 6)
        # the floor of this access pattern: the matrix's own column indices read once and x gathered through
        # them, nothing else (no values, no rows, no output)
        probe_out = torch.empty(512 * 8 * 148, device=dev)
        floor = time_kernel(torch, lambda i: rt_check(rt_lib.appy_probe_gather_f32(
            sets[i][3].data_ptr(), sets[i][2].data_ptr(), Am.nnz, probe_out.data_ptr(), stream_of(torch))), 2, 40)
        if world > 1:
            tf = torch.tensor([floor], dtype=torch.float64, device="cuda")
            import torch.distributed as dist
            dist.all_reduce(tf, op=dist.ReduceOp.MAX)
            floor = float(tf.item())
        rows[f"C3 spmv {kind} M=2^20 nnz={Am.nnz}"].update({
            "gather_floor_us": round(floor, 2), "floor_is": "x[indices[k]] summed over all non-zeros, no values/rows/output",
            "kernel_over_floor": round(rows[f"C3 spmv {kind} M=2^20 nnz={Am.nnz}"]["us"] / floor, 3)})
        Asp = _scipy_csr(Am)
        if Asp is not None:
            host(f"C3 spmv {kind} M=2^20 nnz={Am.nnz}", lambda: Asp @ xv)
        del sets
    # C5
    Am, B = W.spmm(seed=rank)
    d = [torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, B)]
    Cm = torch.empty((Am.shape[0], B.shape[1]), device=dev)
    b1, b2 = W.bytes_spmm(Am.shape[0], B.shape[0], Am.nnz, B.shape[1])
    M = Am.shape[0]
    us = time_kernel(torch, lambda i: L.spmm(d[0], d[1], d[2], d[3], Cm, M), 1, 10)
    add(f"C5 spmm M=2^18 nnz={Am.nnz} B=2^18x128", b1, us,
        {"gather_bytes": int(b2), "gather_gbs": round(b2 / us / 1e3, 1), "l2": "403 MB working set"})
    probe_out = torch.empty(512 * 8 * 148, device=dev)
    ceil_us = time_kernel(torch, lambda i: rt_check(rt_lib.appy_probe_row_gather_f32(
        d[3].data_ptr(), B.shape[1], d[2].data_ptr(), Am.nnz, 128, probe_out.data_ptr(), stream_of(torch))), 1, 10)
    if world > 1:
        tf = torch.tensor([ceil_us], dtype=torch.float64, device="cuda")
        import torch.distributed as dist
        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
        ceil_us = float(tf.item())
    rows[f"C5 spmm M=2^18 nnz={Am.nnz} B=2^18x128"].update({
        "gather_ceiling_us": round(ceil_us, 2), "kernel_over_ceiling": round(us / ceil_us, 3),
        "ceiling_is": "the B rows named by the matrix's column indices gathered and summed, 8 rows in flight per "
                      "warp; no coefficients, row ends or output"})
    tri(f"C5 spmm M=2^18 nnz={Am.nnz} B=2^18x128", b1, lambda i: TK.spmm(d[0], d[1], d[2], d[3], Cm, M), 1, 2)
    Asp = _scipy_csr(Am)
    if Asp is not None:
        host(f"C5 spmm M=2^18 nnz={Am.nnz} B=2^18x128", lambda: Asp @ B, reps=1)
    return rows


def strong_table(torch, L, peak, rank, world, quick=False, use_p2p=True):
    """The configured problems split over the ranks (`@jit(distribute=True)`): contiguous ranges of the
    outer index, balanced by non-zeros for the CSR loops; the gathered operands (x, B) whole on every
    GPU; every rank writes its own slice of the result, which stays where it is.  Inputs are the same on
    every rank and resident before the timed launches.  Per kernel: `us` = maximum over ranks of the
    rank's own average launch time, `one_gpu_us` = the same loop on the whole problem on one GPU
    (maximum over ranks, same run), `strong_speedup` = their ratio.  Each rank rotates over enough
    copies of its inputs that consecutive launches find nothing of theirs in the 126 MB L2."""
    import torch.distributed as dist
    from appy_b200 import workloads as W
    dev = "cuda"
    rows = {}
    L2 = 126e6

    def copies(per_gpu_bytes):
        return int(max(2, min(24, -(-2.2 * L2 // max(per_gpu_bytes, 1)))))

    def both(name, byts, one_fn, dist_fn, rot, iters, note, after=None):
        t1 = time_kernel(torch, one_fn, rot, max(4, iters // 2))
        tn = time_kernel(torch, dist_fn, rot, iters, after=after)
        t = torch.tensor([t1, tn], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t1, tn = float(t[0]), float(t[1])
        rows[name] = {"us": round(tn, 2), "one_gpu_us": round(t1, 2), "strong_speedup": round(t1 / tn, 2),
                      "gbs": round(byts / tn / 1e3, 1), "frac_per_gpu": round(byts / world / tn / 1e3 / peak, 4),
                      "bytes": int(byts), "split": note, "copies_rotated": rot}

    # C1
    n = 1 << 24
    a, b = W.vec_add(n, seed=0)
    rot = copies(W.bytes_vec_add(n) / world)
    sets = [(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev), torch.empty(n, device=dev)) for _ in range(rot)]
    both("C1 vec_add f32 n=2^24", W.bytes_vec_add(n), lambda i: L.vec_add(*sets[i]), lambda i: L.d_vec_add(*sets[i]),
         rot, 8 * rot, "contiguous index ranges, cuts at multiples of 32")
    from appy_b200.backends.cuda_sm100 import multi_gpu as mg
    lo, hi = mg.split_range(0, n, world, rank)
    assert np.array_equal(sets[0][2][lo:hi].cpu().numpy(), (a + b)[lo:hi])
    del sets
    # C2a with the combine inside the kernel's tail
    n = N_HEADLINE
    av = W.vec_sum(n, seed=0)
    rot = copies(W.bytes_sum(n) / world)
    das = [torch.from_numpy(av).to(dev) for _ in range(rot)]
    cell = torch.zeros(1, dtype=torch.float64, device=dev)
    d_sum = L.d_sum_into_split if use_p2p else L.d_sum_into
    flush = None
    if use_p2p:
        from appy_b200.backends.cuda_sm100 import multi_gpu as _mg
        flush = _mg.combiner().flush
    both("C2a sum f32 n=2^26", W.bytes_sum(n), lambda i: L.sum_into(das[i], cell), lambda i: d_sum(das[i], cell),
         rot, 8 * rot, "contiguous index ranges; the scalar is combined " +
         ("over peer mailboxes, split phase (posted and collected by the following launches, the last ones by a "
          "flush inside the timed region)" if use_p2p else "by an NCCL all-reduce"), after=flush)
    cell.zero_()
    d_sum(das[0], cell)
    if flush is not None:
        flush()
    assert np.isclose(float(cell.item()), float(np.sum(av, dtype=np.float64)), rtol=1e-5)
    del das
    # C4
    al, A, x = W.gemv(16384, seed=0)
    rot = copies(W.bytes_gemv(16384, 16384) / world)
    dAs = [torch.from_numpy(A).to(dev) for _ in range(rot)]
    dx, dy = torch.from_numpy(x).to(dev), torch.empty(16384, device=dev)
    both("C4 gemv f32 16384x16384", W.bytes_gemv(16384, 16384), lambda i: L.gemv(1.0, dAs[i], dx, dy),
         lambda i: L.d_gemv(1.0, dAs[i], dx, dy), rot, 6 * rot, "row blocks; x on every GPU")
    del dAs, A
    if quick:
        return rows
    # C3
    for kind in ("poisson", "zipf"):
        Am, xv = W.spmv(kind=kind, seed=0)
        byts = W.bytes_spmv(Am.shape[0], Am.shape[1], Am.nnz)
        rot = copies(byts / world)
        sets = []
        for _ in range(rot):
            sets.append([torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, xv)] +
                        [torch.empty(Am.shape[0], device=dev)])
        M = Am.shape[0]
        both(f"C3 spmv {kind} M=2^20 nnz={Am.nnz}", byts,
             lambda i: L.spmv(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M),
             lambda i: L.d_spmv(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M),
             rot, 8 * rot, "row ranges balanced by non-zeros; x on every GPU")
        del sets
    # C5
    Am, B = W.spmm(seed=0)
    b1, b2 = W.bytes_spmm(Am.shape[0], B.shape[0], Am.nnz, B.shape[1])
    rot = 2
    sets = []
    for _ in range(rot):
        sets.append([torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, B)] +
                    [torch.empty((Am.shape[0], B.shape[1]), device=dev)])
    M = Am.shape[0]
    both(f"C5 spmm M=2^18 nnz={Am.nnz} B=2^18x128", b1,
         lambda i: L.spmm(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M),
         lambda i: L.d_spmm(sets[i][0], sets[i][1], sets[i][2], sets[i][3], sets[i][4], M),
         rot, 6 * rot, "row ranges balanced by non-zeros; B (134 MB) on every GPU, never read from a peer")
    return rows


# --------------------------------------------------------------------------- CPU arms
_cpu_inputs = {}


def cpu_port_numbers(n_sample: int, reps: int):
    """Oracle C port (OpenMP) of the two headline loops on n_sample elements per loop, on every core
    this process may use: the thread count is set explicitly, whatever OMP_NUM_THREADS the launcher
    exported (torch.distributed.run sets it to 1)."""
    from appy_b200 import workloads as W
    from oracle import c_loops
    threads = c_loops.set_threads(c_loops.host_cores())
    if n_sample not in _cpu_inputs:
        _cpu_inputs.clear()
        _cpu_inputs[n_sample] = W.masked_sum(n_sample, seed=0)
    a, m = _cpu_inputs[n_sample]
    c_loops.vec_sum(a)
    t0 = time.perf_counter()
    for _ in range(reps):
        c_loops.vec_sum(a)
        c_loops.masked_sum(a, m)
    dt = (time.perf_counter() - t0) / reps
    byts = 9 * n_sample
    return byts / dt / 1e9, dt, threads


def python_loop_number(n_sample: int):
    """The reference's literal CPU execution: the undecorated Python loops."""
    from appy_b200 import workloads as W
    from oracle import python_loops as PL
    a, m = W.masked_sum(n_sample, seed=0)
    t0 = time.perf_counter()
    PL.vec_sum(a)
    PL.masked_sum_ternary(a, m)
    dt = time.perf_counter() - t0
    return 9 * n_sample / dt / 1e9, dt


def run_reference(args, rank):
    """The CPU arm: the same two loops on the same n = 2**26 elements per loop, every step one full pass
    of both, on all the host cores this process may use.  Rank 0 only; other ranks leave at once."""
    if rank != 0:
        return
    n = args.n
    for _ in range(max(args.warmup, 1)):
        cpu_port_numbers(n, 1)
    gbs, dt, threads = cpu_port_numbers(n, args.steps)
    py_gbs, py_dt = python_loop_number(1 << 20)
    line = {
        "impl": "reference", "metric": "effective HBM GB/s of the generated-kernel path (shared-scalar reductions)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2 shared-scalar reductions: (a) sum, (b) masked sum (Bernoulli 0.5 bool mask), "
                               f"f32, n={n} per GPU, through @appy_b200.jit",
                   "l2": "inputs larger than L2 (256 MiB + 64 MiB read per step)",
                   "accumulate": "float64 (the shared scalar is a float64 cell, as in the reference)",
                   "collective": "none"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"oracle/loops.c with OpenMP on the full n={n} elements per loop, {args.steps} "
                                   f"passes, {threads} threads set explicitly; the interpreted Python loops (the "
                                   f"reference's own CPU execution) reach {py_gbs:.5f} GB/s on n=2^20 on 1 core"},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_only(args):
    """One configuration, device-resident inputs, --warmup + --steps launches through the jit path."""
    import torch
    from appy_b200 import workloads as W
    from appy_b200.backends.cuda_sm100 import runtime as rt
    torch.cuda.set_device(0)
    rt.init(0)
    L = define_loops()
    k, sc = args.only, max(1, args.scale)
    dev = "cuda"
    if k == "vec_add":
        # four rotating buffer sets, as in the per-kernel table: 201 MB per set is close to the L2 size, and a
        # single set would leave part of the previous launch's output in L2
        n = (1 << 24) // sc
        a, b = W.vec_add(n)
        sets = [(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev), torch.empty(n, device=dev)) for _ in range(4)]
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % 4
            L.vec_add(*sets[turn[0]])
        byts = W.bytes_vec_add(n)
        for _ in range(4):
            fn()
    elif k in ("sum", "masked_sum"):
        n = (1 << 26) // sc
        a, m = W.masked_sum(n)
        da, dm = torch.from_numpy(a).to(dev), torch.from_numpy(m).to(dev)
        out = torch.zeros(1, dtype=torch.float64, device=dev)
        fn = (lambda: L.sum_into(da, out)) if k == "sum" else (lambda: L.masked_sum_into(da, dm, out))
        byts = W.bytes_sum(n) if k == "sum" else W.bytes_masked_sum(n)
    elif k == "gemv":
        n = 16384 // sc
        _al, A, x = W.gemv(n)
        dA, dx, dy = torch.from_numpy(A).to(dev), torch.from_numpy(x).to(dev), torch.empty(n, device=dev)
        fn, byts = (lambda: L.gemv(1.0, dA, dx, dy)), W.bytes_gemv(n, n)
    elif k in ("spmv_poisson", "spmv_zipf"):
        Am, xv = W.spmv((1 << 20) // sc, kind=k.split("_")[1])
        d = [torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, xv)]
        dy = torch.empty(Am.shape[0], device=dev)
        M = Am.shape[0]
        fn, byts = (lambda: L.spmv(d[0], d[1], d[2], d[3], dy, M)), W.bytes_spmv(M, M, Am.nnz)
    elif k == "spmm":
        Am, B = W.spmm((1 << 18) // sc)
        d = [torch.from_numpy(v).to(dev) for v in (Am.data, Am.indptr, Am.indices, B)]
        Cm = torch.empty((Am.shape[0], B.shape[1]), device=dev)
        M = Am.shape[0]
        fn, byts = (lambda: L.spmm(d[0], d[1], d[2], d[3], Cm, M)), W.bytes_spmm(M, M, Am.nnz, B.shape[1])[0]
    else:
        raise SystemExit(f"unknown --only {k}")
    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    e1.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"only": k, "scale": sc, "us_per_launch": round(us, 2), "algorithmic_bytes": int(byts),
                      "gbs": round(byts / us / 1e3, 1)}), flush=True)


def run_ceilings(args):
    """Gather ceilings of the two sparse kernels, measured with the library's probe kernels
    (appy_probe_row_gather_f32 / appy_probe_gather_f32): 2^23 random rows of a 2^18 x 128 float32 matrix,
    taken whole (512 B), in halves (256 B) and in quarters (128 B), from all of it (134 MB), half of its
    rows (67 MB) and a quarter (34 MB); and x[indices[k]] over the column indices of both C3 matrices.
    L2 is flushed before every timed launch.  Prints one JSON object."""
    import torch
    from appy_b200 import workloads as W
    from appy_b200.backends.cuda_sm100 import runtime as rt
    torch.cuda.set_device(0)
    rt.init(0)
    L = rt.lib()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def cold(fn, iters=6):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return float(np.median(ts))

    M, n = 1 << 18, 1 << 23
    B = torch.rand((M, 128), device="cuda")
    out = torch.empty(512 * 8 * 148, device="cuda")
    res = {"row_gather": [], "spmv_gather": []}
    g = torch.Generator(device="cuda").manual_seed(0)
    for frac, label in ((1, "134 MB"), (2, "67 MB"), (4, "34 MB")):
        rows = torch.randint(0, M // frac, (n,), device="cuda", dtype=torch.int32, generator=g)
        for floats in (128, 64, 32):
            us = cold(lambda: rt.check(L.appy_probe_row_gather_f32(B.data_ptr(), 128, rows.data_ptr(), n, floats,
                                                                     out.data_ptr(), None)))
            res["row_gather"].append({"operand": label, "bytes_per_row": 4 * floats, "rows": n, "us": round(us, 1),
                                      "gbs": round(n * 4 * floats / us / 1e3)})
    for kind in ("poisson", "zipf"):
        Am, xv = W.spmv(kind=kind)
        idx, x = torch.from_numpy(Am.indices).cuda(), torch.from_numpy(xv).cuda()
        us = cold(lambda: rt.check(L.appy_probe_gather_f32(x.data_ptr(), idx.data_ptr(), Am.nnz, out.data_ptr(), None)))
        res["spmv_gather"].append({"matrix": kind, "nnz": Am.nnz, "us": round(us, 1)})
    print(json.dumps(res), flush=True)


# --------------------------------------------------------------------------- main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="appy_b200")
    ap.add_argument("--no-table", action="store_true")
    ap.add_argument("--quick-table", action="store_true")
    ap.add_argument("--n", type=int, default=N_HEADLINE)
    ap.add_argument("--only", default=None,
                    help="run a single configuration's kernel --steps times and exit (for profilers): "
                         "vec_add, sum, masked_sum, gemv, spmv_poisson, spmv_zipf, spmm")
    ap.add_argument("--ceilings", action="store_true",
                    help="measure the gather ceilings of the sparse kernels with the library's probe kernels and exit")
    ap.add_argument("--scale", type=int, default=1, help="with --only: divide the problem size by this factor")
    ap.add_argument("--combine", default="p2p", choices=["nccl", "p2p", "p2p-immediate"],
                    help="N > 1: how the two result scalars are combined across GPUs: peer mailboxes inside "
                         "the reduction kernels (no collective call; falls back to NCCL when peer mappings "
                         "cannot be made), or an NCCL all-reduce per step")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.ceilings:
        run_ceilings(args)
        return
    if args.only:
        run_only(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL writes its version banner to stdout; stdout is reserved for the one JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", os.path.join(tempfile.gettempdir(), "appy_bench_nccl.%h.%p.log"))
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from appy_b200 import workloads as W
    from appy_b200.backends.cuda_sm100 import runtime as rt
    rt.init(local_rank)
    L = define_loops()
    peak, peak_src = measured_peak()
    n = args.n

    a_h, m_h = W.masked_sum(n, seed=rank)
    a = torch.from_numpy(a_h).cuda()
    m = torch.from_numpy(m_h).cuda()
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    out_a, out_b = out[0:1], out[1:2]

    # The two result cells of a step are combined across ranks by one all-reduce, ordered on the
    # launch stream.  (Overlapping it with the next step's kernels through a second buffer was
    # measured slower: the reduction kernels occupy every SM, so the NCCL kernel waits for them anyway.)
    outs = [out]
    part = torch.zeros(2, dtype=torch.float64, device="cuda")
    use_p2p = world > 1 and args.combine in ("p2p", "p2p-immediate")
    if use_p2p:
        from appy_b200.backends.cuda_sm100 import multi_gpu as mg
        try:
            combiner = mg.enable_p2p()
            mapped = 1
        except Exception as exc:                  # no peer access between some pair of GPUs
            sys.stderr.write(f"[bench] rank {rank}: peer mailboxes unavailable ({exc}); using NCCL\n")
            mapped = 0
        flag = torch.tensor([mapped], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)       # every rank takes the same path
        use_p2p = bool(flag.item())

    split = use_p2p and args.combine == "p2p"       # split-phase: post in this kernel, collect in the next

    def step():
        # the two result cells accumulate over the steps (`out[0] += a[i]`); they are zeroed before the timed
        # region and checked against steps x the per-step totals after it
        if split:
            L.sum_into_split(a, out_a)
            L.masked_sum_into_split(a, m, out_b)
        elif use_p2p:
            L.sum_into_p2p(a, out_a)
            L.masked_sum_into_p2p(a, m, out_b)
        elif world > 1:
            # NCCL: this step's per-GPU sums go to a scratch pair, one all-reduce combines both, the
            # result is added to the accumulating cells
            part.zero_()
            L.sum_into(a, part[0:1])
            L.masked_sum_into(a, m, part[1:2])
            dist.all_reduce(part)
            out.add_(part)
        else:
            L.sum_into(a, out_a)
            L.masked_sum_into(a, m, out_b)

    def drain():
        if split:
            combiner.flush()        # the last launch's totals: collected inside the timed region

    for _ in range(args.warmup):
        step()
    drain()
    torch.cuda.synchronize()
    # parity of the warm-up result (rank-local part is checked before the all-reduce mixes ranks)
    out.zero_()
    L.sum_into(a, out_a)
    L.masked_sum_into(a, m, out_b)
    got = out.cpu().numpy()
    ref = [float(np.sum(a_h, dtype=np.float64)), float(np.sum(a_h[m_h], dtype=np.float64))]
    assert np.allclose(got, ref, rtol=1e-5, atol=0), (got, ref)

    sampler = ClockSampler(local_rank)          # every rank watches its own GPU
    sampler.start()
    for _ in range(20):                         # clocks under load before the region, as during it
        step()
    drain()                                     # nothing of the warm-up steps is left to collect
    out.zero_()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = rt.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark("timed_start")
    e0.record()
    for _ in range(args.steps):
        step()
    drain()
    e1.record()
    torch.cuda.synchronize()
    sampler.mark("timed_end")
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    launches = rt.launch_count() - launches0
    # every rank's cells hold the sums of all ranks, accumulated over the timed steps
    if world > 1:
        tot = torch.tensor(ref, dtype=torch.float64, device="cuda")
        dist.all_reduce(tot)
        for buf in outs:
            assert np.allclose(buf.cpu().numpy(), args.steps * tot.cpu().numpy(), rtol=1e-5, atol=0), (buf, tot)
    else:
        for buf in outs:
            assert np.allclose(buf.cpu().numpy(), args.steps * np.asarray(ref), rtol=1e-5, atol=0), (buf, ref)
    if use_p2p:
        assert not combiner.timed_out(), "a peer-mailbox wait ran out"
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # keep the clocks sampler running through the per-kernel timings as well
    bytes_step = (W.bytes_sum(n) + W.bytes_masked_sum(n)) * world
    value = bytes_step * args.steps / (ms * 1e-3) / 1e9

    # ---- roofline of the dominant kernel, timed alone on the launch stream
    us_sum = time_kernel(torch, lambda i: L.sum_into(a, out_a), 1, 100)
    us_msk = time_kernel(torch, lambda i: L.masked_sum_into(a, m, out_b), 1, 100)
    if world > 1:      # per-kernel times: maximum over ranks
        tk = torch.tensor([us_sum, us_msk], dtype=torch.float64, device="cuda")
        dist.all_reduce(tk, op=dist.ReduceOp.MAX)
        us_sum, us_msk = float(tk[0].item()), float(tk[1].item())
    dom_bytes, dom_us, dom_name = (W.bytes_masked_sum(n), us_msk, "masked sum (T2 reduction template)") \
        if us_msk >= us_sum else (W.bytes_sum(n), us_sum, "sum (T2 reduction template)")
    achieved = dom_bytes / dom_us / 1e3

    # ---- e2e: NumPy host buffers through the public API, copies inside the timed region.
    # (a) the step as a user of the reference's API writes it when two loops share an input: upload the
    #     step's inputs once with appy.to_gpu, run both loops on the resident copies, read the two results;
    # (b) the same two loops called with the NumPy arrays themselves: every call re-uploads its arguments
    #     (what the reference's generated host code does), so `a` crosses PCIe twice per step.
    import appy_b200 as appy
    e2e_steps = max(3, min(10, args.steps))

    def step_resident():
        da, dm = appy.to_gpu(a_h, m_h)
        return L.vec_sum(da), L.masked_sum(da, dm)

    def step_numpy_args():
        return L.vec_sum(a_h), L.masked_sum(a_h, m_h)

    def step_numpy_resident():
        # (c) NumPy arguments declared resident: the step's new data is reported with `touch`, the first
        #     loop uploads `a`, the second finds it on the device and uploads only the mask
        appy.touch(a_h, m_h)
        return L.vec_sum(a_h), L.masked_sum(a_h, m_h)

    e2e = {}
    for name, fn in (("resident", step_resident), ("numpy_args", step_numpy_args),
                     ("numpy_resident", step_numpy_resident)):
        if name == "numpy_resident":
            appy.resident(a_h, m_h)
        fn(); fn()                                    # mirrors, pinning and launch records settle
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            r1, r2 = fn()
        e2e_s = time.perf_counter() - t0
        assert np.isclose(r1, ref[0], rtol=1e-5) and np.isclose(r2, ref[1], rtol=1e-5)
        te = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e[name] = bytes_step * e2e_steps / float(te.item()) / 1e9
    appy.release(a_h, m_h)
    e2e_val = e2e["resident"]
    h2d = a_h.nbytes + m_h.nbytes + 16
    d2h = 16

    table = {}
    if not args.no_table:
        table = kernel_table(torch, L, peak, rank, quick=args.quick_table, with_triton=(rank == 0 and world == 1),
                             world=world)
        TK = _triton_arm() if (rank == 0 and world == 1) else None
        tri_sum = tri_msk = tri_if = None
        if TK is not None:
            try:
                tb = torch.zeros(1, dtype=torch.float64, device="cuda")
                tri_sum = time_kernel(torch, lambda i: TK.vec_sum(a, tb), 1, 5, warm=2)
                tri_msk = time_kernel(torch, lambda i: TK.masked_sum_ternary(a, m, tb), 1, 5, warm=2)
                tri_if = time_kernel(torch, lambda i: TK.masked_sum_if(a, m, tb), 1, 2, warm=1)
            except Exception as e:
                sys.stderr.write(f"[bench] Triton reduction kernels failed: {e!r}\n")
        table["C2a sum f32 n=2^26"] = {"us": round(us_sum, 2), "gbs": round(world * W.bytes_sum(n) / us_sum / 1e3, 1),
                                       "frac": round(W.bytes_sum(n) / us_sum / 1e3 / peak, 4),
                                       "bytes": W.bytes_sum(n), "l2": "256 MiB input"}
        table["C2b masked sum f32+bool n=2^26"] = {"us": round(us_msk, 2),
                                                   "gbs": round(world * W.bytes_masked_sum(n) / us_msk / 1e3, 1),
                                                   "frac": round(W.bytes_masked_sum(n) / us_msk / 1e3 / peak, 4),
                                                   "bytes": W.bytes_masked_sum(n), "l2": "320 MiB input"}
        if tri_sum:
            table["C2a sum f32 n=2^26"].update({"triton_us": round(tri_sum, 2),
                                                "triton_gbs": round(W.bytes_sum(n) / tri_sum / 1e3, 1),
                                                "speedup_vs_triton": round(tri_sum / us_sum, 2)})
        if tri_msk:
            table["C2b masked sum f32+bool n=2^26"].update({
                "triton_us": round(tri_msk, 2), "triton_gbs": round(W.bytes_masked_sum(n) / tri_msk / 1e3, 1),
                "speedup_vs_triton": round(tri_msk / us_msk, 2),
                "triton_if_form_us": round(tri_if, 2) if tri_if else None})
        if world == 1:      # the vectorised NumPy statements of the two loops on the host cores
            for name, us, fn in (("C2a sum f32 n=2^26", us_sum, lambda: np.sum(a_h, dtype=np.float64)),
                                 ("C2b masked sum f32+bool n=2^26", us_msk,
                                  lambda: np.sum(a_h, where=m_h, dtype=np.float64))):
                fn()
                best = min(_wall(fn) for _ in range(2))
                table[name].update({"numpy_ms": round(best * 1e3, 2), "numpy_threads": os.cpu_count(),
                                    "speedup_vs_numpy": round(best * 1e6 / us, 1)})

    strong = None
    if world > 1 and not args.no_table:
        strong = strong_table(torch, L, peak, rank, world, quick=args.quick_table, use_p2p=use_p2p)

    clocks = sampler.stop()                     # covers the timed region and the per-kernel tables
    if world > 1:                               # one line per rank's GPU: median MHz, minimum MHz, readings
        mine = torch.tensor([clocks.get("sm_mhz") or 0.0, clocks.get("sm_mhz_min") or 0.0,
                             float(clocks.get("samples") or 0),
                             float(sum(1 << i for i, (nm, _b) in enumerate(ClockSampler.REASONS)
                                       if nm in clocks.get("reasons", [])))], dtype=torch.float64, device="cuda")
        allc = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allc, mine)
        clocks["per_rank"] = [{"sm_mhz": float(c[0]), "sm_mhz_min": float(c[1]), "samples": int(c[2]),
                               "reasons": [nm for i, (nm, _b) in enumerate(ClockSampler.REASONS)
                                           if int(c[3]) >> i & 1]} for c in allc]
        for c in clocks["per_rank"]:            # a throttle seen on any rank's GPU counts for the run
            clocks["reasons"] = sorted(set(clocks["reasons"]) | set(c["reasons"]))

    # host cost of one call through the whole @jit path (wall clock; the kernel on 4096 elements is
    # shorter than the call, so the loop is host-bound and wall time per call is the launch path)
    small, small_out = a[:4096], torch.zeros(1, dtype=torch.float64, device="cuda")
    for _ in range(20):
        L.sum_into(small, small_out)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(500):
        L.sum_into(small, small_out)
    host_launch_us = (time.perf_counter() - t0) / 500 * 1e6
    torch.cuda.synchronize()

    cpu = None
    if rank == 0 and world == 1:
        _cpu_inputs[n] = (a_h, m_h)
        cpu_port_numbers(n, 1)
        gbs, dt, threads = cpu_port_numbers(n, 10)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"oracle/loops.c (OpenMP, {threads} threads set explicitly) on the full n={n} elements "
                         "per loop, 10 passes"}

    if rank == 0:
        line = {
            "metric": "effective HBM GB/s of the generated-kernel path (shared-scalar reductions)",
            "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2 shared-scalar reductions: (a) sum, (b) masked sum (Bernoulli 0.5 bool mask), "
                                   f"f32, n={n} per GPU, through @appy_b200.jit",
                       "l2": "inputs larger than L2 (256 MiB + 64 MiB read per step)",
                       "accumulate": "float64 (the shared scalar is a float64 cell, as in the reference)",
                       "collective": ("none" if world == 1 else
                                      "peer mailboxes, split phase: every reduction kernel posts its totals with P2P "
                                      "stores over NVLink and collects those of the kernel before it" if split else
                                      "peer mailboxes inside the reduction kernels (P2P stores over NVLink)" if use_p2p
                                      else "NCCL all-reduce of the two result scalars per step")},
            "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": round(achieved, 1), "peak": peak,
                         "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None,
                         "peak_source": f"{peak_src} copy bandwidth", "us_per_launch": round(dom_us, 2),
                         "algorithmic_bytes": dom_bytes},
            "cpu_baseline": cpu,
            "e2e": {"value": round(e2e_val, 3), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps,
                    "form": "per step: appy.to_gpu(a, mask) from NumPy buffers (pinned in place), both loops on the "
                            "resident copies, the two float64 results read back",
                    "numpy_args_value": round(e2e["numpy_args"], 3),
                    "numpy_args_h2d_bytes_per_step": 2 * a_h.nbytes + m_h.nbytes + 16,
                    "numpy_resident_value": round(e2e["numpy_resident"], 3),
                    "numpy_resident_form": "the loops called with the NumPy arrays after appy.resident(a, mask); every "
                                           "step appy.touch(a, mask) reports new data, so each array crosses PCIe "
                                           "once per step"},
            "gpu_launches": int(launches),
            "host_launch_us": round(host_launch_us, 2),
            "clocks": clocks,
            "kernels": table,
        }
        if strong is not None:
            line["strong"] = {"what": "the configured problems split over the GPUs with @jit(distribute=True); "
                                      "time = maximum over ranks; strong_speedup = one_gpu_us / us", "kernels": strong}
        traffic = ncu_traffic()
        if n == N_HEADLINE:
            t = traffic.get("masked_sum" if dom_name.startswith("masked") else "sum")
            line["roofline"]["traffic"] = t["dram_bytes"] if t else None
            line["roofline"]["traffic_source"] = t["source"] if t else None
            keys = {"C1": "vec_add", "C2a": "sum", "C2b": "masked_sum", "C4": "gemv", "C3 spmv poisson": "spmv_poisson",
                    "C3 spmv zipf": "spmv_zipf", "C5": "spmm"}
            for row, vals in table.items():
                for prefix, key in keys.items():
                    if row.startswith(prefix) and key in traffic:
                        vals["traffic"] = traffic[key]["dram_bytes"]
                        vals["traffic_over_algorithmic"] = round(traffic[key]["dram_bytes"] / vals["bytes"], 3)
                        vals["traffic_source"] = traffic[key]["source"]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
