/*
 * libappy_sm100 — C ABI of the cuda_sm100 execution backend for APPy-style
 * annotated loops.
 *
 * The reference (habanero-lab/APPy) is pure Python: a loop marked
 * `#pragma parallel for` is turned into Triton source by
 * appy/backends/triton/codegen.py:9-73, and the generated host function
 * (appy/backends/triton/passes/gen_host_code.py:25-42) moves data with torch
 * (host_passes/gen_data_movement.py:14-96) and launches through Triton
 * (host_passes/gen_kernel_launch.py:4-73).  This library is what those three
 * steps bind to instead: compile a CUDA C instantiation of a kernel template
 * (NVRTC, sm_100a), move data (pinned registration, async copies, cached
 * device mirrors), launch, and split an iteration space across GPUs.
 *
 * Conventions
 *   - every function returns 0 on success and a negative code on failure;
 *     appy_last_error() then returns a message for the calling thread;
 *   - all pointers are plain C pointers; `stream` is a cudaStream_t passed as
 *     void* (NULL = the legacy default stream, which orders with torch's
 *     default stream);
 *   - device pointers named d* must belong to the device made current by
 *     appy_init();
 *   - handles returned by appy_compile are immutable and may be launched from
 *     any thread; the caches behind appy_compile / appy_mirror are guarded by
 *     one mutex.
 */
#ifndef APPY_SM100_H
#define APPY_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define APPY_OK 0
#define APPY_ERR_CUDA (-1)
#define APPY_ERR_NVRTC (-2)
#define APPY_ERR_ARG (-3)
#define APPY_ERR_STATE (-4)

/* ---- runtime ----------------------------------------------------------- */

/* Make `device` current for the calling thread, create the backend's streams and
 * reduction workspaces on first use.  Replaces the implicit torch/Triton context
 * set-up of the reference (appy/dispatcher.py:36-41). */
int appy_init(int device);
int appy_shutdown(void);
const char* appy_last_error(void);
int appy_device_count(int* count);
/* sm_count, l2_bytes, cc (major*10+minor), total memory of `device` */
int appy_device_info(int device, int* sm_count, int* l2_bytes, int* cc, size_t* total_mem);
/* which: 0 = compute stream, 1 = copy stream of the current device */
int appy_get_stream(int which, void** stream);
int appy_sync(void* stream);
/* number of kernel launches issued through this library since load (or last reset) */
int64_t appy_launch_count(void);
void appy_reset_launch_count(void);

/* ---- memory ------------------------------------------------------------ */

/* Cached device allocator (replaces `tensor.to('cuda')` allocations,
 * host_passes/gen_data_movement.py:48-64). */
int appy_malloc(void** dptr, size_t bytes);
int appy_free(void* dptr);
int appy_trim(void);
int appy_memset(void* dptr, int value, size_t bytes, void* stream);
/* Pin a caller-owned host range in place so copies from it are true DMA. */
int appy_register_host(void* hptr, size_t bytes);
int appy_unregister_host(void* hptr);
/* Device mirror of a host range, created on first use and then reused
 * (the residency cache).  `created` (optional) is set to 1 when the mirror is new. */
int appy_mirror(const void* hptr, size_t bytes, void** dptr, int* created);
int appy_evict(const void* hptr);
int appy_h2d_async(void* dptr, const void* hptr, size_t bytes, void* stream);
int appy_d2h_async(void* hptr, const void* dptr, size_t bytes, void* stream);
/* Upload from PAGEABLE host memory through two pinned 8 MiB staging buffers: the CPU copy of one
 * chunk overlaps the DMA of the previous one.  Returns when the last chunk has been queued. */
int appy_h2d_staged(void* dptr, const void* hptr, size_t bytes, void* stream);
int appy_d2d_async(void* dst, const void* src, size_t bytes, void* stream);
/* One page (4096 bytes) of mapped, pinned host memory of the current device, for the cells of shared
 * scalars: *hptr is the host address, *dptr the address kernels use for the same bytes.  A kernel that
 * updates a cell with ONE read and ONE write at its very end (the ordered commit of the reduction
 * templates; atomics on host memory cross PCIe one by one) needs no upload and no download, only
 * appy_sync.  Replaces, for a shared scalar, the pair `__tg_s = __tc_s.to('cuda')` / `__tc_s.copy_(__tg_s)`
 * of the reference's generated host code (appy/backends/triton/passes/host_passes/gen_data_movement.py:14-96).
 * The page lives until appy_shutdown; the caller hands out its bytes. */
int appy_host_cells(void** hptr, void** dptr, size_t* bytes);

/* ---- compile / launch -------------------------------------------------- */

/* Compile CUDA C `src` with NVRTC for sm_100a and return a handle to the
 * extern "C" kernel `kernel_name`.  `options` is a '\n'-separated list of extra
 * NVRTC options (e.g. "-I<dir>\n-DNAME=1").  Results are cached in memory and,
 * when `cache_dir` is not NULL, as cubin files under that directory.
 * Replaces utils.load_module_from_str + Triton's JIT (appy/utils.py:46-80). */
int appy_compile(const char* src, const char* kernel_name, const char* options,
                 const char* cache_dir, void** handle);
/* NVRTC step of appy_compile alone: needs no GPU.  Used to syntax-check generated
 * sources on build machines. */
int appy_compile_check(const char* src, const char* kernel_name, const char* options,
                       size_t* cubin_bytes);
/* The cubin of appy_compile without loading it (needs no GPU), through the same on-disk cache:
 * `from_cache` receives 1 when a valid entry was found.  A cache entry is keyed by SHA-256 of the
 * source, the options, the contents of every -I directory, the NVRTC version and the target
 * architecture, and carries its key and length in a header: an entry that is truncated, torn or
 * belongs to another key is compiled afresh and replaced, never loaded.  (The reference leaves one
 * /tmp/appy_temp_<uuid>.py per compile and keeps no cache across processes, appy/utils.py:46-80.) */
int appy_compile_image(const char* src, const char* kernel_name, const char* options,
                       const char* cache_dir, size_t* cubin_bytes, int* from_cache);
/* compile log of the last appy_compile on this thread (warnings or errors) */
const char* appy_compile_log(void);
/* regs per thread, static shared bytes, max threads per block of a compiled kernel */
int appy_kernel_info(void* handle, int* regs, int* static_smem, int* max_threads);
int appy_occupancy(void* handle, int block, size_t dyn_smem, int* blocks_per_sm);
/* args: array of pointers to the kernel arguments, as for cudaLaunchKernel.
 * Replaces `_kernel[grid](..., num_warps=4)` (host_passes/gen_kernel_launch.py:56-69). */
int appy_launch(void* handle, unsigned grid, unsigned block, size_t dyn_smem, void** args,
                void* stream);
/* Launch `iters` times back to back between two events; returns total milliseconds.
 * Used by the block-size autotuner. */
int appy_time_launches(void* handle, unsigned grid, unsigned block, size_t dyn_smem, void** args,
                       void* stream, int warmup, int iters, float* total_ms);
/* Zero-initialised reduction workspace of the current device for `stream`
 * (ticket + per-CTA partial cells); `bytes` receives its size. */
int appy_workspace(void* stream, void** dptr, size_t* bytes);
/* Scratch buffer of at least `bytes` bytes of the current device for kernels queued on `stream`
 * (grow-only, one per stream, contents undefined).  The two-kernel CSR x dense template keeps
 * the pieces of rows cut by share boundaries there between its two launches; the reference's
 * lowering of that loop needs no such buffer because it sends every row through C itself, once
 * per non-zero (examples/06-spmm.py:4-11 after appy/backends/triton/passes/block_loop.py:77-159).
 * Growing the buffer waits for the work queued on the stream. */
int appy_scratch(void* stream, size_t bytes, void** dptr);

/* ---- multi-GPU partitioning (host-side integer work) ------------------- */

/* Split [lo, hi) into `parts` contiguous ranges whose cut points are multiples of
 * `align` (relative to 0); bounds has parts+1 entries. */
int appy_partition_range(int64_t lo, int64_t hi, int parts, int64_t align, int64_t* bounds);
/* Split rows [0, nrows) of a CSR matrix into `parts` contiguous row ranges with
 * near-equal non-zero counts; indptr is a host array of nrows+1 int32 or int64
 * entries (idx_bytes = 4 or 8). */
int appy_partition_rows(const void* indptr, int idx_bytes, int64_t nrows, int parts,
                        int64_t* bounds);
/* The same with a fixed cost per row beside its non-zeros: the ranges are balanced by
 * (non-zeros + row_cost * rows).  A row costs a kernel its pointer loads, its reduction and its store
 * whatever its length, so a range of many short rows takes longer than its non-zeros say; row_cost = 0
 * is appy_partition_rows.  (The reference is single-GPU; north_star asks for nnz-balanced row splits.) */
int appy_partition_rows_weighted(const void* indptr, int idx_bytes, int64_t nrows, int parts, int64_t row_cost,
                                 int64_t* bounds);
/* Row-length histogram of a device-resident indptr: counts[b] = rows whose length
 * lies in [2^(b-1), 2^b) (b = 0: empty rows), 32 bins; also the longest row. */
int appy_row_histogram(const void* d_indptr, int idx_bytes, int64_t nrows, int64_t* counts32,
                       int64_t* max_len, void* stream);

/* ---- peer mailboxes: combining shared(...) scalars across the GPUs of one box ----
 * No counterpart in the reference (it is single-GPU).  One process per GPU.  Each rank
 * creates a small mailbox in its own HBM and exports it as a CUDA IPC handle (64 bytes);
 * after the ranks exchanged their handles (any host transport), appy_p2p_open maps the
 * peers' mailboxes and returns the device descriptor that reduction kernels built with the
 * `combine="p2p"` option take as an argument: they write their totals into every rank's
 * mailbox over NVLink and fold the slots of their own mailbox in rank order, inside the
 * kernel's tail.  Waits are bounded (spin_limit polls of about 1 us per source rank, 0 = default
 * of 2^23); appy_p2p_status reports, and clears, whether one ran out.  all_handles == NULL opens
 * the context in loop-back: no peer process exists and the other ranks never post, which is how
 * the time-out path is exercised on a single GPU. */
int appy_p2p_create(int world, int rank, void** ctx, void* ipc_handle_out /* 64 bytes */);
int appy_p2p_open(void* ctx, const void* all_handles /* world x 64 bytes */, unsigned spin_limit,
                  void** device_descriptor);
/* The same for ranks that live in ONE process (a host that drives several GPUs itself, or several ranks on
 * one GPU whose kernels are queued one after another on one stream): contexts[r] is the context created for
 * rank r in this process; the mailboxes are wired by address, no IPC handle is opened.  With ranks on
 * different GPUs the caller enables peer access first.  Kernels of ranks that share a GPU must not wait for
 * one another: only the split-phase exchange, whose collect finds the words already posted, fits that use. */
int appy_p2p_open_local(void* ctx, void* const* contexts, unsigned spin_limit, void** device_descriptor);
int appy_p2p_status(void* ctx, int* timed_out);
int appy_p2p_destroy(void* ctx);
/* Combine `count` (1..4) device scalars of one type across all ranks, in place: every rank ends with
 * the fold, in rank order, of all ranks' values.  For callers of the prebuilt kernels, whose results
 * are per-GPU (the generated kernels do this exchange in their own tail).  `seq` numbers the
 * combining launches of this context: it starts at 1 and grows by one per launch that uses the
 * mailboxes (this call or a `combine="p2p"` kernel), identically on all ranks. */
enum { APPY_OP_ADD = 0, APPY_OP_MUL = 1, APPY_OP_MAX = 2, APPY_OP_MIN = 3 };
enum { APPY_F32 = 0, APPY_F64 = 1, APPY_I32 = 2, APPY_I64 = 3 };
int appy_p2p_combine(void* ctx, uint64_t seq, int op, int dtype, void* dvalues, int count, void* stream);
/* Split-phase form of the exchange: kernels generated with `combine="p2p", defer=True` end like a
 * single-GPU reduction (every CTA stores its partial); one warp at the start of the next such kernel folds
 * those partials and posts the GPU's totals, and one launch later collects the ranks' totals into the
 * shared(...) cells, so that no kernel ends waiting for the slowest rank or for an NVLink round trip.
 * appy_p2p_flush runs those two steps for launches that no later kernel serves (call it twice to complete
 * the last launch: once to fold and post it, once to collect it).  `pending` points to
 *   struct { record fold, coll; void* unused; }   with
 *   record = { uint64 seq (0 = none); int32 nv, grid, slot, pad; void* partials; void* cell[4];
 *              int32 op[4] (APPY_OP_*); int32 dtype[4] (APPY_F32..) }
 * as the kernels take it; a launch's partials live in the stream's workspace (appy_workspace) from byte
 * 256 + 8*4*65536 on, 8*4*4096 bytes per launch parity.  Collective like the kernels themselves: every
 * rank flushes at the same point of its launch sequence.
 * (The reference has no multi-GPU path; north_star asks for the combine of shared(...) scalars.) */
int appy_p2p_flush(void* ctx, const void* pending, void* stream);

/* ---- prebuilt instantiations of the five templates (float32 / int32) ----
 * Device pointers; asynchronous on `stream`.  Each is the canonical
 * instantiation of a template that appy_compile would otherwise build from
 * generated source. */

/* c[i] = a[i] + b[i]            — examples/01-vec_add.py:7-13 */
int appy_vec_add_f32(const float* da, const float* db, float* dc, int64_t n, void* stream);
/* *dresult += sum(a[0:n]), double accumulator — examples/02-vec_sum.py:5-11
 * (shared scalar is float64: appy/frontend/process_shared.py:37-41).
 * ordered != 0 selects the scheduling-independent commit. */
int appy_sum_f32(const float* da, int64_t n, double* dresult, int ordered, void* stream);
/* *dresult += sum(a[i] for mask[i])          — examples/04-masked_sum.py:7-23 */
int appy_masked_sum_f32(const float* da, const uint8_t* dmask, int64_t n, double* dresult,
                        int ordered, void* stream);
/* y[i] = sum_k data[k] * x[indices[k]], rows [row_lo,row_hi) — examples/03-spmv.py:5-16.
 * strategy: 0 = row-tile streaming, 2..32 = that many lanes per row. */
int appy_spmv_csr_f32(const float* ddata, const int32_t* dindptr, const int32_t* dindices,
                      const float* dx, float* dy, int64_t row_lo, int64_t row_hi, int strategy,
                      void* stream);
/* y[i] = sum_j alpha * A[i,j] * x[j]          — examples/05-gemv.py:7-17.
 * lda in elements; lanes: 32 = warp per row, 0 = CTA per pair of rows (the faster choice for
 * rows of a few thousand elements or more). */
int appy_gemv_f32(float alpha, const float* dA, int64_t lda, const float* dx, float* dy,
                  int64_t row_lo, int64_t row_hi, int64_t ncols, int lanes, void* stream);
/* C[i,:] = sum_k data[k] * B[indices[k],:]    — examples/06-spmm.py:4-11.
 * ncols <= 512; ldb/ldc in elements. */
int appy_spmm_csr_f32(const float* ddata, const int32_t* dindptr, const int32_t* dindices,
                      const float* dB, int64_t ldb, float* dC, int64_t ldc, int64_t row_lo,
                      int64_t row_hi, int ncols, void* stream);

/* ---- gather ceilings (measurement aids; no counterpart in the reference) ----
 * What the memory system delivers for the gathers of the two sparse kernels alone, so that their times can
 * be set against a measured floor instead of an assumed one.
 * appy_probe_row_gather_f32: every warp sums rows drows[k] (k < n, rounded down to whole blocks of 32 per
 * warp) of the row-major matrix dB, `row_floats` (128, 64 or 32) leading floats of each, eight rows in
 * flight per warp — the gathers of appy_spmm_csr_f32 without coefficients, row ends or output.
 * appy_probe_gather_f32: sums dx[didx[k]] — the gathers of appy_spmv_csr_f32 without values and rows.
 * dout receives one float per thread of the probe's grid (at most 512 * 8 * the number of SMs). */
int appy_probe_row_gather_f32(const float* dB, int64_t ldb, const int32_t* drows, int64_t n, int row_floats,
                              float* dout, void* stream);
int appy_probe_gather_f32(const float* dx, const int32_t* didx, int64_t n, float* dout, void* stream);

/* ---- allocation-free variant ---------------------------------------------
 * No counterpart in the reference (it has no native code and allocates through torch).
 *
 * The same value as appy_sum_f32(da, n, dresult, 1, stream) up to floating-point association:
 * *dresult += sum(a[0:n]) with a float64 accumulator and a commit that does not depend on CTA
 * scheduling, so the result is the same on every run for a given n and alignment of `da`; the
 * partial sums are formed per 8192-element tile here and per CTA of a persistent grid there, so the
 * two entry points may differ in the last bits (the test allows rtol 1e-5).  It is meant for
 * callers that must not allocate device memory where they reduce (inside a memory budget
 * fixed by a host application, between a pool allocator's sync points, or where the
 * device-wide synchronisation of a first-use cudaMalloc is unacceptable).  The scratch
 * (one ticket + one 8-byte partial per 8192-element tile) is a 128.25 KiB array inside the
 * library image, present on every GPU that loads the library.
 *   - n may not exceed 134,217,728 elements (16384 tiles) for a 16-byte aligned `da`, a
 *     quarter of that otherwise; longer inputs return APPY_ERR_ARG and launch nothing;
 *   - the first call on a device looks up the array's device address and keeps it; make that
 *     call before any stream capture begins.  A cudaDeviceReset by the host application makes
 *     the kept address stale: do not call this entry point again on that device afterwards;
 *   - all calls share the array: calls that can overlap on the GPU race, so keep them
 *     ordered (one stream, or events between streams);
 *   - no cudaMalloc / cudaFree / allocating library routine is called. */
int appy_sum_f32_noalloc(const float* da, int64_t n, double* dresult, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* APPY_SM100_H */
