// T3 (streaming form): CSR row reduction with the non-zeros, not the rows, dealt out to the warps
//
//   #pragma parallel for
//   for i in range(lo, hi):
//       start, end = indptr[i], indptr[i+1]
//       s = <identity>
//       #pragma simd
//       for k in range(start, end):
//           s = s (op) term(k)              e.g. A_data[k] * x[A_indices[k]]
//       finish(i, s)                        e.g. y[i] = s
//
// (reference: examples/03-spmv.py:5-16, tests/integration/triton/tutorial/test_spmv.py:10-21.)
//
// The grid is one wave of resident CTAs.  The non-zeros of rows [lo, hi) are one contiguous span
// of the CSR arrays; it is cut into one equal share per warp, and a warp walks its share in
// blocks of 32 non-zeros: lane j evaluates term(k) of the block's j-th non-zero (coalesced value
// and index loads, one gather), U blocks in flight.  Every lane does the same amount of work
// whatever the row lengths are, so a matrix with a long-tailed row-length distribution runs at
// the speed of a regular one with the same number of non-zeros.
//
// Rows are put back together inside the warp.  The row ends inside a block are found as in
// t_csr_dense_stream.cuh (a window of 32 consecutive rows held one per lane, a bit mask of the
// positions at which a row ends, the row numbers in a 32-entry table in shared memory); a
// segmented inclusive scan by shuffles then leaves, at every such position, the fold of that
// row's terms within the block; the first row end of a block also takes the carry of the row
// that was open when the block began.  A row cut by a share boundary leaves its pieces in a
// scratch buffer ("tail" in the share it begins in, "head" in the following ones) and a second,
// small kernel folds them in share order and runs finish(); it also runs finish() with the
// operator's identity for rows without non-zeros.  No atomics; the result does not depend on
// scheduling.  The terms of a row are folded as a tree per block and block by block in order,
// not one by one as the sequential loop does.
//
//   struct Body {                               // same functor as t_csr_rows.cuh
//     typedef <T> Acc;  typedef <op> Op;
//     Acc  term(i64 k) const;
//     void finish(i64 i, Acc total) const;
//   };
//
// Scratch layout (bytes): [0, 16) header {int workers}; [16, 16 + 16*workers) one record
// {head_row, head_closed, tail_row, unused} per worker (rows relative to lo, -1 = none); then,
// 256-byte aligned, workers x 2 cells of 8 bytes (head, tail).
#pragma once
#include "t_csr_dense_stream.cuh"

#define APPY_SR_SCRATCH_BYTES(workers) ((16 + 16 * (size_t)(workers) + 255) / 256 * 256 + (size_t)(workers) * 16)

template <class Acc> APPY_DEV Acc* appy_sr_cell(void* scratch, i64 workers, i64 w, int slot) {
  const size_t off = (16 + 16 * (size_t)workers + 255) / 256 * 256;
  return reinterpret_cast<Acc*>(reinterpret_cast<char*>(scratch) + off + ((size_t)w * 2 + slot) * 8);
}

// blockDim.x == 32*NWARPS; smem_raw holds NWARPS*32 ints.
template <int NWARPS, int U, class IdxT, class Body>
APPY_DEV void appy_csr_rows_stream(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi, void* scratch,
                                   void* smem_raw) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int* s_row = reinterpret_cast<int*>(smem_raw) + warp * 32;
  const i64 workers = (i64)gridDim.x * NWARPS;
  const i64 w = (i64)blockIdx.x * NWARPS + warp;
  const int nrows = (int)(hi - lo);
  const i64 s = (i64)appy_ldg1(indptr + lo), e = (i64)appy_ldg1(indptr + hi);
  i64 chunk = ((e - s) + workers - 1) / workers;
  chunk = (chunk + 32 * U - 1) / (32 * U) * (32 * U);
  const i64 ks = s + w * chunk;
  const int n_tot = (ks >= e) ? 0 : (int)((e - ks < chunk) ? e - ks : chunk);
  appy_sd_meta meta;
  meta.head_row = meta.tail_row = -1;
  meta.head_closed = meta.pad = 0;
  if (w == 0 && lane == 0) *reinterpret_cast<int*>(scratch) = (int)workers;
  if (n_tot > 0) {
    // row that holds non-zero ks: the largest r with indptr[lo + r] <= ks (32 probes per round)
    int r0 = 0;
    {
      int len = nrows;
      while (len > 1) {
        const int step = (len + 31) / 32;
        const int probe = r0 + (lane + 1) * step;
        const bool le = probe < r0 + len && (i64)appy_ldg1(indptr + lo + probe) <= ks;
        const int c = __popc(__ballot_sync(APPY_FULL_MASK, le));
        const int end = r0 + len;
        r0 += c * step;
        len = (end - r0 < step) ? end - r0 : step;
      }
    }
    int wbase = r0, sr, er;
    appy_sd_row_span<IdxT>(indptr, lo, wbase + lane, nrows, ks, n_tot + 32, sr, er);
    bool entered = __shfl_sync(APPY_FULL_MASK, sr, 0) < 0;     // the open row began before ks
    Acc carry = Op::template id<Acc>();                        // fold of the open row's terms so far
    unsigned ends = 0;
    int n = 0;
    for (int kb0 = 0; kb0 < n_tot; kb0 += 32 * U) {
      Acc v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int p = kb0 + u * 32 + lane;
        v[u] = (p < n_tot) ? body.term(ks + p) : Op::template id<Acc>();
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int kb = kb0 + u * 32;
        if (kb >= n_tot) break;
        n = (n_tot - kb < 32) ? n_tot - kb : 32;
        // rows that end inside [kb, kb + 32): bit of their last non-zero, row number into the table
        ends = 0;
        __syncwarp();
        for (;;) {
          const bool has = sr < er && er > kb && er <= kb + 32;
          if (has) s_row[er - 1 - kb] = wbase + lane;
          ends |= __reduce_or_sync(APPY_FULL_MASK, has ? 1u << (er - 1 - kb) : 0u);
          if (__shfl_sync(APPY_FULL_MASK, er, 31) > kb + 32) break;   // the window reaches past this block
          wbase += 32;
          appy_sd_row_span<IdxT>(indptr, lo, wbase + lane, nrows, ks, n_tot + 32, sr, er);
        }
        __syncwarp();
        // segmented inclusive scan: a lane's segment begins after the last row end below it
        const int seg0 = 32 - __clz(ends & ((1u << lane) - 1u));
        Acc x = v[u];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const Acc t = appy_shfl_up<Acc>(x, d);
          if (lane - d >= seg0) x = Op::template op<Acc>(t, x);
        }
        if (ends) {
          const int first = __ffs(ends) - 1;
          if ((ends >> lane) & 1u) {
            const Acc total = (lane == first) ? Op::template op<Acc>(carry, x) : x;
            if (lane == first && entered)      // the row was open when this share began: its piece is a head
              *appy_sr_cell<Acc>(scratch, workers, w, 0) = total;
            else
              body.finish(lo + s_row[lane], total);
          }
          if (entered) {
            meta.head_row = s_row[first];
            meta.head_closed = 1;
            entered = false;
          }
          carry = Op::template id<Acc>();
        }
        // what follows the last row end of the block belongs to a row that is still open
        const Acc open = appy_shfl<Acc>(x, 31, 32);
        if (((ends >> (n - 1)) & 1u) == 0) carry = Op::template op<Acc>(carry, open);
      }
    }
    if (((ends >> (n - 1)) & 1u) == 0) {
      // the share ended inside a row: the first row of the window that reaches past the share
      const unsigned m = __ballot_sync(APPY_FULL_MASK, sr < er && er > n_tot);
      const int row = wbase + __ffs(m) - 1;
      if (entered) {
        if (lane == 0) *appy_sr_cell<Acc>(scratch, workers, w, 0) = carry;
        meta.head_row = row;
        meta.head_closed = 0;
      } else {
        if (lane == 0) *appy_sr_cell<Acc>(scratch, workers, w, 1) = carry;
        meta.tail_row = row;
      }
    }
  }
  if (lane == 0) appy_sd_metas(scratch)[w] = meta;
}

// Second kernel: finish() with the identity for rows without non-zeros, and for every row cut by share
// boundaries the fold of its pieces in share order.  Any grid.
template <class IdxT, class Body>
APPY_DEV void appy_csr_rows_fixup(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi, void* scratch) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  const i64 gt = (i64)blockIdx.x * blockDim.x + threadIdx.x, nt = (i64)gridDim.x * blockDim.x;
  for (i64 i = lo + gt; i < hi; i += nt)
    if (appy_ldg1(indptr + i) == appy_ldg1(indptr + i + 1)) body.finish(i, Op::template id<Acc>());
  const int workers = *reinterpret_cast<const int*>(scratch);
  const appy_sd_meta* metas = appy_sd_metas(scratch);
  for (i64 w = gt; w < workers; w += nt) {
    const int row = metas[w].tail_row;
    if (row < 0) continue;
    Acc total = *appy_sr_cell<Acc>(scratch, workers, w, 1);
    for (i64 v = w + 1; v < workers; ++v) {
      if (metas[v].head_row != row) break;
      total = Op::template op<Acc>(total, *appy_sr_cell<Acc>(scratch, workers, v, 0));
      if (metas[v].head_closed) break;
    }
    body.finish(lo + row, total);
  }
}
