// T3: CSR row loop (sparse row reduction)
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
// (reference: examples/03-spmv.py:5-16 and
// tests/integration/triton/tutorial/test_spmv.py:10-21; its Triton lowering gives
// every row a 128-thread program and a 256-wide masked tile, so a 16-element row
// leaves 94 % of the lanes idle.)
//
// Two lowerings are provided; the dispatcher picks from the row-length histogram.
//
// (1) appy_csr_stream — row-tile streaming.  A CTA owns BLOCK consecutive rows.
//     Because CSR rows are contiguous, the tile's non-zeros are one contiguous
//     span [indptr[r0], indptr[r0+BLOCK)): all threads stream it with perfectly
//     coalesced loads, evaluate term(k) and park the products in shared memory;
//     then thread t folds the products of row r0+t.  Rows longer than LONG are
//     folded by a whole warp instead.  Spans longer than CHUNK are processed in
//     several passes, so one very long row is simply streamed by the whole CTA:
//     no row binning, no atomics, and the result does not depend on scheduling.
//
// (2) appy_csr_vector — a group of G lanes per row (G = 1..32), with rows that are
//     too long for a group deferred to a warp, and rows too long for a warp to the
//     whole CTA.
//
//   struct Body {
//     typedef <T> Acc;  typedef <op> Op;
//     Acc  term(i64 k) const;
//     void finish(i64 i, Acc total) const;
//   };
#pragma once
#include "t_group.cuh"

template <int BLOCK, int CHUNK, int LONG, class IdxT, class Body>
APPY_DEV void appy_csr_stream(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi,
                              void* smem_raw) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  // shared memory: products first (largest alignment), then the row pointers
  Acc* prod = reinterpret_cast<Acc*>(smem_raw);
  i64* s_ptr = reinterpret_cast<i64*>(prod + CHUNK);
  const int tid = threadIdx.x;
  const int lane = tid & 31;

  for (i64 r0 = lo + (i64)blockIdx.x * BLOCK; r0 < hi; r0 += (i64)gridDim.x * BLOCK) {
    const int nr = (hi - r0 < BLOCK) ? (int)(hi - r0) : BLOCK;
    if (tid < nr) s_ptr[tid] = (i64)appy_ldg1(indptr + r0 + tid);
    if (tid == 0) s_ptr[nr] = (i64)appy_ldg1(indptr + r0 + nr);
    __syncthreads();
    const i64 s = s_ptr[0], e = s_ptr[nr];
    const i64 my_a = (tid < nr) ? s_ptr[tid] : e;
    const i64 my_b = (tid < nr) ? s_ptr[tid + 1] : e;
    Acc acc = Op::template id<Acc>();

    for (i64 c = s; c < e; c += CHUNK) {
      const i64 ce = (c + CHUNK < e) ? c + CHUNK : e;
      // ---- stream: coalesced over the span, 4 independent gathers in flight per thread
      i64 k = c + tid;
      for (; k + 3 * BLOCK < ce; k += 4 * BLOCK) {
        const Acc t0 = body.term(k);
        const Acc t1 = body.term(k + BLOCK);
        const Acc t2 = body.term(k + 2 * BLOCK);
        const Acc t3 = body.term(k + 3 * BLOCK);
        prod[k - c] = t0;
        prod[k - c + BLOCK] = t1;
        prod[k - c + 2 * BLOCK] = t2;
        prod[k - c + 3 * BLOCK] = t3;
      }
      for (; k < ce; k += BLOCK) prod[k - c] = body.term(k);
      __syncthreads();
      // ---- fold: thread t owns row r0+t; the part of it that lies in this chunk
      const i64 a64 = my_a > c ? my_a : c;
      const i64 b64 = my_b < ce ? my_b : ce;
      const int a = (int)(a64 - c), b = (int)(b64 - c);
      const bool is_long = (b - a) > LONG;
      if (!is_long) {
        for (int q = a; q < b; ++q) acc = Op::template op<Acc>(acc, prod[q]);
      }
      unsigned longmask = __ballot_sync(APPY_FULL_MASK, is_long);
      while (longmask) {
        const int src = __ffs(longmask) - 1;
        longmask &= longmask - 1;
        const int ra = __shfl_sync(APPY_FULL_MASK, a, src);
        const int rb = __shfl_sync(APPY_FULL_MASK, b, src);
        Acc p = Op::template id<Acc>();
        for (int q = ra + lane; q < rb; q += 32) p = Op::template op<Acc>(p, prod[q]);
        p = appy_group_reduce<Op, 32, Acc>(p);
        if (lane == src) acc = Op::template op<Acc>(acc, p);
      }
      __syncthreads();
    }
    if (tid < nr) body.finish(r0 + tid, acc);
    // s_ptr is rewritten at the top of the next tile; the barrier that ends the last
    // chunk (or the one after the s_ptr loads when the span is empty) orders it.
    if (e <= s) __syncthreads();
  }
}

// fold non-zeros [s, e) of one row with `gs` lanes striding from `lane`; two gathers in flight
template <class Body>
APPY_DEV typename Body::Acc appy_csr_fold(const Body& body, i64 s, i64 e, int lane, int gs) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  Acc a0 = Op::template id<Acc>(), a1 = Op::template id<Acc>();
  Acc a2 = Op::template id<Acc>(), a3 = Op::template id<Acc>();
  i64 k = s + lane;
  for (; k + 3 * gs < e; k += 4 * gs) {
    const Acc t0 = body.term(k);
    const Acc t1 = body.term(k + gs);
    const Acc t2 = body.term(k + 2 * gs);
    const Acc t3 = body.term(k + 3 * gs);
    a0 = Op::template op<Acc>(a0, t0);
    a1 = Op::template op<Acc>(a1, t1);
    a2 = Op::template op<Acc>(a2, t2);
    a3 = Op::template op<Acc>(a3, t3);
  }
  for (; k < e; k += gs) a0 = Op::template op<Acc>(a0, body.term(k));
  return Op::template op<Acc>(Op::template op<Acc>(a0, a1), Op::template op<Acc>(a2, a3));
}

// (2) appy_csr_vector: a CTA owns ROWS consecutive rows.
//   phase 1: groups of G lanes take the rows whose length is <= T_WARP;
//   phase 2: rows in (T_WARP, T_BLOCK] are taken by one warp each;
//   phase 3: rows longer than T_BLOCK are taken by the whole CTA, one after another.
// Deferred rows are queued in shared memory, so no row list has to be prepared by
// the host and the per-row result does not depend on scheduling.
// blockDim.x == BLOCK; shared memory: (2*ROWS + 2) ints + 32 Acc.
template <int G, int BLOCK, int ROWS, int T_WARP, int T_BLOCK, class IdxT, class Body>
APPY_DEV void appy_csr_vector(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi,
                              void* smem_raw) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  Acc* s_red = reinterpret_cast<Acc*>(smem_raw);            // 32 cells for the CTA reduction
  int* s_cnt = reinterpret_cast<int*>(s_red + 32);          // [0] warp-queue size, [1] CTA-queue size
  int* s_q1 = s_cnt + 2;                                    // rows for phase 2
  int* s_q2 = s_q1 + ROWS;                                  // rows for phase 3
  appy_grp<G> g;
  g.init(nullptr);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int GPB = BLOCK / G;                                // groups per CTA

  for (i64 r0 = lo + (i64)blockIdx.x * ROWS; r0 < hi; r0 += (i64)gridDim.x * ROWS) {
    if (tid < 2) s_cnt[tid] = 0;
    __syncthreads();
    const int nr = (hi - r0 < ROWS) ? (int)(hi - r0) : ROWS;
    // ---- phase 1
    for (int j = tid / G; j < nr; j += GPB) {
      const i64 i = r0 + j;
      const i64 s = (i64)appy_ldg1(indptr + i), e = (i64)appy_ldg1(indptr + i + 1);
      const i64 len = e - s;
      if (len > T_WARP) {
        if (g.lane == 0) {
          if (len > T_BLOCK) s_q2[atomicAdd(&s_cnt[1], 1)] = j;
          else s_q1[atomicAdd(&s_cnt[0], 1)] = j;
        }
        continue;
      }
      Acc a = appy_csr_fold<Body>(body, s, e, g.lane, G);
      a = g.template reduce<Op, Acc>(a);
      if (g.lane == 0) body.finish(i, a);
    }
    __syncthreads();
    // ---- phase 2: a warp per row
    const int n1 = s_cnt[0], n2 = s_cnt[1];
    for (int q = warp; q < n1; q += BLOCK / 32) {
      const i64 i = r0 + s_q1[q];
      const i64 s = (i64)appy_ldg1(indptr + i), e = (i64)appy_ldg1(indptr + i + 1);
      Acc a = appy_csr_fold<Body>(body, s, e, lane, 32);
      a = appy_group_reduce<Op, 32, Acc>(a);
      if (lane == 0) body.finish(i, a);
    }
    // ---- phase 3: the CTA per row
    for (int q = 0; q < n2; ++q) {
      const i64 i = r0 + s_q2[q];
      const i64 s = (i64)appy_ldg1(indptr + i), e = (i64)appy_ldg1(indptr + i + 1);
      Acc a = appy_csr_fold<Body>(body, s, e, tid, BLOCK);
      a = appy_block_reduce<Op, Acc>(a, s_red);
      if (tid == 0) body.finish(i, a);
    }
    __syncthreads();
  }
}
