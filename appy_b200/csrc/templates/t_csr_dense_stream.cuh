// T5 (streaming form): CSR x dense with the non-zeros, not the rows, dealt out to the warps
//
//   #pragma parallel for
//   for i in range(lo, hi):
//       start, end = indptr[i], indptr[i+1]
//       C[i, :] = init
//       for k in range(start, end):
//           C[i, :] += coef(k) * B[brow(k), :]
//
// (reference: examples/06-spmm.py:4-11.)
//
// The grid is one wave of resident CTAs.  The non-zeros of rows [lo, hi) are one contiguous
// span of the CSR arrays; it is cut into one equal share per warp of the grid, and a warp
// streams its share from start to end: 32 (coef, brow) pairs per coalesced load (fetched one
// block ahead), the C row in registers, and D B rows in flight at all times: the rows travel by
// asynchronous 16-byte copies (cp.async) into a ring of D slots in shared memory, one commit group
// per non-zero; before a row is folded the warp waits for the oldest group, and at once refills
// the slot with the row D non-zeros ahead.  A lane reads back only the 16 bytes it copied itself,
// so the ring needs no barrier, and the rows in flight cost no registers.  A warp therefore runs
// one long, uniform pipeline whatever the row lengths are: a matrix with a few very long rows
// and many short ones costs the same as a regular one, and no warp idles while a CTA starts
// up or drains.
//
// Row ends are found on the fly.  A warp keeps a window of 32 consecutive rows (lane j holds
// the start and end position of row window+j, relative to the share's first non-zero); for
// every block of 32 non-zeros the lanes whose row ends inside the block set the bit of the
// row's last non-zero and leave the row number in a 32-entry table in shared memory; the
// window moves on when its last row ends inside the block.  Rows without non-zeros never set
// a bit; the fix-up kernel below writes them.
//
// A row that lies wholly inside a share is stored straight from registers.  A row cut by a
// share boundary leaves partial rows in a scratch buffer: the warp in whose share the row
// begins writes a "tail", every later warp a "head" (a warp whose whole share lies inside one
// row writes only a head).  A second, small kernel adds the pieces of each cut row in share
// order and stores it, so there are no atomics and the result does not depend on scheduling.
//
//   struct Body {                                // same functor as t_csr_dense.cuh
//     typedef <T> Elt;
//     typedef <unsigned|i64> Off;
//     Elt   coef(i64 k) const;
//     Off   brow_off(i64 k) const;
//     const Elt* bbase() const;
//     Elt*  crow_ptr(i64 i) const;
//     Elt   init() const;
//   };
//
// Scratch layout (bytes): [0, 16) header {int workers}; [16, 16 + 16*workers) one record
// {head_row, head_closed, tail_row, unused} per worker (rows relative to lo, -1 = none);
// then, 256-byte aligned, workers x 2 partial rows of 32*V*T elements (head, tail).
#pragma once
#include "t_csr_dense.cuh"

struct appy_sd_meta {
  int head_row;      // row (relative to lo) of the partial in the head slot, -1 if none
  int head_closed;   // 1: that row ended inside this share; 0: it runs on into the next share
  int tail_row;      // row of the partial in the tail slot (the row begins in this share), -1 if none
  int pad;
};

APPY_DEV appy_sd_meta* appy_sd_metas(void* scratch) {
  return reinterpret_cast<appy_sd_meta*>(reinterpret_cast<char*>(scratch) + 16);
}
template <class Elt> APPY_DEV Elt* appy_sd_parts(void* scratch, i64 workers) {
  const size_t off = (16 + 16 * (size_t)workers + 255) / 256 * 256;
  return reinterpret_cast<Elt*>(reinterpret_cast<char*>(scratch) + off);
}
// bytes of scratch for `workers` warps and rows of `w` padded elements of `esize` bytes
#define APPY_SD_SCRATCH_BYTES(workers, w, esize) \
  ((16 + 16 * (size_t)(workers) + 255) / 256 * 256 + (size_t)(workers) * 2 * (size_t)(w) * (size_t)(esize))

// start/end of row `row` (relative to lo) as positions relative to ks, clamped to [-1, cap]
// (cap lies beyond the end of every block of the share, so a clamped end never falls inside one)
template <class IdxT>
APPY_DEV void appy_sd_row_span(const IdxT* __restrict__ indptr, i64 lo, int row, int nrows, i64 ks, int cap,
                               int& sr, int& er) {
  if (row < nrows) {
    const i64 a = (i64)appy_ldg1(indptr + lo + row) - ks, b = (i64)appy_ldg1(indptr + lo + row + 1) - ks;
    sr = a < -1 ? -1 : (a > cap ? cap : (int)a);
    er = b < -1 ? -1 : (b > cap ? cap : (int)b);
  } else {
    sr = er = 0x7fffffff;      // past the last row: never ends, never empty-tested
  }
}

// ---- asynchronous 4/8/16-byte copies global -> shared (cp.async), one group per non-zero ----
APPY_DEV unsigned appy_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
template <int BYTES> APPY_DEV void appy_cp_async(unsigned saddr, const void* g) {
  if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
  else if (BYTES == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(saddr), "l"(g) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(saddr), "l"(g) : "memory");
}
APPY_DEV void appy_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> APPY_DEV void appy_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
template <class T, int V> APPY_DEV appy_pack<T, V> appy_ld_shared(unsigned saddr) {
  union { unsigned r[4]; appy_pack<T, V> k; } u;
  if (sizeof(T) * V == 16)
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.r[0]), "=r"(u.r[1]), "=r"(u.r[2]), "=r"(u.r[3]) : "r"(saddr) : "memory");
  else if (sizeof(T) * V == 8)
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(u.r[0]), "=r"(u.r[1]) : "r"(saddr) : "memory");
  else
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.r[0]) : "r"(saddr) : "memory");
  return u.k;
}

// bytes of dynamic shared memory: the warps' rings of D rows, then 32 row numbers per warp
#define APPY_SD_SMEM_BYTES(nwarps, d, w, esize) ((size_t)(nwarps) * (d) * (w) * (esize) + (size_t)(nwarps) * 32 * 4)

// Copy of B row piece [off + lane*V + t*32*V, +V) for t < T into ring slot `slot` (this lane's own 16 bytes
// of every 512: a lane later reads back exactly what it copied, so the ring needs no barrier).
template <int V, int T, int NC, class Body>
APPY_DEV void appy_sd_fetch(const typename Body::Elt* blane, typename Body::Off off, unsigned slot_addr, int lane,
                            int ncols) {
  typedef typename Body::Elt Elt;
#pragma unroll
  for (int t = 0; t < T; ++t)
    if (NC > 0 || (t * 32 + lane) * V < ncols)
      appy_cp_async<(int)sizeof(Elt) * V>(slot_addr + t * 32 * V * (int)sizeof(Elt), blane + off + t * 32 * V);
}

// blockDim.x == 32*NWARPS; smem_raw: APPY_SD_SMEM_BYTES(NWARPS, D, 32*V*T, sizeof(Elt)) bytes, 16-byte aligned.
// D (rows in flight per warp) divides 32 and is at most 16.
// SMEM = false keeps the ring in registers instead (plain ld.global.nc into D packs per lane, refilled as
// they are folded; smem_raw then only holds the NWARPS*32 row numbers): half the traffic through the
// L1/shared-memory pipe, but the registers bound the rows in flight.  Measured on the 2^18-row, 128-column
// case: shared-memory ring 404 us whether the gathered rows fit L2 or not; register ring 441 us when they
// do not (134 MB of rows), 327 us when they do (34 MB).
template <int V, int T, int D, int NWARPS, int NC, bool SMEM, class IdxT, class Body>
APPY_DEV void appy_csr_dense_stream(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi, int ncols,
                                    void* scratch, void* smem_raw) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Off Off;
  const int W = 32 * V * T;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // this lane's first element of slot 0 of the warp's ring; slot j is j*W elements further
  const unsigned ring = SMEM ? appy_smem_addr(reinterpret_cast<Elt*>(smem_raw) + (size_t)warp * D * W + lane * V) : 0u;
  int* s_row = reinterpret_cast<int*>(reinterpret_cast<Elt*>(smem_raw) + (SMEM ? (size_t)NWARPS * D * W : 0)) + warp * 32;
  appy_pack<Elt, V> rr[SMEM ? 1 : D][T];      // the ring in registers (SMEM == false)
  const i64 workers = (i64)gridDim.x * NWARPS;
  const i64 w = (i64)blockIdx.x * NWARPS + warp;
  const int nrows = (int)(hi - lo);
  const i64 s = (i64)appy_ldg1(indptr + lo), e = (i64)appy_ldg1(indptr + hi);
  i64 chunk = ((e - s) + workers - 1) / workers;
  chunk = (chunk + 31) / 32 * 32;
  const i64 ks = s + w * chunk;
  const int n_tot = (ks >= e) ? 0 : (int)((e - ks < chunk) ? e - ks : chunk);
  appy_sd_meta* meta = appy_sd_metas(scratch) + w;     // written by lane 0 only
  if (lane == 0) {
    meta->head_row = meta->tail_row = -1;
    meta->head_closed = 0;
    if (w == 0) *reinterpret_cast<int*>(scratch) = (int)workers;
  }
  if (n_tot <= 0) return;
  const Elt* blane = body.bbase() + lane * V;
  // the first two blocks' coefficients and offsets, and the first D rows, travel while the start row is searched
  Elt my_c = Elt(0), nxt_c = Elt(0);
  Off my_off = 0, nxt_off = 0;
  if (lane < n_tot) {
    nxt_c = body.coef(ks + lane);
    nxt_off = body.brow_off(ks + lane);
  }
#pragma unroll
  for (int j = 0; j < D; ++j) {
    const Off o = appy_shfl<Off>(nxt_off, j, 32);
    if (SMEM) {
      if (j < n_tot) appy_sd_fetch<V, T, NC, Body>(blane, o, ring + j * W * (int)sizeof(Elt), lane, ncols);
      appy_cp_commit();
    } else if (j < n_tot) {
      appy_csr_dense_load<V, T, NC, Body>(blane, o, lane, ncols, rr[SMEM ? 0 : j]);
    }
  }
  // row that holds non-zero ks: the largest r with indptr[lo + r] <= ks (32 probes per round)
  int wbase = 0;
  {
    int len = nrows;                       // answer in [wbase, wbase + len)
    while (len > 1) {
      const int step = (len + 31) / 32;
      const int probe = wbase + (lane + 1) * step;
      const bool le = probe < wbase + len && (i64)appy_ldg1(indptr + lo + probe) <= ks;
      const int c = __popc(__ballot_sync(APPY_FULL_MASK, le));
      const int end = wbase + len;
      wbase += c * step;
      len = (end - wbase < step) ? end - wbase : step;
    }
  }
  int sr, er;
  appy_sd_row_span<IdxT>(indptr, lo, wbase + lane, nrows, ks, n_tot + 32, sr, er);
  bool entered = __shfl_sync(APPY_FULL_MASK, sr, 0) < 0;     // the open row began before ks
  appy_rowacc<V, T, Body> acc;
  acc.fill(entered ? Elt(0) : body.init());
  unsigned ends = 0;
  int n = 0;
  for (int kb = 0; kb < n_tot; kb += 32) {
    n = (n_tot - kb < 32) ? n_tot - kb : 32;
    my_c = nxt_c;
    my_off = nxt_off;
    if (kb + 32 + lane < n_tot) {          // next block's coefficients and offsets, one block ahead
      nxt_c = body.coef(ks + kb + 32 + lane);
      nxt_off = body.brow_off(ks + kb + 32 + lane);
    }
    // rows that end inside [kb, kb + 32): bit of their last non-zero, row number into the table
    // (D rows of this block are in flight already, so this bookkeeping costs no memory time)
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
    if (n == 32 && kb + 32 + D <= n_tot) {
      // Full block, and every refill of it exists: no position or range checks.  The block's coefficients
      // and offsets are rotated down by D lanes per group, so that the group's non-zeros sit in lanes
      // 0..D-1 and the D after them in lanes D..2D-1: every shuffle below has a constant source lane.
      Elt rc = my_c;
      Off ro = my_off;
#pragma unroll 1
      for (int q = 0; q < 32; q += D) {
        const unsigned m = (ends >> q) & ((1u << D) - 1u);          // row ends among this group's non-zeros
        const bool last = q + D == 32;                              // then the refills come from the next block
#pragma unroll
        for (int j = 0; j < D; ++j) {
          appy_pack<Elt, V> b[T];
          if (SMEM) {
            appy_cp_wait<D - 1>();           // the oldest of the D groups in flight has landed
#pragma unroll
            for (int t = 0; t < T; ++t)
              if (NC > 0 || (t * 32 + lane) * V < ncols)
                b[t] = appy_ld_shared<Elt, V>(ring + (j * W + t * 32 * V) * (int)sizeof(Elt));
          } else {
#pragma unroll
            for (int t = 0; t < T; ++t) b[t] = rr[SMEM ? 0 : j][t];
          }
          appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(rc, j, 32), b);
          if (m != 0 && ((m >> j) & 1u)) {
            const int row = s_row[q + j];
            if (entered) {     // the row was open when this share began: its piece goes to the head slot
              appy_csr_dense_park<V, T, Body>(appy_sd_parts<Elt>(scratch, workers) + (size_t)w * 2 * W, lane, acc);
              if (lane == 0) {
                meta->head_row = row;
                meta->head_closed = 1;
              }
              entered = false;
            } else {
              appy_csr_dense_store<V, T, NC, Body>(body, lo + row, lane, ncols, acc);
            }
            acc.fill(body.init());
          }
          const Off ahead_off = last ? appy_shfl<Off>(nxt_off, j, 32) : appy_shfl<Off>(ro, (j + D) & 31, 32);
          if (SMEM) {
            appy_sd_fetch<V, T, NC, Body>(blane, ahead_off, ring + j * W * (int)sizeof(Elt), lane, ncols);
            appy_cp_commit();
          } else {
            appy_csr_dense_load<V, T, NC, Body>(blane, ahead_off, lane, ncols, rr[SMEM ? 0 : j]);
          }
        }
        rc = appy_shfl<Elt>(rc, (lane + D) & 31, 32);
        ro = appy_shfl<Off>(ro, (lane + D) & 31, 32);
      }
    } else {
#pragma unroll 1
      for (int q = 0; q < 32; q += D) {
#pragma unroll
        for (int j = 0; j < D; ++j) {
          if (q + j < n) {
            appy_pack<Elt, V> b[T];
            if (SMEM) {
              appy_cp_wait<D - 1>();
#pragma unroll
              for (int t = 0; t < T; ++t)
                if (NC > 0 || (t * 32 + lane) * V < ncols)
                  b[t] = appy_ld_shared<Elt, V>(ring + (j * W + t * 32 * V) * (int)sizeof(Elt));
            } else {
#pragma unroll
              for (int t = 0; t < T; ++t) b[t] = rr[SMEM ? 0 : j][t];
            }
            appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(my_c, q + j, 32), b);
            if ((ends >> (q + j)) & 1u) {
              const int row = s_row[q + j];
              if (entered) {
                appy_csr_dense_park<V, T, Body>(appy_sd_parts<Elt>(scratch, workers) + (size_t)w * 2 * W, lane, acc);
                if (lane == 0) {
                  meta->head_row = row;
                  meta->head_closed = 1;
                }
                entered = false;
              } else {
                appy_csr_dense_store<V, T, NC, Body>(body, lo + row, lane, ncols, acc);
              }
              acc.fill(body.init());
            }
          }
          // refill the slot with the row D non-zeros ahead (from this block's offsets or the next block's)
          const int ahead = q + j + D;
          const Off o = appy_shfl<Off>(ahead < 32 ? my_off : nxt_off, ahead & 31, 32);
          if (SMEM) {
            if (kb + ahead < n_tot) appy_sd_fetch<V, T, NC, Body>(blane, o, ring + j * W * (int)sizeof(Elt), lane, ncols);
            appy_cp_commit();                  // one group per step, empty or not, keeps the count uniform
          } else if (kb + ahead < n_tot) {
            appy_csr_dense_load<V, T, NC, Body>(blane, o, lane, ncols, rr[SMEM ? 0 : j]);
          }
        }
      }
    }
  }
  if (SMEM) appy_cp_wait<0>();
  if (((ends >> (n - 1)) & 1u) == 0) {
    // the share ended inside a row: the first row of the window that reaches past the share
    const unsigned m = __ballot_sync(APPY_FULL_MASK, sr < er && er > n_tot);
    const int row = wbase + __ffs(m) - 1;
    Elt* part = appy_sd_parts<Elt>(scratch, workers) + (size_t)w * 2 * W;
    if (entered) {
      appy_csr_dense_park<V, T, Body>(part, lane, acc);
      if (lane == 0) {
        meta->head_row = row;
        meta->head_closed = 0;
      }
    } else {
      appy_csr_dense_park<V, T, Body>(part + W, lane, acc);
      if (lane == 0) meta->tail_row = row;
    }
  }
}

// Second kernel: rows without non-zeros get `init`; every row cut by share boundaries is summed in
// share order (tail of the share it begins in, then the heads of the following shares up to the one
// it ends in) and stored.  Any grid; blockDim.x a multiple of 32.
template <int V, int T, int NC, class IdxT, class Body>
APPY_DEV void appy_csr_dense_fixup(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi, int ncols,
                                   void* scratch) {
  typedef typename Body::Elt Elt;
  const int W = 32 * V * T;
  const int lane = threadIdx.x & 31;
  const i64 gw = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((i64)gridDim.x * blockDim.x) >> 5;
  const i64 nrows = hi - lo;
  for (i64 base = gw * 32; base < nrows; base += nw * 32) {
    const i64 row = base + lane;
    const bool empty = row < nrows && appy_ldg1(indptr + lo + row) == appy_ldg1(indptr + lo + row + 1);
    unsigned m = __ballot_sync(APPY_FULL_MASK, empty);
    while (m) {
      const int j = __ffs(m) - 1;
      m &= m - 1;
      appy_rowacc<V, T, Body> z;
      z.fill(body.init());
      appy_csr_dense_store<V, T, NC, Body>(body, lo + base + j, lane, ncols, z);
    }
  }
  const int workers = *reinterpret_cast<const int*>(scratch);
  const appy_sd_meta* metas = appy_sd_metas(scratch);
  const Elt* parts = appy_sd_parts<Elt>(scratch, workers);
  for (i64 w = gw; w < workers; w += nw) {
    const int row = metas[w].tail_row;
    if (row < 0) continue;
    appy_rowacc<V, T, Body> sum;
    const Elt* p = parts + ((size_t)w * 2 + 1) * W;
#pragma unroll
    for (int t = 0; t < T; ++t)
#pragma unroll
      for (int x = 0; x < V; ++x) sum.a[t].v[x] = p[(t * 32 + lane) * V + x];
    for (i64 v = w + 1; v < workers; ++v) {
      if (metas[v].head_row != row) break;
      p = parts + (size_t)v * 2 * W;
#pragma unroll
      for (int t = 0; t < T; ++t)
#pragma unroll
        for (int x = 0; x < V; ++x) sum.a[t].v[x] = sum.a[t].v[x] + p[(t * 32 + lane) * V + x];
      if (metas[v].head_closed) break;
    }
    appy_csr_dense_store<V, T, NC, Body>(body, lo + row, lane, ncols, sum);
  }
}
