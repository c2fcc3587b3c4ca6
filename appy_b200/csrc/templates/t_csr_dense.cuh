// T5: CSR x dense (sparse row times dense matrix, row-slice accumulation)
//
//   #pragma parallel for
//   for i in range(lo, hi):
//       start, end = indptr[i], indptr[i+1]
//       C[i, :] = init
//       for k in range(start, end):
//           C[i, :] += coef(k) * B[brow(k), :]
//
// (reference: examples/06-spmm.py:4-11.  Its slice statements become 256-lane simd
// loops, so the C row makes a global-memory round trip for every non-zero.)
//
// Here the C row lives in registers for the whole k loop: lane l of a warp holds
// columns [l*V + t*32*V, +V) for t = 0..T-1 (32*V*T >= ncols), so a B row is fetched
// by one coalesced 16-byte load per lane and C is written once.
//
// Work is balanced by non-zeros, not by rows.  A CTA owns R consecutive rows; in CSR
// their non-zeros are one contiguous span, which is cut into NWARPS equal shares.
// Each warp streams its share: 32 (coef, brow) pairs per coalesced load, handed round
// by shuffle, D B-row gathers in flight.  Row boundaries are crossed on the fly.  A
// row that lies wholly inside a share is stored straight from registers; a row cut
// by a share boundary leaves a partial row in shared memory (at most two per warp:
// the one entering and the one leaving its share), and after a barrier the partials
// of each cut row are added in warp order and stored.  So a very long row is simply
// split over the warps of its CTA, short rows never drain the pipeline, there are no
// atomics, and the result does not depend on scheduling.
//
//   struct Body {
//     typedef <T> Elt;
//     typedef <unsigned|i64> Off;              // element offset of a B row (32-bit when B is small enough)
//     Elt   coef(i64 k) const;                 // A_data[k]
//     Off   brow_off(i64 k) const;             // A_indices[k] * (row stride of B)
//     const Elt* bbase() const;                // &B[0, 0]
//     Elt*  crow_ptr(i64 i) const;             // &C[i, 0]
//     Elt   init() const;
//   };
#pragma once
#include "appy_device.cuh"

template <int V, int T, class Body>
struct appy_rowacc {
  typedef typename Body::Elt Elt;
  appy_pack<Elt, V> a[T];
  APPY_DEV void fill(Elt v) {
#pragma unroll
    for (int t = 0; t < T; ++t)
#pragma unroll
      for (int x = 0; x < V; ++x) a[t].v[x] = v;
  }
};

// NC > 0: the number of columns is the compile-time constant NC and equals 32*V*T exactly
// (no column guard); NC == 0: `ncols` is a run-time value and every access is guarded.
template <int V, int T, int NC, class Body>
APPY_DEV void appy_csr_dense_load(const typename Body::Elt* blane, typename Body::Off off, int lane, int ncols,
                                  appy_pack<typename Body::Elt, V> (&b)[T]) {
  typedef typename Body::Elt Elt;
  const Elt* p = blane + off;
#pragma unroll
  for (int t = 0; t < T; ++t) {
    if (NC > 0 || (t * 32 + lane) * V < ncols) b[t] = appy_ld_nc<Elt, V>(p + t * 32 * V);
  }
}

template <int V, int T, class Body>
APPY_DEV void appy_csr_dense_fma(appy_rowacc<V, T, Body>& acc, typename Body::Elt c,
                                 const appy_pack<typename Body::Elt, V> (&b)[T]) {
#pragma unroll
  for (int t = 0; t < T; ++t)
#pragma unroll
    for (int x = 0; x < V; ++x) acc.a[t].v[x] = acc.a[t].v[x] + c * b[t].v[x];
}

template <int V, int T, int NC, class Body>
APPY_DEV void appy_csr_dense_store(const Body& body, i64 i, int lane, int ncols,
                                   const appy_rowacc<V, T, Body>& acc) {
  typedef typename Body::Elt Elt;
  Elt* p = body.crow_ptr(i);
#pragma unroll
  for (int t = 0; t < T; ++t) {
    const int col = (t * 32 + lane) * V;
    if (NC > 0 || col < ncols) appy_st_cs<Elt, V>(p + col, acc.a[t]);
  }
}

template <int V, int T, class Body>
APPY_DEV void appy_csr_dense_park(typename Body::Elt* dst, int lane, const appy_rowacc<V, T, Body>& acc) {
#pragma unroll
  for (int t = 0; t < T; ++t)
#pragma unroll
    for (int x = 0; x < V; ++x) dst[(t * 32 + lane) * V + x] = acc.a[t].v[x];
}

// shared memory bytes needed by appy_csr_dense
template <int V, int T, int NWARPS, int R, class Elt>
struct appy_csr_dense_smem {
  static const int bytes = NWARPS * 2 * 32 * V * T * (int)sizeof(Elt) + (int)sizeof(i64) * (R + 1) +
                           (int)sizeof(int) * 2 * NWARPS;
};

// One group of up to D non-zeros of the current 32-wide block: D gathers are issued, then folded in
// order; after a non-zero that ends its row (bit set in `ends`) the row is written out.
// GUARD = false is the fast path for a full block (all 32 positions valid).
template <int V, int T, int D, int NC, bool GUARD, class Body>
APPY_DEV void appy_csr_dense_group(const Body& body, const typename Body::Elt* blane, int q, int n, unsigned ends,
                                   typename Body::Elt my_c, typename Body::Off my_off, int my_row, i64 r0,
                                   bool& entered, typename Body::Elt* park0, int* tag0, int lane, int ncols,
                                   appy_rowacc<V, T, Body>& acc) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Off Off;
  appy_pack<Elt, V> b[D][T];
#pragma unroll
  for (int j = 0; j < D; ++j)
    if (!GUARD || q + j < n)
      appy_csr_dense_load<V, T, NC, Body>(blane, appy_shfl<Off>(my_off, q + j, 32), lane, ncols, b[j]);
#pragma unroll
  for (int j = 0; j < D; ++j) {
    if (!GUARD || q + j < n) {
      appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(my_c, q + j, 32), b[j]);
      if ((ends >> (q + j)) & 1u) {
        const int row = __shfl_sync(APPY_FULL_MASK, my_row, q + j, 32);
        if (entered) {   // the row was already open when this warp's share began: park the partial
          appy_csr_dense_park<V, T, Body>(park0, lane, acc);
          if (lane == 0) *tag0 = row;
          entered = false;
        } else {
          appy_csr_dense_store<V, T, NC, Body>(body, r0 + row, lane, ncols, acc);
        }
        acc.fill(body.init());
      }
    }
  }
}

// Rolling variant of the group above: `ring` always holds the gathers of the next D non-zeros.
// Each pack is folded and at once refilled with the gather D positions ahead (from this block's
// offsets, or from the next block's, which were fetched one block earlier), so the number of
// gathers in flight does not drop to zero between groups.
template <int V, int T, int D, int NC, bool GUARD, class Body>
APPY_DEV void appy_csr_dense_roll(const Body& body, const typename Body::Elt* blane, i64 kb, i64 ke, int q, int n,
                                  unsigned ends, typename Body::Elt my_c, typename Body::Off my_off,
                                  typename Body::Off nxt_off, int my_row, i64 r0, bool& entered,
                                  typename Body::Elt* park0, int* tag0, int lane, int ncols,
                                  appy_pack<typename Body::Elt, V> (&ring)[D][T], appy_rowacc<V, T, Body>& acc) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Off Off;
  const Off src_off = (q + D < 32) ? my_off : nxt_off;
#pragma unroll
  for (int j = 0; j < D; ++j) {
    if (!GUARD || q + j < n) {
      appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(my_c, q + j, 32), ring[j]);
      if ((ends >> (q + j)) & 1u) {
        const int row = __shfl_sync(APPY_FULL_MASK, my_row, q + j, 32);
        if (entered) {
          appy_csr_dense_park<V, T, Body>(park0, lane, acc);
          if (lane == 0) *tag0 = row;
          entered = false;
        } else {
          appy_csr_dense_store<V, T, NC, Body>(body, r0 + row, lane, ncols, acc);
        }
        acc.fill(body.init());
      }
      if (kb + q + j + D < ke)
        appy_csr_dense_load<V, T, NC, Body>(blane, appy_shfl<Off>(src_off, (q + j + D) & 31, 32), lane, ncols, ring[j]);
    }
  }
}

// blockDim.x == 32*NWARPS.  ROLL selects the rolling gather pipeline.
template <int V, int T, int D, int NWARPS, int R, int NC, bool ROLL, class IdxT, class Body>
APPY_DEV void appy_csr_dense(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi,
                             int ncols, void* smem_raw) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Off Off;
  const int W = 32 * V * T;                                          // padded row width
  Elt* s_part = reinterpret_cast<Elt*>(smem_raw);                    // [NWARPS][2][W]
  i64* s_ptr = reinterpret_cast<i64*>(s_part + NWARPS * 2 * W);      // [R+1] row starts
  int* s_tag = reinterpret_cast<int*>(s_ptr + (R + 1));              // [NWARPS][2] row of each partial
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const Elt* blane = body.bbase() + lane * V;

  for (i64 r0 = lo + (i64)blockIdx.x * R; r0 < hi; r0 += (i64)gridDim.x * R) {
    const int nr = (hi - r0 < R) ? (int)(hi - r0) : R;
    for (int t = threadIdx.x; t <= nr; t += 32 * NWARPS) s_ptr[t] = (i64)appy_ldg1(indptr + r0 + t);
    if (threadIdx.x < 2 * NWARPS) s_tag[threadIdx.x] = -1;
    __syncthreads();
    const i64 s = s_ptr[0], e = s_ptr[nr];
    // rows without non-zeros are just `init`
    for (int j = warp; j < nr; j += NWARPS) {
      if (s_ptr[j + 1] == s_ptr[j]) {
        appy_rowacc<V, T, Body> z;
        z.fill(body.init());
        appy_csr_dense_store<V, T, NC, Body>(body, r0 + j, lane, ncols, z);
      }
    }
    // this warp's share [ks, ke) of the tile's non-zeros
    i64 chunk = ((e - s) + NWARPS - 1) / NWARPS;
    chunk = (chunk + 31) / 32 * 32;
    const i64 ks = s + (i64)warp * chunk;
    const i64 ke = (ks + chunk < e) ? ks + chunk : e;
    if (ks < ke) {
      appy_rowacc<V, T, Body> acc;
      bool entered;       // the open row began before ks (its first part belongs to another warp)
      {
        int row = 0, hi_r = nr;      // largest row with s_ptr[row] <= ks: the row that holds non-zero ks
        while (hi_r - row > 1) {
          const int mid = (row + hi_r) >> 1;
          if (s_ptr[mid] <= ks) row = mid; else hi_r = mid;
        }
        entered = s_ptr[row] < ks;
      }
      acc.fill(entered ? Elt(0) : body.init());
      Elt nxt_c = Elt(0);
      Off nxt_off = 0;
      if (ks + lane < ke) {
        nxt_c = body.coef(ks + lane);
        nxt_off = body.brow_off(ks + lane);
      }
      int last_row = 0;
      bool open = true;   // the row holding the last processed non-zero has not ended yet
      appy_pack<Elt, V> ring[ROLL ? D : 1][T];
      if (ROLL) {
#pragma unroll
        for (int j = 0; j < (ROLL ? D : 1); ++j)
          if (ks + j < ke)
            appy_csr_dense_load<V, T, NC, Body>(blane, appy_shfl<Off>(nxt_off, j, 32), lane, ncols, ring[j]);
      }
      for (i64 kb = ks; kb < ke; kb += 32) {
        const int n = (ke - kb < 32) ? (int)(ke - kb) : 32;
        const Elt my_c = nxt_c;
        const Off my_off = nxt_off;
        if (kb + 32 + lane < ke) {   // next block's coefficients and offsets, one block ahead
          nxt_c = body.coef(kb + 32 + lane);
          nxt_off = body.brow_off(kb + 32 + lane);
        }
        // lane j: which row holds non-zero kb+j, and is it that row's last one?
        int my_row = 0;
        bool is_last = false;
        if (lane < n) {
          const i64 pos = kb + lane;
          int hi_r = nr;
          while (hi_r - my_row > 1) {
            const int mid = (my_row + hi_r) >> 1;
            if (s_ptr[mid] <= pos) my_row = mid; else hi_r = mid;
          }
          is_last = s_ptr[my_row + 1] == pos + 1;
        }
        const unsigned ends = __ballot_sync(APPY_FULL_MASK, is_last);
        Elt* park0 = s_part + (size_t)(warp * 2) * W;
        if (ROLL) {
          if (n == 32) {
#pragma unroll 1
            for (int q = 0; q < 32; q += D)
              appy_csr_dense_roll<V, T, (ROLL ? D : 1), NC, false, Body>(
                  body, blane, kb, ke, q, 32, ends, my_c, my_off, nxt_off, my_row, r0, entered, park0,
                  &s_tag[warp * 2], lane, ncols, ring, acc);
          } else {
#pragma unroll 1
            for (int q = 0; q < n; q += D)
              appy_csr_dense_roll<V, T, (ROLL ? D : 1), NC, true, Body>(
                  body, blane, kb, ke, q, n, ends, my_c, my_off, nxt_off, my_row, r0, entered, park0,
                  &s_tag[warp * 2], lane, ncols, ring, acc);
          }
        } else if (n == 32) {
#pragma unroll 1
          for (int q = 0; q < 32; q += D)
            appy_csr_dense_group<V, T, D, NC, false, Body>(body, blane, q, 32, ends, my_c, my_off, my_row, r0,
                                                           entered, park0, &s_tag[warp * 2], lane, ncols, acc);
        } else {
#pragma unroll 1
          for (int q = 0; q < n; q += D)
            appy_csr_dense_group<V, T, D, NC, true, Body>(body, blane, q, n, ends, my_c, my_off, my_row, r0,
                                                          entered, park0, &s_tag[warp * 2], lane, ncols, acc);
        }
        last_row = __shfl_sync(APPY_FULL_MASK, my_row, n - 1, 32);
        open = ((ends >> (n - 1)) & 1u) == 0;
      }
      if (open) {   // the share ended inside a row: park what was gathered so far
        const int slot = entered ? 0 : 1;
        appy_csr_dense_park<V, T, Body>(s_part + (size_t)(warp * 2 + slot) * W, lane, acc);
        if (lane == 0) s_tag[warp * 2 + slot] = last_row;
      }
    }
    __syncthreads();
    // cut rows: the warp that holds the first partial of a row adds the others in order
    for (int slot = 0; slot < 2; ++slot) {
      const int b0 = warp * 2 + slot;
      const int row = s_tag[b0];
      if (row < 0) continue;
      bool first = true;
      for (int bb = 0; bb < b0; ++bb) first = first && (s_tag[bb] != row);
      if (!first) continue;
      appy_rowacc<V, T, Body> sum;
#pragma unroll
      for (int t = 0; t < T; ++t)
#pragma unroll
        for (int x = 0; x < V; ++x) sum.a[t].v[x] = s_part[(size_t)b0 * W + (t * 32 + lane) * V + x];
      for (int bb = b0 + 1; bb < 2 * NWARPS; ++bb) {
        if (s_tag[bb] != row) continue;
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
          for (int x = 0; x < V; ++x) sum.a[t].v[x] = sum.a[t].v[x] + s_part[(size_t)bb * W + (t * 32 + lane) * V + x];
      }
      appy_csr_dense_store<V, T, NC, Body>(body, r0 + row, lane, ncols, sum);
    }
    __syncthreads();
  }
}
