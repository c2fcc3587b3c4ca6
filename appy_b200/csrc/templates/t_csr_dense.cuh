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
//     typedef <int|i64> Row;
//     Elt   coef(i64 k) const;                 // A_data[k]
//     Row   brow(i64 k) const;                 // A_indices[k]
//     const Elt* brow_ptr(Row r) const;        // &B[r, 0]
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

template <int V, int T, class Body>
APPY_DEV void appy_csr_dense_load(const Body& body, typename Body::Row r, int lane, int ncols,
                                  appy_pack<typename Body::Elt, V> (&b)[T]) {
  typedef typename Body::Elt Elt;
  const Elt* p = body.brow_ptr(r);
#pragma unroll
  for (int t = 0; t < T; ++t) {
    const int col = (t * 32 + lane) * V;
    if (col < ncols) b[t] = appy_ld_nc<Elt, V>(p + col);
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

template <int V, int T, class Body>
APPY_DEV void appy_csr_dense_store(const Body& body, i64 i, int lane, int ncols,
                                   const appy_rowacc<V, T, Body>& acc) {
  typedef typename Body::Elt Elt;
  Elt* p = body.crow_ptr(i);
#pragma unroll
  for (int t = 0; t < T; ++t) {
    const int col = (t * 32 + lane) * V;
    if (col < ncols) appy_st_cs<Elt, V>(p + col, acc.a[t]);
  }
}

// shared memory bytes needed by appy_csr_dense
template <int V, int T, int NWARPS, int R, class Elt>
struct appy_csr_dense_smem {
  static const int bytes = NWARPS * 2 * 32 * V * T * (int)sizeof(Elt) + (int)sizeof(i64) * (R + 1) +
                           (int)sizeof(int) * 2 * NWARPS;
};

// blockDim.x == 32*NWARPS.
template <int V, int T, int D, int NWARPS, int R, class IdxT, class Body>
APPY_DEV void appy_csr_dense(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi,
                             int ncols, void* smem_raw) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Row Row;
  const int W = 32 * V * T;                                          // padded row width
  Elt* s_part = reinterpret_cast<Elt*>(smem_raw);                    // [NWARPS][2][W]
  i64* s_ptr = reinterpret_cast<i64*>(s_part + NWARPS * 2 * W);      // [R+1] row starts
  int* s_tag = reinterpret_cast<int*>(s_ptr + (R + 1));              // [NWARPS][2] row of each partial
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

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
        appy_csr_dense_store<V, T, Body>(body, r0 + j, lane, ncols, z);
      }
    }
    // this warp's share [ks, ke) of the tile's non-zeros
    i64 chunk = ((e - s) + NWARPS - 1) / NWARPS;
    chunk = (chunk + 31) / 32 * 32;
    const i64 ks = s + (i64)warp * chunk;
    const i64 ke = (ks + chunk < e) ? ks + chunk : e;
    if (ks < ke) {
      int cur = 0;
      {  // largest row index with s_ptr[row] <= ks (the non-empty row that holds non-zero ks)
        int hi_r = nr;
        while (hi_r - cur > 1) {
          const int mid = (cur + hi_r) >> 1;
          if (s_ptr[mid] <= ks) cur = mid; else hi_r = mid;
        }
      }
      i64 cur_end = s_ptr[cur + 1];
      appy_rowacc<V, T, Body> acc;
      acc.fill(s_ptr[cur] >= ks ? body.init() : Elt(0));
      Elt nxt_c = Elt(0);
      Row nxt_r = 0;
      if (ks + lane < ke) {
        nxt_c = body.coef(ks + lane);
        nxt_r = body.brow(ks + lane);
      }
      for (i64 kb = ks; kb < ke; kb += 32) {
        const int n = (ke - kb < 32) ? (int)(ke - kb) : 32;
        const Elt my_c = nxt_c;
        const Row my_r = nxt_r;
        if (kb + 32 + lane < ke) {   // next block's coefficients and row numbers, one block ahead
          nxt_c = body.coef(kb + 32 + lane);
          nxt_r = body.brow(kb + 32 + lane);
        }
#pragma unroll 1
        for (int q = 0; q < n; q += D) {
          appy_pack<Elt, V> b[D][T];
#pragma unroll
          for (int j = 0; j < D; ++j)
            if (q + j < n) appy_csr_dense_load<V, T, Body>(body, appy_shfl<Row>(my_r, q + j, 32), lane, ncols, b[j]);
#pragma unroll
          for (int j = 0; j < D; ++j) {
            if (q + j < n) {
              if (kb + q + j >= cur_end) {
                // row `cur` is complete: store it, or park it if a share boundary cut it
                if (s_ptr[cur] >= ks) {
                  appy_csr_dense_store<V, T, Body>(body, r0 + cur, lane, ncols, acc);
                } else {
                  Elt* mine = s_part + (size_t)(warp * 2) * W;
#pragma unroll
                  for (int t = 0; t < T; ++t)
#pragma unroll
                    for (int x = 0; x < V; ++x) mine[(t * 32 + lane) * V + x] = acc.a[t].v[x];
                  if (lane == 0) s_tag[warp * 2] = cur;
                }
                do { ++cur; } while (s_ptr[cur + 1] == s_ptr[cur]);
                cur_end = s_ptr[cur + 1];
                acc.fill(body.init());
              }
              appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(my_c, q + j, 32), b[j]);
            }
          }
        }
      }
      // the row that was open when the share ended
      if (s_ptr[cur] >= ks && cur_end <= ke) {
        appy_csr_dense_store<V, T, Body>(body, r0 + cur, lane, ncols, acc);
      } else {
        const int slot = (s_ptr[cur] >= ks) ? 1 : 0;
        Elt* mine = s_part + (size_t)(warp * 2 + slot) * W;
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
          for (int x = 0; x < V; ++x) mine[(t * 32 + lane) * V + x] = acc.a[t].v[x];
        if (lane == 0) s_tag[warp * 2 + slot] = cur;
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
      appy_csr_dense_store<V, T, Body>(body, r0 + row, lane, ncols, sum);
    }
    __syncthreads();
  }
}
