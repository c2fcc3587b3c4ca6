// T5, bulk-copy variant: CSR x dense with the B rows fetched by asynchronous bulk copies
//
// Same loop shape, work split and row-boundary handling as t_csr_dense.cuh; what differs is how a
// B row reaches the multiply-add.  There a warp gathers a row with one 16-byte load per lane and
// holds D rows in registers, so registers bound the number of rows in flight.  Here lane 0 of the
// warp issues one `cp.async.bulk` per non-zero (the whole B row, NC * sizeof(Elt) bytes, global ->
// shared memory) into a ring of S slots owned by the warp; each slot has an mbarrier on which the
// copy signals its bytes.  The warp then waits for the slot, reads it with one 16-byte
// `ld.shared` per lane, multiplies, and at once re-arms the slot with the row S non-zeros ahead.
// Rows in flight per SM = warps x S, limited by shared memory (S x row bytes per warp), not by
// registers, and the load/store units see one instruction per row instead of 32 lanes' worth.
//
// Conditions: the column count is the compile-time NC = 32*V*T (no ragged columns), a row is a
// multiple of 16 bytes and every B row starts on a 16-byte boundary (what the vector path
// requires anyway), S is a power of two <= 32.
//
// Every wait on an mbarrier is bounded: after `spin_limit` unsuccessful polls the warp raises
// *err, stops issuing copies, waits (bounded again) for the copies it still has in flight, and
// falls through to the tile's barriers, so the kernel returns with a status instead of hanging.
//
// Dynamic shared memory: NWARPS * S * (NC * sizeof(Elt) + 8) bytes (ring + barriers); the static
// part is the one of t_csr_dense.cuh.
#pragma once
#include "t_csr_dense.cuh"

APPY_DEV unsigned appy_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
APPY_DEV void appy_mbar_init(u64* bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(appy_smem_addr(bar)), "r"(arrivals) : "memory");
}
APPY_DEV void appy_mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// one arrival and `bytes` expected from the copy that follows
APPY_DEV void appy_mbar_expect(u64* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(appy_smem_addr(bar)), "r"(bytes)
               : "memory");
}
APPY_DEV bool appy_mbar_try_wait(u64* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(appy_smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
APPY_DEV bool appy_mbar_wait(u64* bar, unsigned parity, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i)
    if (appy_mbar_try_wait(bar, parity)) return true;
  return false;
}
// `bytes` from global memory to this CTA's shared memory; completion is counted on `bar`
APPY_DEV void appy_bulk_load(void* smem_dst, const void* gsrc, unsigned bytes, u64* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   appy_smem_addr(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(appy_smem_addr(bar))
               : "memory");
}

template <int V, int T, int S, int NWARPS, class Elt>
struct appy_csr_dense_bulk_smem {
  static const int row_bytes = 32 * V * T * (int)sizeof(Elt);
  static const int bytes = NWARPS * S * (row_bytes + 8);
};

// blockDim.x == 32*NWARPS.  `dyn` is the dynamic shared memory (128-byte aligned).
template <int V, int T, int S, int NWARPS, int R, int NC, class IdxT, class Body>
APPY_DEV void appy_csr_dense_bulk(const Body& body, const IdxT* __restrict__ indptr, i64 lo, i64 hi,
                                  void* smem_raw, void* dyn, unsigned* err, unsigned spin_limit) {
  typedef typename Body::Elt Elt;
  typedef typename Body::Off Off;
  static_assert(NC == 32 * V * T, "the bulk variant needs full, compile-time rows");
  static_assert((S & (S - 1)) == 0 && S >= 2 && S <= 32, "S must be a power of two in 2..32");
  static_assert((NC * sizeof(Elt)) % 16 == 0, "a row must be a multiple of 16 bytes");
  const int W = NC;
  const unsigned ROWB = NC * sizeof(Elt);
  Elt* s_part = reinterpret_cast<Elt*>(smem_raw);                    // [NWARPS][2][W]
  i64* s_ptr = reinterpret_cast<i64*>(s_part + NWARPS * 2 * W);      // [R+1] row starts
  int* s_tag = reinterpret_cast<int*>(s_ptr + (R + 1));              // [NWARPS][2] row of each partial
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Elt* ring = reinterpret_cast<Elt*>(dyn) + (size_t)warp * S * NC;   // this warp's S rows
  u64* bars = reinterpret_cast<u64*>(reinterpret_cast<char*>(dyn) + (size_t)NWARPS * S * ROWB) + warp * S;
  const Elt* bbase = body.bbase();

  if (lane < S) appy_mbar_init(&bars[lane], 1);
  appy_mbar_init_fence();
  __syncthreads();
  unsigned consumed = 0, issued = 0;   // rows of this warp taken from / put into the ring so far
  bool dead = false;                   // a wait ran out: no more copies are issued

  for (i64 r0 = lo + (i64)blockIdx.x * R; r0 < hi; r0 += (i64)gridDim.x * R) {
    const int nr = (hi - r0 < R) ? (int)(hi - r0) : R;
    for (int t = threadIdx.x; t <= nr; t += 32 * NWARPS) s_ptr[t] = (i64)appy_ldg1(indptr + r0 + t);
    if (threadIdx.x < 2 * NWARPS) s_tag[threadIdx.x] = -1;
    __syncthreads();
    const i64 s = s_ptr[0], e = s_ptr[nr];
    for (int j = warp; j < nr; j += NWARPS) {      // rows without non-zeros are just `init`
      if (s_ptr[j + 1] == s_ptr[j]) {
        appy_rowacc<V, T, Body> z;
        z.fill(body.init());
        appy_csr_dense_store<V, T, NC, Body>(body, r0 + j, lane, NC, z);
      }
    }
    i64 chunk = ((e - s) + NWARPS - 1) / NWARPS;
    chunk = (chunk + 31) / 32 * 32;
    const i64 ks = s + (i64)warp * chunk;
    const i64 ke = (ks + chunk < e) ? ks + chunk : e;
    if (ks < ke) {
      appy_rowacc<V, T, Body> acc;
      bool entered;
      {
        int row = 0, hi_r = nr;
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
      // fill the ring with the first S rows of the share
#pragma unroll
      for (int j = 0; j < S; ++j) {
        const Off off = appy_shfl<Off>(nxt_off, j, 32);
        if (!dead && ks + j < ke) {
          if (lane == 0) {
            const unsigned slot = issued & (S - 1);
            appy_mbar_expect(&bars[slot], ROWB);
            appy_bulk_load(ring + (size_t)slot * NC, bbase + off, ROWB, &bars[slot]);
          }
          ++issued;
        }
      }
      int last_row = 0;
      bool open = true;
      for (i64 kb = ks; kb < ke; kb += 32) {
        const int n = (ke - kb < 32) ? (int)(ke - kb) : 32;
        const Elt my_c = nxt_c;
        const Off my_off = nxt_off;
        if (kb + 32 + lane < ke) {
          nxt_c = body.coef(kb + 32 + lane);
          nxt_off = body.brow_off(kb + 32 + lane);
        }
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
#pragma unroll 2
        for (int j = 0; j < n; ++j) {
          const unsigned slot = consumed & (S - 1);
          if (!dead) {
            const bool ok = appy_mbar_wait(&bars[slot], (consumed / S) & 1u, spin_limit);
            if (!__all_sync(APPY_FULL_MASK, ok)) {
              dead = true;
              if (lane == 0) atomicExch(err, 1u);
            }
          }
          if (!dead) {
            appy_pack<Elt, V> b[T];
            const Elt* row = ring + (size_t)slot * NC + lane * V;
#pragma unroll
            for (int t = 0; t < T; ++t) b[t] = *reinterpret_cast<const appy_pack<Elt, V>*>(row + t * 32 * V);
            appy_csr_dense_fma<V, T, Body>(acc, appy_shfl<Elt>(my_c, j, 32), b);
          }
          if ((ends >> j) & 1u) {
            const int rowi = __shfl_sync(APPY_FULL_MASK, my_row, j, 32);
            if (entered) {
              appy_csr_dense_park<V, T, Body>(s_part + (size_t)(warp * 2) * W, lane, acc);
              if (lane == 0) s_tag[warp * 2] = rowi;
              entered = false;
            } else {
              appy_csr_dense_store<V, T, NC, Body>(body, r0 + rowi, lane, NC, acc);
            }
            acc.fill(body.init());
          }
          __syncwarp();                       // every lane has read the slot before it is refilled
          if (!dead) ++consumed;              // once dead, [consumed, issued) are the copies still in flight
          const Off off = appy_shfl<Off>((j + S < 32) ? my_off : nxt_off, (j + S) & 31, 32);
          if (!dead && kb + j + S < ke) {
            if (lane == 0) {
              appy_mbar_expect(&bars[slot], ROWB);
              appy_bulk_load(ring + (size_t)slot * NC, bbase + off, ROWB, &bars[slot]);
            }
            ++issued;
          }
        }
        last_row = __shfl_sync(APPY_FULL_MASK, my_row, n - 1, 32);
        open = ((ends >> (n - 1)) & 1u) == 0;
      }
      if (dead) {     // copies still in flight must land before the CTA may give up its shared memory
        while (consumed != issued) {
          appy_mbar_wait(&bars[consumed & (S - 1)], (consumed / S) & 1u, spin_limit);
          ++consumed;
        }
      }
      if (open) {
        const int slot2 = entered ? 0 : 1;
        appy_csr_dense_park<V, T, Body>(s_part + (size_t)(warp * 2 + slot2) * W, lane, acc);
        if (lane == 0) s_tag[warp * 2 + slot2] = last_row;
      }
    }
    __syncthreads();
    for (int slot = 0; slot < 2; ++slot) {      // cut rows: partials are added in warp order
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
      appy_csr_dense_store<V, T, NC, Body>(body, r0 + row, lane, NC, sum);
    }
    __syncthreads();
  }
}
