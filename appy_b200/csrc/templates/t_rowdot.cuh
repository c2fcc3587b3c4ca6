// T4: row-dot / dense row reduction
//
//   #pragma parallel for
//   for i in range(lo, hi):
//       acc = <identity>
//       #pragma simd
//       for j in range(jlo, jhi):
//           acc = acc (op) term(i, j)
//       finish(i, acc)                      e.g. y[i] = acc
//
// (reference: examples/05-gemv.py:7-17; its Triton lowering runs a 256-lane tile
// with a cross-warp tl.sum on every inner iteration,
// appy/backends/triton/passes/block_loop.py:10-74.)
//
// Here a group of G lanes (a warp slice, or the whole CTA for G = 0) owns a row.
// Each lane walks 16-byte chunks of the row with U chunks in flight, keeps U
// private accumulators for the whole row, and the group reduces exactly once per
// row.  Read-only operands go through ld.global.nc.
//
//   struct Body {
//     typedef <T> Acc;  typedef <op> Op;  struct Regs;
//     void bounds(i64 i, i64& jlo, i64& jhi) const;
//     void load(i64 i, i64 j0, Regs&) const;               // chunk [j0, j0+V), j0 % V == 0
//     Acc  fold(i64 i, i64 j0, const Regs&, Acc) const;    // fold V terms into acc
//     Acc  one(i64 i, i64 j, Acc) const;                   // ragged edges
//     void finish(i64 i, Acc total) const;                 // executed by lane 0
//   };
#pragma once
#include "t_group.cuh"

template <int G, int V, int U, class Body>
APPY_DEV void appy_rowdot_row(const Body& body, i64 i, const appy_grp<G>& g) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  i64 jlo, jhi;
  body.bounds(i, jlo, jhi);
  Acc acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = Op::template id<Acc>();
  const int gs = g.size();
  // aligned interior [a_lo, a_hi) in units of chunks
  i64 c_lo = (jlo + V - 1) / V, c_hi = jhi / V;   // jlo >= 0 for array indices
  if (c_hi < c_lo) c_hi = c_lo;
  const i64 head_end = (c_lo * V < jhi) ? c_lo * V : jhi;
  for (i64 j = jlo + g.lane; j < head_end; j += gs) acc[0] = body.one(i, j, acc[0]);
  i64 c = c_lo + g.lane;
  for (; c + (i64)(U - 1) * gs < c_hi; c += (i64)U * gs) {
    typename Body::Regs r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) body.load(i, (c + (i64)u * gs) * V, r[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = body.fold(i, (c + (i64)u * gs) * V, r[u], acc[u]);
  }
  for (; c < c_hi; c += gs) {
    typename Body::Regs r;
    body.load(i, c * V, r);
    acc[0] = body.fold(i, c * V, r, acc[0]);
  }
  const i64 tail_begin = (c_hi * V > head_end) ? c_hi * V : head_end;
  for (i64 j = tail_begin + g.lane; j < jhi; j += gs) acc[0] = body.one(i, j, acc[0]);
#pragma unroll
  for (int u = 1; u < U; ++u) acc[0] = Op::template op<Acc>(acc[0], acc[u]);
  const Acc total = g.template reduce<Op, Acc>(acc[0]);
  if (g.lane == 0) body.finish(i, total);
}

// R consecutive rows at once: the group walks the same chunk of all R rows before it moves on,
// so operands that depend on the inner index only (x[j]) are fetched once per chunk (identical
// read-only loads are merged by the compiler) and every lane keeps R x U chunks in flight.
// Rows whose inner bounds differ (triangular loops) are processed one after the other.
template <int G, int V, int U, int R, class Body>
APPY_DEV void appy_rowdot_rows(const Body& body, i64 i, const appy_grp<G>& g) {
  typedef typename Body::Acc Acc;
  typedef typename Body::Op Op;
  i64 jlo, jhi;
  body.bounds(i, jlo, jhi);
  bool same = true;
#pragma unroll
  for (int r = 1; r < R; ++r) {
    i64 a, b;
    body.bounds(i + r, a, b);
    same = same && a == jlo && b == jhi;
  }
  if (!same) {
    for (int r = 0; r < R; ++r) appy_rowdot_row<G, V, U, Body>(body, i + r, g);
    return;
  }
  Acc acc[R][U];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int u = 0; u < U; ++u) acc[r][u] = Op::template id<Acc>();
  const int gs = g.size();
  i64 c_lo = (jlo + V - 1) / V, c_hi = jhi / V;
  if (c_hi < c_lo) c_hi = c_lo;
  const i64 head_end = (c_lo * V < jhi) ? c_lo * V : jhi;
  for (i64 j = jlo + g.lane; j < head_end; j += gs)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = body.one(i + r, j, acc[r][0]);
  i64 c = c_lo + g.lane;
  for (; c + (i64)(U - 1) * gs < c_hi; c += (i64)U * gs) {
    typename Body::Regs rg[R][U];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int u = 0; u < U; ++u) body.load(i + r, (c + (i64)u * gs) * V, rg[r][u]);
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int u = 0; u < U; ++u) acc[r][u] = body.fold(i + r, (c + (i64)u * gs) * V, rg[r][u], acc[r][u]);
  }
  for (; c < c_hi; c += gs) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      typename Body::Regs rg;
      body.load(i + r, c * V, rg);
      acc[r][0] = body.fold(i + r, c * V, rg, acc[r][0]);
    }
  }
  const i64 tail_begin = (c_hi * V > head_end) ? c_hi * V : head_end;
  for (i64 j = tail_begin + g.lane; j < jhi; j += gs)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = body.one(i + r, j, acc[r][0]);
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int u = 1; u < U; ++u) acc[r][0] = Op::template op<Acc>(acc[r][0], acc[r][u]);
    const Acc total = g.template reduce<Op, Acc>(acc[r][0]);
    if (g.lane == 0) body.finish(i + r, total);
  }
}

template <int G, int V, int U, int R, class Body>
APPY_DEV void appy_rowdot(const Body& body, i64 lo, i64 hi, void* smem) {
  appy_grp<G> g;
  g.init(smem);
  const int gg = G ? G : 1;
  const int gpb = G ? blockDim.x / gg : 1;                       // groups per CTA
  const i64 gid = G ? (i64)blockIdx.x * gpb + threadIdx.x / gg : (i64)blockIdx.x;
  const i64 ngroups = (i64)gridDim.x * gpb;
  const i64 nfull = (hi - lo) / R;                               // units of R rows
  for (i64 b = gid; b < nfull; b += ngroups) {
    if (R == 1) appy_rowdot_row<G, V, U, Body>(body, lo + b, g);
    else appy_rowdot_rows<G, V, U, R, Body>(body, lo + b * R, g);
  }
  for (i64 i = lo + nfull * R + gid; i < hi; i += ngroups) appy_rowdot_row<G, V, U, Body>(body, i, g);
}
