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

template <int G, int V, int U, class Body>
APPY_DEV void appy_rowdot(const Body& body, i64 lo, i64 hi, void* smem) {
  appy_grp<G> g;
  g.init(smem);
  if (G == 0) {
    for (i64 i = lo + blockIdx.x; i < hi; i += gridDim.x) appy_rowdot_row<G, V, U, Body>(body, i, g);
  } else {
    const int gg = G ? G : 1;
    const int gpb = blockDim.x / gg;
    const i64 gid = (i64)blockIdx.x * gpb + threadIdx.x / gg;
    const i64 ngroups = (i64)gridDim.x * gpb;
    for (i64 i = lo + gid; i < hi; i += ngroups) appy_rowdot_row<G, V, U, Body>(body, i, g);
  }
}
