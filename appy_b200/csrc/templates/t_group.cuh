// Group lowering of `#pragma parallel for` loops whose body holds inner
// `#pragma simd` loops (reference lowering: one Triton program per outer
// iteration, appy/backends/triton/passes/device_passes/remove_loop_head.py:3-55,
// inner loops tiled by 256 lanes with a cross-warp tl.sum per tile,
// appy/backends/triton/passes/block_loop.py:10-74).
//
// Here a *group* of G threads owns one outer iteration.  G is 1,2,4,8,16,32
// (a slice of a warp: reductions are shuffles restricted to the group's lanes)
// or 0, meaning the whole CTA (reductions through shared memory).  Inner simd
// loops are strided over the group's lanes; a scalar statement is executed by
// every lane redundantly and its memory stores by lane 0 only.
//
//   struct Body { template <class Grp> void iter(i64 i, const Grp& g); };
#pragma once
#include "appy_device.cuh"

template <int G> struct appy_grp {
  int lane;        // 0..G-1 inside the group
  u32 mask;        // warp lanes that form this group
  void* smem;      // unused for sub-warp groups
  int seg;         // which of the SEG column segments of the outer iteration this group works on
  static const int size_static = G;
  APPY_DEV int size() const { return G; }
  APPY_DEV void init(void* s) {
    const int wl = threadIdx.x & 31;
    lane = wl & (G - 1);
    mask = (G == 32) ? APPY_FULL_MASK : (((1u << G) - 1u) << (wl & ~(G - 1)));
    smem = s;
    seg = 0;
  }
  APPY_DEV void barrier() const {
    if (G > 1) __syncwarp(mask);
  }
  template <class Op, class T> APPY_DEV T reduce(T v) const {
#pragma unroll
    for (int m = G >> 1; m > 0; m >>= 1) {
      T o;
      if (sizeof(T) == 8) {
        union { T t; u64 u; } x; x.t = v;
        x.u = __shfl_xor_sync(mask, x.u, m, 32);
        o = x.t;
      } else {
        o = __shfl_xor_sync(mask, v, m, 32);
      }
      v = Op::template op<T>(v, o);
    }
    return v;
  }
};

// whole-CTA group
template <> struct appy_grp<0> {
  int lane;
  u32 mask;
  void* smem;
  int seg;
  static const int size_static = 0;
#ifdef P_BLOCK
  // generated kernels are compiled for one CTA size: a constant stride lets the compiler prove that
  // unrolled iterations of a lane touch different elements and overlap their loads
  APPY_DEV int size() const { return P_BLOCK; }
#else
  APPY_DEV int size() const { return blockDim.x; }
#endif
  APPY_DEV void init(void* s) { lane = threadIdx.x; mask = APPY_FULL_MASK; smem = s; seg = 0; }
  APPY_DEV void barrier() const { __syncthreads(); }
  template <class Op, class T> APPY_DEV T reduce(T v) const {
    return appy_block_reduce<Op, T>(v, reinterpret_cast<T*>(smem));
  }
};

// SEG > 1 (perfect nests only: the outer body is one simd loop without reductions): an outer
// iteration is cut into SEG column segments worked on by different groups, so that a few long
// rows still fill the machine.  The generated inner loop takes its bounds from g.seg.
template <int G, int SEG, class Body>
APPY_DEV void appy_group_rows(Body& body, i64 lo, i64 hi, void* smem) {
  appy_grp<G> g;
  g.init(smem);
  const i64 units = (hi - lo) * SEG;
  if (G == 0) {
    for (i64 u = blockIdx.x; u < units; u += gridDim.x) {
      g.seg = (int)(u % SEG);
      body.iter(lo + u / SEG, g);
    }
  } else {
    const int gpb = blockDim.x / (G ? G : 1);                 // groups per CTA
    const i64 gid = (i64)blockIdx.x * gpb + threadIdx.x / (G ? G : 1);
    const i64 ngroups = (i64)gridDim.x * gpb;
    for (i64 u = gid; u < units; u += ngroups) {
      g.seg = (int)(u % SEG);
      body.iter(lo + u / SEG, g);
    }
  }
}
