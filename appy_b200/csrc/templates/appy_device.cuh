// Device-side building blocks shared by every kernel template of the cuda_sm100
// backend.  This header is compiled two ways: by nvcc into the prebuilt kernels
// of libappy_sm100.so, and by NVRTC (passed as an in-memory header) for every
// loop the Python code generator instantiates.  It therefore includes nothing
// and relies only on CUDA built-ins.
//
// Contents: fixed-width aliases, 4/8/16-byte packs with read-only (ld.global.nc)
// and streaming load/store, reduction operators with identities, group (2..32
// lanes) / block reductions by warp shuffle + shared memory, and atomics for
// every reduction operator the loop front end can detect (+, max, min, *).
#pragma once

typedef long long i64;
typedef unsigned long long u64;
typedef unsigned int u32;
typedef unsigned char u8;

#define APPY_DEV __device__ __forceinline__
#define APPY_FULL_MASK 0xffffffffu

// ---------------------------------------------------------------------------
// numeric limits without <limits> / <cmath>
// ---------------------------------------------------------------------------
template <class T> struct appy_lim;
template <> struct appy_lim<float> {
  static APPY_DEV float inf() { return __int_as_float(0x7f800000); }
  static APPY_DEV float lowest() { return -inf(); }
  static APPY_DEV float highest() { return inf(); }
};
template <> struct appy_lim<double> {
  static APPY_DEV double inf() { return __longlong_as_double(0x7ff0000000000000LL); }
  static APPY_DEV double lowest() { return -inf(); }
  static APPY_DEV double highest() { return inf(); }
};
template <> struct appy_lim<int> {
  static APPY_DEV int lowest() { return -2147483647 - 1; }
  static APPY_DEV int highest() { return 2147483647; }
};
template <> struct appy_lim<i64> {
  static APPY_DEV i64 lowest() { return -9223372036854775807LL - 1; }
  static APPY_DEV i64 highest() { return 9223372036854775807LL; }
};
template <> struct appy_lim<u8> {
  static APPY_DEV u8 lowest() { return 0; }
  static APPY_DEV u8 highest() { return 255; }
};

// ---------------------------------------------------------------------------
// packs: V consecutive elements moved with one 4/8/16-byte instruction
// ---------------------------------------------------------------------------
template <class T, int V> struct __align__(sizeof(T) * V) appy_pack { T v[V]; };

template <int BYTES> struct appy_raw;
template <> struct appy_raw<1> { typedef unsigned char type; };
template <> struct appy_raw<2> { typedef unsigned short type; };
template <> struct appy_raw<4> { typedef unsigned int type; };
template <> struct appy_raw<8> { typedef uint2 type; };
template <> struct appy_raw<16> { typedef uint4 type; };

// read-only path (ld.global.nc): operand is never written by the running kernel
template <class T, int V> APPY_DEV appy_pack<T, V> appy_ld_nc(const T* p) {
  typedef typename appy_raw<sizeof(T) * V>::type R;
  union { R r; appy_pack<T, V> k; } u;
  u.r = __ldg(reinterpret_cast<const R*>(p));
  return u.k;
}
// streaming read-only load: evict-first in L1/L2, for data touched exactly once
template <class T, int V> APPY_DEV appy_pack<T, V> appy_ld_cs(const T* p) {
  typedef typename appy_raw<sizeof(T) * V>::type R;
  union { R r; appy_pack<T, V> k; } u;
  u.r = __ldcs(reinterpret_cast<const R*>(p));
  return u.k;
}
// plain (coherent) load: operand may also be stored by this kernel
template <class T, int V> APPY_DEV appy_pack<T, V> appy_ld(const T* p) {
  typedef typename appy_raw<sizeof(T) * V>::type R;
  union { R r; appy_pack<T, V> k; } u;
  u.r = *reinterpret_cast<const R*>(p);
  return u.k;
}
template <class T, int V> APPY_DEV void appy_st(T* p, const appy_pack<T, V>& k) {
  typedef typename appy_raw<sizeof(T) * V>::type R;
  union { R r; appy_pack<T, V> k; } u;
  u.k = k;
  *reinterpret_cast<R*>(p) = u.r;
}
// streaming store (st.global.cs): output is not re-read by this kernel
template <class T, int V> APPY_DEV void appy_st_cs(T* p, const appy_pack<T, V>& k) {
  typedef typename appy_raw<sizeof(T) * V>::type R;
  union { R r; appy_pack<T, V> k; } u;
  u.k = k;
  __stcs(reinterpret_cast<R*>(p), u.r);
}
template <class T> APPY_DEV T appy_ldg1(const T* p) { return appy_ld_nc<T, 1>(p).v[0]; }

// ---------------------------------------------------------------------------
// reduction operators
// ---------------------------------------------------------------------------
struct appy_add {
  template <class T> static APPY_DEV T id() { return T(0); }
  template <class T> static APPY_DEV T op(T a, T b) { return a + b; }
};
struct appy_mul {
  template <class T> static APPY_DEV T id() { return T(1); }
  template <class T> static APPY_DEV T op(T a, T b) { return a * b; }
};
struct appy_max {
  template <class T> static APPY_DEV T id() { return appy_lim<T>::lowest(); }
  template <class T> static APPY_DEV T op(T a, T b) { return a > b ? a : b; }
};
struct appy_min {
  template <class T> static APPY_DEV T id() { return appy_lim<T>::highest(); }
  template <class T> static APPY_DEV T op(T a, T b) { return a < b ? a : b; }
};

template <class T> APPY_DEV T appy_shfl_xor(T v, int m, int width) {
  if (sizeof(T) == 8) {
    union { T t; u64 u; } x; x.t = v;
    x.u = __shfl_xor_sync(APPY_FULL_MASK, x.u, m, width);
    return x.t;
  } else {
    return __shfl_xor_sync(APPY_FULL_MASK, v, m, width);
  }
}
template <class T> APPY_DEV T appy_shfl(T v, int src, int width) {
  if (sizeof(T) == 8) {
    union { T t; u64 u; } x; x.t = v;
    x.u = __shfl_sync(APPY_FULL_MASK, x.u, src, width);
    return x.t;
  } else {
    return __shfl_sync(APPY_FULL_MASK, v, src, width);
  }
}

// all-reduce over a group of G consecutive lanes (G a power of two, 1..32);
// every lane of the group receives the result.  All 32 lanes of the warp must
// reach the call (groups never diverge from one another in the templates).
template <class Op, int G, class T> APPY_DEV T appy_group_reduce(T v) {
#pragma unroll
  for (int m = G >> 1; m > 0; m >>= 1) v = Op::template op<T>(v, appy_shfl_xor<T>(v, m, G));
  return v;
}

// all-reduce over the whole CTA; `smem` holds >= 32 elements of T and may be
// reused after the call returns (ends with a barrier).  blockDim.x % 32 == 0.
template <class Op, class T> APPY_DEV T appy_block_reduce(T v, T* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = appy_group_reduce<Op, 32, T>(v);
  if (nwarp == 1) return v;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  T r = lane < nwarp ? smem[lane] : Op::template id<T>();
  r = appy_group_reduce<Op, 32, T>(r);
  __syncthreads();
  return r;
}

// floor(a / b) for chunk arithmetic on signed iteration ranges
APPY_DEV i64 appy_floor_div_i64(i64 a, i64 b) {
  i64 q = a / b;
  return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
}

// Element `idx` of the run [lo[NL-1] .. lo[0], p.v[0] .. p.v[V-1], hi[0] .. hi[NH-1]] (a pack with the
// scalar elements below and above it).  `idx` is a constant after unrolling, so this is a register pick.
template <class T, int V, int NL, int NH>
APPY_DEV T appy_side(const appy_pack<T, V>& p, const T (&lo)[NL], const T (&hi)[NH], int idx) {
  if (idx < 0) return lo[-idx - 1];
  if (idx >= V) return hi[idx - V];
  return p.v[idx];
}

// ---------------------------------------------------------------------------
// atomics on a shared(...) scalar, one per block
// ---------------------------------------------------------------------------
APPY_DEV void appy_atomic(appy_add, double* p, double v) { atomicAdd(p, v); }
APPY_DEV void appy_atomic(appy_add, float* p, float v) { atomicAdd(p, v); }
APPY_DEV void appy_atomic(appy_add, int* p, int v) { atomicAdd(p, v); }
APPY_DEV void appy_atomic(appy_add, i64* p, i64 v) { atomicAdd(reinterpret_cast<u64*>(p), (u64)v); }
APPY_DEV void appy_atomic(appy_max, int* p, int v) { atomicMax(p, v); }
APPY_DEV void appy_atomic(appy_min, int* p, int v) { atomicMin(p, v); }
APPY_DEV void appy_atomic(appy_max, i64* p, i64 v) { atomicMax(p, v); }
APPY_DEV void appy_atomic(appy_min, i64* p, i64 v) { atomicMin(p, v); }

template <class Op> APPY_DEV void appy_atomic_cas64(double* p, double v) {
  u64* a = reinterpret_cast<u64*>(p);
  u64 old = *a, assumed;
  do {
    assumed = old;
    double cur = __longlong_as_double((i64)assumed);
    double nxt = Op::template op<double>(cur, v);
    if (nxt == cur) break;
    old = atomicCAS(a, assumed, (u64)__double_as_longlong(nxt));
  } while (old != assumed);
}
template <class Op> APPY_DEV void appy_atomic_cas32(float* p, float v) {
  u32* a = reinterpret_cast<u32*>(p);
  u32 old = *a, assumed;
  do {
    assumed = old;
    float cur = __uint_as_float(assumed);
    float nxt = Op::template op<float>(cur, v);
    if (nxt == cur) break;
    old = atomicCAS(a, assumed, __float_as_uint(nxt));
  } while (old != assumed);
}
APPY_DEV void appy_atomic(appy_max, double* p, double v) { appy_atomic_cas64<appy_max>(p, v); }
APPY_DEV void appy_atomic(appy_min, double* p, double v) { appy_atomic_cas64<appy_min>(p, v); }
APPY_DEV void appy_atomic(appy_max, float* p, float v) { appy_atomic_cas32<appy_max>(p, v); }
APPY_DEV void appy_atomic(appy_min, float* p, float v) { appy_atomic_cas32<appy_min>(p, v); }
// products: CAS loop without the early exit on unchanged value being wrong
// (x * 1 == x leaves the value untouched, which is the right result).
APPY_DEV void appy_atomic(appy_mul, double* p, double v) { appy_atomic_cas64<appy_mul>(p, v); }
APPY_DEV void appy_atomic(appy_mul, float* p, float v) { appy_atomic_cas32<appy_mul>(p, v); }

// ---------------------------------------------------------------------------
// Python arithmetic semantics
// ---------------------------------------------------------------------------
template <class T> APPY_DEV T appy_floordiv(T a, T b) {
  T q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}
template <class T> APPY_DEV T appy_pymod(T a, T b) {
  T r = a % b;
  if (r != 0 && ((r < 0) != (b < 0))) r += b;
  return r;
}
APPY_DEV double appy_floordiv(double a, double b) { return floor(a / b); }
APPY_DEV float appy_floordiv(float a, float b) { return floorf(a / b); }
APPY_DEV double appy_pymod(double a, double b) {
  double r = fmod(a, b);
  if (r != 0.0 && ((r < 0.0) != (b < 0.0))) r += b;
  return r;
}
APPY_DEV float appy_pymod(float a, float b) {
  float r = fmodf(a, b);
  if (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) r += b;
  return r;
}
// float32 division as the reference's Triton backend performs it: div.full.f32 (full range, 2 ulp)
APPY_DEV float appy_div_full(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// tanh.approx.f32, the instruction behind libdevice's fast_tanhf
APPY_DEV float appy_tanh_approx(float a) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}
template <class T> APPY_DEV T appy_tmax(T a, T b) { return a > b ? a : b; }
template <class T> APPY_DEV T appy_tmin(T a, T b) { return a < b ? a : b; }
