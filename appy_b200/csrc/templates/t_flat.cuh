// T1 / T2: flat lowering of `#pragma parallel for simd` loops
// (reference lowering: appy/backends/triton/passes/block_loop.py:77-159 tiles the
// loop by 256 and device_passes/remove_loop_head.py:3-55 gives one tile to each
// program; device_passes/rewrite_par_reduce_to_atomics.py:10-88 issues one atomic
// per tile for shared(...) reductions).
//
// Here one thread owns V consecutive iterations (one 16-byte access per array),
// a CTA owns U such chunks per thread, and the grid strides over CTA tiles.
// The body is a functor generated per loop (or hand-written for the prebuilt
// kernels) with this interface:
//
//   struct Body {
//     struct Regs { ... };                      // streamed operands of one chunk
//     void load(i64 i0, Regs&) const;           // issue the 16-byte loads of chunk [i0, i0+V)
//     void compute(i64 i0, const Regs&);        // evaluate V iterations, store, accumulate
//     void one(i64 i);                          // one iteration, scalar accesses (ragged edges)
//     void finish(void* smem);                  // reduction epilogue (empty for T1)
//   };
//
// `load` for all U chunks is issued before any `compute`, so every thread keeps
// U x (#streamed arrays) 16-byte loads in flight regardless of what the compiler
// can prove about aliasing between inputs and outputs.
#pragma once
#include "appy_device.cuh"

template <int V, int U, class Body>
APPY_DEV void appy_flat(Body& body, i64 lo, i64 hi, void* smem) {
  if (hi > lo) {
    // chunk c covers iterations [c*V, c*V+V); chunks are aligned to multiples of V in
    // absolute index space so that 16-byte aligned bases stay aligned for any lo.
    const i64 c_lo = appy_floor_div_i64(lo, V);
    const i64 c_hi = appy_floor_div_i64(hi - 1, V) + 1;
    const i64 c_full_lo = appy_floor_div_i64(lo + V - 1, V);   // first chunk fully inside
    const i64 c_full_hi = appy_floor_div_i64(hi, V);           // one past last chunk fully inside
    const i64 tile = (i64)blockDim.x * U;
    for (i64 t = c_lo + (i64)blockIdx.x * tile; t < c_hi; t += (i64)gridDim.x * tile) {
      if (t >= c_full_lo && t + tile <= c_full_hi) {
        typename Body::Regs r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) body.load((t + (i64)u * blockDim.x + threadIdx.x) * V, r[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) body.compute((t + (i64)u * blockDim.x + threadIdx.x) * V, r[u]);
      } else {
#pragma unroll 1
        for (int u = 0; u < U; ++u) {
          const i64 c = t + (i64)u * blockDim.x + threadIdx.x;
          if (c >= c_full_lo && c < c_full_hi) {
            typename Body::Regs r;
            body.load(c * V, r);
            body.compute(c * V, r);
          } else if (c < c_hi) {
#pragma unroll 1
            for (int k = 0; k < V; ++k) {
              const i64 i = c * V + k;
              if (i >= lo && i < hi) body.one(i);
            }
          }
        }
      }
    }
  }
  body.finish(smem);
}

// ---------------------------------------------------------------------------
// Grid-level commit of one reduction variable.
//
// Mode A (atomic): thread 0 of every CTA issues one atomic on the target scalar.
// Mode B (ordered): every CTA publishes its partial into a workspace slot; the CTA
// that draws the last ticket folds the partials in slot order and updates the target
// with a plain read-modify-write, so the result does not depend on CTA scheduling.
// The ticket counter wraps back to zero by itself (atomicInc with limit gridDim.x-1),
// so the workspace needs zeroing only once, when it is created.
//
// Workspace layout (bytes): [0,4) ticket, [256, 256 + 8*slots*gridDim.x) partials,
// variable r using elements [r*gridDim.x, (r+1)*gridDim.x) of 8-byte cells.
// ---------------------------------------------------------------------------
struct appy_ws {
  unsigned* ticket;
  double* cells;   // 8-byte cells, reinterpret per variable type
};
APPY_DEV appy_ws appy_ws_from(void* base) {
  appy_ws w;
  w.ticket = reinterpret_cast<unsigned*>(base);
  w.cells = reinterpret_cast<double*>(reinterpret_cast<char*>(base) + 256);
  return w;
}

template <class T> APPY_DEV void appy_ws_publish(const appy_ws& w, int var, T v) {
  if (threadIdx.x == 0) {
    T* cell = reinterpret_cast<T*>(w.cells + (size_t)var * gridDim.x + blockIdx.x);
    __stcg(cell, v);
  }
}
// returns true (to every thread of the CTA) in the CTA that arrives last
APPY_DEV bool appy_ws_arrive(const appy_ws& w, void* smem) {
  int* flag = reinterpret_cast<int*>(smem);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned t = atomicInc(w.ticket, gridDim.x - 1);
    *flag = (t == gridDim.x - 1);
  }
  __syncthreads();
  const bool last = *flag != 0;
  __syncthreads();
  if (last) __threadfence();
  return last;
}
template <class Op, class T> APPY_DEV T appy_ws_collect(const appy_ws& w, int var, void* smem) {
  // fixed association order: thread t folds cells t, t+B, t+2B, ... then the block tree
  const T* cells = reinterpret_cast<const T*>(w.cells + (size_t)var * gridDim.x);
  T acc = Op::template id<T>();
  for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
    const T* cell = reinterpret_cast<const T*>(reinterpret_cast<const double*>(cells) + b);
    acc = Op::template op<T>(acc, __ldcg(cell));
  }
  return appy_block_reduce<Op, T>(acc, reinterpret_cast<T*>(smem));
}

// ---------------------------------------------------------------------------
// Cross-GPU combine of shared(...) scalars, fused into the reduction kernel's tail.
//
// Every rank (one process per GPU) owns a mailbox in its own HBM and holds peer pointers to
// the mailboxes of all ranks (CUDA IPC mappings; NVLink/NVSwitch).  After the ordered commit
// has produced this GPU's totals, the first warp of the last CTA runs the exchange, lane r
// talking to rank r:
//   1. lane r stores the totals into this rank's slot of rank r's mailbox;
//   2. lane r polls (bounded) the slot of rank r in this rank's OWN mailbox;
//   3. the warp folds the world's totals in rank order, so every rank obtains the same bits.
// A value travels as 8-byte words {32 payload bits, 32-bit tag of the launch}: an aligned
// 8-byte store is single-copy atomic, payload and tag arrive together, and neither side needs
// a fence or a separate flag (the scheme of low-latency collective protocols).  A total of up
// to 8 bytes takes two words.  No kernel reads a peer's memory; only these words cross GPUs.
// Slots are double-buffered by the parity of the launch sequence number: a rank can be at most
// one launch ahead of the slowest rank, because finishing launch s needs every rank's words
// of launch s.  The tag is the low 31 bits of s with bit 31 set, so it differs from the tag
// two launches earlier and from freshly zeroed memory.
// The wait is limited; on expiry the error word is set and floating-point results are set to NaN,
// so a missing rank makes the launch return with a status the host reads, never a hang.
//
// Mailbox of one rank: [parity 0..1][source rank 0..world-1] x 8 words of 8 bytes;
// variable v (up to 4 per loop) uses words 2v (low half) and 2v+1 (high half).
// ---------------------------------------------------------------------------
struct appy_mailbox {
  int world;
  int rank;
  unsigned spin_limit;      // polls per source rank before giving up (20 ns, later 1 us apart)
  unsigned reserved;
  unsigned* err;            // set to 1 when a wait ran out
  u64* peer[16];            // peer[r] = mailbox of rank r as mapped into this process
  u64* own;                 // peer[rank], so that it can be read without knowing the rank first
};

APPY_DEV void appy_st_relaxed_sys(u64* p, u64 v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
APPY_DEV u64 appy_ld_relaxed_sys(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

template <class T> APPY_DEV u64 appy_to_bits(T v) {
  union { T t; u64 u; } x;
  x.u = 0;
  x.t = v;
  return x.u;
}
template <class T> APPY_DEV T appy_from_bits(u64 u) {
  union { T t; u64 u; } x;
  x.u = u;
  return x.t;
}

// Steps 1 and 2, called by the 32 threads of warp 0.  In: x[v] = this rank's total of variable v
// (raw bits, same in every lane).  Out: in lane r < world, x[v] = rank r's total of variable v.
// Returns false (to every lane) when some rank's words did not arrive within the limit.
template <int NV> APPY_DEV bool appy_p2p_exchange(const appy_mailbox* mb, u64 seq, u64 (&x)[NV]) {
  const int world = mb->world, rank = mb->rank;
  const int lane = threadIdx.x & 31;
  const u64 tag = (u64)((unsigned)seq | 0x80000000u) << 32;
  bool ok = true;
  if (lane < world) {
    u64* dst = mb->peer[lane] + ((seq & 1) * world + rank) * 8;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      appy_st_relaxed_sys(dst + 2 * v, tag | (x[v] & 0xffffffffull));
      appy_st_relaxed_sys(dst + 2 * v + 1, tag | (x[v] >> 32));
    }
    const u64* src = mb->peer[rank] + ((seq & 1) * world + lane) * 8;
    const unsigned limit = mb->spin_limit;
    unsigned spins = 0;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      u64 lo, hi;
      for (;;) {
        lo = appy_ld_relaxed_sys(src + 2 * v);
        hi = appy_ld_relaxed_sys(src + 2 * v + 1);
        if (((lo ^ tag) >> 32) == 0 && ((hi ^ tag) >> 32) == 0) break;
        if (!ok || ++spins > limit) {
          ok = false;
          break;
        }
        __nanosleep(spins < 256 ? 20 : 1000);
      }
      x[v] = (hi << 32) | (lo & 0xffffffffull);
    }
    if (!ok) atomicExch(mb->err, 1u);
  }
  return __all_sync(0xffffffffu, ok) != 0;
}
// A combine that timed out must not look like a result: floating-point totals become NaN (integer
// totals cannot be marked; the status word is the only sign there).
template <class T> APPY_DEV T appy_p2p_poison(T v) { return v; }
template <> APPY_DEV float appy_p2p_poison<float>(float) { return __int_as_float(0x7fc00000); }
template <> APPY_DEV double appy_p2p_poison<double>(double) { return __longlong_as_double(0x7ff8000000000000ll); }
// Step 3, called by the 32 threads of warp 0 with lane r holding rank r's total.
template <class Op, class T> APPY_DEV T appy_p2p_fold(const appy_mailbox* mb, u64 bits) {
  const int world = mb->world;
  T total = Op::template id<T>();
  for (int r = 0; r < world; ++r)
    total = Op::template op<T>(total, appy_from_bits<T>(__shfl_sync(0xffffffffu, bits, r)));
  return total;
}

// ---------------------------------------------------------------------------
// Split-phase form of the exchange (`@jit(combine="p2p", defer=True)`).
//
// The exchange above makes every reduction kernel end with a chain of waits: the ordered commit (a fence, a
// ticket, the last CTA's fold of all partials), then the slowest rank and one NVLink round trip.  Here the
// kernel's tail is only what a single-GPU reduction has: every CTA stores its partial and is done.  The rest
// moves to the START of the next two kernels, where one warp (warp 0 of the last CTA) does it beside the
// kernel's own work:
//   launch k      every CTA stores its partial (slot of parity k in the workspace);
//   launch k + 1  that warp FOLDS the partials of launch k — complete, because launch k has ended — and POSTS
//                 the GPU's totals: stores into every rank's mailbox, its own included;
//   launch k + 2  that warp COLLECTS launch k: the ranks' words have long arrived, it folds them in rank
//                 order and applies the result to the shared(...) cells.
// A stand-alone one-warp kernel (flush) runs the same two steps for the launches that no later kernel
// serves.  The cells of a loop hold their final value once the second launch after it, or the flush, has
// run, and must be left alone until then.
//
// Posted words live in a ring of APPY_MB_RING slots per mailbox, indexed by the count of split-phase
// launches, at byte offset 4096 (after the two slots of the immediate exchange).  A rank posts launch k + 8
// only after it collected k + 6, which needs every rank's words of k + 6, posted after those ranks read k:
// a slot is never overwritten unread.  A launch is described by values alone (cell addresses, operator and
// type codes, the address and number of its partials), because the kernel that serves it was generated for
// another loop.
// ---------------------------------------------------------------------------
#define APPY_MB_RING 8
enum { APPY_PEND_ADD = 0, APPY_PEND_MUL = 1, APPY_PEND_MAX = 2, APPY_PEND_MIN = 3 };
enum { APPY_PEND_F32 = 0, APPY_PEND_F64 = 1, APPY_PEND_I32 = 2, APPY_PEND_I64 = 3 };

struct appy_pending {      // one earlier split-phase launch; seq == 0: none
  u64 seq;                 // its launch number (the tag of its words)
  int nv;                  // its shared(...) variables (1..4)
  int grid;                // its CTAs = partials per variable
  int slot;                // its ring slot
  int pad;
  void* partials;          // its partials: variable r in the 8-byte cells [r*grid, (r+1)*grid)
  void* cell[4];           // the shared(...) cells, in this GPU's memory
  int op[4];               // APPY_PEND_ADD ..
  int ty[4];               // APPY_PEND_F32 ..
};
struct appy_pending2 {
  appy_pending fold;       // the launch before this one: fold its partials and post the totals
  appy_pending coll;       // the launch before that: collect the ranks' totals into its cells
  void* partials;          // where THIS launch's CTAs store their partials
};

APPY_DEV u64* appy_mb_ring_words(u64* mailbox, int slot, int world, int src) {
  return mailbox + 512 + ((u64)slot * (u64)world + src) * 8;
}

template <class T> APPY_DEV T appy_fold_any(int op, T a, T b) {
  if (op == APPY_PEND_ADD) return a + b;
  if (op == APPY_PEND_MUL) return a * b;
  if (op == APPY_PEND_MAX) return a > b ? a : b;
  return a < b ? a : b;
}
APPY_DEV u64 appy_fold_bits(int op, int ty, u64 a, u64 b) {
  if (ty == APPY_PEND_F32) return appy_to_bits<float>(appy_fold_any<float>(op, appy_from_bits<float>(a), appy_from_bits<float>(b)));
  if (ty == APPY_PEND_F64) return appy_to_bits<double>(appy_fold_any<double>(op, appy_from_bits<double>(a), appy_from_bits<double>(b)));
  if (ty == APPY_PEND_I32) return appy_to_bits<int>(appy_fold_any<int>(op, appy_from_bits<int>(a), appy_from_bits<int>(b)));
  return appy_to_bits<i64>(appy_fold_any<i64>(op, appy_from_bits<i64>(a), appy_from_bits<i64>(b)));
}
template <class T> APPY_DEV u64 appy_identity_of(int op) {
  if (op == APPY_PEND_ADD) return appy_to_bits<T>(appy_add::id<T>());
  if (op == APPY_PEND_MUL) return appy_to_bits<T>(appy_mul::id<T>());
  if (op == APPY_PEND_MAX) return appy_to_bits<T>(appy_max::id<T>());
  return appy_to_bits<T>(appy_min::id<T>());
}
APPY_DEV u64 appy_identity_bits(int op, int ty) {
  if (ty == APPY_PEND_F32) return appy_identity_of<float>(op);
  if (ty == APPY_PEND_F64) return appy_identity_of<double>(op);
  if (ty == APPY_PEND_I32) return appy_identity_of<int>(op);
  return appy_identity_of<i64>(op);
}

// The descriptor's fields read once, all loads independent of one another (it lives in device memory, and
// every store of the exchange is a compiler barrier that would otherwise force them to be read again).
struct appy_mb_view {
  int world, rank;
  unsigned limit;
  unsigned* err;
  u64* to;       // lane r: mailbox of rank r
  u64* own;      // this rank's mailbox
};
APPY_DEV appy_mb_view appy_mb_open(const appy_mailbox* mb) {
  appy_mb_view v;
  v.world = mb->world;
  v.rank = mb->rank;
  v.limit = mb->spin_limit;
  v.err = mb->err;
  v.to = mb->peer[threadIdx.x & 15];
  v.own = mb->own;
  return v;
}

// What a CTA of a split-phase kernel does in its tail: thread 0 stores the CTA's partial of variable `var`.
template <class T> APPY_DEV void appy_split_publish(void* partials, int var, T v) {
  if (threadIdx.x == 0) {
    T* cell = reinterpret_cast<T*>(reinterpret_cast<double*>(partials) + (size_t)var * gridDim.x + blockIdx.x);
    __stcg(cell, v);
  }
}

struct appy_collect_regs { u64 lo[4], hi[4], cell[4]; };

// Called by the 32 threads of one warp (warp 0 of the last CTA at the start of a split-phase kernel, or the flush
// kernel): folds and posts p.fold, collects p.coll.  The reads that the collect needs go out first, so that
// their latency hides behind the fold.  A wait that runs out sets the error word and turns floating-point
// results into NaN, as in the immediate exchange.
APPY_DEV void appy_split_service(const appy_mailbox* mb, const appy_pending2& p) {
  if (p.fold.seq == 0 && p.coll.seq == 0) return;
  const int lane = threadIdx.x & 31;
  const appy_mb_view mv = appy_mb_open(mb);
  appy_collect_regs r;
  const appy_pending& c = p.coll;
  const u64* src = appy_mb_ring_words(mv.own, c.slot, mv.world, lane < mv.world ? lane : 0);
  if (c.seq != 0) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      if (v < c.nv) {
        r.lo[v] = appy_ld_relaxed_sys(src + 2 * v);
        r.hi[v] = appy_ld_relaxed_sys(src + 2 * v + 1);
        if (lane == 0) {
          if (c.ty[v] == APPY_PEND_F32 || c.ty[v] == APPY_PEND_I32) r.cell[v] = (u64)*reinterpret_cast<const unsigned*>(c.cell[v]);
          else r.cell[v] = *reinterpret_cast<const u64*>(c.cell[v]);
        }
      }
    }
  }
  // ---- fold the partials of the previous launch (fixed order: lane l takes cells l, l+32, ..; then the
  // lanes are folded by a butterfly), and post the totals
  const appy_pending& f = p.fold;
  if (f.seq != 0) {
    const u64 tag = (u64)((unsigned)f.seq | 0x80000000u) << 32;
    u64* dst = appy_mb_ring_words(mv.to, f.slot, mv.world, mv.rank);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      if (v < f.nv) {
        const int op = f.op[v], ty = f.ty[v];
        const bool narrow = ty == APPY_PEND_F32 || ty == APPY_PEND_I32;
        const u64* cells = reinterpret_cast<const u64*>(f.partials) + (size_t)v * f.grid;
        u64 acc = appy_identity_bits(op, ty);
        for (int b = lane; b < f.grid; b += 32) {
          const u64 raw = __ldcg(cells + b);
          acc = appy_fold_bits(op, ty, acc, narrow ? (raw & 0xffffffffull) : raw);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc = appy_fold_bits(op, ty, acc, __shfl_xor_sync(0xffffffffu, acc, m));
        if (lane < mv.world) {
          appy_st_relaxed_sys(dst + 2 * v, tag | (acc & 0xffffffffull));
          appy_st_relaxed_sys(dst + 2 * v + 1, tag | (acc >> 32));
        }
      }
    }
  }
  // ---- collect: words that had not arrived yet are waited for (bounded)
  if (c.seq != 0) {
    const u64 tag = (u64)((unsigned)c.seq | 0x80000000u) << 32;
    unsigned spins = 0;
    bool ok = true;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      if (v < c.nv) {
        u64 lo = r.lo[v], hi = r.hi[v];
        if (lane < mv.world) {
          while (((lo ^ tag) >> 32) != 0 || ((hi ^ tag) >> 32) != 0) {
            if (!ok || ++spins > mv.limit) {
              ok = false;
              break;
            }
            __nanosleep(spins < 256 ? 20 : 1000);
            lo = appy_ld_relaxed_sys(src + 2 * v);
            hi = appy_ld_relaxed_sys(src + 2 * v + 1);
          }
        }
        const bool all_ok = __all_sync(0xffffffffu, ok) != 0;
        const u64 mine = (hi << 32) | (lo & 0xffffffffull);
        u64 total = __shfl_sync(0xffffffffu, mine, 0);
        for (int q = 1; q < mv.world; ++q) total = appy_fold_bits(c.op[v], c.ty[v], total, __shfl_sync(0xffffffffu, mine, q));
        if (lane == 0) {
          const int ty = c.ty[v];
          if (!all_ok) {
            atomicExch(mv.err, 1u);
            if (ty == APPY_PEND_F32) total = appy_to_bits<float>(appy_p2p_poison<float>(0.f));
            if (ty == APPY_PEND_F64) total = appy_to_bits<double>(appy_p2p_poison<double>(0.0));
          }
          const u64 res = appy_fold_bits(c.op[v], ty, r.cell[v], total);
          if (ty == APPY_PEND_F32 || ty == APPY_PEND_I32) *reinterpret_cast<unsigned*>(c.cell[v]) = (unsigned)res;
          else *reinterpret_cast<u64*>(c.cell[v]) = res;
        }
      }
    }
  }
}
