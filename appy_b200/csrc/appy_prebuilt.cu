// Prebuilt (nvcc-compiled) instantiations of the five kernel templates for the
// canonical float32 / int32 workloads, exported through the C ABI.  The bodies
// below are what the Python code generator emits for the corresponding loops;
// they are written out by hand here so that the library is usable from C and so
// that `nvcc -Xptxas -v` reports registers and spills at build time.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/appy_sm100.h"
#include "templates/t_csr_dense_stream.cuh"
#include "templates/t_csr_rows.cuh"
#include "templates/t_flat.cuh"
#include "templates/t_rowdot.cuh"

void appy_note_launch();
int appy_fail_cuda(cudaError_t e, const char* what);
int appy_fail_arg(const char* what);

namespace {

int g_sm_count[16] = {0};
int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 148;
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

int finish_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return appy_fail_cuda(e, what);
  appy_note_launch();
  return APPY_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ------------------------------------------------------------------ T1: c[i] = a[i] + b[i]
template <int V> struct VecAddBody {
  const float* __restrict__ a;
  const float* __restrict__ b;
  float* __restrict__ c;
  struct Regs { appy_pack<float, V> a, b; };
  APPY_DEV void load(i64 i0, Regs& r) const {
    r.a = appy_ld_cs<float, V>(a + i0);
    r.b = appy_ld_cs<float, V>(b + i0);
  }
  APPY_DEV void compute(i64 i0, const Regs& r) {
    appy_pack<float, V> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = r.a.v[k] + r.b.v[k];
    appy_st_cs<float, V>(c + i0, o);
  }
  APPY_DEV void one(i64 i) { c[i] = a[i] + b[i]; }
  APPY_DEV void finish(void*) {}
};

template <int V, int U>
__global__ void __launch_bounds__(256) k_vec_add(const float* a, const float* b, float* c, i64 n) {
  VecAddBody<V> body{a, b, c};
  appy_flat<V, U>(body, 0, n, nullptr);
}

// ------------------------------------------------------------------ T2: b += a[i]  (optionally masked)
template <int V, bool MASKED, bool ORDERED> struct SumBody {
  const float* __restrict__ a;
  const u8* __restrict__ m;
  double* result;
  void* ws;
  float acc[V];   // V independent float32 lanes per thread; folded in double at the end
  struct Regs { appy_pack<float, V> a; appy_pack<u8, V> m; };
  APPY_DEV void init() {
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
  }
  APPY_DEV void load(i64 i0, Regs& r) const {
    r.a = appy_ld_cs<float, V>(a + i0);
    if (MASKED) r.m = appy_ld_cs<u8, V>(m + i0);
  }
  APPY_DEV void compute(i64, const Regs& r) {
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] += (MASKED && !r.m.v[k]) ? 0.f : r.a.v[k];
  }
  APPY_DEV void one(i64 i) {
    if (!MASKED || m[i]) acc[0] += a[i];
  }
  APPY_DEV void finish(void* smem) {
    double t = 0.0;
#pragma unroll
    for (int k = 0; k < V; ++k) t += (double)acc[k];
    t = appy_block_reduce<appy_add, double>(t, reinterpret_cast<double*>(smem));
    if (!ORDERED) {
      if (threadIdx.x == 0) appy_atomic(appy_add(), result, t);
    } else {
      const appy_ws w = appy_ws_from(ws);
      appy_ws_publish<double>(w, 0, t);
      if (appy_ws_arrive(w, smem)) {
        const double total = appy_ws_collect<appy_add, double>(w, 0, smem);
        if (threadIdx.x == 0) *result = *result + total;
      }
    }
  }
};

// 512-thread CTAs, two per SM, register budget left open (second launch bound = 1) so that all U
// loads of a thread are issued before the first add: measured 4-5 % faster on 2^26 elements than
// 256-thread CTAs at eight per SM.
const int kSumBlock = 512, kSumCtasPerSm = 2;

template <int V, int U, bool MASKED, bool ORDERED>
__global__ void __launch_bounds__(kSumBlock, 1) k_sum(const float* a, const u8* m, i64 n, double* result, void* ws) {
  __shared__ double smem[32];
  SumBody<V, MASKED, ORDERED> body;
  body.a = a; body.m = m; body.result = result; body.ws = ws;
  body.init();
  appy_flat<V, U>(body, 0, n, smem);
}

// ------------------------------------------------------------------ T3: SpMV
struct SpmvBody {
  typedef float Acc;
  typedef appy_add Op;
  const float* __restrict__ data;
  const int* __restrict__ indices;
  const float* __restrict__ x;
  float* __restrict__ y;
  APPY_DEV float term(i64 k) const {
    return appy_ld_cs<float, 1>(data + k).v[0] * appy_ldg1(x + appy_ld_cs<int, 1>(indices + k).v[0]);
  }
  APPY_DEV void finish(i64 i, float total) const { y[i] = total; }
};

template <int BLOCK, int CHUNK, int LONG>
__global__ void __launch_bounds__(BLOCK) k_spmv_stream(SpmvBody body, const int* indptr, i64 lo, i64 hi) {
  __shared__ __align__(16) unsigned char smem[CHUNK * sizeof(float) + (BLOCK + 1) * sizeof(i64)];
  appy_csr_stream<BLOCK, CHUNK, LONG, int>(body, indptr, lo, hi, smem);
}
const int kSpmvRows = 64, kSpmvBlock = 128;
template <int G>
__global__ void __launch_bounds__(kSpmvBlock) k_spmv_vector(SpmvBody body, const int* indptr, i64 lo, i64 hi) {
  __shared__ __align__(16) unsigned char smem[32 * sizeof(float) + (2 * kSpmvRows + 2) * sizeof(int)];
  appy_csr_vector<G, kSpmvBlock, kSpmvRows, 16 * G, 512, int>(body, indptr, lo, hi, smem);
}

// ------------------------------------------------------------------ T4: GEMV
template <int V> struct GemvBody {
  typedef float Acc;
  typedef appy_add Op;
  float alpha;
  const float* __restrict__ A;
  i64 lda;
  const float* __restrict__ x;
  float* __restrict__ y;
  i64 ncols;
  struct Regs { appy_pack<float, V> a, x; };
  APPY_DEV void bounds(i64, i64& jlo, i64& jhi) const { jlo = 0; jhi = ncols; }
  APPY_DEV void load(i64 i, i64 j0, Regs& r) const {
    r.a = appy_ld_cs<float, V>(A + i * lda + j0);
    r.x = appy_ld_nc<float, V>(x + j0);
  }
  APPY_DEV float fold(i64, i64, const Regs& r, float acc) const {
#pragma unroll
    for (int k = 0; k < V; ++k) acc = acc + alpha * r.a.v[k] * r.x.v[k];
    return acc;
  }
  APPY_DEV float one(i64 i, i64 j, float acc) const { return acc + alpha * A[i * lda + j] * x[j]; }
  APPY_DEV void finish(i64 i, float total) const { y[i] = total; }
};

template <int G, int V, int U, int R>
__global__ void __launch_bounds__(G == 32 ? 128 : 256, G == 32 ? 4 : 2) k_gemv(GemvBody<V> body, i64 lo, i64 hi) {
  __shared__ float smem[32];
  appy_rowdot<G, V, U, R>(body, lo, hi, smem);
}

// ------------------------------------------------------------------ T5: SpMM
template <class OffT> struct SpmmBody {
  typedef float Elt;
  typedef OffT Off;
  const float* __restrict__ data;
  const int* __restrict__ indices;
  const float* __restrict__ B;
  i64 ldb;
  float* __restrict__ C;
  i64 ldc;
  APPY_DEV float coef(i64 k) const { return appy_ld_cs<float, 1>(data + k).v[0]; }
  APPY_DEV Off brow_off(i64 k) const { return (Off)appy_ld_cs<int, 1>(indices + k).v[0] * (Off)ldb; }
  APPY_DEV const float* bbase() const { return B; }
  APPY_DEV float* crow_ptr(i64 i) const { return C + i * ldc; }
  APPY_DEV float init() const { return 0.f; }
};

const int kSpmmRows = 32;

// One row = one 16-byte pack per lane (V = 4, T = 1): 16 warps per CTA, three CTAs per SM, four gathers in
// flight per warp, no rolling ring (measured best on the 2^18-row, 128-column case: 634 us against 673 us
// for 8 warps x 4 CTAs with a rolling ring of 8).  Wider rows keep 8 warps and fewer, larger gathers.
template <int V, int T, int D, int MINB, int NC, int WARPS, bool ROLL, class OffT>
__global__ void __launch_bounds__(32 * WARPS, MINB)
k_spmm(SpmmBody<OffT> body, const int* indptr, i64 lo, i64 hi, int ncols) {
  __shared__ __align__(16) unsigned char smem[appy_csr_dense_smem<V, T, WARPS, kSpmmRows, float>::bytes];
  appy_csr_dense<V, T, D, WARPS, kSpmmRows, NC, ROLL, int>(body, indptr, lo, hi, ncols, smem);
}

template <int V, int T, int D, int MINB, int NC, class OffT>
int launch_spmm(const SpmmBody<OffT>& body, const int* indptr, i64 lo, i64 hi, int ncols, cudaStream_t s) {
  const i64 tiles = (hi - lo + kSpmmRows - 1) / kSpmmRows;
  const unsigned grid = (unsigned)std::min<i64>(tiles, 1 << 30);
  const int WARPS = (V == 4 && T == 1) ? 16 : 8;
  k_spmm<V, T, D, MINB, NC, WARPS, false, OffT><<<grid, 32 * WARPS, 0, s>>>(body, indptr, lo, hi, ncols);
  return finish_launch("spmm launch");
}

// Streaming form (t_csr_dense_stream.cuh): one wave of CTAs, every warp an equal share of the non-zeros, D rows
// of B in flight per warp in a shared-memory ring, and a second kernel for rows cut by share boundaries and
// rows without non-zeros.  Used from kSpmmStreamRows rows on; below that one CTA per 32 rows is over sooner.
const int kSpmmStreamRows = 4096;

template <int V, int T, int D, int WARPS, int MINB, int NC, class OffT>
__global__ void __launch_bounds__(32 * WARPS, MINB)
k_spmm_stream(SpmmBody<OffT> body, const int* indptr, i64 lo, i64 hi, int ncols, void* scratch) {
  extern __shared__ __align__(16) unsigned char dyn[];
  appy_csr_dense_stream<V, T, D, WARPS, NC, true, int>(body, indptr, lo, hi, ncols, scratch, dyn);
}
template <int V, int T, int NC, class OffT>
__global__ void __launch_bounds__(256)
k_spmm_fixup(SpmmBody<OffT> body, const int* indptr, i64 lo, i64 hi, int ncols, void* scratch) {
  appy_csr_dense_fixup<V, T, NC, int>(body, indptr, lo, hi, ncols, scratch);
}

template <int V, int T, int D, int WARPS, int MINB, int NC, class OffT>
int launch_spmm_stream(const SpmmBody<OffT>& body, const int* indptr, i64 lo, i64 hi, int ncols, cudaStream_t s) {
  const int sms = sm_count();
  const unsigned grid = (unsigned)(sms * MINB);
  const size_t workers = (size_t)grid * WARPS;
  void* scratch = nullptr;
  if (int rc = appy_scratch(s, APPY_SD_SCRATCH_BYTES(workers, 32 * V * T, sizeof(float)), &scratch)) return rc;
  const size_t dyn = APPY_SD_SMEM_BYTES(WARPS, D, 32 * V * T, sizeof(float));
  static bool allowed[16] = {false};       // per instantiation and device: raise the dynamic shared-memory limit once
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !allowed[dev]) {
    cudaError_t e = cudaFuncSetAttribute(k_spmm_stream<V, T, D, WARPS, MINB, NC, OffT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
    if (e != cudaSuccess) return appy_fail_cuda(e, "cudaFuncSetAttribute(spmm stream)");
    allowed[dev] = true;
  }
  k_spmm_stream<V, T, D, WARPS, MINB, NC, OffT><<<grid, 32 * WARPS, dyn, s>>>(body, indptr, lo, hi, ncols, scratch);
  if (int rc = finish_launch("spmm stream launch")) return rc;
  k_spmm_fixup<V, T, NC, OffT><<<(unsigned)(4 * sms), 256, 0, s>>>(body, indptr, lo, hi, ncols, scratch);
  return finish_launch("spmm fix-up launch");
}

// ------------------------------------------------------------------ gather ceilings (measurement aids)
// What the memory system delivers for the gathers of T3 and T5 alone: the same index streams and the same
// gathered operand as the kernels, no values, no row structure, no output besides one word per thread.
template <int V, int D>
__global__ void __launch_bounds__(512) k_probe_rows(const float* __restrict__ B, i64 ldb, const int* __restrict__ rows,
                                                     i64 n, float* out) {
  const int lane = threadIdx.x & 31;
  const i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((i64)gridDim.x * blockDim.x) >> 5;
  const i64 per = ((n + nw - 1) / nw + 31) / 32 * 32;
  const i64 ks = warp * per, ke = ks + per < n ? ks + per : n;
  appy_pack<float, V> acc;
#pragma unroll
  for (int x = 0; x < V; ++x) acc.v[x] = 0.f;
  const float* bl = B + lane * V;
  for (i64 kb = ks; kb + 32 <= ke; kb += 32) {
    const i64 my = (i64)appy_ld_cs<int, 1>(rows + kb + lane).v[0] * ldb;
#pragma unroll 1
    for (int q = 0; q < 32; q += D) {
      appy_pack<float, V> b[D];
#pragma unroll
      for (int j = 0; j < D; ++j) b[j] = appy_ld_nc<float, V>(bl + appy_shfl<i64>(my, q + j, 32));
#pragma unroll
      for (int j = 0; j < D; ++j)
#pragma unroll
        for (int x = 0; x < V; ++x) acc.v[x] += b[j].v[x];
    }
  }
  float s = 0.f;
#pragma unroll
  for (int x = 0; x < V; ++x) s += acc.v[x];
  out[(i64)blockIdx.x * blockDim.x + threadIdx.x] = s;
}
__global__ void __launch_bounds__(256) k_probe_gather(const float* __restrict__ x, const int* __restrict__ idx, i64 n,
                                                       float* out) {
  float s = 0.f;
  const i64 stride = (i64)gridDim.x * blockDim.x;
  i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    int c[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) c[u] = appy_ld_cs<int, 1>(idx + i + u * stride).v[0];
#pragma unroll
    for (int u = 0; u < 4; ++u) s += appy_ldg1(x + c[u]);
  }
  for (; i < n; i += stride) s += appy_ldg1(x + appy_ld_cs<int, 1>(idx + i).v[0]);
  out[(i64)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// ------------------------------------------------------------------ row-length histogram
template <class IdxT>
__global__ void k_row_hist(const IdxT* indptr, i64 nrows, u64* counts, u64* max_len) {
  __shared__ u64 s_counts[32];
  __shared__ u64 s_max;
  if (threadIdx.x < 32) s_counts[threadIdx.x] = 0;
  if (threadIdx.x == 0) s_max = 0;
  __syncthreads();
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < nrows; i += (i64)gridDim.x * blockDim.x) {
    const i64 len = (i64)indptr[i + 1] - (i64)indptr[i];
    int bin = 0;
    if (len > 0) bin = 64 - __clzll((u64)len);   // len in [2^(bin-1), 2^bin)
    if (bin > 31) bin = 31;
    atomicAdd(&s_counts[bin], 1ull);
    atomicMax(&s_max, (u64)(len > 0 ? len : 0));
  }
  __syncthreads();
  if (threadIdx.x < 32 && s_counts[threadIdx.x]) atomicAdd(&counts[threadIdx.x], s_counts[threadIdx.x]);
  if (threadIdx.x == 0) atomicMax(max_len, s_max);
}

}  // namespace

extern "C" {

int appy_vec_add_f32(const float* da, const float* db, float* dc, int64_t n, void* stream) {
  if (n <= 0) return APPY_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int U = 1;
  if (aligned16(da) && aligned16(db) && aligned16(dc)) {
    const i64 chunks = (n + 3) / 4, tiles = (chunks + 256 * U - 1) / (256 * U);
    k_vec_add<4, U><<<(unsigned)std::min<i64>(tiles, 1 << 30), 256, 0, s>>>(da, db, dc, n);
  } else {
    const i64 tiles = (n + 256 * U - 1) / (256 * U);
    k_vec_add<1, U><<<(unsigned)std::min<i64>(tiles, 1 << 30), 256, 0, s>>>(da, db, dc, n);
  }
  return finish_launch("vec_add launch");
}

static int launch_sum(const float* da, const uint8_t* dmask, int64_t n, double* dresult, int ordered,
                      void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* ws = nullptr;
  if (ordered) {
    if (int rc = appy_workspace(stream, &ws, nullptr)) return rc;
  }
  const int U = 4;
  const bool vec = aligned16(da) && (!dmask || (reinterpret_cast<uintptr_t>(dmask) & 3) == 0);
  const int V = vec ? 4 : 1;
  const i64 chunks = (n + V - 1) / V, tiles = std::max<i64>(1, (chunks + kSumBlock * U - 1) / (kSumBlock * U));
  const unsigned grid = (unsigned)std::min<i64>(tiles, (i64)sm_count() * kSumCtasPerSm);
#define APPY_SUM_CASE(VV, MM, OO) \
  k_sum<VV, U, MM, OO><<<grid, kSumBlock, 0, s>>>(da, dmask, n, dresult, ws)
  if (vec) {
    if (dmask) { if (ordered) APPY_SUM_CASE(4, true, true); else APPY_SUM_CASE(4, true, false); }
    else       { if (ordered) APPY_SUM_CASE(4, false, true); else APPY_SUM_CASE(4, false, false); }
  } else {
    if (dmask) { if (ordered) APPY_SUM_CASE(1, true, true); else APPY_SUM_CASE(1, true, false); }
    else       { if (ordered) APPY_SUM_CASE(1, false, true); else APPY_SUM_CASE(1, false, false); }
  }
#undef APPY_SUM_CASE
  return finish_launch("sum launch");
}

int appy_sum_f32(const float* da, int64_t n, double* dresult, int ordered, void* stream) {
  if (!dresult) return appy_fail_arg("appy_sum_f32: dresult is NULL");
  if (n < 0) n = 0;
  return launch_sum(da, nullptr, n, dresult, ordered, stream);
}

int appy_masked_sum_f32(const float* da, const uint8_t* dmask, int64_t n, double* dresult,
                        int ordered, void* stream) {
  if (!dresult || !dmask) return appy_fail_arg("appy_masked_sum_f32: NULL argument");
  if (n < 0) n = 0;
  return launch_sum(da, dmask, n, dresult, ordered, stream);
}

int appy_spmv_csr_f32(const float* ddata, const int32_t* dindptr, const int32_t* dindices,
                      const float* dx, float* dy, int64_t row_lo, int64_t row_hi, int strategy,
                      void* stream) {
  if (row_hi <= row_lo) return APPY_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SpmvBody body{ddata, dindices, dx, dy};
  const i64 rows = row_hi - row_lo;
  if (strategy == 0) {
    const int BLOCK = 256;
    const i64 tiles = (rows + BLOCK - 1) / BLOCK;
    k_spmv_stream<BLOCK, 8192, 64><<<(unsigned)std::min<i64>(tiles, 1 << 30), BLOCK, 0, s>>>(
        body, dindptr, row_lo, row_hi);
  } else {
    const i64 max_grid = 1 << 30;
#define APPY_SPMV_CASE(G)                                                              \
  case G: {                                                                            \
    const i64 blocks = (rows + kSpmvRows - 1) / kSpmvRows;                             \
    k_spmv_vector<G><<<(unsigned)std::min<i64>(blocks, max_grid), kSpmvBlock, 0, s>>>(body, dindptr, row_lo, row_hi); \
  } break;
    switch (strategy) {
      APPY_SPMV_CASE(1)
      APPY_SPMV_CASE(2)
      APPY_SPMV_CASE(4)
      APPY_SPMV_CASE(8)
      APPY_SPMV_CASE(16)
      APPY_SPMV_CASE(32)
      default: return appy_fail_arg("appy_spmv_csr_f32: strategy must be 0, 1, 2, 4, 8, 16 or 32");
    }
#undef APPY_SPMV_CASE
  }
  return finish_launch("spmv launch");
}

int appy_gemv_f32(float alpha, const float* dA, int64_t lda, const float* dx, float* dy,
                  int64_t row_lo, int64_t row_hi, int64_t ncols, int lanes, void* stream) {
  if (row_hi <= row_lo) return APPY_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const i64 rows = row_hi - row_lo;
  const bool vec = aligned16(dA) && aligned16(dx) && (lda % 4 == 0);
  const i64 cap = (i64)sm_count() * 8;
  if (lanes == 32) {
    const unsigned grid = (unsigned)std::min<i64>((rows + 3) / 4, 1 << 30);
    if (vec) { GemvBody<4> b{alpha, dA, lda, dx, dy, ncols}; k_gemv<32, 4, 4, 1><<<grid, 128, 0, s>>>(b, row_lo, row_hi); }
    else     { GemvBody<1> b{alpha, dA, lda, dx, dy, ncols}; k_gemv<32, 1, 4, 1><<<grid, 128, 0, s>>>(b, row_lo, row_hi); }
  } else if (lanes == 0) {
    // a CTA per pair of rows, eight 16-byte chunks per lane and row in flight; the register
    // footprint keeps two CTAs per SM resident: few, deep, contiguous streams
    const unsigned grid = (unsigned)std::min<i64>((rows + 1) / 2, 1 << 30);
    if (vec) { GemvBody<4> b{alpha, dA, lda, dx, dy, ncols}; k_gemv<0, 4, 8, 2><<<grid, 256, 0, s>>>(b, row_lo, row_hi); }
    else     { GemvBody<1> b{alpha, dA, lda, dx, dy, ncols}; k_gemv<0, 1, 4, 1><<<(unsigned)std::min<i64>(rows, cap), 256, 0, s>>>(b, row_lo, row_hi); }
  } else {
    return appy_fail_arg("appy_gemv_f32: lanes must be 32 or 0");
  }
  return finish_launch("gemv launch");
}

int appy_spmm_csr_f32(const float* ddata, const int32_t* dindptr, const int32_t* dindices,
                      const float* dB, int64_t ldb, float* dC, int64_t ldc, int64_t row_lo,
                      int64_t row_hi, int ncols, void* stream) {
  if (row_hi <= row_lo || ncols <= 0) return APPY_OK;
  if (ncols > 512) return appy_fail_arg("appy_spmm_csr_f32: ncols > 512 is not prebuilt");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SpmmBody<i64> body{ddata, dindices, dB, ldb, dC, ldc};
  const bool vec = aligned16(dB) && aligned16(dC) && ldb % 4 == 0 && ldc % 4 == 0 && ncols % 4 == 0;
  if (vec && row_hi - row_lo >= kSpmmStreamRows && row_hi - row_lo < (i64)1 << 31) {
    const int T = (ncols + 127) / 128;
    if (ncols == 128) return launch_spmm_stream<4, 1, 8, 16, 2, 128, i64>(body, dindptr, row_lo, row_hi, ncols, s);
    switch (T) {
      case 1: return launch_spmm_stream<4, 1, 8, 16, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      case 2: return launch_spmm_stream<4, 2, 8, 8, 3, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      case 3: return launch_spmm_stream<4, 3, 4, 8, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      default: return launch_spmm_stream<4, 4, 4, 8, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
    }
  }
  if (vec) {
    const int T = (ncols + 127) / 128;
    if (ncols == 128) return launch_spmm<4, 1, 4, 3, 128, i64>(body, dindptr, row_lo, row_hi, ncols, s);
    switch (T) {
      case 1: return launch_spmm<4, 1, 4, 3, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      case 2: return launch_spmm<4, 2, 4, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      case 3: return launch_spmm<4, 3, 2, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
      default: return launch_spmm<4, 4, 2, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
    }
  }
  const int T = (ncols + 31) / 32;
  if (T <= 1) return launch_spmm<1, 1, 4, 5, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
  if (T <= 2) return launch_spmm<1, 2, 4, 5, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
  if (T <= 4) return launch_spmm<1, 4, 4, 4, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
  if (T <= 8) return launch_spmm<1, 8, 2, 3, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
  return launch_spmm<1, 16, 2, 2, 0, i64>(body, dindptr, row_lo, row_hi, ncols, s);
}

int appy_probe_row_gather_f32(const float* dB, int64_t ldb, const int32_t* drows, int64_t n, int row_floats,
                              float* dout, void* stream) {
  if (!dB || !drows || !dout || n < 0) return appy_fail_arg("appy_probe_row_gather_f32: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(sm_count() * 2);
  switch (row_floats) {
    case 128: k_probe_rows<4, 8><<<grid, 512, 0, s>>>(dB, ldb, drows, n, dout); break;
    case 64: k_probe_rows<2, 8><<<grid, 512, 0, s>>>(dB, ldb, drows, n, dout); break;
    case 32: k_probe_rows<1, 8><<<grid, 512, 0, s>>>(dB, ldb, drows, n, dout); break;
    default: return appy_fail_arg("appy_probe_row_gather_f32: row_floats must be 128, 64 or 32");
  }
  return finish_launch("row-gather probe launch");
}

int appy_probe_gather_f32(const float* dx, const int32_t* didx, int64_t n, float* dout, void* stream) {
  if (!dx || !didx || !dout || n < 0) return appy_fail_arg("appy_probe_gather_f32: bad arguments");
  k_probe_gather<<<(unsigned)(sm_count() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(dx, didx, n, dout);
  return finish_launch("gather probe launch");
}

int appy_row_histogram(const void* d_indptr, int idx_bytes, int64_t nrows, int64_t* counts32,
                       int64_t* max_len, void* stream) {
  if (!d_indptr || !counts32 || !max_len || (idx_bytes != 4 && idx_bytes != 8))
    return appy_fail_arg("appy_row_histogram: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  u64* dbuf = nullptr;
  if (int rc = appy_malloc(reinterpret_cast<void**>(&dbuf), 33 * sizeof(u64))) return rc;
  cudaError_t e = cudaMemsetAsync(dbuf, 0, 33 * sizeof(u64), s);
  if (e != cudaSuccess) { appy_free(dbuf); return appy_fail_cuda(e, "cudaMemsetAsync"); }
  if (nrows > 0) {
    const unsigned grid = (unsigned)std::min<i64>((nrows + 255) / 256, (i64)sm_count() * 8);
    if (idx_bytes == 4)
      k_row_hist<int><<<grid, 256, 0, s>>>(static_cast<const int*>(d_indptr), nrows, dbuf, dbuf + 32);
    else
      k_row_hist<i64><<<grid, 256, 0, s>>>(static_cast<const i64*>(d_indptr), nrows, dbuf, dbuf + 32);
    if (int rc = finish_launch("row histogram launch")) { appy_free(dbuf); return rc; }
  }
  u64 host[33];
  e = cudaMemcpyAsync(host, dbuf, sizeof host, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  appy_free(dbuf);
  if (e != cudaSuccess) return appy_fail_cuda(e, "row histogram readback");
  for (int b = 0; b < 32; ++b) counts32[b] = (int64_t)host[b];
  *max_len = (int64_t)host[32];
  return APPY_OK;
}

}  // extern "C"
