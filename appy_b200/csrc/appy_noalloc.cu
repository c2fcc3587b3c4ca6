// appy_sum_f32_noalloc: the scheduling-independent float32 sum without any allocation.
//
// Who this is for.  Some callers are not allowed to allocate device memory at the
// point where they need a reduction: code running between a stream-ordered
// allocator's sync points, plug-ins that were handed a fixed memory budget by their
// host application, and latency-critical loops where a first-use cudaMalloc (which
// synchronises the device) is not acceptable.  appy_sum_f32(..., ordered = 1) is not
// usable there, because it takes its per-stream workspace from cudaMalloc the first
// time a stream is seen.  This entry point does the same reduction with its scratch
// in a fixed array that is part of the library image.
//
// What the scratch is.  One 4-byte arrival ticket and one 8-byte partial sum per CTA.
// A CTA sums one tile of kTile elements, publishes its partial, and the CTA that
// arrives last adds the partials in tile order and updates *dresult, so the result
// does not depend on how the CTAs were scheduled.  The array holds kMaxTiles partials:
// inputs longer than kMaxTiles * kTile = 134,217,728 elements are rejected.  Every GPU
// on which the library's code is loaded carries the array (128.25 KiB) until the
// process exits.
//
// What the caller must know.
//  * The first call on each device looks the array's device address up
//    (cudaGetSymbolAddress) and remembers it; make that first call outside any stream
//    capture.  Later calls only enqueue a 256-byte memset of the ticket and the kernel.
//  * All calls share the one array and it keeps whatever the previous call left in
//    it.  The ticket is cleared at the start of every call; the partials need no
//    clearing because every cell that is read has been written by the same launch.
//    Two calls that overlap on the GPU (different streams, or the same stream on two
//    host threads without ordering) race on the array and give wrong sums: order them.
//  * Nothing here calls cudaMalloc, cudaFree, or any routine that allocates device
//    memory; inputs and the output cell are the caller's.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/appy_sm100.h"
#include "templates/t_flat.cuh"

void appy_note_launch();
int appy_fail_cuda(cudaError_t e, const char* what);
int appy_fail_arg(const char* what);

namespace {

const int kBlock = 256, kVec = 4, kUnroll = 8;
const int64_t kTile = (int64_t)kBlock * kVec * kUnroll;   // 8192 elements per CTA
const int kMaxTiles = 16384;
const size_t kScratchBytes = 256 + 8 * (size_t)kMaxTiles;

// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

std::mutex g_setup_mu;
void* g_scratch_ptr[16] = {nullptr};

template <int V> struct OrderedSumBody {
  const float* __restrict__ a;
  double* result;
  void* ws;
  double acc;
  struct Regs { appy_pack<float, V> a; };
  APPY_DEV void load(i64 i0, Regs& r) const { r.a = appy_ld_cs<float, V>(a + i0); }
  APPY_DEV void compute(i64, const Regs& r) {
#pragma unroll
    for (int k = 0; k < V; ++k) acc += (double)r.a.v[k];
  }
  APPY_DEV void one(i64 i) { acc += (double)a[i]; }
  APPY_DEV void finish(void* smem) {
    const double t = appy_block_reduce<appy_add, double>(acc, reinterpret_cast<double*>(smem));
    const appy_ws w = appy_ws_from(ws);
    appy_ws_publish<double>(w, 0, t);
    if (appy_ws_arrive(w, smem)) {
      const double total = appy_ws_collect<appy_add, double>(w, 0, smem);
      if (threadIdx.x == 0) *result = *result + total;
    }
  }
};

template <int V>
__global__ void __launch_bounds__(kBlock) k_sum_noalloc(const float* a, i64 n, double* result, void* ws) {
  __shared__ double smem[32];
  OrderedSumBody<V> body;
  body.a = a;
  body.result = result;
  body.ws = ws;
  body.acc = 0.0;
  appy_flat<V, kUnroll>(body, 0, n, smem);
}

// once per device, with that device current
int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return appy_fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= 16) return appy_fail_arg("appy_sum_f32_noalloc: device index out of range");
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return appy_fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return APPY_OK;
}

}  // namespace

extern "C" int appy_sum_f32_noalloc(const float* da, int64_t n, double* dresult, void* stream) {
  if (!dresult) return appy_fail_arg("appy_sum_f32_noalloc: dresult is NULL");
  if (n <= 0) return APPY_OK;
  if (!da) return appy_fail_arg("appy_sum_f32_noalloc: da is NULL");
  // one CTA per tile; a misaligned input is walked one element per thread, V = 1
  const bool vec = (reinterpret_cast<uintptr_t>(da) & 15) == 0;
  const int64_t per_cta = vec ? kTile : kTile / kVec;
  const int64_t tiles = (n + per_cta - 1) / per_cta;
  if (tiles > kMaxTiles)
    return appy_fail_arg(
        "appy_sum_f32_noalloc: input too long for the built-in scratch "
        "(at most 134,217,728 elements for a 16-byte aligned input, a quarter of that otherwise); "
        "use appy_sum_f32 instead");
  void* ws = nullptr;
  if (int rc = scratch_for_current_device(&ws)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(ws, 0, 256, s);   // the ticket must start at zero
  if (e != cudaSuccess) return appy_fail_cuda(e, "cudaMemsetAsync(scratch ticket)");
  if (vec)
    k_sum_noalloc<kVec><<<(unsigned)tiles, kBlock, 0, s>>>(da, n, dresult, ws);
  else
    k_sum_noalloc<1><<<(unsigned)tiles, kBlock, 0, s>>>(da, n, dresult, ws);
  e = cudaGetLastError();
  if (e != cudaSuccess) return appy_fail_cuda(e, "appy_sum_f32_noalloc launch");
  appy_note_launch();
  return APPY_OK;
}
