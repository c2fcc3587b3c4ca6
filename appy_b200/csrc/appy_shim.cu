// Runtime half of libappy_sm100: context set-up, cached device allocator,
// pinned-host registration, device mirrors of host ranges, NVRTC compile with
// an in-memory and on-disk cubin cache, kernel launch, timing, and the host-side
// integer work for multi-GPU partitioning.  Declarations and the reference
// interfaces they replace are in include/appy_sm100.h.
#include <cuda_runtime.h>
#include <nvrtc.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <dirent.h>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/appy_sm100.h"
#include "templates/t_flat.cuh"      // peer-mailbox exchange used by appy_p2p_combine

namespace {

thread_local std::string g_err;
thread_local std::string g_log;
std::mutex g_mu;
std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CK(call)                                                                          \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess)                                                                \
      return fail(APPY_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_),  \
                  __FILE__, __LINE__);                                                    \
  } while (0)

// ticket + 4 variables x 65536 CTAs of the ordered commit, then the partials of split-phase launches:
// two parities x 4 variables x 4096 CTAs
const size_t kWorkspaceSplitOffset = 256 + 8 * 4 * 65536;
const size_t kWorkspaceSplitBytes = 2 * 8 * 4 * 4096;
const size_t kWorkspaceBytes = kWorkspaceSplitOffset + kWorkspaceSplitBytes;

struct DeviceState {
  bool ready = false;
  cudaStream_t streams[2] = {nullptr, nullptr};
  std::unordered_map<cudaStream_t, void*> workspaces;
  std::multimap<size_t, void*> free_blocks;          // cached allocator: size -> block
  std::unordered_map<void*, size_t> live_blocks;     // block -> rounded size
  std::unordered_set<void*> free_set;                // blocks that sit in free_blocks right now
  struct Scratch { void* dptr; size_t bytes; };
  std::unordered_map<cudaStream_t, Scratch> scratch; // grow-only scratch of the two-kernel templates, per stream
  struct Mirror { void* dptr; size_t bytes; uint64_t last_use; };
  std::unordered_map<const void*, Mirror> mirrors;   // host pointer -> device mirror
  size_t mirror_bytes = 0;
  uint64_t tick = 0;
  std::unordered_map<const void*, size_t> pinned;    // host ranges registered by us
};
DeviceState g_dev[16];

const size_t kStageBytes = 8u << 20;
struct Staging {
  void* buf[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
};
Staging g_stage[16];

const size_t kHostCellBytes = 4096;           // mapped pinned page for shared scalars (appy_host_cells)
void* g_host_cells[16] = {nullptr};
void* g_host_cells_dev[16] = {nullptr};

int staging_for(int dev, Staging** out) {
  Staging& st = g_stage[dev];
  if (!st.buf[0]) {
    for (int i = 0; i < 2; ++i) {
      CK(cudaHostAlloc(&st.buf[i], kStageBytes, cudaHostAllocPortable));
      CK(cudaEventCreateWithFlags(&st.done[i], cudaEventDisableTiming));
    }
  }
  *out = &st;
  return APPY_OK;
}

int cur_device(int* dev) {
  CK(cudaGetDevice(dev));
  if (*dev < 0 || *dev >= 16) return fail(APPY_ERR_STATE, "device index %d out of range", *dev);
  return APPY_OK;
}

size_t round_block(size_t bytes) {
  if (bytes < 512) return 512;
  if (bytes <= (1u << 20)) {  // next power of two
    size_t r = 512;
    while (r < bytes) r <<= 1;
    return r;
  }
  const size_t q = 2u << 20;  // 2 MiB granules above 1 MiB
  return (bytes + q - 1) / q * q;
}

struct Kernel {
  cudaLibrary_t lib = nullptr;
  cudaKernel_t kern = nullptr;
  std::string name;
  std::atomic<size_t> dyn_smem_allowed{48 * 1024};   // raised on demand, once per size
};
std::unordered_map<std::string, Kernel*> g_kernels;  // key: hash + name

// SHA-256 (FIPS 180-4), used for the key of the compiled-kernel cache
struct Sha256 {
  uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
  unsigned char buf[64];
  size_t fill = 0;
  uint64_t total = 0;
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const unsigned char* p) {
    static const uint32_t K[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const void* data, size_t n) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    total += n;
    while (n) {
      const size_t take = std::min(n, sizeof buf - fill);
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  void update(const std::string& t) { update(t.data(), t.size()); }
  std::string hex() {
    const uint64_t bits = total * 8;
    const unsigned char one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    unsigned char len[8];
    for (int i = 0; i < 8; ++i) len[i] = (unsigned char)(bits >> (56 - 8 * i));
    update(len, 8);
    char out[65];
    for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", h[i]);
    return std::string(out, 64);
  }
};

// Digest of every file in a template directory (the generated sources only say
// `#include "t_flat.cuh"`, so the headers' contents have to enter the cache key themselves).
std::unordered_map<std::string, std::string> g_dir_digest;
std::string dir_digest(const std::string& dir) {
  auto it = g_dir_digest.find(dir);
  if (it != g_dir_digest.end()) return it->second;
  std::vector<std::string> names;
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* e = readdir(d))
      if (e->d_name[0] != '.') names.push_back(e->d_name);
    closedir(d);
  }
  std::sort(names.begin(), names.end());
  Sha256 sh;
  for (auto& n : names) {
    std::ifstream f(dir + "/" + n, std::ios::binary);
    if (!f) continue;
    std::string body((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    sh.update(n);
    sh.update("\x1f");
    sh.update(body);
    sh.update("\x1e");
  }
  return g_dir_digest[dir] = sh.hex();
}

// A cache file is: "APPYCUBIN1\n" + 64 hex digits of the key + "\n" + 16 hex digits of the image
// length + "\n" + the image.  Anything else (another key, a torn or truncated file) is not loaded.
const char kCacheMagic[] = "APPYCUBIN1\n";
bool read_cache_file(const std::string& path, const std::string& key_hex, std::vector<char>& image) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::string all((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  const size_t head = sizeof kCacheMagic - 1 + 64 + 1 + 16 + 1;
  if (all.size() < head || all.compare(0, sizeof kCacheMagic - 1, kCacheMagic) != 0) return false;
  if (all.compare(sizeof kCacheMagic - 1, 64, key_hex) != 0) return false;
  unsigned long long len = 0;
  if (sscanf(all.c_str() + sizeof kCacheMagic - 1 + 65, "%16llx", &len) != 1) return false;
  if (all.size() != head + len || len == 0) return false;
  image.assign(all.begin() + head, all.end());
  return true;
}
void write_cache_file(const std::string& path, const std::string& key_hex, const std::vector<char>& image,
                      const void* unique) {
  const std::string tmp = path + ".tmp" + std::to_string((unsigned long long)(uintptr_t)unique);
  std::ofstream f(tmp, std::ios::binary);
  if (!f) return;
  char len[18];
  snprintf(len, sizeof len, "%016llx\n", (unsigned long long)image.size());
  f << kCacheMagic << key_hex << "\n" << len;
  f.write(image.data(), (std::streamsize)image.size());
  f.close();
  if (f) std::rename(tmp.c_str(), path.c_str());    // readers never see a torn file
  else std::remove(tmp.c_str());
}

int load_cubin(const std::vector<char>& image, const char* name, Kernel** out) {
  Kernel* k = new Kernel;
  k->name = name;
  cudaError_t e = cudaLibraryLoadData(&k->lib, image.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (e != cudaSuccess) {
    delete k;
    return fail(APPY_ERR_CUDA, "cudaLibraryLoadData failed: %s", cudaGetErrorString(e));
  }
  e = cudaLibraryGetKernel(&k->kern, k->lib, name);
  if (e != cudaSuccess) {
    cudaLibraryUnload(k->lib);
    delete k;
    return fail(APPY_ERR_CUDA, "kernel `%s` not found in compiled image: %s", name,
                cudaGetErrorString(e));
  }
  *out = k;
  return APPY_OK;
}

int nvrtc_build(const char* src, const char* kernel_name, const std::vector<std::string>& opts,
                std::vector<char>& image) {
  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, src, (std::string(kernel_name) + ".cu").c_str(), 0,
                                     nullptr, nullptr);
  if (r != NVRTC_SUCCESS)
    return fail(APPY_ERR_NVRTC, "nvrtcCreateProgram: %s", nvrtcGetErrorString(r));
  std::vector<const char*> copts;
  for (auto& o : opts) copts.push_back(o.c_str());
  r = nvrtcCompileProgram(prog, (int)copts.size(), copts.data());
  size_t logsz = 0;
  nvrtcGetProgramLogSize(prog, &logsz);
  if (logsz > 1) {
    g_log.resize(logsz);
    nvrtcGetProgramLog(prog, &g_log[0]);
  }
  if (r != NVRTC_SUCCESS) {
    nvrtcDestroyProgram(&prog);
    return fail(APPY_ERR_NVRTC, "NVRTC compilation of `%s` failed: %s\n%s", kernel_name,
                nvrtcGetErrorString(r), g_log.c_str());
  }
  size_t sz = 0;
  r = nvrtcGetCUBINSize(prog, &sz);
  if (r != NVRTC_SUCCESS || sz == 0) {
    nvrtcDestroyProgram(&prog);
    return fail(APPY_ERR_NVRTC, "nvrtcGetCUBINSize: %s", nvrtcGetErrorString(r));
  }
  image.resize(sz);
  nvrtcGetCUBIN(prog, image.data());
  nvrtcDestroyProgram(&prog);
  return APPY_OK;
}

std::vector<std::string> nvrtc_options(const char* options) {
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device"};
  if (options) {
    std::stringstream ss(options);
    std::string line;
    while (std::getline(ss, line, '\n'))
      if (!line.empty()) opts.push_back(line);
  }
  return opts;
}

}  // namespace

extern "C" {

const char* appy_last_error(void) { return g_err.c_str(); }
const char* appy_compile_log(void) { return g_log.c_str(); }
int64_t appy_launch_count(void) { return g_launches.load(); }
void appy_reset_launch_count(void) { g_launches.store(0); }
}

// used by the prebuilt kernels' host wrappers
void appy_note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
int appy_fail_cuda(cudaError_t e, const char* what) {
  return fail(APPY_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
}
int appy_fail_arg(const char* what) { return fail(APPY_ERR_ARG, "%s", what); }

extern "C" {

int appy_device_count(int* count) {
  if (!count) return fail(APPY_ERR_ARG, "count is NULL");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    *count = 0;
    return fail(APPY_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
  }
  return APPY_OK;
}

int appy_device_info(int device, int* sm_count, int* l2_bytes, int* cc, size_t* total_mem) {
  cudaDeviceProp p;
  CK(cudaGetDeviceProperties(&p, device));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (l2_bytes) *l2_bytes = p.l2CacheSize;
  if (cc) *cc = p.major * 10 + p.minor;
  if (total_mem) *total_mem = p.totalGlobalMem;
  return APPY_OK;
}

int appy_init(int device) {
  if (device < 0 || device >= 16) return fail(APPY_ERR_ARG, "device index %d out of range", device);
  CK(cudaSetDevice(device));
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (d.ready) return APPY_OK;
  for (int i = 0; i < 2; ++i) CK(cudaStreamCreateWithFlags(&d.streams[i], cudaStreamNonBlocking));
  d.ready = true;
  return APPY_OK;
}

int appy_shutdown(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (int dev = 0; dev < 16; ++dev) {
    DeviceState& d = g_dev[dev];
    if (!d.ready) continue;
    if (cudaSetDevice(dev) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    for (auto& kv : d.pinned) cudaHostUnregister(const_cast<void*>(kv.first));
    d.pinned.clear();
    for (auto& kv : d.mirrors) d.free_blocks.emplace(d.live_blocks[kv.second.dptr], kv.second.dptr);
    d.mirrors.clear();
    d.mirror_bytes = 0;
    for (auto& kv : d.workspaces) cudaFree(kv.second);
    d.workspaces.clear();
    for (int i = 0; i < 2; ++i) {
      if (g_stage[dev].buf[i]) { cudaFreeHost(g_stage[dev].buf[i]); g_stage[dev].buf[i] = nullptr; }
      if (g_stage[dev].done[i]) { cudaEventDestroy(g_stage[dev].done[i]); g_stage[dev].done[i] = nullptr; }
    }
    if (g_host_cells[dev]) {
      cudaFreeHost(g_host_cells[dev]);
      g_host_cells[dev] = g_host_cells_dev[dev] = nullptr;
    }
    for (auto& kv : d.live_blocks) cudaFree(kv.first);
    d.live_blocks.clear();
    d.free_blocks.clear();
    for (int i = 0; i < 2; ++i)
      if (d.streams[i]) cudaStreamDestroy(d.streams[i]);
    d.streams[0] = d.streams[1] = nullptr;
    d.ready = false;
  }
  return APPY_OK;
}

int appy_get_stream(int which, void** stream) {
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  if (!g_dev[dev].ready) return fail(APPY_ERR_STATE, "appy_init(%d) has not been called", dev);
  if (which < 0 || which > 1 || !stream) return fail(APPY_ERR_ARG, "bad stream selector");
  *stream = g_dev[dev].streams[which];
  return APPY_OK;
}

int appy_sync(void* stream) {
  CK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return APPY_OK;
}

// ---------------------------------------------------------------- memory

int appy_malloc(void** dptr, size_t bytes) {
  if (!dptr) return fail(APPY_ERR_ARG, "dptr is NULL");
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  const size_t want = round_block(bytes ? bytes : 1);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  auto it = d.free_blocks.lower_bound(want);
  if (it != d.free_blocks.end() && it->first <= 2 * want) {
    *dptr = it->second;
    d.free_set.erase(it->second);
    d.free_blocks.erase(it);
    return APPY_OK;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, want);
  if (e == cudaErrorMemoryAllocation) {  // give cached blocks back and retry once
    cudaGetLastError();
    for (auto& kv : d.free_blocks) {
      cudaFree(kv.second);
      d.live_blocks.erase(kv.second);
    }
    d.free_blocks.clear();
    d.free_set.clear();
    e = cudaMalloc(&p, want);
  }
  if (e != cudaSuccess)
    return fail(APPY_ERR_CUDA, "cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
  d.live_blocks[p] = want;
  *dptr = p;
  return APPY_OK;
}

int appy_free(void* dptr) {
  if (!dptr) return APPY_OK;
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  auto it = d.live_blocks.find(dptr);
  if (it == d.live_blocks.end()) return fail(APPY_ERR_ARG, "appy_free: unknown block %p", dptr);
  if (d.free_set.count(dptr)) return fail(APPY_ERR_ARG, "appy_free: block %p is already free", dptr);
  for (auto& m : d.mirrors)
    if (m.second.dptr == dptr)
      return fail(APPY_ERR_ARG, "appy_free: block %p is the mirror of a host range; use appy_evict", dptr);
  d.free_blocks.emplace(it->second, dptr);
  d.free_set.insert(dptr);
  return APPY_OK;
}

int appy_trim(void) {
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  CK(cudaDeviceSynchronize());
  for (auto& kv : d.free_blocks) {
    cudaFree(kv.second);
    d.live_blocks.erase(kv.second);
  }
  d.free_blocks.clear();
  d.free_set.clear();
  return APPY_OK;
}

int appy_memset(void* dptr, int value, size_t bytes, void* stream) {
  CK(cudaMemsetAsync(dptr, value, bytes, static_cast<cudaStream_t>(stream)));
  return APPY_OK;
}

int appy_register_host(void* hptr, size_t bytes) {
  if (!hptr || !bytes) return fail(APPY_ERR_ARG, "appy_register_host: empty range");
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  auto it = d.pinned.find(hptr);
  if (it != d.pinned.end()) {
    if (it->second >= bytes) return APPY_OK;
    cudaHostUnregister(hptr);
    d.pinned.erase(it);
  }
  cudaError_t e = cudaHostRegister(hptr, bytes, cudaHostRegisterPortable);
  if (e == cudaErrorHostMemoryAlreadyRegistered) {  // pinned by someone else (e.g. torch): fine
    cudaGetLastError();
    return APPY_OK;
  }
  if (e != cudaSuccess)
    return fail(APPY_ERR_CUDA, "cudaHostRegister(%p, %zu) failed: %s", hptr, bytes,
                cudaGetErrorString(e));
  d.pinned[hptr] = bytes;
  return APPY_OK;
}

int appy_unregister_host(void* hptr) {
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  auto it = d.pinned.find(hptr);
  if (it == d.pinned.end()) return APPY_OK;
  cudaHostUnregister(hptr);
  d.pinned.erase(it);
  return APPY_OK;
}

// Mirrors are a cache: beyond kMirrorMaxCount entries or kMirrorMaxBytes the least recently used ones
// are dropped (their blocks return to the cached allocator).  A mirror is only referenced between the
// appy_mirror call and the stream synchronisation that ends the same host-array launch, so dropping an
// older one is safe.
const size_t kMirrorMaxCount = 1024;
const size_t kMirrorMaxBytes = (size_t)16 << 30;

static void drop_mirror_locked(DeviceState& d, std::unordered_map<const void*, DeviceState::Mirror>::iterator it) {
  d.mirror_bytes -= it->second.bytes;
  d.free_blocks.emplace(d.live_blocks[it->second.dptr], it->second.dptr);
  d.free_set.insert(it->second.dptr);
  d.mirrors.erase(it);
}

int appy_mirror(const void* hptr, size_t bytes, void** dptr, int* created) {
  if (!hptr || !dptr) return fail(APPY_ERR_ARG, "appy_mirror: NULL argument");
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[dev];
    auto it = d.mirrors.find(hptr);
    if (it != d.mirrors.end()) {
      if (it->second.bytes >= bytes && it->second.bytes <= 2 * round_block(bytes)) {
        it->second.last_use = ++d.tick;
        *dptr = it->second.dptr;
        if (created) *created = 0;
        return APPY_OK;
      }
      drop_mirror_locked(d, it);
    }
    const size_t want = round_block(bytes ? bytes : 1);
    while (!d.mirrors.empty() &&
           (d.mirrors.size() >= kMirrorMaxCount || d.mirror_bytes + want > kMirrorMaxBytes)) {
      auto oldest = d.mirrors.begin();
      for (auto jt = d.mirrors.begin(); jt != d.mirrors.end(); ++jt)
        if (jt->second.last_use < oldest->second.last_use) oldest = jt;
      // the 64 most recent acquisitions may belong to the launch being prepared: never drop those
      if (oldest->second.last_use + 64 > d.tick) break;
      drop_mirror_locked(d, oldest);
    }
  }
  void* p = nullptr;
  if (int rc = appy_malloc(&p, bytes)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  const size_t got = round_block(bytes ? bytes : 1);
  d.mirrors[hptr] = DeviceState::Mirror{p, got, ++d.tick};
  d.mirror_bytes += got;
  *dptr = p;
  if (created) *created = 1;
  return APPY_OK;
}

int appy_evict(const void* hptr) {
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  auto it = d.mirrors.find(hptr);
  if (it == d.mirrors.end()) return APPY_OK;
  drop_mirror_locked(d, it);
  return APPY_OK;
}

int appy_h2d_async(void* dptr, const void* hptr, size_t bytes, void* stream) {
  if (!bytes) return APPY_OK;
  CK(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return APPY_OK;
}
int appy_d2h_async(void* hptr, const void* dptr, size_t bytes, void* stream) {
  if (!bytes) return APPY_OK;
  CK(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return APPY_OK;
}
// Pageable host memory: stage through two pinned buffers so that the CPU copy of chunk k+1 overlaps
// the DMA of chunk k (a plain cudaMemcpyAsync from pageable memory is staged by the driver and
// blocks the calling thread for the whole transfer).
int appy_h2d_staged(void* dptr, const void* hptr, size_t bytes, void* stream) {
  if (!bytes) return APPY_OK;
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::lock_guard<std::mutex> lk(g_mu);     // the two buffers are shared by all callers of a device
  Staging* st = nullptr;
  if (int rc = staging_for(dev, &st)) return rc;
  size_t off = 0;
  int which = 0;
  while (off < bytes) {
    const size_t n = std::min(kStageBytes, bytes - off);
    CK(cudaEventSynchronize(st->done[which]));          // the previous DMA out of this buffer is over
    memcpy(st->buf[which], static_cast<const char*>(hptr) + off, n);
    CK(cudaMemcpyAsync(static_cast<char*>(dptr) + off, st->buf[which], n, cudaMemcpyHostToDevice, s));
    CK(cudaEventRecord(st->done[which], s));
    off += n;
    which ^= 1;
  }
  return APPY_OK;
}

// Cells for shared scalars: one page of mapped, pinned host memory per device.  A reduction kernel that is
// given the device address of a cell reads the initial value and writes the result over PCIe itself, so
// the host needs neither an upload nor a download, only the wait for the stream (measured on a 4096-element
// sum: 17.6 us per call against 31.5 us with a mirror, an 8-byte upload and an 8-byte download).
int appy_host_cells(void** hptr, void** dptr, size_t* bytes) {
  if (!hptr || !dptr) return fail(APPY_ERR_ARG, "appy_host_cells: NULL argument");
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_host_cells[dev]) {
    void* h = nullptr;
    CK(cudaHostAlloc(&h, kHostCellBytes, cudaHostAllocMapped | cudaHostAllocPortable));
    void* d = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
    if (e != cudaSuccess) {
      cudaFreeHost(h);
      return appy_fail_cuda(e, "cudaHostGetDevicePointer(host cells)");
    }
    memset(h, 0, kHostCellBytes);
    g_host_cells[dev] = h;
    g_host_cells_dev[dev] = d;
  }
  *hptr = g_host_cells[dev];
  *dptr = g_host_cells_dev[dev];
  if (bytes) *bytes = kHostCellBytes;
  return APPY_OK;
}

int appy_d2d_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (!bytes) return APPY_OK;
  CK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return APPY_OK;
}

int appy_workspace(void* stream, void** dptr, size_t* bytes) {
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto it = d.workspaces.find(s);
  if (it == d.workspaces.end()) {
    void* p = nullptr;
    CK(cudaMalloc(&p, kWorkspaceBytes));
    CK(cudaMemset(p, 0, kWorkspaceBytes));
    it = d.workspaces.emplace(s, p).first;
  }
  if (dptr) *dptr = it->second;
  if (bytes) *bytes = kWorkspaceBytes;
  return APPY_OK;
}

int appy_scratch(void* stream, size_t bytes, void** dptr) {
  if (!dptr) return fail(APPY_ERR_ARG, "appy_scratch: NULL argument");
  int dev;
  if (int rc = cur_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto it = d.scratch.find(s);
  if (it == d.scratch.end() || it->second.bytes < bytes) {
    const size_t want = std::max<size_t>((bytes + (1u << 20) - 1) >> 20 << 20, 1u << 20);
    void* p = nullptr;
    CK(cudaMalloc(&p, want));
    if (it != d.scratch.end()) {
      // kernels queued on this stream may still use the old buffer: let them finish first
      CK(cudaStreamSynchronize(s));
      CK(cudaFree(it->second.dptr));
      it->second = DeviceState::Scratch{p, want};
    } else {
      it = d.scratch.emplace(s, DeviceState::Scratch{p, want}).first;
    }
  }
  *dptr = it->second.dptr;
  return APPY_OK;
}

// ---------------------------------------------------------------- compile / launch

// Key of a compiled kernel: source, options, contents of every include directory, NVRTC version and
// target architecture.  Caller holds g_mu.
static std::string compile_key(const char* src, const std::vector<std::string>& opts) {
  int nv_major = 0, nv_minor = 0;
  nvrtcVersion(&nv_major, &nv_minor);
  Sha256 sh;
  sh.update(src);
  sh.update("\x1f");
  for (auto& o : opts) {
    sh.update(o);
    sh.update("\x1f");
    if (o.compare(0, 2, "-I") == 0) sh.update(dir_digest(o.substr(2)));
  }
  sh.update("nvrtc " + std::to_string(nv_major) + "." + std::to_string(nv_minor) + " sm_100a");
  return sh.hex();
}

// The cubin of `src`, from the cache directory when it holds a valid entry for the key, otherwise
// compiled (and then written there, best effort).  Caller holds g_mu.
static int image_through_cache(const char* src, const char* kernel_name, const std::vector<std::string>& opts,
                               const std::string& hex, const char* cache_dir, std::vector<char>& image,
                               bool* from_cache, bool force_compile) {
  std::string path;
  *from_cache = false;
  if (cache_dir && *cache_dir) {
    path = std::string(cache_dir) + "/" + hex + ".cubin";
    if (!force_compile && read_cache_file(path, hex, image)) {
      *from_cache = true;
      return APPY_OK;
    }
    image.clear();
  }
  if (int rc = nvrtc_build(src, kernel_name, opts, image)) return rc;
  if (!path.empty()) write_cache_file(path, hex, image, &image);
  return APPY_OK;
}

int appy_compile(const char* src, const char* kernel_name, const char* options,
                 const char* cache_dir, void** handle) {
  if (!src || !kernel_name || !handle) return fail(APPY_ERR_ARG, "appy_compile: NULL argument");
  g_log.clear();
  std::vector<std::string> opts = nvrtc_options(options);
  std::lock_guard<std::mutex> lk(g_mu);
  const std::string hex = compile_key(src, opts);
  const std::string key = hex + ":" + kernel_name;
  auto it = g_kernels.find(key);
  if (it != g_kernels.end()) {
    *handle = it->second;
    return APPY_OK;
  }
  std::vector<char> image;
  bool from_cache = false;
  if (int rc = image_through_cache(src, kernel_name, opts, hex, cache_dir, image, &from_cache, false)) return rc;
  Kernel* k = nullptr;
  if (load_cubin(image, kernel_name, &k) != APPY_OK) {
    if (!from_cache) return APPY_ERR_CUDA;
    // an entry the driver refuses (or that lacks this kernel): compile afresh and replace it
    if (int rc = image_through_cache(src, kernel_name, opts, hex, cache_dir, image, &from_cache, true)) return rc;
    if (int rc = load_cubin(image, kernel_name, &k)) return rc;
  }
  g_kernels[key] = k;
  *handle = k;
  return APPY_OK;
}

int appy_compile_image(const char* src, const char* kernel_name, const char* options, const char* cache_dir,
                       size_t* cubin_bytes, int* from_cache) {
  if (!src || !kernel_name) return fail(APPY_ERR_ARG, "appy_compile_image: NULL argument");
  g_log.clear();
  std::vector<std::string> opts = nvrtc_options(options);
  std::lock_guard<std::mutex> lk(g_mu);
  const std::string hex = compile_key(src, opts);
  std::vector<char> image;
  bool cached = false;
  if (int rc = image_through_cache(src, kernel_name, opts, hex, cache_dir, image, &cached, false)) return rc;
  if (cubin_bytes) *cubin_bytes = image.size();
  if (from_cache) *from_cache = cached ? 1 : 0;
  return APPY_OK;
}

int appy_compile_check(const char* src, const char* kernel_name, const char* options,
                       size_t* cubin_bytes) {
  if (!src || !kernel_name) return fail(APPY_ERR_ARG, "appy_compile_check: NULL argument");
  g_log.clear();
  std::vector<char> image;
  if (int rc = nvrtc_build(src, kernel_name, nvrtc_options(options), image)) return rc;
  if (cubin_bytes) *cubin_bytes = image.size();
  return APPY_OK;
}

int appy_kernel_info(void* handle, int* regs, int* static_smem, int* max_threads) {
  if (!handle) return fail(APPY_ERR_ARG, "NULL kernel handle");
  Kernel* k = static_cast<Kernel*>(handle);
  cudaFuncAttributes a;
  CK(cudaFuncGetAttributes(&a, (const void*)k->kern));
  if (regs) *regs = a.numRegs;
  if (static_smem) *static_smem = (int)a.sharedSizeBytes;
  if (max_threads) *max_threads = a.maxThreadsPerBlock;
  return APPY_OK;
}

int appy_occupancy(void* handle, int block, size_t dyn_smem, int* blocks_per_sm) {
  if (!handle || !blocks_per_sm) return fail(APPY_ERR_ARG, "NULL argument");
  Kernel* k = static_cast<Kernel*>(handle);
  CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, (const void*)k->kern, block,
                                                   dyn_smem));
  return APPY_OK;
}

int appy_launch(void* handle, unsigned grid, unsigned block, size_t dyn_smem, void** args,
                void* stream) {
  if (!handle) return fail(APPY_ERR_ARG, "NULL kernel handle");
  if (grid == 0) return APPY_OK;
  Kernel* k = static_cast<Kernel*>(handle);
  if (dyn_smem > k->dyn_smem_allowed.load(std::memory_order_relaxed)) {
    CK(cudaFuncSetAttribute((const void*)k->kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                            (int)dyn_smem));
    k->dyn_smem_allowed.store(dyn_smem, std::memory_order_relaxed);
  }
  CK(cudaLaunchKernel((const void*)k->kern, dim3(grid), dim3(block), args, dyn_smem,
                      static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return APPY_OK;
}

int appy_time_launches(void* handle, unsigned grid, unsigned block, size_t dyn_smem, void** args,
                       void* stream, int warmup, int iters, float* total_ms) {
  if (!total_ms || iters <= 0) return fail(APPY_ERR_ARG, "bad timing arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < warmup; ++i)
    if (int rc = appy_launch(handle, grid, block, dyn_smem, args, stream)) return rc;
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0, s));
  for (int i = 0; i < iters; ++i)
    if (int rc = appy_launch(handle, grid, block, dyn_smem, args, stream)) {
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      return rc;
    }
  CK(cudaEventRecord(e1, s));
  CK(cudaEventSynchronize(e1));
  CK(cudaEventElapsedTime(total_ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return APPY_OK;
}

// ---------------------------------------------------------------- partitioning

int appy_partition_range(int64_t lo, int64_t hi, int parts, int64_t align, int64_t* bounds) {
  if (parts <= 0 || !bounds || align <= 0) return fail(APPY_ERR_ARG, "bad partition arguments");
  if (hi < lo) hi = lo;
  const int64_t n = hi - lo;
  bounds[0] = lo;
  for (int p = 1; p < parts; ++p) {
    // ideal cut, then round to the nearest multiple of `align` in absolute index space
    const int64_t ideal = lo + (int64_t)((__int128)n * p / parts);
    int64_t cut = (ideal + align / 2) / align * align;
    cut = std::max(cut, bounds[p - 1]);
    cut = std::min(cut, hi);
    bounds[p] = cut;
  }
  bounds[parts] = hi;
  return APPY_OK;
}

int appy_partition_rows_weighted(const void* indptr, int idx_bytes, int64_t nrows, int parts, int64_t row_cost,
                                 int64_t* bounds) {
  if (!indptr || parts <= 0 || !bounds || nrows < 0 || row_cost < 0 || (idx_bytes != 4 && idx_bytes != 8))
    return fail(APPY_ERR_ARG, "bad partition arguments");
  auto at = [&](int64_t i) -> int64_t {
    return idx_bytes == 4 ? (int64_t) static_cast<const int32_t*>(indptr)[i]
                          : static_cast<const int64_t*>(indptr)[i];
  };
  // cost of rows [0, i): their non-zeros plus row_cost per row; non-decreasing in i
  const int64_t first = at(0);
  auto cost = [&](int64_t i) -> int64_t { return at(i) - first + row_cost * i; };
  const int64_t total = cost(nrows);
  bounds[0] = 0;
  for (int p = 1; p < parts; ++p) {
    const int64_t target = (int64_t)((__int128)total * p / parts);
    // first row r with cost(r) >= target
    int64_t a = bounds[p - 1], b = nrows;
    while (a < b) {
      const int64_t m = a + (b - a) / 2;
      if (cost(m) < target) a = m + 1; else b = m;
    }
    // choose the nearer of the two neighbouring row boundaries
    if (a > bounds[p - 1] && a <= nrows && (cost(a) - target) > (target - cost(a - 1))) --a;
    bounds[p] = std::min(std::max(a, bounds[p - 1]), nrows);
  }
  bounds[parts] = nrows;
  return APPY_OK;
}

int appy_partition_rows(const void* indptr, int idx_bytes, int64_t nrows, int parts,
                        int64_t* bounds) {
  return appy_partition_rows_weighted(indptr, idx_bytes, nrows, parts, 0, bounds);
}

// ---------------------------------------------------------------- peer mailboxes (multi-GPU scalar combine)

struct P2PContext {
  int world = 0, rank = 0;
  void* local = nullptr;        // this rank's mailbox (cudaMalloc)
  void* peers[16] = {nullptr};  // mapped mailboxes of all ranks (peers[rank] == local)
  void* d_desc = nullptr;       // device copy of the descriptor the kernels read
  unsigned* d_err = nullptr;
  bool loopback = false;
  bool opened = false;
};

typedef appy_mailbox MailboxDesc;   // the descriptor the kernels read (templates/t_flat.cuh)

// the device-side descriptor of an opened context: every rank's mailbox, own mailbox, limits
static int p2p_finish_open(P2PContext* c, unsigned spin_limit, void** device_descriptor) {
  MailboxDesc d;
  memset(&d, 0, sizeof d);
  d.world = c->world;
  d.rank = c->rank;
  d.spin_limit = spin_limit ? spin_limit : (1u << 23);
  d.err = c->d_err;
  for (int r = 0; r < 16; ++r) d.peer[r] = static_cast<unsigned long long*>(c->peers[r < c->world ? r : c->rank]);
  d.own = static_cast<unsigned long long*>(c->peers[c->rank]);
  CK(cudaMemcpy(c->d_desc, &d, sizeof d, cudaMemcpyHostToDevice));
  c->opened = true;
  *device_descriptor = c->d_desc;
  return APPY_OK;
}

int appy_p2p_create(int world, int rank, void** ctx, void* ipc_handle_out) {
  if (!ctx || !ipc_handle_out || world < 1 || world > 16 || rank < 0 || rank >= world)
    return fail(APPY_ERR_ARG, "appy_p2p_create: bad arguments");
  P2PContext* c = new P2PContext;
  c->world = world;
  c->rank = rank;
  // [0, 4096): the two slots of the immediate exchange; from 4096: the ring of the split-phase exchange
  const size_t bytes = 4096 + (size_t)APPY_MB_RING * world * 8 * sizeof(unsigned long long);
  cudaError_t e = cudaMalloc(&c->local, bytes);
  if (e == cudaSuccess) e = cudaMemset(c->local, 0, bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&c->d_err), 256);
  if (e == cudaSuccess) e = cudaMemset(c->d_err, 0, 256);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_desc, sizeof(MailboxDesc));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->local);
  if (e != cudaSuccess) {
    cudaFree(c->local); cudaFree(c->d_err); cudaFree(c->d_desc);
    delete c;
    return fail(APPY_ERR_CUDA, "appy_p2p_create failed: %s", cudaGetErrorString(e));
  }
  memcpy(ipc_handle_out, &h, sizeof h);
  c->peers[rank] = c->local;
  *ctx = c;
  return APPY_OK;
}

int appy_p2p_open(void* ctx, const void* all_handles, unsigned spin_limit, void** device_descriptor) {
  if (!ctx || !device_descriptor) return fail(APPY_ERR_ARG, "appy_p2p_open: NULL argument");
  P2PContext* c = static_cast<P2PContext*>(ctx);
  const cudaIpcMemHandle_t* hs = static_cast<const cudaIpcMemHandle_t*>(all_handles);
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (!hs) {                     // loop-back: no peer process; the other ranks never post
      c->peers[r] = c->local;
      c->loopback = true;
      continue;
    }
    cudaError_t e = cudaIpcOpenMemHandle(&c->peers[r], hs[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return fail(APPY_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d) failed: %s", r, cudaGetErrorString(e));
  }
  return p2p_finish_open(c, spin_limit, device_descriptor);
}

int appy_p2p_open_local(void* ctx, void* const* contexts, unsigned spin_limit, void** device_descriptor) {
  if (!ctx || !contexts || !device_descriptor) return fail(APPY_ERR_ARG, "appy_p2p_open_local: NULL argument");
  P2PContext* c = static_cast<P2PContext*>(ctx);
  for (int r = 0; r < c->world; ++r) {
    const P2PContext* o = static_cast<const P2PContext*>(contexts[r]);
    if (!o || o->world != c->world || o->rank != r)
      return fail(APPY_ERR_ARG, "appy_p2p_open_local: contexts[%d] is not rank %d of a world of %d", r, r, c->world);
    c->peers[r] = o->local;
  }
  if (contexts[c->rank] != ctx) return fail(APPY_ERR_ARG, "appy_p2p_open_local: contexts[rank] is another context");
  c->loopback = true;              // nothing was opened through IPC, so nothing is closed
  return p2p_finish_open(c, spin_limit, device_descriptor);
}

}  // extern "C"

namespace {
// One warp: exchange up to four device scalars with all ranks and fold them in rank order, in place.
template <class Op, class T>
__global__ void __launch_bounds__(32) k_p2p_combine(const appy_mailbox* mb, u64 seq, T* values, int count) {
  u64 x[4];
#pragma unroll
  for (int v = 0; v < 4; ++v) x[v] = v < count ? appy_to_bits<T>(values[v]) : 0ull;
  const bool ok = appy_p2p_exchange<4>(mb, seq, x);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    T t = appy_p2p_fold<Op, T>(mb, x[v]);
    if (!ok) t = appy_p2p_poison<T>(t);
    if (threadIdx.x == 0 && v < count) values[v] = t;
  }
}
template <class T>
cudaError_t launch_p2p_combine(int op, const appy_mailbox* mb, u64 seq, void* values, int count, cudaStream_t s) {
  T* v = static_cast<T*>(values);
  switch (op) {
    case APPY_OP_ADD: k_p2p_combine<appy_add, T><<<1, 32, 0, s>>>(mb, seq, v, count); break;
    case APPY_OP_MUL: k_p2p_combine<appy_mul, T><<<1, 32, 0, s>>>(mb, seq, v, count); break;
    case APPY_OP_MAX: k_p2p_combine<appy_max, T><<<1, 32, 0, s>>>(mb, seq, v, count); break;
    default:          k_p2p_combine<appy_min, T><<<1, 32, 0, s>>>(mb, seq, v, count); break;
  }
  return cudaGetLastError();
}
}  // namespace

extern "C" {

int appy_p2p_combine(void* ctx, uint64_t seq, int op, int dtype, void* dvalues, int count, void* stream) {
  if (!ctx || !dvalues) return fail(APPY_ERR_ARG, "appy_p2p_combine: NULL argument");
  if (count < 1 || count > 4) return fail(APPY_ERR_ARG, "appy_p2p_combine: count must be 1..4");
  if (op < APPY_OP_ADD || op > APPY_OP_MIN) return fail(APPY_ERR_ARG, "appy_p2p_combine: unknown operator %d", op);
  P2PContext* c = static_cast<P2PContext*>(ctx);
  if (!c->opened) return fail(APPY_ERR_ARG, "appy_p2p_combine: appy_p2p_open has not been called");
  const appy_mailbox* mb = static_cast<const appy_mailbox*>(c->d_desc);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  switch (dtype) {
    case APPY_F32: e = launch_p2p_combine<float>(op, mb, seq, dvalues, count, s); break;
    case APPY_F64: e = launch_p2p_combine<double>(op, mb, seq, dvalues, count, s); break;
    case APPY_I32: e = launch_p2p_combine<int>(op, mb, seq, dvalues, count, s); break;
    case APPY_I64: e = launch_p2p_combine<i64>(op, mb, seq, dvalues, count, s); break;
    default: return fail(APPY_ERR_ARG, "appy_p2p_combine: unknown dtype %d", dtype);
  }
  if (e != cudaSuccess) return fail(APPY_ERR_CUDA, "appy_p2p_combine launch failed: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return APPY_OK;
}

}  // extern "C"

namespace {
// One warp: what the start of a split-phase kernel does for the launches before it (fold and post one,
// collect the other), for launches that no later kernel serves.
__global__ void __launch_bounds__(32) k_p2p_flush(const appy_mailbox* mb, appy_pending2 pend) {
  appy_split_service(mb, pend);
}
}  // namespace

extern "C" {

int appy_p2p_flush(void* ctx, const void* pending, void* stream) {
  if (!ctx || !pending) return fail(APPY_ERR_ARG, "appy_p2p_flush: NULL argument");
  P2PContext* c = static_cast<P2PContext*>(ctx);
  if (!c->opened) return fail(APPY_ERR_ARG, "appy_p2p_flush: appy_p2p_open has not been called");
  appy_pending2 pend;
  memcpy(&pend, pending, sizeof pend);
  const appy_pending* both[2] = {&pend.fold, &pend.coll};
  for (const appy_pending* e : both)
    if (e->seq != 0 && (e->nv < 1 || e->nv > 4 || e->slot < 0 || e->slot >= APPY_MB_RING))
      return fail(APPY_ERR_ARG, "appy_p2p_flush: a pending launch must carry 1..4 variables and a ring slot");
  if (pend.fold.seq != 0 && (pend.fold.grid < 1 || pend.fold.grid > 4096 || !pend.fold.partials))
    return fail(APPY_ERR_ARG, "appy_p2p_flush: the launch to fold needs its partials and 1..4096 CTAs");
  k_p2p_flush<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const appy_mailbox*>(c->d_desc), pend);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(APPY_ERR_CUDA, "appy_p2p_flush launch failed: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return APPY_OK;
}

int appy_p2p_status(void* ctx, int* timed_out) {
  if (!ctx || !timed_out) return fail(APPY_ERR_ARG, "appy_p2p_status: NULL argument");
  P2PContext* c = static_cast<P2PContext*>(ctx);
  unsigned v = 0;
  CK(cudaMemcpy(&v, c->d_err, sizeof v, cudaMemcpyDeviceToHost));
  *timed_out = (int)v;
  if (v) CK(cudaMemset(c->d_err, 0, sizeof v));   // reading clears the flag
  return APPY_OK;
}

int appy_p2p_destroy(void* ctx) {
  if (!ctx) return APPY_OK;
  P2PContext* c = static_cast<P2PContext*>(ctx);
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank && c->peers[r] && !c->loopback) cudaIpcCloseMemHandle(c->peers[r]);
  cudaFree(c->local);
  cudaFree(c->d_err);
  cudaFree(c->d_desc);
  delete c;
  return APPY_OK;
}

}  // extern "C"
