// Library-level pieces of the C ABI: error text, launch counters, tuning knobs,
// allocators for host-resident tables.
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <sys/mman.h>
#include <utility>

#include "tbe_common.cuh"

namespace tbe {
namespace {
thread_local char g_error[512] = "";
std::atomic<int64_t> g_kernel_launches{0};
std::atomic<int64_t> g_library_launches{0};
std::atomic<int> g_tuning[kTuneCount];
const char* const kTuningNames[kTuneCount] = {"fwd_unroll", "fwd_threads", "bwd_threads", "bwd_unroll",
                                              "long_segment", "fwd_blocks_per_sm", "bwd_blocks_per_sm", "bwd_vpl",
                                              "bwd_sort", "sort_bucket", "split_runs", "bwd_stride"};
}  // namespace

namespace {
struct TimedLaunch {
  const char* name;
  cudaEvent_t start, stop;
};
std::atomic<int> g_timing_on{0};
std::mutex g_timing_mutex;
std::vector<TimedLaunch> g_timed;
}  // namespace

KernelTimer::KernelTimer(const char* name, cudaStream_t stream) : name_(name), stream_(stream) {
  if (!g_timing_on.load(std::memory_order_relaxed)) return;
  if (cudaEventCreate(&start_) != cudaSuccess) {
    start_ = nullptr;
    return;
  }
  cudaEventRecord(start_, stream_);
}

KernelTimer::~KernelTimer() {
  if (!start_) return;
  cudaEvent_t stop = nullptr;
  if (cudaEventCreate(&stop) != cudaSuccess) {
    cudaEventDestroy(start_);
    return;
  }
  cudaEventRecord(stop, stream_);
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  g_timed.push_back({name_, start_, stop});
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_kernel_launch(int n) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }
void count_library_launch(int n) { g_library_launches.fetch_add(n, std::memory_order_relaxed); }
int tuning(int which) { return g_tuning[which].load(std::memory_order_relaxed); }

int device_sm_count() {
  // cached per device ordinal; 64 is far above any box this runs on
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cache[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

int64_t device_l2_bytes() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 126ll << 20;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) != cudaSuccess || v <= 0) v = 126 << 20;
    cache[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}
}  // namespace tbe

extern "C" int tbe_abi_version(void) { return 5; }

extern "C" const char* tbe_last_error_string(void) { return tbe::g_error; }

extern "C" int64_t tbe_kernel_launch_count(void) { return tbe::g_kernel_launches.load(); }
extern "C" int64_t tbe_library_launch_count(void) { return tbe::g_library_launches.load(); }

extern "C" int tbe_set_tuning(const char* name, int value) {
  if (!name) return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_set_tuning: null name");
  for (int i = 0; i < tbe::kTuneCount; ++i) {
    if (std::strcmp(name, tbe::kTuningNames[i]) == 0) {
      tbe::g_tuning[i].store(value);
      return TBE_OK;
    }
  }
  return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_set_tuning: unknown knob '%s'", name);
}

extern "C" int tbe_kernel_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(tbe::g_timing_mutex);
  for (auto& t : tbe::g_timed) {
    cudaEventDestroy(t.start);
    cudaEventDestroy(t.stop);
  }
  tbe::g_timed.clear();
  tbe::g_timing_on.store(on ? 1 : 0);
  return TBE_OK;
}

extern "C" int64_t tbe_kernel_timing_read(char* buffer, int64_t buffer_bytes) {
  if (!buffer || buffer_bytes <= 0) return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_kernel_timing_read: no buffer");
  std::map<std::string, std::pair<int64_t, double>> acc;
  {
    std::lock_guard<std::mutex> lock(tbe::g_timing_mutex);
    for (auto& t : tbe::g_timed) {
      float ms = 0.f;
      cudaError_t e = cudaEventSynchronize(t.stop);
      if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t.start, t.stop);
      cudaEventDestroy(t.start);
      cudaEventDestroy(t.stop);
      if (e != cudaSuccess) {
        tbe::g_timed.clear();
        return tbe::fail(TBE_ERR_CUDA, "tbe_kernel_timing_read: %s", cudaGetErrorString(e));
      }
      auto& slot = acc[t.name];
      slot.first += 1;
      slot.second += ms;
    }
    tbe::g_timed.clear();
  }
  std::string out;
  char line[256];
  for (auto& kv : acc) {
    snprintf(line, sizeof(line), "%s %lld %.6f\n", kv.first.c_str(), (long long)kv.second.first, kv.second.second);
    out += line;
  }
  if (static_cast<int64_t>(out.size()) + 1 > buffer_bytes)
    return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_kernel_timing_read: buffer too small");
  std::memcpy(buffer, out.c_str(), out.size() + 1);
  return static_cast<int64_t>(out.size());
}

// ------------------------------------------------------------------ allocators
extern "C" int tbe_alloc_managed(void** ptr, int64_t bytes) {
  TBE_REQUIRE(ptr && bytes > 0, "tbe_alloc_managed: bad arguments");
  int dev = 0;
  TBE_CUDA_TRY(cudaGetDevice(&dev));
  void* p = nullptr;
  TBE_CUDA_TRY(cudaMallocManaged(&p, static_cast<size_t>(bytes)));
  cudaError_t e = cudaMemAdvise(p, static_cast<size_t>(bytes), cudaMemAdviseSetPreferredLocation, cudaCpuDeviceId);
  if (e == cudaSuccess) e = cudaMemAdvise(p, static_cast<size_t>(bytes), cudaMemAdviseSetAccessedBy, dev);
  if (e != cudaSuccess) {
    cudaFree(p);
    return tbe::fail(TBE_ERR_CUDA, "cudaMemAdvise failed: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return TBE_OK;
}

extern "C" int tbe_free_managed(void* ptr) {
  TBE_CUDA_TRY(cudaFree(ptr));
  return TBE_OK;
}

namespace tbe {
namespace {
// Large host-mapped allocations made from anonymous memory: {aligned address -> (mapping base, mapping length)}.
std::mutex g_mapped_mu;
std::map<void*, std::pair<void*, size_t>> g_mapped;
constexpr size_t kHugePage = 2u << 20;
}  // namespace
}  // namespace tbe

extern "C" int tbe_alloc_host_mapped(void** host_ptr, void** device_ptr, int64_t bytes) {
  TBE_REQUIRE(host_ptr && device_ptr && bytes > 0, "tbe_alloc_host_mapped: bad arguments");
  void* h = nullptr;
  // A table of a gigabyte or more comes from anonymous memory that asks for transparent huge pages and
  // is then registered with CUDA.  The GPU does not care, but the host side of the staged cache fill
  // gathers and scatters random rows of it, and with 4 KB pages every such row is a TLB miss whose
  // page walk misses the caches as well.  (Best effort: where that is refused, cudaHostAlloc below.)
  if (bytes >= (1ll << 30)) {
    const size_t len = (static_cast<size_t>(bytes) + 2 * tbe::kHugePage - 1) & ~(tbe::kHugePage - 1);
    void* base = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (base != MAP_FAILED) {
      void* aligned = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(base) + tbe::kHugePage - 1) &
                                              ~static_cast<uintptr_t>(tbe::kHugePage - 1));
      madvise(aligned, len - tbe::kHugePage, MADV_HUGEPAGE);
      if (cudaHostRegister(aligned, static_cast<size_t>(bytes), cudaHostRegisterMapped | cudaHostRegisterPortable) ==
          cudaSuccess) {
        std::lock_guard<std::mutex> lk(tbe::g_mapped_mu);
        tbe::g_mapped[aligned] = std::make_pair(base, len);
        h = aligned;
      } else {
        cudaGetLastError();
        munmap(base, len);
      }
    }
  }
  if (h == nullptr)
    TBE_CUDA_TRY(cudaHostAlloc(&h, static_cast<size_t>(bytes), cudaHostAllocMapped | cudaHostAllocPortable));
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
  if (e != cudaSuccess) {
    tbe_free_host_mapped(h);
    return tbe::fail(TBE_ERR_CUDA, "cudaHostGetDevicePointer failed: %s", cudaGetErrorString(e));
  }
  *host_ptr = h;
  *device_ptr = d;
  return TBE_OK;
}

extern "C" int tbe_free_host_mapped(void* host_ptr) {
  tbe::host_pool_wait();  // no worker may still be writing evicted rows into the table
  std::pair<void*, size_t> mapping(nullptr, 0);
  {
    std::lock_guard<std::mutex> lk(tbe::g_mapped_mu);
    auto it = tbe::g_mapped.find(host_ptr);
    if (it != tbe::g_mapped.end()) {
      mapping = it->second;
      tbe::g_mapped.erase(it);
    }
  }
  if (mapping.first != nullptr) {
    cudaError_t e = cudaHostUnregister(host_ptr);
    munmap(mapping.first, mapping.second);
    if (e != cudaSuccess) return tbe::fail(TBE_ERR_CUDA, "cudaHostUnregister failed: %s", cudaGetErrorString(e));
    return TBE_OK;
  }
  TBE_CUDA_TRY(cudaFreeHost(host_ptr));
  return TBE_OK;
}
