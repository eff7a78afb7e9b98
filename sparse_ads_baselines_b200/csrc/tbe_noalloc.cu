// Exact-SGD backward for callers that cannot hand over a scratch buffer.
//
// Some hosts of this library have no way to allocate device memory at all: a program that binds the
// C ABI through a bare FFI (cgo, JNI, ctypes without a tensor library) owns no device allocator, and
// a serving process whose HBM is budgeted completely at start-up forbids a cudaMalloc in the request
// path (besides failing when the budget is spent, cudaMalloc synchronises the whole device).  For
// them the sort scratch of tbe_backward_sgd lives inside the library, in a fixed array in device
// memory.  CUDA materialises a library's device image lazily, so a GPU starts holding the array at
// the first call made on it (a warm-up call at start-up reserves it) and keeps it until exit.
//
// The array is shared by all calls on a device and keeps whatever the previous call left in it:
// each call re-initialises the few words that must start at zero (the long-run counters) before it
// uses them.  Two calls whose GPU work overlaps in time (different streams, different threads)
// would overwrite each other's sorted lookups: callers must keep calls on one device in one stream
// order.
#include "tbe_common.cuh"

#include <atomic>
#include <mutex>

namespace {

// 20 MiB: enough for TBE_NOALLOC_MAX_LOOKUPS lookups (about 28 bytes each plus CUB's temp storage).
constexpr size_t kScratchBytes = 20u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

// Never launched: it names the array from device code so that the array is kept in the device image.
#pragma nv_diag_suppress 177
__global__ void noalloc_scratch_anchor(unsigned char** out) { *out = g_noalloc_scratch; }

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices];  // device address of the array on each device, 0 = not looked up yet
std::atomic<bool> g_scratch_ready[kMaxDevices];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address valid on the current device comes from cudaGetSymbolAddress, looked up once per device.
int scratch_for_current_device(void** out) {
  int dev = 0;
  TBE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return tbe::fail(TBE_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!g_scratch_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ready[dev].load(std::memory_order_relaxed)) {
      void* p = nullptr;
      TBE_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
      if (p == nullptr) return tbe::fail(TBE_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
      g_scratch_address[dev] = p;
      g_scratch_ready[dev].store(true, std::memory_order_release);
    }
  }
  *out = g_scratch_address[dev];
  return TBE_OK;
}

}  // namespace

extern "C" int64_t tbe_noalloc_scratch_bytes(void) { return static_cast<int64_t>(kScratchBytes); }

extern "C" int tbe_backward_sgd_noalloc(const void* grad_output, int64_t stride_b, int64_t stride_t, void* weights,
                                        const int32_t* table_offsets, const int32_t* indices,
                                        const int32_t* offsets, int64_t T, int64_t B, int64_t D, int64_t N,
                                        int64_t total_rows, int dtype, int pooling, float lr,
                                        int64_t max_rows_per_table, void* stream) {
  if (N > TBE_NOALLOC_MAX_LOOKUPS)
    return tbe::fail(TBE_ERR_WORKSPACE_TOO_SMALL,
                     "tbe_backward_sgd_noalloc: %lld lookups exceed the built-in scratch's limit of %lld; use "
                     "tbe_backward_sgd with a caller-owned workspace",
                     (long long)N, (long long)TBE_NOALLOC_MAX_LOOKUPS);
  const int64_t need = tbe_backward_workspace_bytes(N < 0 ? 0 : N, total_rows);
  if (need < 0) return static_cast<int>(need);
  if (need > static_cast<int64_t>(kScratchBytes))
    return tbe::fail(TBE_ERR_WORKSPACE_TOO_SMALL,
                     "tbe_backward_sgd_noalloc: %lld lookups need %lld bytes of scratch, the built-in array has %lld",
                     (long long)N, (long long)need, (long long)kScratchBytes);
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != TBE_OK) return rc;
  // tbe_backward_sgd clears the counters it relies on (cudaMemsetAsync on `stream`) before its kernels
  // read them, so stale contents of the shared array are harmless.
  return tbe_backward_sgd(grad_output, stride_b, stride_t, weights, table_offsets, indices, offsets, T, B, D, N,
                          total_rows, dtype, pooling, lr, max_rows_per_table, /*plan_ready=*/0, scratch,
                          static_cast<int64_t>(kScratchBytes), stream);
}
