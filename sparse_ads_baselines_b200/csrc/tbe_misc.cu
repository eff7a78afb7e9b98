// Input-side helpers: per-bag length construction and device-side input validation.
#include "tbe_common.cuh"

namespace tbe {
namespace {

__global__ void construct_offsets_kernel(const int32_t* __restrict__ begin,   // [T][B]
                                         const int32_t* __restrict__ totals,  // [T]
                                         int32_t* __restrict__ out, int32_t B, int64_t nbags) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i == 0) out[0] = 0;
  if (i >= nbags) return;
  const int t = static_cast<int>(i / B);
  const int b = static_cast<int>(i - static_cast<int64_t>(t) * B);
  const int32_t hi = (b != B - 1) ? __ldg(begin + i + 1) : __ldg(totals + t);
  out[1 + i] = hi - __ldg(begin + i);
}

// Bag-wise gather of ragged index lists: destination bag g takes the indices of source bag
// src_bag[g].  One warp per destination bag.
__global__ void __launch_bounds__(256) permute_bags_kernel(const int32_t* __restrict__ src_indices,
                                                          const int32_t* __restrict__ src_offsets,
                                                          const int32_t* __restrict__ src_bag,
                                                          const int32_t* __restrict__ dst_offsets,
                                                          int32_t* __restrict__ dst_indices, int64_t nbags) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); g < nbags; g += wstride) {
    const int32_t sb = __ldg(src_bag + g);
    const int32_t s = __ldg(src_offsets + sb), n = __ldg(src_offsets + sb + 1) - s;
    const int32_t d = __ldg(dst_offsets + g);
    for (int32_t i = lane; i < n; i += 32) dst_indices[d + i] = __ldg(src_indices + s + i);
  }
}

// err[0] = violation kind (first writer wins), err[1..3] = details.
enum Violation { kNone = 0, kFirstOffset = 1, kDecreasing = 2, kLastOffset = 3, kIndexRange = 4 };

__device__ void report(int32_t* err, int kind, int32_t a, int32_t b, int32_t c) {
  if (atomicCAS(err, kNone, kind) == kNone) {
    err[1] = a;
    err[2] = b;
    err[3] = c;
  }
}

__global__ void check_inputs_kernel(const int32_t* __restrict__ indices, const int32_t* __restrict__ offsets,
                                    const int32_t* __restrict__ rows_per_table, int32_t B, int64_t nbags,
                                    int64_t N, int32_t* err) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int32_t s = __ldg(offsets + bag), e = __ldg(offsets + bag + 1);
    if (lane == 0) {
      if (bag == 0 && s != 0) report(err, kFirstOffset, s, 0, 0);
      if (bag == nbags - 1 && e != N) report(err, kLastOffset, e, static_cast<int32_t>(N), 0);
      if (e < s) report(err, kDecreasing, static_cast<int32_t>(bag), s, e);
    }
    if (e < s || s < 0 || e > N) continue;  // never dereference a broken extent
    const int t = static_cast<int>(bag / B);
    const int32_t rows = __ldg(rows_per_table + t);
    for (int p = s + lane; p < e; p += 32) {
      const int32_t idx = __ldg(indices + p);
      if (idx < 0 || idx >= rows) report(err, kIndexRange, p, idx, t);
    }
  }
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_construct_offsets(const int32_t* batch_offsets_per_table, const int32_t* total_indices_per_table,
                                     int32_t* lengths_out, int64_t T, int64_t B, void* stream) {
  using namespace tbe;
  TBE_REQUIRE(batch_offsets_per_table && total_indices_per_table && lengths_out,
              "tbe_construct_offsets: null pointer argument");
  TBE_REQUIRE(T > 0 && B > 0 && T * B < (1ll << 31), "tbe_construct_offsets: T and B must be > 0 and T*B < 2^31");
  const int64_t nbags = T * B;
  const int threads = 256;
  const int64_t blocks = (nbags + threads - 1) / threads;
  construct_offsets_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      batch_offsets_per_table, total_indices_per_table, lengths_out, static_cast<int32_t>(B), nbags);
  TBE_CHECK_LAUNCH("construct_offsets_kernel");
  return TBE_OK;
}

extern "C" int tbe_check_inputs(const int32_t* indices, const int32_t* offsets, const int32_t* rows_per_table,
                                int64_t T, int64_t B, int64_t N, void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(offsets && rows_per_table && (indices || N == 0), "tbe_check_inputs: null pointer argument");
  TBE_REQUIRE(T > 0 && B > 0 && N >= 0 && T * B < (1ll << 31) && N < (1ll << 31), "tbe_check_inputs: sizes out of range");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int32_t* err = nullptr;
  // four words of pinned, device-visible memory: the result is read on the host after the sync
  TBE_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&err), 16, cudaHostAllocMapped));
  err[0] = err[1] = err[2] = err[3] = 0;
  int32_t* derr = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&derr), err, 0);
  if (e == cudaSuccess) {
    const int64_t nbags = T * B;
    int64_t blocks = (nbags + 7) / 8;
    const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    check_inputs_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(indices, offsets, rows_per_table,
                                                                          static_cast<int32_t>(B), nbags, N, derr);
    e = cudaGetLastError();
    if (e == cudaSuccess) {
      count_kernel_launch();
      e = cudaStreamSynchronize(stream);
    }
  }
  const int32_t kind = err[0], a = err[1], b = err[2], c = err[3];
  cudaFreeHost(err);
  if (e != cudaSuccess) return fail(TBE_ERR_CUDA, "tbe_check_inputs: %s", cudaGetErrorString(e));
  switch (kind) {
    case kNone: return TBE_OK;
    case kFirstOffset: return fail(TBE_ERR_BAD_INPUT_DATA, "offsets[0] is %d, expected 0", a);
    case kDecreasing: return fail(TBE_ERR_BAD_INPUT_DATA, "offsets decrease at bag %d: %d > %d", a, b, c);
    case kLastOffset: return fail(TBE_ERR_BAD_INPUT_DATA, "offsets[T*B] is %d, expected N = %d", a, b);
    default: return fail(TBE_ERR_BAD_INPUT_DATA, "indices[%d] = %d is outside table %d", a, b, c);
  }
}

extern "C" int tbe_permute_bags(const int32_t* src_indices, const int32_t* src_offsets, const int32_t* src_bag,
                                const int32_t* dst_offsets, int32_t* dst_indices, int64_t nbags, void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(src_offsets && src_bag && dst_offsets, "tbe_permute_bags: null pointer argument");
  TBE_REQUIRE(nbags >= 0 && nbags < (1ll << 31), "tbe_permute_bags: bag count out of range");
  if (nbags == 0) return TBE_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int64_t blocks = (nbags + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  {
    KernelTimer timer("permute_bags_kernel", stream);
    permute_bags_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src_indices, src_offsets, src_bag,
                                                                          dst_offsets, dst_indices, nbags);
  }
  TBE_CHECK_LAUNCH("permute_bags_kernel");
  return TBE_OK;
}
