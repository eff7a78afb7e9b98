// Deterministic TBE backward with the optimizer fused into the write-back (sm_100a).
//
// Pipeline per call (all on the caller's stream, scratch in the caller's workspace):
//   1. linearize   : key[p] = table_offsets[t] + indices[p], value[p] = bag id (t*B+b)
//   2. radix sort  : (key,value) pairs by key over ceil(log2(total_rows)) bits (CUB, stable,
//                    so the entries of one row stay in ascending index position)
//   3. run starts  : positions where the sorted key changes, compacted (CUB select)
//   4. segment kernel: one lane group per run ("segment" = all lookups of one row):
//                    G = sum of the bags' gradient rows in sorted order, then the optimizer
//                    update of that row, written once.  Runs longer than `long_segment`
//                    entries are queued and
//   5. long-segment kernel: one CTA per queued run, lane groups sum strided slices, the
//                    slices are folded in a fixed order in shared memory.
// Every row is read once and written once; gradients of repeated rows are summed before
// the update, so the result does not depend on scheduling.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include "tbe_common.cuh"

namespace tbe {
namespace {

enum Opt { kSGD = 0, kExactAdagrad = 1, kApproxAdagrad = 2 };

constexpr int kDefaultLongSegment = 96;
constexpr int kBwdThreads = 256;

// ------------------------------------------------------------------ workspace
struct Workspace {
  uint32_t* keys[2];
  int32_t* vals[2];
  int32_t* seg_starts;   // N + 1
  int32_t* long_list;    // N / 2 + 1 (a run on the list has >= 2 entries)
  int32_t* bag_of_pos;   // N (approx adagrad only)
  float* bag_g2;         // unused slot kept for the approx path: sized by caller when needed
  int32_t* counters;     // [0] = number of runs, [1] = number of long runs
  void* cub_temp;
  size_t cub_bytes;
  size_t total;
};

// Predicate over positions of the sorted key array: true where a run starts.
struct RunStart {
  const uint32_t* keys;
  __host__ __device__ bool operator()(int32_t i) const { return i == 0 || keys[i] != keys[i - 1]; }
};

size_t cub_temp_bytes(int64_t N, int end_bit, cudaError_t* err) {
  size_t sort_bytes = 0, sel_bytes = 0;
  cub::DoubleBuffer<uint32_t> dk(nullptr, nullptr);
  cub::DoubleBuffer<int32_t> dv(nullptr, nullptr);
  cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, dk, dv, static_cast<int64_t>(N), 0, end_bit);
  if (e != cudaSuccess) {
    *err = e;
    return 0;
  }
  thrust::counting_iterator<int32_t> it(0);
  e = cub::DeviceSelect::If(nullptr, sel_bytes, it, static_cast<int32_t*>(nullptr),
                            static_cast<int32_t*>(nullptr), static_cast<int64_t>(N), RunStart{nullptr});
  if (e != cudaSuccess) {
    *err = e;
    return 0;
  }
  *err = cudaSuccess;
  return sort_bytes > sel_bytes ? sort_bytes : sel_bytes;
}

int key_bits(int64_t total_rows) {
  int bits = 1;
  while (bits < 32 && (1ll << bits) < total_rows) ++bits;
  return bits;
}

// Carves the workspace; with base == nullptr only sizes are computed.
int carve(void* base, int64_t N, int64_t total_rows, Workspace* ws) {
  cudaError_t err = cudaSuccess;
  const size_t cub_bytes = cub_temp_bytes(N > 0 ? N : 1, key_bits(total_rows), &err);
  if (err != cudaSuccess) return fail(TBE_ERR_CUDA, "CUB temp-storage query failed: %s", cudaGetErrorString(err));
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* r = p ? p + off : nullptr;
    off += align_up(bytes, 256);
    return r;
  };
  const size_t n = static_cast<size_t>(N > 0 ? N : 1);
  ws->keys[0] = static_cast<uint32_t*>(take(n * 4));
  ws->keys[1] = static_cast<uint32_t*>(take(n * 4));
  ws->vals[0] = static_cast<int32_t*>(take(n * 4));
  ws->vals[1] = static_cast<int32_t*>(take(n * 4));
  ws->seg_starts = static_cast<int32_t*>(take((n + 1) * 4));
  ws->long_list = static_cast<int32_t*>(take((n / 2 + 1) * 4));
  ws->bag_of_pos = static_cast<int32_t*>(take(n * 4));
  ws->bag_g2 = nullptr;
  ws->counters = static_cast<int32_t*>(take(64));
  ws->cub_temp = take(cub_bytes);
  ws->cub_bytes = cub_bytes;
  ws->total = off;
  return TBE_OK;
}

// ------------------------------------------------------------------ step 1: linearize
// One warp per bag, lanes stride over the bag's index positions.
template <bool WITH_POS>
__global__ void __launch_bounds__(256) linearize_kernel(const int32_t* __restrict__ table_offsets,
                                                       const int32_t* __restrict__ indices,
                                                       const int32_t* __restrict__ offsets, int32_t B,
                                                       int64_t nbags, uint32_t* __restrict__ keys,
                                                       int32_t* __restrict__ vals,
                                                       int32_t* __restrict__ bag_of_pos) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int t = static_cast<int>(bag / B);
    const uint32_t row0 = static_cast<uint32_t>(__ldg(table_offsets + t));
    const int s = __ldg(offsets + bag), e = __ldg(offsets + bag + 1);
    for (int p = s + lane; p < e; p += 32) {
      keys[p] = row0 + static_cast<uint32_t>(__ldg(indices + p));
      if (WITH_POS) {
        vals[p] = p;
        bag_of_pos[p] = static_cast<int32_t>(bag);
      } else {
        vals[p] = static_cast<int32_t>(bag);
      }
    }
  }
}

struct Plan {
  const uint32_t* sorted_rows;
  const int32_t* sorted_vals;
};

// Steps 1-3.  Leaves ws.counters[0] = number of runs, ws.counters[1] = 0.
int build_plan(const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, int64_t T,
               int64_t B, int64_t N, int64_t total_rows, bool with_pos, Workspace& ws, Plan* plan,
               cudaStream_t stream) {
  TBE_CUDA_TRY(cudaMemsetAsync(ws.counters, 0, 64, stream));
  const int64_t nbags = T * B;
  {
    const int wpb = 256 / 32;
    int64_t blocks = (nbags + wpb - 1) / wpb;
    const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    KernelTimer timer("linearize_kernel", stream);
    if (with_pos) {
      linearize_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
          table_offsets, indices, offsets, static_cast<int32_t>(B), nbags, ws.keys[0], ws.vals[0], ws.bag_of_pos);
    } else {
      linearize_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
          table_offsets, indices, offsets, static_cast<int32_t>(B), nbags, ws.keys[0], ws.vals[0], nullptr);
    }
  }
  TBE_CHECK_LAUNCH("linearize_kernel");
  cub::DoubleBuffer<uint32_t> dk(ws.keys[0], ws.keys[1]);
  cub::DoubleBuffer<int32_t> dv(ws.vals[0], ws.vals[1]);
  size_t bytes = ws.cub_bytes;
  {
    KernelTimer timer("cub_radix_sort_pairs", stream);
    TBE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(ws.cub_temp, bytes, dk, dv, static_cast<int64_t>(N), 0,
                                                key_bits(total_rows), stream));
  }
  count_library_launch();
  plan->sorted_rows = dk.Current();
  plan->sorted_vals = dv.Current();
  bytes = ws.cub_bytes;
  thrust::counting_iterator<int32_t> it(0);
  {
    KernelTimer timer("cub_select_run_starts", stream);
    TBE_CUDA_TRY(cub::DeviceSelect::If(ws.cub_temp, bytes, it, ws.seg_starts, ws.counters,
                                       static_cast<int64_t>(N), RunStart{plan->sorted_rows}, stream));
  }
  count_library_launch();
  return TBE_OK;
}

// ------------------------------------------------------------------ steps 4/5: segment kernels
struct BwdArgs {
  const void* grad;
  int64_t stride_b, stride_t;  // elements
  void* weights;
  float* state;
  const uint32_t* sorted_rows;
  const int32_t* sorted_vals;  // bag id (exact/SGD) or index position (approx)
  const int32_t* seg_starts;
  const int32_t* counters;     // [0] runs, [1] long runs
  int32_t* long_list;
  int32_t* long_count;
  const int32_t* offsets;      // bag extents (mean pooling)
  const int32_t* bag_of_pos;   // approx only
  const void* psw;             // approx only, nullable
  const float* bag_g2;         // approx only
  int32_t B, D, N;
  int32_t lpr_log2, nvec, nchunks;
  int32_t long_threshold;
  float lr, eps;
  uint64_t sr_seed, sr_offset;
};

template <typename T, int VB, bool SR>
__device__ __forceinline__ Raw<VB> pack_out(const typename Acc<T>::type* v, Philox* rng) {
  return pack_rn<T, VB>(v);
}
template <>
__device__ __forceinline__ Raw<16> pack_out<__half, 16, true>(const float* v, Philox* rng) {
  Raw<16> r;
  const uint4 r0 = rng->next(), r1 = rng->next();
  const uint32_t rnd[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half lo = sr_half(v[2 * i], rnd[2 * i]), hi = sr_half(v[2 * i + 1], rnd[2 * i + 1]);
    r.w[i] = static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
  }
  return r;
}
template <>
__device__ __forceinline__ Raw<8> pack_out<__half, 8, true>(const float* v, Philox* rng) {
  Raw<8> r;
  const uint4 r0 = rng->next();
  const uint32_t rnd[4] = {r0.x, r0.y, r0.z, r0.w};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const __half lo = sr_half(v[2 * i], rnd[2 * i]), hi = sr_half(v[2 * i + 1], rnd[2 * i + 1]);
    r.w[i] = static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
  }
  return r;
}

// Sums the gradient rows of entries [s + first, s + first + step, ...) < s + len of one run
// for vector v of the row.  All lanes of the warp call this with a warp-uniform `iters`.
template <typename T, int VB, bool MEAN, int UNROLL>
__device__ __forceinline__ void sum_grads(const BwdArgs& a, int s, int len, int first, int step, int iters,
                                          int v, bool vact, typename Acc<T>::type* acc) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const char* __restrict__ G = static_cast<const char*>(a.grad);
  for (int it = 0; it < iters; it += UNROLL) {
    Raw<VB> r[UNROLL];
    acc_t sc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int i = first + (it + u) * step;
      r[u] = raw_zero<VB>();
      sc[u] = 1;
      if (i < len) {
        const uint32_t bag = static_cast<uint32_t>(__ldg(a.sorted_vals + s + i));
        const uint32_t t = bag / static_cast<uint32_t>(a.B);
        const uint32_t b = bag - t * static_cast<uint32_t>(a.B);
        if (vact) {
          r[u] = ld_stream<VB>(G + (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                                       static_cast<int64_t>(sizeof(T)) +
                               static_cast<int64_t>(v) * VB);
        }
        if (MEAN) {
          const int L = __ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag);
          sc[u] = static_cast<acc_t>(L);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      acc_t e[NE];
      unpack<T, VB>(r[u], e);
#pragma unroll
      for (int k = 0; k < NE; ++k) {
        if (MEAN) {
          acc[k] += e[k] / sc[u];
        } else {
          acc[k] += e[k];
        }
      }
    }
  }
}

template <typename A>
__device__ __forceinline__ A sq_sum(const A* v, int n) {
  A s = 0;
  for (int k = 0; k < n; ++k) s += v[k] * v[k];
  return s;
}

// w -= mult * G for one vector, then store.
template <typename T, int VB, bool SR>
__device__ __forceinline__ void apply_update(char* wp, const Raw<VB>& wraw, const typename Acc<T>::type* G,
                                             typename Acc<T>::type mult, Philox* rng) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  acc_t w[NE];
  unpack<T, VB>(wraw, w);
#pragma unroll
  for (int k = 0; k < NE; ++k) w[k] -= G[k] * mult;
  st_row<VB>(wp, pack_out<T, VB, SR>(w, rng));
}

// One lane group per run.  OPT is kSGD or kExactAdagrad.
template <typename T, int VB, int OPT, bool MEAN, bool SR, int UNROLL>
__global__ void __launch_bounds__(kBwdThreads) segment_kernel(const BwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int lpr_log2 = a.lpr_log2;
  const int gpw = 32 >> lpr_log2;  // groups per warp
  const int sub = lane & ((1 << lpr_log2) - 1);
  const int slot = lane >> lpr_log2;
  const int U = __ldg(a.counters);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  Philox rng(a.sr_seed, static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x, a.sr_offset);

  for (int64_t seg0 = warp_global * gpw; seg0 < U; seg0 += warps_total * gpw) {
    const int64_t seg = seg0 + slot;
    bool has = seg < U;
    int s = 0, len = 0;
    uint32_t row = 0;
    if (has) {
      s = __ldg(a.seg_starts + seg);
      const int e = (seg + 1 < U) ? __ldg(a.seg_starts + seg + 1) : a.N;
      len = e - s;
      row = __ldg(a.sorted_rows + s);
      if (len > a.long_threshold) {
        if (sub == 0) a.long_list[atomicAdd(a.long_count, 1)] = static_cast<int32_t>(seg);
        has = false;
        len = 0;
      }
    }
    const int maxlen = __reduce_max_sync(kFullMask, len);
    char* wrow = static_cast<char*>(a.weights) + static_cast<int64_t>(row) * row_bytes;

    acc_t g2 = 0;
    if (OPT == kExactAdagrad && a.nchunks > 1) {
      for (int c = 0; c < a.nchunks; ++c) {
        const int v = (c << 5) + sub;
        const bool vact = v < a.nvec;
        acc_t acc[NE];
#pragma unroll
        for (int k = 0; k < NE; ++k) acc[k] = 0;
        sum_grads<T, VB, MEAN, UNROLL>(a, s, len, 0, 1, maxlen, v, vact, acc);
        g2 += sq_sum(acc, NE);
      }
      g2 = group_sum(g2, lpr_log2);
    }
    acc_t mult = static_cast<acc_t>(a.lr);
    for (int c = 0; c < a.nchunks; ++c) {
      const int v = (c << 5) + sub;
      const bool vact = v < a.nvec;
      Raw<VB> wraw = raw_zero<VB>();
      if (has && vact) wraw = ld_rw<VB>(wrow + static_cast<int64_t>(v) * VB);
      acc_t acc[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) acc[k] = 0;
      sum_grads<T, VB, MEAN, UNROLL>(a, s, len, 0, 1, maxlen, v, vact, acc);
      if (OPT == kExactAdagrad && c == 0) {
        if (a.nchunks == 1) g2 = group_sum(sq_sum(acc, NE), lpr_log2);
        const float st = (has ? a.state[row] : 0.f) + static_cast<float>(g2);
        __syncwarp();
        if (has && sub == 0) a.state[row] = st;
        mult = static_cast<acc_t>(a.lr * (1.0f / (sqrtf(st) + a.eps)));
      }
      if (has && vact) apply_update<T, VB, SR>(wrow + static_cast<int64_t>(v) * VB, wraw, acc, mult, &rng);
    }
  }
}

// One CTA per queued long run.
template <typename T, int VB, int OPT, bool MEAN, bool SR>
__global__ void __launch_bounds__(kBwdThreads) long_segment_kernel(const BwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  __shared__ acc_t part[kBwdThreads * NE];
  const int lane = threadIdx.x & 31;
  const int lpr_log2 = a.lpr_log2;
  const int lpr = 1 << lpr_log2;
  const int sub = lane & (lpr - 1);
  const int gid = threadIdx.x >> lpr_log2;
  const int groups = blockDim.x >> lpr_log2;
  const int U = __ldg(a.counters);
  const int nlong = __ldg(a.counters + 1);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  Philox rng(a.sr_seed, (static_cast<uint64_t>(gridDim.x) + 1 + blockIdx.x) * blockDim.x + threadIdx.x + (1ull << 40),
             a.sr_offset);

  for (int li = blockIdx.x; li < nlong; li += gridDim.x) {
    const int seg = a.long_list[li];
    const int s = __ldg(a.seg_starts + seg);
    const int e = (seg + 1 < U) ? __ldg(a.seg_starts + seg + 1) : a.N;
    const int len = e - s;
    const uint32_t row = __ldg(a.sorted_rows + s);
    char* wrow = static_cast<char*>(a.weights) + static_cast<int64_t>(row) * row_bytes;
    const int iters = (len + groups - 1) / groups;  // block-uniform

    // Folds the groups' partial sums for vector v in group order; every thread of warp 0 returns
    // the total of its own `sub`, other warps return garbage they never use.
    auto reduce_chunk = [&](int c, acc_t* total) {
      const int v = (c << 5) + sub;
      const bool vact = v < a.nvec;
      acc_t acc[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) acc[k] = 0;
      sum_grads<T, VB, MEAN, 4>(a, s, len, gid, groups, iters, v, vact, acc);
      __syncthreads();  // previous use of `part` finished
#pragma unroll
      for (int k = 0; k < NE; ++k) part[threadIdx.x * NE + k] = acc[k];
      __syncthreads();
#pragma unroll
      for (int k = 0; k < NE; ++k) total[k] = 0;
      if (threadIdx.x < 32) {
        for (int g = 0; g < groups; ++g) {
#pragma unroll
          for (int k = 0; k < NE; ++k) total[k] += part[(g * lpr + sub) * NE + k];
        }
      }
    };

    acc_t g2 = 0;
    if (OPT == kExactAdagrad && a.nchunks > 1) {
      for (int c = 0; c < a.nchunks; ++c) {
        acc_t tot[NE];
        reduce_chunk(c, tot);
        const int v = (c << 5) + sub;
        if (v < a.nvec) g2 += sq_sum(tot, NE);
      }
      if (threadIdx.x < 32) g2 = group_sum(g2, lpr_log2);
    }
    acc_t mult = static_cast<acc_t>(a.lr);
    for (int c = 0; c < a.nchunks; ++c) {
      const int v = (c << 5) + sub;
      const bool vact = v < a.nvec;
      acc_t tot[NE];
      reduce_chunk(c, tot);
      if (threadIdx.x < 32) {
        if (OPT == kExactAdagrad && c == 0) {
          if (a.nchunks == 1) g2 = group_sum(vact ? sq_sum(tot, NE) : acc_t(0), lpr_log2);
          const float st = a.state[row] + static_cast<float>(g2);
          __syncwarp();
          if (lane == 0) a.state[row] = st;
          mult = static_cast<acc_t>(a.lr * (1.0f / (sqrtf(st) + a.eps)));
        }
        if (gid == 0 && vact) {
          const Raw<VB> wraw = ld_rw<VB>(wrow + static_cast<int64_t>(v) * VB);
          apply_update<T, VB, SR>(wrow + static_cast<int64_t>(v) * VB, wraw, tot, mult, &rng);
        }
      }
    }
  }
}

template <typename T, int VB, int OPT, bool MEAN, bool SR>
int launch_segments(const BwdArgs& a, cudaStream_t stream) {
  int threads = tuning(kTuneBwdThreads);
  if (threads <= 0) threads = kBwdThreads;
  if (threads > kBwdThreads || threads % 32 != 0)
    return fail(TBE_ERR_INVALID_ARGUMENT, "bwd_threads must be a multiple of 32 <= %d", kBwdThreads);
  const int unroll = tuning(kTuneBwdUnroll) > 0 ? tuning(kTuneBwdUnroll) : 2;
  void (*kernel)(const BwdArgs) = nullptr;
  switch (unroll) {
    case 1: kernel = segment_kernel<T, VB, OPT, MEAN, SR, 1>; break;
    case 2: kernel = segment_kernel<T, VB, OPT, MEAN, SR, 2>; break;
    case 4: kernel = segment_kernel<T, VB, OPT, MEAN, SR, 4>; break;
    default: return fail(TBE_ERR_INVALID_ARGUMENT, "bwd_unroll must be 1, 2 or 4");
  }
  int per_sm = 0;
  TBE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
  if (per_sm < 1) per_sm = 1;
  const int gpw = 32 >> a.lpr_log2;
  const int64_t groups_per_block = static_cast<int64_t>(threads / 32) * gpw;
  int64_t blocks = (static_cast<int64_t>(a.N) + groups_per_block - 1) / groups_per_block;  // U <= N
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  if (blocks > resident) blocks = resident;
  if (blocks < 1) blocks = 1;
  {
    KernelTimer timer("segment_kernel", stream);
    kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("segment_kernel");
  {
    KernelTimer timer("long_segment_kernel", stream);
    long_segment_kernel<T, VB, OPT, MEAN, SR><<<device_sm_count() * 2, kBwdThreads, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("long_segment_kernel");
  return TBE_OK;
}

template <typename T, int VB, int OPT>
int dispatch_flags(const BwdArgs& a, bool mean, bool sr, cudaStream_t stream) {
  if (mean) {
    if (sr) return launch_segments<T, VB, OPT, true, true>(a, stream);
    return launch_segments<T, VB, OPT, true, false>(a, stream);
  }
  if (sr) return launch_segments<T, VB, OPT, false, true>(a, stream);
  return launch_segments<T, VB, OPT, false, false>(a, stream);
}

template <int OPT>
int dispatch_bwd(const BwdArgs& a, int dtype, int vb, bool mean, bool sr, cudaStream_t stream) {
  switch (dtype) {
    case TBE_F16:
      if (vb == 16) return dispatch_flags<__half, 16, OPT>(a, mean, sr, stream);
      return dispatch_flags<__half, 8, OPT>(a, mean, sr, stream);
    case TBE_F32:
      return dispatch_flags<float, 16, OPT>(a, mean, false, stream);
    case TBE_F64:
      return dispatch_flags<double, 16, OPT>(a, mean, false, stream);
  }
  return fail(TBE_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

int check_common(const char* who, const void* grad, const void* weights, const int32_t* table_offsets,
                 const int32_t* indices, const int32_t* offsets, int64_t T, int64_t B, int64_t D, int64_t N,
                 int64_t total_rows, int dtype, const void* workspace) {
  TBE_REQUIRE(grad && weights && table_offsets && indices && offsets, "%s: null pointer argument", who);
  TBE_REQUIRE(workspace != nullptr, "%s: workspace is null", who);
  TBE_REQUIRE(T > 0 && B > 0, "%s: T and B must be > 0", who);
  TBE_REQUIRE(D > 0 && D % 4 == 0, "%s: D must be a positive multiple of 4 (got %lld)", who, (long long)D);
  TBE_REQUIRE(N >= 0 && N < (1ll << 31) - 1, "%s: N out of range", who);
  TBE_REQUIRE(T * B < (1ll << 31), "%s: B*T out of range", who);
  TBE_REQUIRE(total_rows > 0 && total_rows < (1ll << 31), "%s: total_rows out of range", who);
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "%s: bad dtype %d", who, dtype);
  return TBE_OK;
}

int exact_backward(int opt, const void* grad, int64_t stride_b, int64_t stride_t, void* weights,
                   const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, float* state,
                   int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, int pooling,
                   float lr, float eps, int sr, uint64_t sr_seed, uint64_t sr_offset, void* workspace,
                   int64_t workspace_bytes, void* stream_v) {
  const char* who = opt == kSGD ? "tbe_backward_sgd" : "tbe_backward_exact_rowwise_adagrad";
  int rc = check_common(who, grad, weights, table_offsets, indices, offsets, T, B, D, N, total_rows, dtype, workspace);
  if (rc != TBE_OK) return rc;
  TBE_REQUIRE(pooling == TBE_POOL_SUM || pooling == TBE_POOL_MEAN, "%s: bad pooling %d", who, pooling);
  TBE_REQUIRE(opt == kSGD || state != nullptr, "%s: optimizer_state is null", who);
  if (N == 0) return TBE_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  Workspace ws;
  rc = carve(workspace, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  if (static_cast<int64_t>(ws.total) > workspace_bytes)
    return fail(TBE_ERR_WORKSPACE_TOO_SMALL, "%s: workspace has %lld bytes, %lld needed", who,
                (long long)workspace_bytes, (long long)ws.total);
  TBE_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "%s: workspace must be 256-byte aligned", who);
  Plan plan;
  rc = build_plan(table_offsets, indices, offsets, T, B, N, total_rows, false, ws, &plan, stream);
  if (rc != TBE_OK) return rc;

  BwdArgs a{};
  a.grad = grad;
  a.stride_b = stride_b;
  a.stride_t = stride_t;
  a.weights = weights;
  a.state = state;
  a.sorted_rows = plan.sorted_rows;
  a.sorted_vals = plan.sorted_vals;
  a.seg_starts = ws.seg_starts;
  a.counters = ws.counters;
  a.long_list = ws.long_list;
  a.long_count = ws.counters + 1;
  a.offsets = offsets;
  a.B = static_cast<int32_t>(B);
  a.D = static_cast<int32_t>(D);
  a.N = static_cast<int32_t>(N);
  const int es = elem_size(dtype);
  // the gradient rows must allow the same vector width as the weight rows
  const bool grad16 = reinterpret_cast<uintptr_t>(grad) % 16 == 0 && (stride_b * es) % 16 == 0 && (stride_t * es) % 16 == 0;
  const RowGeom g = make_geom(D, dtype, weights, grad16 ? nullptr : reinterpret_cast<const void*>(uintptr_t(8)));
  TBE_REQUIRE(g.vb == 16 || dtype == TBE_F16, "%s: weights and grad_output rows must be 16-byte aligned", who);
  if (g.vb == 8)
    TBE_REQUIRE(reinterpret_cast<uintptr_t>(grad) % 8 == 0 && (stride_b * es) % 8 == 0 && (stride_t * es) % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(weights) % 8 == 0,
                "%s: weights and grad_output rows must be 8-byte aligned", who);
  a.lpr_log2 = g.lpr_log2;
  a.nvec = g.nvec;
  a.nchunks = g.nchunks;
  a.long_threshold = tuning(kTuneLongSegment) > 0 ? tuning(kTuneLongSegment) : kDefaultLongSegment;
  a.lr = lr;
  a.eps = eps;
  a.sr_seed = sr_seed;
  a.sr_offset = sr_offset;
  const bool mean = pooling == TBE_POOL_MEAN;
  const bool use_sr = sr != 0 && dtype == TBE_F16;
  if (opt == kSGD) return dispatch_bwd<kSGD>(a, dtype, g.vb, mean, use_sr, stream);
  return dispatch_bwd<kExactAdagrad>(a, dtype, g.vb, mean, use_sr, stream);
}

}  // namespace
}  // namespace tbe

extern "C" int64_t tbe_backward_workspace_bytes(int64_t N, int64_t total_rows) {
  if (N < 0 || total_rows <= 0) return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_backward_workspace_bytes: bad sizes");
  tbe::Workspace ws;
  const int rc = tbe::carve(nullptr, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  return static_cast<int64_t>(ws.total);
}

extern "C" int tbe_backward_sgd(const void* grad_output, int64_t stride_b, int64_t stride_t, void* weights,
                                const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets,
                                int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype,
                                int pooling, float lr, void* workspace, int64_t workspace_bytes, void* stream) {
  return tbe::exact_backward(tbe::kSGD, grad_output, stride_b, stride_t, weights, table_offsets, indices, offsets,
                             nullptr, T, B, D, N, total_rows, dtype, pooling, lr, 0.f, 0, 0, 0, workspace,
                             workspace_bytes, stream);
}

extern "C" int tbe_backward_exact_rowwise_adagrad(const void* grad_output, int64_t stride_b, int64_t stride_t,
                                                  void* weights, const int32_t* table_offsets,
                                                  const int32_t* indices, const int32_t* offsets,
                                                  float* optimizer_state, int64_t T, int64_t B, int64_t D,
                                                  int64_t N, int64_t total_rows, int dtype, int pooling, float lr,
                                                  float eps, int stochastic_rounding, uint64_t sr_seed,
                                                  uint64_t sr_offset, void* workspace, int64_t workspace_bytes,
                                                  void* stream) {
  return tbe::exact_backward(tbe::kExactAdagrad, grad_output, stride_b, stride_t, weights, table_offsets, indices,
                             offsets, optimizer_state, T, B, D, N, total_rows, dtype, pooling, lr, eps,
                             stochastic_rounding, sr_seed, sr_offset, workspace, workspace_bytes, stream);
}

extern "C" int tbe_sort_segments(const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets,
                                 int64_t T, int64_t B, int64_t N, int64_t total_rows, int32_t* sorted_rows,
                                 int32_t* sorted_bags, int32_t* segment_starts, int32_t* num_segments,
                                 void* workspace, int64_t workspace_bytes, void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(table_offsets && indices && offsets && sorted_rows && sorted_bags && segment_starts && num_segments &&
                  workspace,
              "tbe_sort_segments: null pointer argument");
  TBE_REQUIRE(T > 0 && B > 0 && N >= 0 && N < (1ll << 31) - 1 && total_rows > 0 && total_rows < (1ll << 31),
              "tbe_sort_segments: sizes out of range");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (N == 0) {
    TBE_CUDA_TRY(cudaMemsetAsync(num_segments, 0, 4, stream));
    TBE_CUDA_TRY(cudaMemsetAsync(segment_starts, 0, 4, stream));
    return TBE_OK;
  }
  Workspace ws;
  int rc = carve(workspace, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  if (static_cast<int64_t>(ws.total) > workspace_bytes)
    return fail(TBE_ERR_WORKSPACE_TOO_SMALL, "tbe_sort_segments: workspace has %lld bytes, %lld needed",
                (long long)workspace_bytes, (long long)ws.total);
  Plan plan;
  rc = build_plan(table_offsets, indices, offsets, T, B, N, total_rows, false, ws, &plan, stream);
  if (rc != TBE_OK) return rc;
  TBE_CUDA_TRY(cudaMemcpyAsync(sorted_rows, plan.sorted_rows, N * 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(sorted_bags, plan.sorted_vals, N * 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(segment_starts, ws.seg_starts, N * 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(num_segments, ws.counters, 4, cudaMemcpyDeviceToDevice, stream));
  return TBE_OK;
}
