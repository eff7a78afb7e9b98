// Deterministic TBE backward with the optimizer fused into the write-back (sm_100a).
//
// Two phases, both on the caller's stream with scratch in the caller's workspace:
//
//  plan (depends on the indices only, so a caller may build it while the forward runs):
//   1. linearize  : key[p] = table_offsets[t] + indices[p], value[p] = bag id (t*B+b)
//   2. radix sort : (key,value) pairs by key over ceil(log2(total_rows)) bits (CUB, stable,
//                   so the lookups of one row stay in ascending index position)
//
//  apply:
//   3. run kernel : a warp walks 32 consecutive sorted entries at a time ("tile").  The tile's keys
//                   and values are loaded coalesced, one per lane, and the next tile is prefetched
//                   while this one is processed.  Run starts are found with one shuffle and a
//                   ballot; every run that STARTS in the tile is owned by one lane group of the
//                   warp, which already holds the row id and the bag ids in registers, so the
//                   gradient rows and the weight row are requested without any dependent load.
//                   G = sum of the run's gradient rows in sorted order; then the optimizer update
//                   of the row, written once.  A run that continues past its tile is followed by
//                   its owner; if it is longer than `long_segment` entries it is queued instead.
//   4. long-run kernel: one CTA per queued run; lane groups sum strided slices that are folded in
//                   a fixed order in shared memory.
//
// Every touched row is read once and written once; gradients of repeated rows are summed before
// the update in an order fixed by the sort, so results do not depend on scheduling.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include <type_traits>

#include "tbe_plan.cuh"

namespace tbe {

// ------------------------------------------------------------------ shared host helpers (tbe_plan.cuh)
// Predicate over positions of the sorted key array: true where a run starts.
struct RunStart {
  const uint32_t* keys;
  __host__ __device__ bool operator()(int32_t i) const { return i == 0 || keys[i] != keys[i - 1]; }
};

size_t cub_temp_bytes(int64_t N, int end_bit, cudaError_t* err) {
  size_t sort_bytes = 0, sel_bytes = 0;
  cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<const uint32_t*>(nullptr),
                                                  static_cast<uint32_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                                                  static_cast<int32_t*>(nullptr), static_cast<int64_t>(N), 0, end_bit);
  if (e != cudaSuccess) {
    *err = e;
    return 0;
  }
  thrust::counting_iterator<int32_t> it(0);
  e = cub::DeviceSelect::If(nullptr, sel_bytes, it, static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                            static_cast<int64_t>(N), RunStart{nullptr});
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
  const size_t cub_bytes = cub_temp_bytes(N > 0 ? N : 1, 32, &err);
  if (err != cudaSuccess) return fail(TBE_ERR_CUDA, "CUB temp-storage query failed: %s", cudaGetErrorString(err));
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* r = p ? p + off : nullptr;
    off += align_up(bytes, 256);
    return r;
  };
  const size_t n = static_cast<size_t>(N > 0 ? N : 1);
  ws->counters = static_cast<int32_t*>(take(64));
  ws->keys = static_cast<uint32_t*>(take(n * 4));
  ws->vals = static_cast<int32_t*>(take(n * 4));
  ws->long_list = static_cast<int2*>(take((n / 32 + 2) * sizeof(int2)));
  ws->keys_in = static_cast<uint32_t*>(take(n * 4));
  ws->vals_in = static_cast<int32_t*>(take(n * 4));
  ws->seg_starts = static_cast<int32_t*>(take((n + 1) * 4));
  ws->entry_bag = static_cast<int32_t*>(take(n * 4));
  ws->entry_g2 = static_cast<float*>(take(n * 4));
  ws->hist_cap = static_cast<int64_t>(n / 16 + 4096);
  ws->queue_cap = static_cast<int64_t>(n / kBucketSortMaxGroup + 2);
  ws->hist = static_cast<int32_t*>(take(ws->hist_cap * 4));
  ws->bucket_start = static_cast<int32_t*>(take(ws->hist_cap * 4));
  ws->oversize = static_cast<int2*>(take(ws->queue_cap * sizeof(int2)));
  ws->cub_temp = take(cub_bytes);
  ws->cub_bytes = cub_bytes;
  ws->total = off;
  return TBE_OK;
}

KeyLayout key_layout(int64_t T, int64_t total_rows, int64_t max_rows_per_table, bool full_order) {
  KeyLayout k;
  int ib = 0, tb = 0;
  if (max_rows_per_table > 0) {
    ib = 1;
    while (ib < 32 && (1ll << ib) < max_rows_per_table) ++ib;
    while ((1ll << tb) < T) ++tb;
  }
  if (ib == 0 || ib + tb > 32) {
    k.idx_bits = 0;
    k.sort_bits = key_bits(total_rows);
  } else {
    k.idx_bits = ib;
    k.sort_bits = full_order ? (ib + tb > 0 ? ib + tb : 1) : ib;
  }
  return k;
}

int check_sizes(const char* who, int64_t T, int64_t B, int64_t N, int64_t total_rows) {
  TBE_REQUIRE(T > 0 && B > 0, "%s: T and B must be > 0", who);
  TBE_REQUIRE(N >= 0 && N < (1ll << 31) - 65536, "%s: N out of range", who);  // kernels look a tile ahead in int32
  TBE_REQUIRE(T * B < (1ll << 31), "%s: B*T out of range", who);
  TBE_REQUIRE(total_rows > 0 && total_rows < (1ll << 31), "%s: total_rows out of range", who);
  return TBE_OK;
}

int prepare_workspace(const char* who, void* workspace, int64_t workspace_bytes, int64_t N, int64_t total_rows,
                      Workspace* ws) {
  TBE_REQUIRE(workspace != nullptr, "%s: workspace is null", who);
  TBE_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "%s: workspace must be 256-byte aligned", who);
  const int rc = carve(workspace, N, total_rows, ws);
  if (rc != TBE_OK) return rc;
  if (static_cast<int64_t>(ws->total) > workspace_bytes)
    return fail(TBE_ERR_WORKSPACE_TOO_SMALL, "%s: workspace has %lld bytes, %lld needed", who,
                (long long)workspace_bytes, (long long)ws->total);
  return TBE_OK;
}


int sort_pairs(Workspace& ws, int64_t N, int sort_bits, cudaStream_t stream) {
  size_t bytes = ws.cub_bytes;
  {
    KernelTimer timer("cub_radix_sort_pairs", stream);
    TBE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(ws.cub_temp, bytes, static_cast<const uint32_t*>(ws.keys_in),
                                                ws.keys, static_cast<const int32_t*>(ws.vals_in), ws.vals, N, 0,
                                                sort_bits, stream));
  }
  count_library_launch();
  return TBE_OK;
}

int select_run_starts(Workspace& ws, int64_t N, cudaStream_t stream) {
  size_t bytes = ws.cub_bytes;
  thrust::counting_iterator<int32_t> it(0);
  {
    KernelTimer timer("cub_select_run_starts", stream);
    TBE_CUDA_TRY(cub::DeviceSelect::If(ws.cub_temp, bytes, it, ws.seg_starts, ws.counters, N, RunStart{ws.keys}, stream));
  }
  count_library_launch();
  return TBE_OK;
}

namespace {

enum Opt { kSGD = 0, kExactAdagrad = 1, kApproxAdagrad = 2 };

constexpr int kDefaultLongSegment = 64;
constexpr int kMinSplitPart = 256;  // entries per part of a split long run (doubled until the scratch fits)
constexpr int kBwdThreads = 256;

// ------------------------------------------------------------------ step 1: linearize
// One warp per bag, lanes stride over the bag's index positions.
__global__ void __launch_bounds__(256) linearize_kernel(const int32_t* __restrict__ table_offsets,
                                                       const int32_t* __restrict__ indices,
                                                       const int32_t* __restrict__ offsets, int32_t B,
                                                       int64_t nbags, int idx_bits, uint32_t* __restrict__ keys,
                                                       int32_t* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int t = static_cast<int>(bag / B);
    // composite key (table << idx_bits | index) when idx_bits > 0, else the linear row id
    const uint32_t row0 = idx_bits ? (static_cast<uint32_t>(t) << idx_bits) : static_cast<uint32_t>(__ldg(table_offsets + t));
    const int s = __ldg(offsets + bag), e = __ldg(offsets + bag + 1);
    for (int p = s + lane; p < e; p += 32) {
      keys[p] = row0 + static_cast<uint32_t>(__ldg(indices + p));
      vals[p] = static_cast<int32_t>(bag);
    }
  }
}

__global__ void __launch_bounds__(256) keys_to_rows_kernel(const int32_t* __restrict__ table_offsets, int idx_bits,
                                                          const uint32_t* __restrict__ keys,
                                                          int32_t* __restrict__ rows, int64_t N) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i < N) rows[i] = static_cast<int32_t>(key_to_row(table_offsets, idx_bits, keys[i]));
}

// Steps 1-2.  Leaves the sorted pairs in ws.keys / ws.vals.
int build_plan(const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, int64_t T,
               int64_t B, int64_t N, int64_t max_rows_per_table, KeyLayout layout, Workspace& ws,
               cudaStream_t stream) {
  BucketGeometry geom;
  if (bucket_geometry(T, N, max_rows_per_table, layout, ws, &geom))
    return bucket_sort_plan(indices, offsets, T, B, N, layout, geom, ws, stream);
  const int64_t nbags = T * B;
  {
    const int wpb = 256 / 32;
    int64_t blocks = (nbags + wpb - 1) / wpb;
    const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    KernelTimer timer("linearize_kernel", stream);
    linearize_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        table_offsets, indices, offsets, static_cast<int32_t>(B), nbags, layout.idx_bits, ws.keys_in, ws.vals_in);
  }
  TBE_CHECK_LAUNCH("linearize_kernel");
  return sort_pairs(ws, N, layout.sort_bits, stream);
}

// ------------------------------------------------------------------ steps 3/4: run kernels
struct BwdArgs {
  const void* grad;
  int64_t stride_b, stride_t;  // elements
  void* weights;
  float* state;
  const uint32_t* keys;   // sorted row ids
  const int32_t* vals;    // bag id of every sorted entry
  int2* long_list;
  int32_t* long_count;
  const int32_t* offsets;  // bag extents (mean pooling)
  const int32_t* table_offsets;
  int32_t idx_bits;        // > 0: keys are (table << idx_bits | index)
  FastDiv divB;            // bag id / B
  int32_t B, D, N;
  int32_t lpr_log2;          // run_kernel: lanes per row when a lane owns VPL vectors
  int32_t lpr1_log2, nchunks;  // wide / long-run kernels: one vector per lane, rows walked in chunks
  int32_t nvec;
  int32_t long_threshold;
  float lr, eps;
  uint64_t sr_seed, sr_offset;
  const float* bag_g2;       // approximate Adagrad: squared gradient norm of every bag
  int32_t* tile_ticket;      // run_kernel: tiles handed out so far beyond every warp's first (null: fixed stride)
  // long runs cut into parts (0 = off): a part is split_len entries (the last one up to twice that)
  int32_t split_len, max_parts;
  int4* part_list;           // dense list of parts: {first entry, end entry, list index of the run's first part, parts of the run}
  int32_t* part_count;       // parts listed so far
  int32_t* part_tickets;     // at the list index of a run's first part: parts of the run finished so far
  float* part_sums;          // [max_parts][D] partial sums, one slot per listed part
};

// Queues a run of sorted entries [s, e) that is too long for the lane groups of run_kernel; called by the
// first lane of the group that found it.  A run of at least two parts is also cut into parts: they take
// consecutive places in the part list, and the ticket of the run starts at zero.
__device__ __forceinline__ void enqueue_long_run(const BwdArgs& a, int s, int e) {
  a.long_list[atomicAdd(a.long_count, 1)] = make_int2(s, e);
  const int part = a.split_len;
  if (part > 0 && e - s >= 2 * part) {
    const int nparts = (e - s) / part;
    const int base = atomicAdd(a.part_count, nparts);  // at most N / split_len parts exist in total
    a.part_tickets[base] = 0;
    for (int k = 0; k < nparts; ++k) {
      const int ps = s + k * part;
      a.part_list[base + k] = make_int4(ps, k == nparts - 1 ? e : ps + part, base, nparts);
    }
  }
}

// Step size of approximate rowwise Adagrad after the state has reached s.
__device__ __forceinline__ float approx_step(const BwdArgs& a, float s) { return a.lr * (1.0f / (sqrtf(s) + a.eps)); }

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

// Requests vector v of the gradient row of `bag`; for mean pooling *scale receives 1/L of the bag.
// Gradient rows are re-read once per lookup, so they are kept in L2 (evict-last policy `keep`).
template <typename T, int VB, bool MEAN>
__device__ __forceinline__ Raw<VB> load_grad(const BwdArgs& a, uint32_t bag, int v, uint64_t keep,
                                             typename Acc<T>::type* scale) {
  using acc_t = typename Acc<T>::type;
  const uint32_t t = fastdiv(bag, a.divB);
  const uint32_t b = bag - t * static_cast<uint32_t>(a.B);
  if (MEAN) *scale = acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag));
  return ld_stream_hint<VB>(static_cast<const char*>(a.grad) +
                                (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                                    static_cast<int64_t>(sizeof(T)) +
                                static_cast<int64_t>(v) * VB,
                            keep);
}

template <typename T, int VB, bool MEAN>
__device__ __forceinline__ void add_grad(const Raw<VB>& r, typename Acc<T>::type scale, typename Acc<T>::type* acc) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  if (MEAN) {
    acc_t e[NE];
    unpack<T, VB>(r, e);
#pragma unroll
    for (int k = 0; k < NE; ++k) acc[k] += e[k] * scale;
  } else {
    accumulate<T, VB>(r, acc);
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
                                             typename Acc<T>::type mult, Philox* rng, uint64_t streaming) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  acc_t w[NE];
  unpack<T, VB>(wraw, w);
#pragma unroll
  for (int k = 0; k < NE; ++k) w[k] -= G[k] * mult;
  st_row_hint<VB>(wp, pack_out<T, VB, SR>(w, rng), streaming);
}

// First position >= lo in the sorted keys whose key differs from `row` (keys[lo-1] == row).  Most runs
// end a few entries further on, so the end is bracketed by doubling steps before it is bisected.
__device__ __forceinline__ int run_end(const uint32_t* __restrict__ keys, int lo, int N, uint32_t row) {
  int hi = N;
  for (int step = 1; step < (1 << 30) && static_cast<int64_t>(lo) + step < N; step <<= 1) {
    if (__ldg(keys + lo + step - 1) != row) {
      hi = lo + step - 1;
      break;
    }
    lo += step;
  }
  while (lo < hi) {
    const int mid = lo + ((hi - lo) >> 1);
    if (__ldg(keys + mid) == row) {
      lo = mid + 1;
    } else {
      hi = mid;
    }
  }
  return lo;
}

// Registers of one tile of 32 sorted entries: key/val of entry p0+lane and a halo word (lane 0: the
// key before the tile, lane 31: the key after it).
struct Tile {
  uint32_t key, halo;
  int32_t val;
};

__device__ __forceinline__ Tile load_tile(const uint32_t* __restrict__ keys, const int32_t* __restrict__ vals,
                                          int64_t tile, int lane, int N) {
  Tile t;
  const int64_t p = (tile << 5) + lane;
  t.key = 0xffffffffu;
  t.val = 0;
  t.halo = 0xffffffffu;
  if (p < N) {
    t.key = __ldg(keys + p);
    t.val = __ldg(vals + p);
  }
  if (lane == 0 && p > 0) t.halo = __ldg(keys + p - 1);
  if (lane == 31 && p + 1 < N) t.halo = __ldg(keys + p + 1);
  return t;
}

// Rows of up to 32*VPL vectors (the common case).
//
// Work that is per sorted ENTRY is done by all 32 lanes at once, one entry per lane, once per tile:
// decoding the key into a weight row, turning the bag id into the offset of its gradient row (and
// 1/L for mean pooling), and measuring the run that starts at the lane.  Work that is per RUN is
// done by a lane group that reads those per-lane results with shuffles: a run costs a handful of
// shuffles, two address computations and its row loads.  A lane owns VPL vectors of a row (vector
// sub, sub + lpr, ...: every load instruction of the warp covers contiguous 16*lpr-byte pieces), so
// a 256-byte row needs only 4 lanes and a warp works on 8 runs at a time; each group keeps SEGS
// runs in flight: the weight row, the optimizer state and the first two gradient rows of each are
// requested first, then the runs are finished one after the other.
//
// Approximate rowwise Adagrad (OPT == kApproxAdagrad) applies every lookup of a row on its own:
// state += g2(bag), row -= lr / (sqrt(state) + eps) * grad(bag), in bag order.  The state after the
// k-th lookup of a run is state_0 plus a prefix sum of the bags' g2, so the whole run is again a
// weighted sum of gradient rows: the tile computes the prefix sums with a segmented scan across its
// lanes, turns them into per-entry step sizes, and the run reduction below uses them exactly as mean
// pooling uses 1/L.
//
// Register budget: 64 (4 CTAs of 256 threads per SM).  Variants squeezed to 56 and 48 registers (9 and
// 10 CTAs of 128 threads per SM) were measured 6 % to 30 % slower on the headline batch, and two runs
// in flight per lane group at 80 registers (3 CTAs per SM) 29 % slower: the kernel is short neither
// of resident warps nor of loads in flight per warp.
template <typename T, int VB, int OPT, bool MEAN, bool SR, int SEGS, int VPL>
__global__ void __launch_bounds__(kBwdThreads, 4) run_kernel(const BwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  constexpr bool APPROX = OPT == kApproxAdagrad;
  constexpr bool SCALED = MEAN || APPROX;  // every gradient row is multiplied by a per-entry factor
  const int lane = threadIdx.x & 31;
  const int lpr_log2 = a.lpr_log2;
  const int lpr = 1 << lpr_log2;
  const int sub = lane & (lpr - 1);
  const int slot = lane >> lpr_log2;
  const int N = a.N;
  const int32_t ntiles = static_cast<int32_t>((static_cast<int64_t>(N) + 31) >> 5);  // N < 2^31
  // A warp starts on the tile of its own number and then takes whichever tile is next on the ticket
  // counter: tiles differ a lot in cost (a tile inside a long run costs nothing, one with 32 runs 32
  // row updates), and with a fixed stride the warps with the dearest tiles would finish last.
  const int32_t wstride = static_cast<int32_t>(gridDim.x * (blockDim.x >> 5));
  const bool ticketed = a.tile_ticket != nullptr;
  int32_t tile = static_cast<int32_t>(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
  if (tile >= ntiles) return;
  int32_t ntile = tile + wstride;
  if (ticketed) {
    int32_t tk = 0;
    if (lane == 0) tk = atomicAdd(a.tile_ticket, 1);
    ntile = wstride + __shfl_sync(kFullMask, tk, 0);
  }
  const uint32_t row_bytes = static_cast<uint32_t>(a.D) * static_cast<uint32_t>(sizeof(T));
  const uint32_t* __restrict__ keys = a.keys;
  const int32_t* __restrict__ vals = a.vals;
  // byte offset of this lane's j-th vector inside a row; lanes beyond the row's end re-read vector 0
  // (a valid address) and never store
  bool vact[VPL];
  uint32_t voff[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = sub + j * lpr;
    vact[j] = v < a.nvec;
    voff[j] = vact[j] ? static_cast<uint32_t>(v) * VB : 0u;
  }
  char* const wbase = static_cast<char*>(a.weights);
  const char* const gbase = static_cast<const char*>(a.grad);
  // gradient row offsets are kept in units of VB bytes so that they fit one 32-bit shuffle
  const uint32_t sb_units = static_cast<uint32_t>(a.stride_b * static_cast<int64_t>(sizeof(T)) / VB);
  const uint32_t st_units = static_cast<uint32_t>(a.stride_t * static_cast<int64_t>(sizeof(T)) / VB);
  // the random stream belongs to the (tile, lane), not to the thread: the result does not depend on
  // which warp came to process a tile
  Philox rng(a.sr_seed, static_cast<uint64_t>(tile) * 32 + lane, a.sr_offset);
  const uint64_t keep = l2_policy_evict_last(), streaming = l2_policy_evict_first();
  const int ngroups = 32 >> lpr_log2;  // lane groups of the warp; the tile's runs are dealt out to them in turn

  // offset (in VB-byte units) of the gradient row of a bag, and 1/L of the bag for mean pooling
  auto grad_units = [&](uint32_t bag, acc_t* scale) -> uint32_t {
    const uint32_t t = fastdiv(bag, a.divB);
    const uint32_t b = bag - t * static_cast<uint32_t>(a.B);
    if (MEAN) *scale = acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag));
    return b * sb_units + t * st_units;
  };
  auto grad_ptr = [&](uint32_t units, int j) -> const char* {
    return gbase + static_cast<uint64_t>(units) * static_cast<uint32_t>(VB) + voff[j];
  };

  Tile cur = load_tile(keys, vals, tile, lane, N);
  while (true) {
    Tile nxt = cur;
    int32_t ticket = 0;  // (requested now, read at the end of the tile)
    if (ntile < ntiles) {
      nxt = load_tile(keys, vals, ntile, lane, N);
      if (ticketed && lane == 0) ticket = atomicAdd(a.tile_ticket, 1);
    }

    // ---- per entry, all lanes at once
    const int p0 = tile << 5;
    const int nvalid = min(32, N - p0);
    const bool valid = lane < nvalid;
    uint32_t prev = __shfl_up_sync(kFullMask, cur.key, 1);
    if (lane == 0) prev = cur.halo;
    const bool is_start = valid && (p0 + lane == 0 || cur.key != prev);
    const unsigned smask = __ballot_sync(kFullMask, is_start);
    const unsigned above = (lane >= 31) ? 0u : (smask & ~((2u << lane) - 1u));
    const int my_end = above ? (__ffs(above) - 1) : nvalid;  // first lane behind the run starting here
    const int my_len = my_end - lane;
    const uint32_t after = __shfl_sync(kFullMask, cur.halo, 31);
    const bool crosses = is_start && my_end == 32 && p0 + 32 < N && after == cur.key;
    const unsigned cmask = __ballot_sync(kFullMask, crosses);  // at most one bit
    // invalid lanes describe entry 0 of the tile so that anything read through them is valid memory
    const uint32_t key0 = __shfl_sync(kFullMask, cur.key, 0);
    const int32_t val0 = __shfl_sync(kFullMask, cur.val, 0);
    const uint32_t my_row = key_to_row(a.table_offsets, a.idx_bits, valid ? cur.key : key0);
    acc_t my_scale = 1;
    const uint32_t my_goff = grad_units(static_cast<uint32_t>(valid ? cur.val : val0), &my_scale);
    float my_state = 0.f;  // approximate Adagrad: the row's state after this entry's lookup
    if (APPROX) {
      float x = valid ? __ldg(a.bag_g2 + cur.val) : 0.f;
      // inclusive scan inside runs: add the value `o` lanes back while that lane belongs to the same run
      const unsigned upto = smask & ((lane >= 31) ? kFullMask : ((2u << lane) - 1u));
      const int dist = upto ? lane - (31 - __clz(upto)) : 32;  // lanes since the run's start (32: it started in an earlier tile)
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(kFullMask, x, o);
        if (dist < 32 && o <= dist) x += y;
      }
      my_state = a.state[my_row] + x;
      my_scale = static_cast<acc_t>(approx_step(a, my_state));
    }
    // the k-th run of the tile goes to lane group k mod ngroups: every group gets its share whatever
    // the lengths of the runs are (runs dealt out by the lanes they start in would leave a group with
    // one long run idle while its neighbour works through eight short ones)
    unsigned mine = smask;
    if (ngroups > 1) {
      const int turn = __popc(smask & ((1u << lane) - 1u)) & (ngroups - 1);
      for (int g = 0; g < ngroups; ++g) {
        const unsigned m = __ballot_sync(kFullMask, is_start && turn == g);
        if (g == slot) mine = m;
      }
    }
    const int rounds = (__popc(smask) + ngroups - 1) >> (5 - lpr_log2);

    // ---- per run
    for (int k = 0; k < rounds; k += SEGS) {
      bool has[SEGS];
      int first[SEGS], len[SEGS], tail_lo[SEGS], tail_hi[SEGS];
      uint32_t wid[SEGS];
      Raw<VB> wraw[SEGS][VPL], g0[SEGS][VPL], g1[SEGS][VPL];
      acc_t s0[SEGS], s1[SEGS];
      float st_old[SEGS];
      float st_run[SEGS];  // approximate Adagrad: state after the run's last lookup seen so far

      // phase 1: pick the runs and request their rows (an idle group re-reads lane 0's rows)
#pragma unroll
      for (int q = 0; q < SEGS; ++q) {
        has[q] = mine != 0u;
        const int i = has[q] ? (__ffs(mine) - 1) : 0;
        mine &= mine - 1u;  // (0 stays 0)
        first[q] = i;
        wid[q] = __shfl_sync(kFullMask, my_row, i);
        len[q] = __shfl_sync(kFullMask, my_len, i);
        if (!has[q]) len[q] = 0;
        const uint32_t off0 = __shfl_sync(kFullMask, my_goff, i);
        const uint32_t off1 = __shfl_sync(kFullMask, my_goff, (i + 1) & 31);
        s0[q] = s1[q] = 1;
        if (SCALED) {
          s0[q] = __shfl_sync(kFullMask, my_scale, i);
          s1[q] = __shfl_sync(kFullMask, my_scale, (i + 1) & 31);
        }
        if (APPROX) st_run[q] = __shfl_sync(kFullMask, my_state, (i + len[q] - 1) & 31);
        tail_lo[q] = tail_hi[q] = 0;
        if (has[q] && ((cmask >> i) & 1u)) {  // the run continues behind the tile (rare)
          tail_lo[q] = p0 + 32;
          tail_hi[q] = run_end(keys, tail_lo[q] + 1, N, after);
          if (len[q] + (tail_hi[q] - tail_lo[q]) > a.long_threshold) {
            if (sub == 0) enqueue_long_run(a, p0 + i, tail_hi[q]);
            has[q] = false;
            len[q] = 0;
            tail_hi[q] = tail_lo[q];
          }
        }
        const char* wrow = wbase + static_cast<uint64_t>(wid[q]) * row_bytes;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          wraw[q][j] = ld_rw_hint<VB>(wrow + voff[j], streaming);
          g0[q][j] = ld_stream_hint<VB>(grad_ptr(off0, j), keep);
          g1[q][j] = raw_zero<VB>();
          if (len[q] > 1) g1[q][j] = ld_stream_hint<VB>(grad_ptr(off1, j), keep);
        }
        if (OPT == kExactAdagrad) st_old[q] = a.state[wid[q]];
      }

      // phase 2: finish the runs one by one
#pragma unroll
      for (int q = 0; q < SEGS; ++q) {
        acc_t acc[VPL][NE];
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          unpack<T, VB>(g0[q][j], acc[j]);
          if (SCALED) {
#pragma unroll
            for (int kk = 0; kk < NE; ++kk) acc[j][kk] *= s0[q];
          }
        }
        const int maxlen = __reduce_max_sync(kFullMask, len[q]);
        if (maxlen > 1) {
#pragma unroll
          for (int j = 0; j < VPL; ++j) add_grad<T, VB, SCALED>(g1[q][j], s1[q], acc[j]);
          for (int e = 2; e < maxlen; e += 2) {  // warp-uniform; runs of 3+ entries inside the tile
            const uint32_t o0 = __shfl_sync(kFullMask, my_goff, (first[q] + e) & 31);
            const uint32_t o1 = __shfl_sync(kFullMask, my_goff, (first[q] + e + 1) & 31);
            acc_t t0 = 1, t1 = 1;
            if (SCALED) {
              t0 = __shfl_sync(kFullMask, my_scale, (first[q] + e) & 31);
              t1 = __shfl_sync(kFullMask, my_scale, (first[q] + e + 1) & 31);
            }
            Raw<VB> r0[VPL], r1[VPL];
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
              r0[j] = raw_zero<VB>();
              r1[j] = raw_zero<VB>();
              if (e < len[q]) r0[j] = ld_stream_hint<VB>(grad_ptr(o0, j), keep);
              if (e + 1 < len[q]) r1[j] = ld_stream_hint<VB>(grad_ptr(o1, j), keep);
            }
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
              add_grad<T, VB, SCALED>(r0[j], t0, acc[j]);
              add_grad<T, VB, SCALED>(r1[j], t1, acc[j]);
            }
          }
        }
        for (int p = tail_lo[q]; p < tail_hi[q]; p += 2) {  // group-uniform; entries behind the tile
          acc_t t0 = 1, t1 = 1;
          const bool two = p + 1 < tail_hi[q];
          const uint32_t bag0 = static_cast<uint32_t>(__ldg(vals + p));
          const uint32_t bag1 = two ? static_cast<uint32_t>(__ldg(vals + p + 1)) : bag0;
          const uint32_t o0 = grad_units(bag0, &t0);
          const uint32_t o1 = two ? grad_units(bag1, &t1) : o0;
          if (APPROX) {  // the state keeps running through the entries behind the tile
            st_run[q] += __ldg(a.bag_g2 + bag0);
            t0 = static_cast<acc_t>(approx_step(a, st_run[q]));
            if (two) {
              st_run[q] += __ldg(a.bag_g2 + bag1);
              t1 = static_cast<acc_t>(approx_step(a, st_run[q]));
            }
          }
          Raw<VB> r0[VPL], r1[VPL];
#pragma unroll
          for (int j = 0; j < VPL; ++j) {
            r0[j] = ld_stream_hint<VB>(grad_ptr(o0, j), keep);
            r1[j] = raw_zero<VB>();
            if (two) r1[j] = ld_stream_hint<VB>(grad_ptr(o1, j), keep);
          }
#pragma unroll
          for (int j = 0; j < VPL; ++j) {
            add_grad<T, VB, SCALED>(r0[j], t0, acc[j]);
            add_grad<T, VB, SCALED>(r1[j], t1, acc[j]);
          }
        }
        acc_t mult = static_cast<acc_t>(a.lr);
        if (APPROX) {  // the step sizes are already inside the sum
          mult = 1;
          if (has[q] && sub == 0) a.state[wid[q]] = st_run[q];
        }
        if (OPT == kExactAdagrad) {
          acc_t part = 0;
#pragma unroll
          for (int j = 0; j < VPL; ++j) {
            if (vact[j]) part += sq_sum(acc[j], NE);
          }
          const acc_t g2 = group_sum(part, lpr_log2);
          const float st = st_old[q] + static_cast<float>(g2);
          if (has[q] && sub == 0) a.state[wid[q]] = st;
          mult = static_cast<acc_t>(a.lr * (1.0f / (sqrtf(st) + a.eps)));
        }
        char* wrow = wbase + static_cast<uint64_t>(wid[q]) * row_bytes;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          if (has[q] && vact[j]) apply_update<T, VB, SR>(wrow + voff[j], wraw[q][j], acc[j], mult, &rng, streaming);
        }
      }
    }

    tile = ntile;
    if (tile >= ntiles) break;
    ntile = ticketed ? wstride + __shfl_sync(kFullMask, ticket, 0) : tile + wstride;
    cur = nxt;
    if (SR) rng = Philox(a.sr_seed, static_cast<uint64_t>(tile) * 32 + lane, a.sr_offset);
  }
}

// Rows wider than 32 vectors: one run per lane group at a time, the row is walked in chunks of 32
// vectors (twice for rowwise Adagrad, whose step size needs the whole row's gradient norm first).
template <typename T, int VB, int OPT, bool MEAN, bool SR>
__global__ void __launch_bounds__(kBwdThreads) run_kernel_wide(const BwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int lpr_log2 = a.lpr1_log2;
  const int gpw = 32 >> lpr_log2;  // lane groups (= concurrent runs) per warp
  const int sub = lane & ((1 << lpr_log2) - 1);
  const int slot = lane >> lpr_log2;
  const int N = a.N;
  const int64_t ntiles = (static_cast<int64_t>(N) + 31) >> 5;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  int64_t tile = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tile >= ntiles) return;
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  const uint32_t* __restrict__ keys = a.keys;
  const int32_t* __restrict__ vals = a.vals;
  Philox rng(a.sr_seed, static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x, a.sr_offset);

  const uint64_t keep = l2_policy_evict_last(), streaming = l2_policy_evict_first();
  // A tile's registers: key/val of entry p0+lane, and a halo word: lane 0 holds the key before the
  // tile, lane 31 the key after it.
  auto load_tile = [&](int64_t tl, uint32_t& key, int32_t& val, uint32_t& halo) {
    const int64_t p = (tl << 5) + lane;
    key = 0xffffffffu;
    val = 0;
    halo = 0xffffffffu;
    if (p < N) {
      key = __ldg(keys + p);
      val = __ldg(vals + p);
    }
    if (lane == 0 && p > 0) halo = __ldg(keys + p - 1);
    if (lane == 31 && p + 1 < N) halo = __ldg(keys + p + 1);
  };

  uint32_t key, halo;
  int32_t val;
  load_tile(tile, key, val, halo);

  while (true) {
    const int64_t ntile = tile + wstride;
    uint32_t nkey = 0, nhalo = 0;
    int32_t nval = 0;
    if (ntile < ntiles) load_tile(ntile, nkey, nval, nhalo);

    const int p0 = static_cast<int>(tile << 5);
    const int nvalid = min(32, N - p0);
    uint32_t prev = __shfl_up_sync(kFullMask, key, 1);
    if (lane == 0) prev = halo;
    const bool is_start = lane < nvalid && (p0 + lane == 0 || key != prev);
    const unsigned smask = __ballot_sync(kFullMask, is_start);
    const int nstarts = __popc(smask);
    const uint32_t after = __shfl_sync(kFullMask, halo, 31);  // key following the tile (if any)
    const bool more_after = p0 + 32 < N;

    for (int k = 0; k < nstarts; k += gpw) {
      const int n = k + slot;
      bool has = n < nstarts;
      const int i = has ? static_cast<int>(__fns(smask, 0, n + 1)) : 0;
      const unsigned rest = (i >= 31) ? 0u : (smask & ~((2u << i) - 1u));
      const int j = rest ? (__ffs(rest) - 1) : nvalid;
      int len = has ? (j - i) : 0;
      const uint32_t row = __shfl_sync(kFullMask, key, i);
      // does the run continue behind the tile?
      int tail_lo = 0, tail_hi = 0;
      if (has && j == 32 && more_after && after == row) {
        tail_lo = p0 + 32;
        tail_hi = run_end(keys, tail_lo + 1, N, row);
        if (len + (tail_hi - tail_lo) > a.long_threshold) {
          if (sub == 0) enqueue_long_run(a, p0 + i, tail_hi);
          has = false;
          len = 0;
          tail_hi = tail_lo;
        }
      }
      const int maxlen = __reduce_max_sync(kFullMask, len);
      const uint32_t wrow_id = has ? key_to_row(a.table_offsets, a.idx_bits, row) : 0u;
      char* wrow = static_cast<char*>(a.weights) + static_cast<int64_t>(wrow_id) * row_bytes;

      // sums vector v of the run's gradient rows into acc (tile part with shuffled bag ids, then the tail)
      auto accumulate = [&](int v, bool vact, acc_t* acc) {
        for (int e = 0; e < maxlen; e += 2) {
          const uint32_t bag0 = static_cast<uint32_t>(__shfl_sync(kFullMask, val, (i + e) & 31));
          const uint32_t bag1 = static_cast<uint32_t>(__shfl_sync(kFullMask, val, (i + e + 1) & 31));
          Raw<VB> r0 = raw_zero<VB>(), r1 = raw_zero<VB>();
          acc_t s0 = 1, s1 = 1;
          if (e < len && vact) r0 = load_grad<T, VB, MEAN>(a, bag0, v, keep, &s0);
          if (e + 1 < len && vact) r1 = load_grad<T, VB, MEAN>(a, bag1, v, keep, &s1);
          add_grad<T, VB, MEAN>(r0, s0, acc);
          add_grad<T, VB, MEAN>(r1, s1, acc);
        }
        for (int q = tail_lo; q < tail_hi; ++q) {  // group-uniform, rare
          acc_t s0 = 1;
          Raw<VB> r0 = raw_zero<VB>();
          if (vact) r0 = load_grad<T, VB, MEAN>(a, static_cast<uint32_t>(__ldg(vals + q)), v, keep, &s0);
          add_grad<T, VB, MEAN>(r0, s0, acc);
        }
      };

      acc_t g2 = 0;
      if (OPT == kExactAdagrad && a.nchunks > 1) {
        for (int c = 0; c < a.nchunks; ++c) {
          const int v = (c << 5) + sub;
          acc_t acc[NE];
#pragma unroll
          for (int kk = 0; kk < NE; ++kk) acc[kk] = 0;
          accumulate(v, v < a.nvec, acc);
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
        for (int kk = 0; kk < NE; ++kk) acc[kk] = 0;
        accumulate(v, vact, acc);
        if (OPT == kExactAdagrad && c == 0) {
          if (a.nchunks == 1) g2 = group_sum(sq_sum(acc, NE), lpr_log2);
          const float st = (has ? a.state[wrow_id] : 0.f) + static_cast<float>(g2);
          __syncwarp();
          if (has && sub == 0) a.state[wrow_id] = st;
          mult = static_cast<acc_t>(a.lr * (1.0f / (sqrtf(st) + a.eps)));
        }
        if (has && vact) apply_update<T, VB, SR>(wrow + static_cast<int64_t>(v) * VB, wraw, acc, mult, &rng, streaming);
      }
    }

    tile = ntile;
    if (tile >= ntiles) break;
    key = nkey;
    val = nval;
    halo = nhalo;
  }
}

// Queued long runs.  A run shorter than two parts (a.split_len entries each) gets one CTA, which sums
// it and applies the update.  A longer run -- a hot row with thousands of lookups -- would make one
// CTA the critical path of the whole kernel, so the lane group that queued it also cut it into parts
// (part_list): every part is summed by whichever CTA picks it and left as an fp32 partial sum,
// and the CTA that finishes a run's LAST outstanding part (a ticket per run) adds the partial sums in
// part order and applies the update.  The order of every summation is fixed by the sorted order and
// the part boundaries, never by scheduling.
template <typename T, int VB, int OPT, bool MEAN, bool SR>
__global__ void __launch_bounds__(kBwdThreads) long_run_kernel(const BwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  constexpr bool APPROX = OPT == kApproxAdagrad;
  constexpr bool SCALED = MEAN || APPROX;
  __shared__ float scan_tot[kBwdThreads / 32];  // approximate Adagrad: block scan of the bags' g2
  __shared__ float carry;                       // ... and the state reached at the end of the previous block of entries
  __shared__ acc_t part[kBwdThreads * NE];
  __shared__ int64_t entry_off[kBwdThreads];   // byte offset of the gradient row of an entry
  __shared__ acc_t entry_scale[kBwdThreads];   // 1/L of its bag (mean pooling)
  __shared__ int ticket;                       // parts of a split run finished before this CTA's
  const int lane = threadIdx.x & 31;
  const int lpr_log2 = a.lpr1_log2;
  const int lpr = 1 << lpr_log2;
  const int sub = lane & (lpr - 1);
  const int gid = threadIdx.x >> lpr_log2;
  const int groups = blockDim.x >> lpr_log2;
  const int nlong = *a.long_count;
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  Philox rng(a.sr_seed, (1ull << 40) + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x, a.sr_offset);
  const uint64_t keep = l2_policy_evict_last(), streaming = l2_policy_evict_first();

  // Sums chunk c of the gradient rows of sorted entries [s, s + len):
  // Folds the groups' partial sums for chunk c in group order; every thread of warp 0 ends with the
  // total of its own `sub`.  The run is taken 256 entries at a time: every thread first turns one
  // entry's bag id into the offset of its gradient row (and 1/L for mean pooling) and leaves it in
  // shared memory, then group g sums entries g, g + groups, ... with eight row loads in flight and
  // no load depending on another.
  auto reduce_range = [&](int c, int s, int len, float st_first, acc_t* total) {
    const int v = (c << 5) + sub;
    const bool vact = v < a.nvec;
    acc_t acc[NE];
#pragma unroll
    for (int k = 0; k < NE; ++k) acc[k] = 0;
    if (APPROX && threadIdx.x == 0) carry = st_first;
    for (int base = 0; base < len; base += kBwdThreads) {
      const int m = min(kBwdThreads, len - base);
      __syncthreads();  // the previous block of entries has been consumed
      float g2 = 0.f;
      if (static_cast<int>(threadIdx.x) < m) {
        const uint32_t bag = static_cast<uint32_t>(__ldg(a.vals + s + base + threadIdx.x));
        if (APPROX) g2 = __ldg(a.bag_g2 + bag);
        const uint32_t t = fastdiv(bag, a.divB);
        const uint32_t b = bag - t * static_cast<uint32_t>(a.B);
        entry_off[threadIdx.x] = (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                                 static_cast<int64_t>(sizeof(T));
        if (MEAN)
          entry_scale[threadIdx.x] =
              acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag));
      }
      if (APPROX) {
        // state after every entry = state so far + inclusive prefix sum of g2 over the block, in a
        // fixed order: shuffles inside a warp, then the totals of the warps in front
        float incl = g2;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float up = __shfl_up_sync(kFullMask, incl, o);
          if (lane >= o) incl += up;
        }
        if (lane == 31) scan_tot[threadIdx.x >> 5] = incl;
        __syncthreads();
        float before = carry;
        for (int w2 = 0; w2 < static_cast<int>(threadIdx.x >> 5); ++w2) before += scan_tot[w2];
        const float st = before + incl;
        entry_scale[threadIdx.x] = static_cast<acc_t>(approx_step(a, st));
        __syncthreads();  // everyone has read `carry`
        if (threadIdx.x == blockDim.x - 1) carry = st;
      }
      __syncthreads();
      for (int i = gid; i < m; i += groups * 8) {
        Raw<VB> r[8];
        acc_t sc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int iu = i + u * groups;
          r[u] = raw_zero<VB>();
          sc[u] = 1;
          if (iu < m && vact) {
            r[u] = ld_stream_hint<VB>(static_cast<const char*>(a.grad) + entry_off[iu] + static_cast<int64_t>(v) * VB,
                                      keep);
            if (SCALED) sc[u] = entry_scale[iu];
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) add_grad<T, VB, SCALED>(r[u], sc[u], acc);
      }
    }
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

  // Applies the optimizer to `row` given a way to obtain the summed gradient of chunk c of the run
  // (every thread of warp 0 receives the total of its own `sub`); all threads of the CTA call it.
  auto apply_run = [&](uint32_t row, auto&& chunk_total) {
    char* wrow = static_cast<char*>(a.weights) + static_cast<int64_t>(row) * row_bytes;
    acc_t g2 = 0;
    if (OPT == kExactAdagrad && a.nchunks > 1) {
      for (int c = 0; c < a.nchunks; ++c) {
        acc_t tot[NE];
        chunk_total(c, tot);
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
      chunk_total(c, tot);
      if (APPROX) {  // the step sizes are inside the sum; `carry` holds the state after the whole run
        mult = 1;
        if (c == 0 && threadIdx.x == 0) a.state[row] = carry;
      }
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
          apply_update<T, VB, SR>(wrow + static_cast<int64_t>(v) * VB, wraw, tot, mult, &rng, streaming);
        }
      }
    }
  };

  const bool splitting = a.split_len > 0;
  for (int li = blockIdx.x; li < nlong; li += gridDim.x) {
    const int2 run = a.long_list[li];
    const int s = run.x, len = run.y - run.x;
    if (splitting && len >= 2 * a.split_len) continue;  // cut into parts: see below
    const uint32_t row = key_to_row(a.table_offsets, a.idx_bits, __ldg(a.keys + s));
    const float st_first = APPROX ? a.state[row] : 0.f;  // read by every thread before thread 0 overwrites it
    apply_run(row, [&](int c, acc_t* total) { reduce_range(c, s, len, st_first, total); });
  }
  if (!splitting) return;

  // parts of split runs
  const int nparts_total = min(*a.part_count, a.max_parts);
  for (int p = blockIdx.x; p < nparts_total; p += gridDim.x) {
    const int4 pm = a.part_list[p];  // {first entry, end entry, list index of the run's first part, parts of the run}
    float* mine = a.part_sums + static_cast<int64_t>(p) * a.D;
    for (int c = 0; c < a.nchunks; ++c) {
      acc_t tot[NE];
      reduce_range(c, pm.x, pm.y - pm.x, 0.f, tot);
      const int v = (c << 5) + sub;
      if (gid == 0 && v < a.nvec) {
#pragma unroll
        for (int k = 0; k < NE; ++k) mine[v * NE + k] = static_cast<float>(tot[k]);
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(a.part_tickets + pm.z, 1);
    __syncthreads();
    if (ticket != pm.w - 1) continue;  // another CTA will find all parts done
    __threadfence();
    const uint32_t row = key_to_row(a.table_offsets, a.idx_bits, __ldg(a.keys + pm.x));
    apply_run(row, [&](int c, acc_t* total) {
      const int v = (c << 5) + sub;
#pragma unroll
      for (int k = 0; k < NE; ++k) total[k] = 0;
      if (threadIdx.x < 32 && v < a.nvec) {
        for (int part_i = 0; part_i < pm.w; ++part_i) {  // part order: fixed
          const float* ps = a.part_sums + static_cast<int64_t>(pm.z + part_i) * a.D + v * NE;
#pragma unroll
          for (int k = 0; k < NE; ++k) total[k] += static_cast<acc_t>(__ldcg(ps + k));
        }
      }
    });
  }
}

// The run_kernel instance for (SEGS, VPL); only 16-byte-vector fp16/fp32 rows get VPL > 1.
template <typename T, int VB, int OPT, bool MEAN, bool SR>
void (*pick_run_kernel(int segs, int vpl))(const BwdArgs) {
  if constexpr (VB == 16 && sizeof(T) <= 4) {
    if (vpl == 4) return segs == 2 ? run_kernel<T, VB, OPT, MEAN, SR, 2, 4> : run_kernel<T, VB, OPT, MEAN, SR, 1, 4>;
    if (vpl == 2) return segs == 2 ? run_kernel<T, VB, OPT, MEAN, SR, 2, 2> : run_kernel<T, VB, OPT, MEAN, SR, 1, 2>;
  }
  return segs == 2 ? run_kernel<T, VB, OPT, MEAN, SR, 2, 1> : run_kernel<T, VB, OPT, MEAN, SR, 1, 1>;
}

template <typename T, int VB, int OPT, bool MEAN, bool SR>
int launch_runs(const BwdArgs& a, cudaStream_t stream) {
  int threads = tuning(kTuneBwdThreads);
  if (threads <= 0) threads = kBwdThreads;
  if (threads > kBwdThreads || threads % 32 != 0)
    return fail(TBE_ERR_INVALID_ARGUMENT, "bwd_threads must be a multiple of 32 <= %d", kBwdThreads);
  void (*kernel)(const BwdArgs) = nullptr;
  BwdArgs args = a;
  // vectors per lane: the most that divides the row, unless a knob says otherwise
  // (two per lane measured best on B200 for 256- and 512-byte rows; four costs too many registers)
  const int vpl_max = (VB != 16 || sizeof(T) == 8) ? 1 : (a.nvec % 4 == 0) ? 4 : (a.nvec % 2 == 0) ? 2 : 1;
  int vpl = vpl_max < 2 ? vpl_max : 2;
  const int knob = tuning(kTuneBwdVpl);
  if ((knob == 1 || knob == 2 || knob == 4) && knob <= vpl_max) vpl = knob;
  const int lanes_needed = (a.nvec + vpl - 1) / vpl;
  if (lanes_needed > 32) {
    if (OPT == kApproxAdagrad) return fail(TBE_ERR_UNSUPPORTED, "rows this wide take the per-run approximate Adagrad path");
    kernel = run_kernel_wide<T, VB, OPT, MEAN, SR>;
  } else {
    int l = 0;
    while ((1 << l) < lanes_needed) ++l;
    args.lpr_log2 = l;
    const int segs = tuning(kTuneBwdUnroll) > 0 ? tuning(kTuneBwdUnroll) : (vpl == 1 ? 2 : 1);
    if (segs != 1 && segs != 2) return fail(TBE_ERR_INVALID_ARGUMENT, "bwd_unroll must be 1 or 2");
    kernel = pick_run_kernel<T, VB, OPT, MEAN, SR>(segs, vpl);
  }
  int per_sm = 0;
  TBE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
  if (per_sm < 1) per_sm = 1;
  if (tuning(kTuneBwdBlocksPerSM) > 0 && tuning(kTuneBwdBlocksPerSM) < per_sm) per_sm = tuning(kTuneBwdBlocksPerSM);
  const int64_t ntiles = (static_cast<int64_t>(a.N) + 31) / 32;
  const int wpb = threads / 32;
  int64_t blocks = (ntiles + wpb - 1) / wpb;
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  if (blocks > resident) blocks = resident;
  if (blocks < 1) blocks = 1;
  {
    KernelTimer timer("run_kernel", stream);
    kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(args);
  }
  TBE_CHECK_LAUNCH("run_kernel");
  {
    KernelTimer timer("long_run_kernel", stream);
    // one CTA per queued run, as many CTAs as fit: the gradient rows of a long run come from L2 and a
    // CTA keeps only a few KB of them in flight
    int long_per_sm = 0;
    TBE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&long_per_sm, long_run_kernel<T, VB, OPT, MEAN, SR>,
                                                               kBwdThreads, 0));
    if (long_per_sm < 1) long_per_sm = 1;
    long_run_kernel<T, VB, OPT, MEAN, SR><<<device_sm_count() * long_per_sm, kBwdThreads, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("long_run_kernel");
  return TBE_OK;
}

template <typename T, int VB, int OPT>
int dispatch_flags(const BwdArgs& a, bool mean, bool sr, cudaStream_t stream) {
  if constexpr (OPT == kApproxAdagrad) {  // sum pooling only
    if (mean) return fail(TBE_ERR_UNSUPPORTED, "approximate rowwise Adagrad supports sum pooling only");
    if (sr) return launch_runs<T, VB, OPT, false, true>(a, stream);
    return launch_runs<T, VB, OPT, false, false>(a, stream);
  }
  if (mean) {
    if (sr) return launch_runs<T, VB, OPT, true, true>(a, stream);
    return launch_runs<T, VB, OPT, true, false>(a, stream);
  }
  if (sr) return launch_runs<T, VB, OPT, false, true>(a, stream);
  return launch_runs<T, VB, OPT, false, false>(a, stream);
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

// g2[bag] = squared norm of the bag's gradient row (approximate Adagrad).  A warp per bag.
template <typename T, int VB>
__global__ void __launch_bounds__(256) bag_g2_kernel(const BwdArgs a, int64_t nbags, float* __restrict__ g2) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int64_t t = bag / a.B, b = bag - t * a.B;
    const char* g = static_cast<const char*>(a.grad) + (b * a.stride_b + t * a.stride_t) * static_cast<int64_t>(sizeof(T));
    acc_t part = 0;
    for (int v = lane; v < a.nvec; v += 32) {
      acc_t e[NE];
      unpack<T, VB>(ld_stream<VB>(g + static_cast<int64_t>(v) * VB), e);
#pragma unroll
      for (int k = 0; k < NE; ++k) part += e[k] * e[k];
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) part += __shfl_xor_sync(kFullMask, part, m);
    if (lane == 0) g2[bag] = static_cast<float>(part);
  }
}

int launch_bag_g2(const BwdArgs& a, int dtype, int vb, int64_t nbags, float* g2, cudaStream_t stream) {
  int64_t blocks = (nbags + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  const unsigned grid = static_cast<unsigned>(blocks);
  {
    KernelTimer timer("bag_g2_kernel", stream);
    if (dtype == TBE_F16 && vb == 16) bag_g2_kernel<__half, 16><<<grid, 256, 0, stream>>>(a, nbags, g2);
    else if (dtype == TBE_F16) bag_g2_kernel<__half, 8><<<grid, 256, 0, stream>>>(a, nbags, g2);
    else if (dtype == TBE_F32) bag_g2_kernel<float, 16><<<grid, 256, 0, stream>>>(a, nbags, g2);
    else bag_g2_kernel<double, 16><<<grid, 256, 0, stream>>>(a, nbags, g2);
  }
  TBE_CHECK_LAUNCH("bag_g2_kernel");
  return TBE_OK;
}

int exact_backward(int opt, const void* grad, int64_t stride_b, int64_t stride_t, void* weights,
                   const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, float* state,
                   int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, int pooling,
                   float lr, float eps, int sr, uint64_t sr_seed, uint64_t sr_offset, int64_t max_rows_per_table,
                   int plan_ready, void* workspace, int64_t workspace_bytes, void* stream_v) {
  const char* who = opt == kSGD ? "tbe_backward_sgd"
                    : opt == kExactAdagrad ? "tbe_backward_exact_rowwise_adagrad"
                                           : "tbe_backward_approx_rowwise_adagrad";
  TBE_REQUIRE(grad && weights && table_offsets && offsets && (indices || N == 0), "%s: null pointer argument", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  TBE_REQUIRE(D > 0 && D % 4 == 0, "%s: D must be a positive multiple of 4 (got %lld)", who, (long long)D);
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "%s: bad dtype %d", who, dtype);
  TBE_REQUIRE(pooling == TBE_POOL_SUM || pooling == TBE_POOL_MEAN, "%s: bad pooling %d", who, pooling);
  TBE_REQUIRE(opt == kSGD || state != nullptr, "%s: optimizer_state is null", who);
  TBE_REQUIRE(stride_b >= 0 && stride_t >= 0 && stride_b * 8 < (1ll << 32) && stride_t * 8 < (1ll << 32),
              "%s: grad_output strides must be non-negative and below 2^29 elements", who);
  Workspace ws;
  rc = prepare_workspace(who, workspace, workspace_bytes, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  if (N == 0) return TBE_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const KeyLayout layout = key_layout(T, total_rows, max_rows_per_table, false);
  if (!plan_ready) {
    rc = build_plan(table_offsets, indices, offsets, T, B, N, max_rows_per_table, layout, ws, stream);
    if (rc != TBE_OK) return rc;
  }
  TBE_CUDA_TRY(cudaMemsetAsync(ws.counters, 0, 64, stream));

  BwdArgs a{};
  a.grad = grad;
  a.stride_b = stride_b;
  a.stride_t = stride_t;
  a.weights = weights;
  a.state = state;
  a.keys = ws.keys;
  a.vals = ws.vals;
  a.long_list = ws.long_list;
  a.long_count = ws.counters + 1;
  // Tickets keep all warps on neighbouring tiles of the sorted order, i.e. on one table's slice of the
  // pooled gradient at a time; that pays once the gradient no longer sits in L2 as a whole (config 5:
  // 1 GB of gradient, run_kernel 10.7 -> 7.6 ms).  A gradient that fits anyway is a little faster with
  // the fixed stride (no ticket traffic).
  {
    const int mode = tuning(kTuneBwdStride);
    const int64_t grad_bytes = B * T * D * elem_size(dtype);
    const bool tickets = mode == 2 || (mode != 1 && grad_bytes * 3 > device_l2_bytes());
    a.tile_ticket = tickets ? ws.counters + 5 : nullptr;  // cleared with the other counters above
  }
  a.offsets = offsets;
  a.table_offsets = table_offsets;
  a.idx_bits = layout.idx_bits;
  a.divB = make_fastdiv(static_cast<uint32_t>(B));
  a.B = static_cast<int32_t>(B);
  a.D = static_cast<int32_t>(D);
  a.N = static_cast<int32_t>(N);
  const int es = elem_size(dtype);
  // the gradient rows must allow the same vector width as the weight rows
  const bool grad16 =
      reinterpret_cast<uintptr_t>(grad) % 16 == 0 && (stride_b * es) % 16 == 0 && (stride_t * es) % 16 == 0;
  const RowGeom g = make_geom(D, dtype, weights, grad16 ? nullptr : reinterpret_cast<const void*>(uintptr_t(8)));
  TBE_REQUIRE(g.vb == 16 || dtype == TBE_F16, "%s: weights and grad_output rows must be 16-byte aligned", who);
  if (g.vb == 8)
    TBE_REQUIRE(reinterpret_cast<uintptr_t>(grad) % 8 == 0 && (stride_b * es) % 8 == 0 && (stride_t * es) % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(weights) % 8 == 0,
                "%s: weights and grad_output rows must be 8-byte aligned", who);
  a.lpr1_log2 = g.lpr_log2;
  a.nvec = g.nvec;
  a.nchunks = g.nchunks;
  a.long_threshold = tuning(kTuneLongSegment) > 0 ? tuning(kTuneLongSegment) : kDefaultLongSegment;
  a.lr = lr;
  a.eps = eps;
  a.sr_seed = sr_seed;
  a.sr_offset = sr_offset;
  const bool mean = pooling == TBE_POOL_MEAN;
  const bool use_sr = sr != 0 && dtype == TBE_F16;
  // Long runs are cut into parts when the part map and the fp32 partial sums fit the stretch of the
  // workspace that the run-start list and the per-position arrays of other entry points occupy
  // (3 N words, unused here).  The part length doubles until they fit.
  a.split_len = 0;
  if (opt != kApproxAdagrad && dtype != TBE_F64 && tuning(kTuneSplitRuns) != 1) {
    const size_t region = static_cast<size_t>(reinterpret_cast<char*>(ws.hist) - reinterpret_cast<char*>(ws.seg_starts));
    for (int64_t part = kMinSplitPart; part <= (1 << 16); part *= 2) {
      const size_t max_parts = static_cast<size_t>(N / part + 1);
      const size_t list_bytes = align_up(max_parts * sizeof(int4), 256), ticket_bytes = align_up(max_parts * sizeof(int32_t), 256);
      if (list_bytes + ticket_bytes + max_parts * static_cast<size_t>(D) * sizeof(float) > region) continue;
      char* base = reinterpret_cast<char*>(ws.seg_starts);
      a.part_list = reinterpret_cast<int4*>(base);
      a.part_tickets = reinterpret_cast<int32_t*>(base + list_bytes);
      a.part_sums = reinterpret_cast<float*>(base + list_bytes + ticket_bytes);
      a.part_count = ws.counters + 3;  // cleared with the other counters above
      a.split_len = static_cast<int32_t>(part);
      a.max_parts = static_cast<int32_t>(max_parts);
      break;
    }
  }
  if (opt == kSGD) return dispatch_bwd<kSGD>(a, dtype, g.vb, mean, use_sr, stream);
  if (opt == kExactAdagrad) return dispatch_bwd<kExactAdagrad>(a, dtype, g.vb, mean, use_sr, stream);
  // approximate Adagrad: the bags' squared gradient norms go where the run-start list and the
  // per-position arrays of the per-run path would be (3 N words, unused on this path)
  const int64_t nbags = T * B;
  if (nbags > 3 * N) return fail(TBE_ERR_UNSUPPORTED, "%s: more than three bags per lookup", who);
  float* bag_g2 = reinterpret_cast<float*>(ws.seg_starts);
  a.bag_g2 = bag_g2;
  rc = launch_bag_g2(a, dtype, g.vb, nbags, bag_g2, stream);
  if (rc != TBE_OK) return rc;
  return dispatch_bwd<kApproxAdagrad>(a, dtype, g.vb, mean, use_sr, stream);
}

}  // namespace

int approx_backward_sorted(const void* grad, int64_t stride_b, int64_t stride_t, void* weights,
                           const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, float* state,
                           int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, float lr,
                           float eps, int sr, uint64_t sr_seed, uint64_t sr_offset, int64_t max_rows_per_table,
                           void* workspace, int64_t workspace_bytes, void* stream) {
  // rows too wide for the lane-group kernel (more than 32 lanes of up to two vectors) keep the per-run path
  const int64_t row_bytes = D * elem_size(dtype);
  const int64_t nvec = row_bytes % 16 == 0 ? row_bytes / 16 : row_bytes / 8;
  const int64_t vpl = (row_bytes % 16 == 0 && nvec % 2 == 0) ? 2 : 1;
  if ((nvec + vpl - 1) / vpl > 32)
    return fail(TBE_ERR_UNSUPPORTED, "rows this wide take the per-run approximate Adagrad path");
  return exact_backward(kApproxAdagrad, grad, stride_b, stride_t, weights, table_offsets, indices, offsets, state, T, B,
                        D, N, total_rows, dtype, TBE_POOL_SUM, lr, eps, sr, sr_seed, sr_offset, max_rows_per_table,
                        /*plan_ready=*/0, workspace, workspace_bytes, stream);
}

}  // namespace tbe

extern "C" int64_t tbe_backward_workspace_bytes(int64_t N, int64_t total_rows) {
  if (N < 0 || total_rows <= 0) return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_backward_workspace_bytes: bad sizes");
  tbe::Workspace ws;
  const int rc = tbe::carve(nullptr, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  return static_cast<int64_t>(ws.total);
}

extern "C" int tbe_backward_plan(const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets,
                                 int64_t T, int64_t B, int64_t N, int64_t total_rows,
                                 int64_t max_rows_per_table, void* workspace, int64_t workspace_bytes,
                                 void* stream) {
  using namespace tbe;
  const char* who = "tbe_backward_plan";
  TBE_REQUIRE(table_offsets && offsets && (indices || N == 0), "%s: null pointer argument", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  Workspace ws;
  rc = prepare_workspace(who, workspace, workspace_bytes, N, total_rows, &ws);
  if (rc != TBE_OK || N == 0) return rc;
  return build_plan(table_offsets, indices, offsets, T, B, N, max_rows_per_table,
                    key_layout(T, total_rows, max_rows_per_table, false), ws,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int tbe_backward_sgd(const void* grad_output, int64_t stride_b, int64_t stride_t, void* weights,
                                const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets,
                                int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype,
                                int pooling, float lr, int64_t max_rows_per_table, int plan_ready, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  return tbe::exact_backward(tbe::kSGD, grad_output, stride_b, stride_t, weights, table_offsets, indices, offsets,
                             nullptr, T, B, D, N, total_rows, dtype, pooling, lr, 0.f, 0, 0, 0, max_rows_per_table,
                             plan_ready, workspace, workspace_bytes, stream);
}

extern "C" int tbe_backward_exact_rowwise_adagrad(const void* grad_output, int64_t stride_b, int64_t stride_t,
                                                  void* weights, const int32_t* table_offsets,
                                                  const int32_t* indices, const int32_t* offsets,
                                                  float* optimizer_state, int64_t T, int64_t B, int64_t D,
                                                  int64_t N, int64_t total_rows, int dtype, int pooling, float lr,
                                                  float eps, int stochastic_rounding, uint64_t sr_seed,
                                                  uint64_t sr_offset, int64_t max_rows_per_table, int plan_ready,
                                                  void* workspace, int64_t workspace_bytes, void* stream) {
  return tbe::exact_backward(tbe::kExactAdagrad, grad_output, stride_b, stride_t, weights, table_offsets, indices,
                             offsets, optimizer_state, T, B, D, N, total_rows, dtype, pooling, lr, eps,
                             stochastic_rounding, sr_seed, sr_offset, max_rows_per_table, plan_ready, workspace,
                             workspace_bytes, stream);
}

extern "C" int tbe_sort_segments(const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets,
                                 int64_t T, int64_t B, int64_t N, int64_t total_rows,
                                 int64_t max_rows_per_table, int32_t* sorted_rows, int32_t* sorted_bags,
                                 int32_t* segment_starts, int32_t* num_segments, void* workspace,
                                 int64_t workspace_bytes, void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_sort_segments";
  TBE_REQUIRE(table_offsets && offsets && (indices || N == 0) && sorted_rows && sorted_bags && segment_starts &&
                  num_segments,
              "%s: null pointer argument", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  Workspace ws;
  rc = prepare_workspace(who, workspace, workspace_bytes, N, total_rows, &ws);
  if (rc != TBE_OK) return rc;
  if (N == 0) {
    TBE_CUDA_TRY(cudaMemsetAsync(num_segments, 0, 4, stream));
    return TBE_OK;
  }
  const KeyLayout layout = key_layout(T, total_rows, max_rows_per_table, true);
  rc = build_plan(table_offsets, indices, offsets, T, B, N, max_rows_per_table, layout, ws, stream);
  if (rc != TBE_OK) return rc;
  rc = select_run_starts(ws, N, stream);
  if (rc != TBE_OK) return rc;
  if (layout.idx_bits > 0) {
    keys_to_rows_kernel<<<static_cast<unsigned>((N + 255) / 256), 256, 0, stream>>>(
        table_offsets, layout.idx_bits, ws.keys, sorted_rows, N);
    TBE_CHECK_LAUNCH("keys_to_rows_kernel");
  } else {
    TBE_CUDA_TRY(cudaMemcpyAsync(sorted_rows, ws.keys, N * 4, cudaMemcpyDeviceToDevice, stream));
  }
  TBE_CUDA_TRY(cudaMemcpyAsync(sorted_bags, ws.vals, N * 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(segment_starts, ws.seg_starts, N * 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(num_segments, ws.counters, 4, cudaMemcpyDeviceToDevice, stream));
  return TBE_OK;
}
