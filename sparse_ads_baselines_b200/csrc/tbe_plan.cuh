// Host-side pieces shared by the backward kernels: the layout of the caller's workspace, the sort
// key layout, and thin wrappers around the two CUB calls (defined once, in tbe_backward.cu, so that
// CUB is instantiated in a single translation unit).
#pragma once

#include "tbe_common.cuh"

namespace tbe {

struct Workspace {
  uint32_t* keys_in;
  uint32_t* keys;       // sorted keys
  int32_t* vals_in;
  int32_t* vals;        // value of every sorted entry: bag id (exact/SGD) or index position (approx)
  int32_t* seg_starts;  // N + 1: first sorted position of every run (approx backward, tbe_sort_segments)
  int2* long_list;      // {first sorted position, end position} of queued runs; N/32 + 2 entries
  int32_t* entry_bag;   // N: bag id of every index position (approx backward)
  float* entry_g2;      // N: squared gradient norm applied by every index position (approx backward)
  int32_t* counters;    // [0] = number of runs, [1] = queued long runs, [8] = queued oversize buckets
  int32_t* hist;        // bucket sort: per (table, slice) bucket histograms, hist_cap entries
  int32_t* bucket_start;  // bucket sort: first sorted position of every (table, bucket), hist_cap entries
  int2* oversize;       // bucket sort: {first, end} position of buckets too large for shared memory, queue_cap entries
  int64_t hist_cap, queue_cap;
  void* cub_temp;
  size_t cub_bytes;
  size_t total;
};

// How the sort keys are formed.  Lookups arrive grouped by table, and a stable sort on the index
// bits alone already brings equal (table, index) pairs together (ordered by index, then table), so
// with composite keys only idx_bits need sorting instead of log2(total_rows).
struct KeyLayout {
  int idx_bits;   // 0: keys are linear row ids; > 0: keys are (table << idx_bits | index)
  int sort_bits;  // bits the radix sort looks at
};

KeyLayout key_layout(int64_t T, int64_t total_rows, int64_t max_rows_per_table, bool full_order);

// Largest bucket the two-level sort finishes in shared memory.
constexpr int kBucketSortCapacity = 2048;
// Most pairs of a bucket that may share one of its level-2 counters (a hot row); a bucket beyond
// either limit is queued for the oversize path, so the queue needs a slot per kBucketSortMaxGroup pairs.
constexpr int kBucketSortMaxGroup = 256;

// Two-level sort geometry: bucket = index >> shift, nb buckets and `slices` position ranges per table.
struct BucketGeometry {
  int shift, nb, slices;
};
// False when the batch does not suit the two-level sort (no composite keys, tables too long,
// scratch too small, or switched off): the caller then uses linearize + sort_pairs.
bool bucket_geometry(int64_t T, int64_t N, int64_t max_rows_per_table, KeyLayout layout, const Workspace& ws,
                     BucketGeometry* g);
// indices/offsets -> ws.keys / ws.vals ordered by (table, index, position).
int bucket_sort_plan(const int32_t* indices, const int32_t* offsets, int64_t T, int64_t B, int64_t N,
                     KeyLayout layout, const BucketGeometry& g, Workspace& ws, cudaStream_t stream);

// Carves the workspace; with base == nullptr only sizes are computed.
int carve(void* base, int64_t N, int64_t total_rows, Workspace* ws);
int check_sizes(const char* who, int64_t T, int64_t B, int64_t N, int64_t total_rows);
int prepare_workspace(const char* who, void* workspace, int64_t workspace_bytes, int64_t N, int64_t total_rows,
                      Workspace* ws);

// keys_in/vals_in -> keys/vals, stable, on the low sort_bits bits.
int sort_pairs(Workspace& ws, int64_t N, int sort_bits, cudaStream_t stream);
// seg_starts[0..U) = first position of every run of equal sorted keys, counters[0] = U.
int select_run_starts(Workspace& ws, int64_t N, cudaStream_t stream);

// Approximate rowwise Adagrad without per-sample weights on the sorted-run kernels of tbe_backward.cu
// (the bags' squared gradient norms, a prefix sum per run, then a weighted segmented reduction).
// Returns TBE_ERR_UNSUPPORTED for shapes that path does not take; the caller then uses its own.
int approx_backward_sorted(const void* grad, int64_t stride_b, int64_t stride_t, void* weights,
                           const int32_t* table_offsets, const int32_t* indices, const int32_t* offsets, float* state,
                           int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, float lr,
                           float eps, int sr, uint64_t sr_seed, uint64_t sr_offset, int64_t max_rows_per_table,
                           void* workspace, int64_t workspace_bytes, void* stream);

// Row of `weights` a sort key stands for.
__device__ __forceinline__ uint32_t key_to_row(const int32_t* __restrict__ table_offsets, int idx_bits, uint32_t key) {
  if (idx_bits == 0) return key;
  return static_cast<uint32_t>(__ldg(table_offsets + (key >> idx_bits))) + (key & ((1u << idx_bits) - 1u));
}

}  // namespace tbe
