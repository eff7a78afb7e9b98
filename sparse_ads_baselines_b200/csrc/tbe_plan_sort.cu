// Table-segmented two-level sort of the (row key, bag id) pairs of a TBE batch (sm_100a).
//
// The backward needs the lookups grouped by row, and inside a group ordered by bag (the order of the
// index positions).  A generic device radix sort spends ~180 us on the 5 M pairs of the headline
// batch, a fifth of the whole forward+backward step, although the input is far from arbitrary:
// lookups arrive grouped by table (table t owns positions [offsets[t*B], offsets[(t+1)*B])), only
// the index inside the table needs ordering, and a table sees far fewer lookups than it has rows.
// This file orders every table independently in two levels that stay in L2:
//
//   1. bucket_count_kernel   : a table's positions are cut into slices; lookups per (table, slice,
//                              bucket), bucket = index >> shift.
//   2. bucket_scatter_kernel : every (slice, table) CTA works out from the histograms where its
//                              slice's share of each bucket lies (slices in order, no global
//                              atomics) and moves (key, bag id) pairs there.  The bag id of a
//                              position comes from a running search in `offsets`, so this kernel
//                              also replaces the separate linearize pass.  The order inside a
//                              slice's share is whatever the shared-memory atomics gave; level 2
//                              makes that irrelevant.
//   3. bucket_rank_kernel    : one CTA per bucket.  A counting sort in shared memory on coarse
//                              counters (one per small group of neighbouring rows) brings the
//                              pairs of a group together; groups with several pairs are then ranked
//                              by (key, bag id).  Equal pairs are indistinguishable, so the output
//                              is the unique order by (table, index, bag): exactly what a stable
//                              sort of the position-ordered input gives, and independent of how the
//                              atomics of any step were served.  A bucket larger than the CTA's
//                              capacity, or with a hot row, is queued instead ...
//   4. oversize_sort_kernel  : ... and sorted by a cluster of eight CTAs with stable radix passes on
//                              (index bits, bag id) in their joint shared memory.  Skewed batches,
//                              where a few hot rows put most of a table in one bucket, land here;
//                              normally the queue is empty.
#include <cooperative_groups.h>

#include <atomic>

#include "tbe_plan.cuh"

namespace cg = cooperative_groups;

namespace tbe {

namespace {

constexpr int kCountThreads = 512;
constexpr int kScatterThreads = 512;
constexpr int kScatterTile = 2048;      // positions a CTA gathers in shared memory at a time ...
constexpr int kScatterTileWide = 4096;  // ... when a table has more than kFewBuckets buckets
constexpr int kRankThreads = 256;
constexpr int kRankItems = kBucketSortCapacity / kRankThreads;  // pairs a thread holds
constexpr int kRankBits = 14;                                   // most index bits level 2 can count on
constexpr int kRankCounterBits = 13;                            // level 2 keeps at most 8192 counters per bucket
constexpr int kRankMaxGroup = kBucketSortMaxGroup;              // most pairs one counter may collect
static_assert(kBucketSortCapacity <= 2048 && kRankMaxGroup < 1024, "packing of bucket_rank_kernel's `where`");
constexpr int kOversizeThreads = 512;
constexpr int kOversizeWarps = kOversizeThreads / 32;
constexpr int kSortCluster = 8;     // CTAs (one cluster) that sort a queued bucket together
constexpr int kSortBlock = 8192;    // pairs of the bucket a CTA of the cluster holds at most
constexpr int kSortDigitBits = 9;   // the in-cluster passes look at up to 9 bits: one digit per thread
constexpr int kSortDigits = 1 << kSortDigitBits;
constexpr size_t kSortSmem = (2 * kSortBlock + kOversizeWarps * (kSortDigits / 2) + 2 * kSortDigits) * sizeof(uint32_t);
static_assert(kSortDigits <= kOversizeThreads && kSortCluster * kSortBlock <= 65536 && kSortBlock % 32 == 0,
              "one digit per thread; positions below 2^16 for the division by multiplication");
constexpr int kMaxDigits = 128;             // radix passes look at up to 7 bits
constexpr int kDigitBits = 7;
constexpr int kFewBuckets = 1024;           // buckets per table the narrow kernel variants hold in shared memory
constexpr int kMaxBuckets = 4096;           // buckets per table (wide variants: busy tables, e.g. 2 lookups per row)
constexpr int kBucketIdBits = 12;           // log2(kMaxBuckets)
static_assert((1 << kBucketIdBits) == kMaxBuckets && kScatterTileWide <= (1 << (31 - kBucketIdBits)), "slot packing");
constexpr int kDefaultBucketTarget = 1400;  // wanted mean bucket size
static_assert(kBucketSortCapacity % kRankThreads == 0 && kBucketSortCapacity < 65536, "16-bit positions");

__device__ __forceinline__ uint32_t bucket_of(int32_t index, int shift, int nb) {
  const uint32_t b = static_cast<uint32_t>(index) >> shift;
  return b < static_cast<uint32_t>(nb) ? b : static_cast<uint32_t>(nb - 1);  // a bad index must not leave the histogram
}

// Position range of slice s of table t.
__device__ __forceinline__ void slice_range(const int32_t* __restrict__ offsets, int64_t t, int32_t B, int s, int S,
                                            int32_t* ts, int32_t* a, int32_t* b) {
  const int32_t t0 = __ldg(offsets + t * B), t1 = __ldg(offsets + (t + 1) * B);
  const int64_t len = t1 - t0;
  *ts = t0;
  *a = t0 + static_cast<int32_t>(len * s / S);
  *b = t0 + static_cast<int32_t>(len * (s + 1) / S);
}

// Share of [a, b) that warp w of W walks: consecutive shares, each a multiple of 32 long.
__device__ __forceinline__ void warp_share(int32_t a, int32_t b, int w, int W, int32_t* ca, int32_t* cb) {
  const int32_t per = (((b - a) + W - 1) / W + 31) & ~31;
  const int64_t lo = static_cast<int64_t>(a) + static_cast<int64_t>(w) * per;
  *ca = lo < b ? static_cast<int32_t>(lo) : b;
  *cb = lo + per < b ? static_cast<int32_t>(lo + per) : b;
}

// Exclusive prefix sum of x over the threads of a CTA: shuffles inside a warp, then the totals of the
// warps in front.  Warps flagged inactive hold zeros and skip the work; every thread must call it,
// and a barrier must separate two calls that share warp_tot (one entry per warp).
template <typename V>
__device__ __forceinline__ V cta_exclusive_scan(V x, V* warp_tot, bool warp_active) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  V incl = x;
  if (warp_active) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const V up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
  }
  if (lane == 31) warp_tot[w] = warp_active ? incl : V(0);
  __syncthreads();
  V base = 0;
  if (warp_active)
    for (int i = 0; i < w; ++i) base += warp_tot[i];
  return base + incl - x;
}

// hist[(t * S + s) * nb + bucket] = lookups of slice s of table t that fall in the bucket.
template <int NBCAP>
__global__ void __launch_bounds__(kCountThreads) bucket_count_kernel(const int32_t* __restrict__ indices,
                                                                     const int32_t* __restrict__ offsets, int32_t B,
                                                                     int shift, int nb, int32_t* __restrict__ hist,
                                                                     int32_t* __restrict__ queue_count) {
  __shared__ int32_t sh[NBCAP];
  const int s = blockIdx.x, S = gridDim.x;
  const int64_t t = blockIdx.y;
  for (int i = threadIdx.x; i < nb; i += kCountThreads) sh[i] = 0;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *queue_count = 0;  // no oversize buckets yet
  __syncthreads();
  int32_t ts, a, b;
  slice_range(offsets, t, B, s, S, &ts, &a, &b);
  for (int32_t p = a + threadIdx.x; p < b; p += 4 * kCountThreads) {
    int32_t index[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) index[j] = p + j * kCountThreads < b ? __ldg(indices + p + j * kCountThreads) : -1;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (p + j * kCountThreads < b) atomicAdd(&sh[bucket_of(index[j], shift, nb)], 1);
  }
  __syncthreads();
  int32_t* out = hist + (t * S + s) * nb;
  for (int i = threadIdx.x; i < nb; i += kCountThreads) out[i] = sh[i];
}

// Largest bag g in [lo, hi) with offsets[g] <= p (offsets[lo] <= p is given).  All lanes call it with
// the same arguments; each round probes 32 evenly spaced bags at once.
__device__ __forceinline__ int32_t warp_find_bag(const int32_t* __restrict__ offsets, int32_t lo, int32_t hi,
                                                 int32_t p, int lane) {
  while (hi - lo > 1) {
    const int32_t step = (hi - lo + 31) >> 5;
    const int64_t probe = static_cast<int64_t>(lo) + static_cast<int64_t>(lane + 1) * step;
    const bool ok = probe < hi && __ldg(offsets + probe) <= p;
    const int c = __popc(__ballot_sync(0xffffffffu, ok));
    lo += c * step;
    hi = min(hi, lo + step);
  }
  return lo;
}

// Lane l receives the end of bag from + l, i.e. offsets[from + 1 + l], clamped to the table's last bag.
__device__ __forceinline__ int32_t load_bag_ends(const int32_t* __restrict__ offsets, int32_t from, int32_t bag_hi,
                                                 int lane) {
  const int64_t i = static_cast<int64_t>(from) + 1 + lane;
  return __ldg(offsets + (i < bag_hi ? i : bag_hi));
}

// Number of the 32 ascending values held one per lane in `ends` that are <= p (each lane its own p).
__device__ __forceinline__ int count_not_above(int32_t ends, int32_t p) {
  int c = 0;
#pragma unroll
  for (int step = 16; step >= 1; step >>= 1) {
    const int32_t v = __shfl_sync(0xffffffffu, ends, c + step - 1);
    if (v <= p) c += step;
  }
  const int32_t last = __shfl_sync(0xffffffffu, ends, 31);
  if (c == 31 && last <= p) c = 32;
  return c;
}

// A CTA moves its slice in steps of TILE pairs.  Every warp owns a contiguous share of the
// slice and contributes its next 32 * kRounds positions to each step (walking one contiguous range
// keeps the search for the bag of a position a matter of a few shuffles).  Per step: count the
// buckets (the old value of a pair's counter is its slot among the step's pairs of that bucket),
// gather the pairs bucket by bucket in shared memory, then copy them out: a bucket's share of the
// step is one contiguous run of 8-byte pairs, so the stores coalesce instead of costing a sector per
// pair.  Where a slice's pairs go inside a bucket follows from the histograms alone: slices in order.
//
// NBCAP buckets per table fit the CTA's shared arrays and TILE pairs are gathered per step: (1024, 2048)
// for the usual sparse batches, (4096, 4096) in dynamic shared memory for busy tables, where a step
// still has to give every bucket more than a pair or two for the copy-out to coalesce.
template <int NBCAP, int TILE>
__global__ void __launch_bounds__(kScatterThreads, NBCAP <= kFewBuckets ? 3 : 2) bucket_scatter_kernel(
    const int32_t* __restrict__ indices, const int32_t* __restrict__ offsets, int32_t B, int64_t T, int idx_bits,
    int shift, int nb, const int32_t* __restrict__ hist, int32_t* __restrict__ bucket_start,
    uint2* __restrict__ pairs) {
  extern __shared__ uint2 scatter_smem[];
  uint2* stage = scatter_smem;                                     // TILE pairs
  int32_t* cnt = reinterpret_cast<int32_t*>(scatter_smem + TILE);  // pairs of the step per bucket, then their first slot in `stage`
  int32_t* delta = cnt + NBCAP;                                    // global position minus slot in `stage`, per bucket
  int32_t* cursor = delta + NBCAP;                                 // next free global position of this slice in every bucket
  __shared__ int32_t warp_tot[kScatterThreads / 32];
  __shared__ int32_t step_total;
  constexpr int kPer = NBCAP / kScatterThreads;  // buckets per thread
  constexpr int kRounds = TILE / kScatterThreads;
  constexpr int kWarps = kScatterThreads / 32;

  const int s = blockIdx.x, S = gridDim.x;
  const int64_t t = blockIdx.y;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int32_t ts, a, b;
  slice_range(offsets, t, B, s, S, &ts, &a, &b);
  const bool scans = w * 32 * kPer < nb;  // this warp's threads own buckets
  {
    int32_t tot[kPer], before[kPer];
    int32_t sum = 0;
    const int32_t* h = hist + t * S * nb;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = threadIdx.x * kPer + j;
      tot[j] = 0;
      before[j] = 0;
      if (i < nb) {
        for (int s2 = 0; s2 < S; ++s2) {
          const int32_t c = __ldg(h + s2 * nb + i);
          if (s2 < s) before[j] += c;
          tot[j] += c;
        }
      }
      sum += tot[j];
    }
    int32_t excl = cta_exclusive_scan(sum, warp_tot, scans);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = threadIdx.x * kPer + j;
      if (i < nb) {
        cursor[i] = ts + excl + before[j];
        cnt[i] = 0;
        if (s == 0) bucket_start[t * nb + i] = ts + excl;
      }
      excl += tot[j];
    }
    if (s == 0 && t == T - 1 && threadIdx.x == 0) bucket_start[T * nb] = __ldg(offsets + T * B);
  }
  const int32_t bag_lo = static_cast<int32_t>(t * B), bag_hi = bag_lo + B;
  const uint32_t key_hi = static_cast<uint32_t>(t) << idx_bits;
  const uint32_t index_mask = (1u << idx_bits) - 1u;
  int32_t ca, cb;
  warp_share(a, b, w, kWarps, &ca, &cb);
  const int32_t share = ((((b - a) + kWarps - 1) / kWarps) + 31) & ~31;  // as in warp_share
  const int steps = (share + 32 * kRounds - 1) / (32 * kRounds);
  // `cur` is a bag that starts at or before the warp's position, `ends` the ends of bags cur..cur+31
  int32_t cur = bag_lo, ends = 0;
  if (ca < cb) {
    cur = warp_find_bag(offsets, bag_lo, bag_hi, ca, lane);
    ends = load_bag_ends(offsets, cur, bag_hi, lane);
  }
  int32_t index[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; ++r) index[r] = ca + r * 32 + lane < cb ? __ldg(indices + ca + r * 32 + lane) : 0;
  __syncthreads();

  for (int k = 0; k < steps; ++k) {
    const int32_t wa = min(cb, ca + k * (32 * kRounds));
    uint32_t key[kRounds], slot[kRounds];
    int32_t bagv[kRounds];
#pragma unroll
    for (int r = 0; r < kRounds; ++r) {
      const int32_t p = wa + r * 32 + lane;
      const bool valid = p < cb;
      key[r] = key_hi | static_cast<uint32_t>(index[r]);
      if (valid) {
        const uint32_t bk = bucket_of(index[r], shift, nb);
        slot[r] = bk | (static_cast<uint32_t>(atomicAdd(&cnt[bk], 1)) << kBucketIdBits);
      }
      const int32_t pn = p + 32 * kRounds;  // the next step's index, in flight during this one
      index[r] = pn < cb ? __ldg(indices + pn) : 0;
    }
    if (wa < cb) {
      // bag of p = cur + number of bag ends that are <= p
      const int32_t last_p = min(cb, wa + 32 * kRounds) - 1;
      if (__shfl_sync(0xffffffffu, ends, 31) > last_p) {
        // Usual case: the window of 32 bag ends reaches past the step.  Ends at or before the
        // step's first position count for all of its positions; the few ends inside the step are
        // broadcast one by one and compared with the lane's positions.
        const int32_t first_bag = cur + __popc(__ballot_sync(0xffffffffu, ends <= wa));
        unsigned inside = __ballot_sync(0xffffffffu, ends > wa && ends <= last_p);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) bagv[r] = first_bag;
        while (inside) {
          const int32_t e = __shfl_sync(0xffffffffu, ends, __ffs(inside) - 1);
          inside &= inside - 1u;
#pragma unroll
          for (int r = 0; r < kRounds; ++r) bagv[r] += (wa + r * 32 + lane >= e) ? 1 : 0;
        }
        const int32_t tail = cur + __popc(__ballot_sync(0xffffffffu, ends <= last_p));  // bag of last_p
        if (tail - cur >= 16) {  // slide the window before it runs out
          cur = tail;
          ends = load_bag_ends(offsets, cur, bag_hi, lane);
        }
      } else {
        // short or empty bags: more than the window's bags end inside the step
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
          const int32_t p = wa + r * 32 + lane;
          const bool valid = p < cb;
          int32_t bag = -1, from = cur, window = ends;
          while (true) {
            const int c = count_not_above(window, p);
            if (bag < 0 && valid && c < 32) bag = from + c;
            if (__all_sync(0xffffffffu, bag >= 0 || !valid)) break;
            from += 32;
            window = load_bag_ends(offsets, from, bag_hi, lane);
          }
          const int32_t tail = __shfl_sync(0xffffffffu, bag, 31);
          if (tail - cur >= 16) {  // (tail is -1 past the share's end)
            cur = tail;
            ends = load_bag_ends(offsets, cur, bag_hi, lane);
          }
          bagv[r] = bag;
        }
      }
    }
    __syncthreads();
    {
      int32_t c[kPer];
      int32_t sum = 0;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x * kPer + j;
        c[j] = i < nb ? cnt[i] : 0;
        sum += c[j];
      }
      int32_t excl = cta_exclusive_scan(sum, warp_tot, scans);
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x * kPer + j;
        if (i < nb) {
          cnt[i] = excl;
          delta[i] = cursor[i] - excl;
          cursor[i] += c[j];
          if (i == nb - 1) step_total = excl + c[j];
        }
        excl += c[j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRounds; ++r)
      if (wa + r * 32 + lane < cb)
        stage[cnt[slot[r] & (kMaxBuckets - 1)] + (slot[r] >> kBucketIdBits)] = make_uint2(key[r], static_cast<uint32_t>(bagv[r]));
    __syncthreads();
    for (int i = threadIdx.x; i < nb; i += kScatterThreads) cnt[i] = 0;
    const int32_t m = step_total;
    for (int i = threadIdx.x; i < m; i += kScatterThreads) {
      const uint2 pr = stage[i];
      pairs[delta[bucket_of(static_cast<int32_t>(pr.x & index_mask), shift, nb)] + i] = pr;
    }
    __syncthreads();
  }
}

// Counter words are moved as 16-byte chunks; a thread scans 8 consecutive chunks at full size, so
// chunk c lives at c ^ ((c >> 3) & 7): the 8 lanes of a quarter warp then hit 8 different bank groups.
__device__ __forceinline__ int swizzle_chunk(int c) { return c ^ ((c >> 3) & 7); }
__device__ __forceinline__ int swizzle_word(int i) { return (swizzle_chunk(i >> 2) << 2) | (i & 3); }

// Level 2, one CTA per bucket of at most kBucketSortCapacity pairs.
//
// A counting sort with one counter per possible row would spend most of its time on counters, not on
// pairs: a bucket of the usual sparse batch holds 1,300 pairs spread over 16,384 rows.  So the
// counters are coarse: one per group of 2^cshift consecutive rows, at most kRankCounters per bucket
// (about 0.6 pairs per counter).  The counting sort brings the pairs of a group together; groups that
// hold several pairs (rows that repeat, or neighbouring rows) are then put in (key, bag id) order by
// ranking every pair against its group, still in shared memory, and the bucket leaves with one
// coalesced copy.  Equal pairs are indistinguishable, so the result is the unique order by
// (table, index, bag id).  A group above kRankMaxGroup pairs (a hot row) would make the ranking
// quadratic: such a bucket is queued for oversize_sort_kernel like one that exceeds the capacity.
//
// Dynamic shared memory: `words` counter words (two 16-bit counters each), then the bucket's keys and
// values in counting-sort order.
__global__ void __launch_bounds__(kRankThreads) bucket_rank_kernel(
    const int32_t* __restrict__ bucket_start, const uint2* __restrict__ pairs, uint32_t* __restrict__ kout,
    int32_t* __restrict__ vout, int bits, int cshift, int words, int32_t* __restrict__ queue_count,
    int2* __restrict__ queue, int queue_cap) {
  extern __shared__ uint4 smem4[];
  uint32_t* cnt = reinterpret_cast<uint32_t*>(smem4);
  uint32_t* sk = cnt + words;
  int32_t* sv = reinterpret_cast<int32_t*>(sk + kBucketSortCapacity);
  __shared__ uint32_t warp_tot[kRankThreads / 32];

  const int32_t start = __ldg(bucket_start + blockIdx.x), end = __ldg(bucket_start + blockIdx.x + 1);
  const int32_t n = end - start;
  if (n <= 0) return;
  auto enqueue = [&]() {
    if (threadIdx.x == 0) {
      const int q = atomicAdd(queue_count, 1);
      if (q < queue_cap) queue[q] = make_int2(start, end);  // always true: the queue has a slot per possible bucket
    }
  };
  if (n > kBucketSortCapacity) {
    enqueue();
    return;
  }
  pairs += start;
  kout += start;
  vout += start;
  uint32_t key[kRankItems], where[kRankItems];
  int32_t val[kRankItems];
#pragma unroll
  for (int j = 0; j < kRankItems; ++j) {  // in flight while the counters are cleared
    const int e = threadIdx.x + j * kRankThreads;
    const uint2 pr = e < n ? __ldg(pairs + e) : make_uint2(0u, 0u);
    key[j] = pr.x;
    val[j] = static_cast<int32_t>(pr.y);
  }
  const uint32_t low_mask = (1u << bits) - 1u;
  const uint32_t last_counter = low_mask >> cshift;
  const int chunks = words >> 2;
  const int cpt = (chunks + kRankThreads - 1) / kRankThreads;  // chunks a thread zeroes and scans
  const int c0 = threadIdx.x * cpt;
  for (int c = c0; c < min(c0 + cpt, chunks); ++c) smem4[swizzle_chunk(c)] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();

  // count: the old value of a pair's counter is its arrival number among the pairs of its group
#pragma unroll
  for (int j = 0; j < kRankItems; ++j) {
    if (threadIdx.x + j * kRankThreads < n) {
      const uint32_t c = (key[j] & low_mask) >> cshift;
      const int half = (c & 1u) * 16;
      where[j] = (atomicAdd(&cnt[swizzle_word(c >> 1)], 1u << half) >> half) & 0xffffu;
    }
  }
  __syncthreads();

  // counts -> first position of every group, in place (positions fit 16 bits)
  bool big_group = false;
  {
    uint32_t packed = 0;
    for (int c = c0; c < min(c0 + cpt, chunks); ++c) {
      const uint4 v = smem4[swizzle_chunk(c)];
      packed += v.x + v.y + v.z + v.w;  // both halves at once: neither can overflow 16 bits
    }
    uint32_t run = cta_exclusive_scan((packed & 0xffffu) + (packed >> 16), warp_tot, true);
    for (int c = c0; c < min(c0 + cpt, chunks); ++c) {
      uint4 v = smem4[swizzle_chunk(c)];
      uint32_t* wv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = wv[i] & 0xffffu, hi = wv[i] >> 16;
        big_group |= lo > kRankMaxGroup || hi > kRankMaxGroup;
        const uint32_t second = run + lo;
        wv[i] = run | (second << 16);
        run = second + hi;
      }
      smem4[swizzle_chunk(c)] = v;
    }
  }
  if (__syncthreads_or(big_group)) {  // (also the barrier the placement below needs)
    enqueue();
    return;
  }

  // place in counting-sort order.  where = position | first position of the group << 11 | pairs in
  // the group << 22 (positions are below 2048, a group holds at most kRankMaxGroup pairs).
#pragma unroll
  for (int j = 0; j < kRankItems; ++j) {
    if (threadIdx.x + j * kRankThreads < n) {
      const uint32_t c = (key[j] & low_mask) >> cshift;
      const int word = c >> 1;
      const uint32_t packed = cnt[swizzle_word(word)];
      uint32_t first, next;
      if (c & 1u) {
        first = packed >> 16;
        next = word + 1 < words ? (cnt[swizzle_word(word + 1)] & 0xffffu) : static_cast<uint32_t>(n);
      } else {
        first = packed & 0xffffu;
        next = packed >> 16;
      }
      if (c == last_counter) next = static_cast<uint32_t>(n);  // the last group of the bucket
      const uint32_t pos = first + where[j];
      sk[pos] = key[j];
      sv[pos] = val[j];
      where[j] = pos | (first << 11) | ((next - first) << 22);
    }
  }
  __syncthreads();

  // groups of several pairs: every pair finds its rank by (key, bag id) among its group; among equal
  // pairs the arrival order stands, which cannot be told apart in the output
#pragma unroll
  for (int j = 0; j < kRankItems; ++j) {
    const uint32_t size = where[j] >> 22;
    if (threadIdx.x + j * kRankThreads < n && size > 1u) {
      const uint32_t pos = where[j] & 2047u, first = (where[j] >> 11) & 2047u;
      const uint32_t k0 = key[j];
      const int32_t v0 = val[j];
      uint32_t rank = 0;
      for (uint32_t q = first; q < first + size; ++q) {
        const uint32_t kq = sk[q];
        const int32_t vq = sv[q];
        rank += (kq < k0) || (kq == k0 && (vq < v0 || (vq == v0 && q < pos)));
      }
      where[j] = (where[j] & ~2047u) | (first + rank);
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kRankItems; ++j) {
    if (threadIdx.x + j * kRankThreads < n && (where[j] >> 22) > 1u) {
      sk[where[j] & 2047u] = key[j];
      sv[where[j] & 2047u] = val[j];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kRankThreads) {
    kout[i] = sk[i];
    vout[i] = sv[i];
  }
}

// One stable radix pass of a CTA of W warps over n pairs, on bits [sh, sh + dbits) of the key or,
// with BY_VAL, of value - vbase.  Every warp owns a contiguous share of the input, counts its
// digits, the counts become start positions in (digit, warp) order, then the warp walks its share 32
// pairs at a time and ranks equal digits with ballots.  cnt: W * kMaxDigits counters, digit_base:
// kMaxDigits.
template <int W, bool BY_VAL>
__device__ __forceinline__ void radix_pass(const uint32_t* sk, const int32_t* sv, uint32_t* dk, int32_t* dv, int32_t n,
                                           int32_t vbase, int sh, int dbits, int32_t* cnt, int32_t* digit_base) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int nd = 1 << dbits;
  const uint32_t mask = static_cast<uint32_t>(nd - 1);
  int32_t ca, cb;
  warp_share(0, n, w, W, &ca, &cb);
  int32_t* my_cnt = cnt + w * kMaxDigits;
  for (int i = lane; i < nd; i += 32) my_cnt[i] = 0;
  __syncwarp();
  for (int32_t p = ca + lane; p < cb; p += 32) {
    const uint32_t x = BY_VAL ? static_cast<uint32_t>(sv[p] - vbase) : sk[p];
    atomicAdd(&my_cnt[(x >> sh) & mask], 1);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < nd; d += W * 32) {
    int32_t run = 0;
#pragma unroll 8
    for (int w2 = 0; w2 < W; ++w2) {
      const int32_t c = cnt[w2 * kMaxDigits + d];
      cnt[w2 * kMaxDigits + d] = run;
      run += c;
    }
    digit_base[d] = run;
  }
  __syncthreads();
  if (w == 0) {  // exclusive scan of the per-digit totals
    constexpr int kPer = kMaxDigits / 32;
    int32_t v[kPer];
    int32_t sum = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int d = lane * kPer + j;
      v[j] = d < nd ? digit_base[d] : 0;
      sum += v[j];
    }
    int32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int32_t run = incl - sum;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int d = lane * kPer + j;
      if (d < nd) digit_base[d] = run;
      run += v[j];
    }
  }
  __syncthreads();
  // the next round's pair is requested before this round's is ranked
  uint32_t key_next = ca + lane < cb ? sk[ca + lane] : 0u;
  int32_t val_next = ca + lane < cb ? sv[ca + lane] : vbase;
  for (int32_t p0 = ca; p0 < cb; p0 += 32) {
    const int32_t p = p0 + lane;
    const bool valid = p < cb;
    const uint32_t key = key_next;
    const int32_t val = val_next;
    key_next = p + 32 < cb ? sk[p + 32] : 0u;
    val_next = p + 32 < cb ? sv[p + 32] : vbase;
    const uint32_t d = ((BY_VAL ? static_cast<uint32_t>(val - vbase) : key) >> sh) & mask;
    uint32_t peers = __ballot_sync(0xffffffffu, valid);
    for (int bit = 0; bit < dbits; ++bit) {
      const bool one = (d >> bit) & 1u;
      const uint32_t set = __ballot_sync(0xffffffffu, one);
      peers &= one ? set : ~set;
    }
    const int r = __popc(peers & ((1u << lane) - 1u));
    if (valid) {
      const int32_t pos = digit_base[d] + my_cnt[d] + r;
      dk[pos] = key;
      dv[pos] = val;
    }
    __syncwarp();
    if (valid && r == 0) my_cnt[d] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
}

// Buckets too large for bucket_rank_kernel (or with a hot row): least-significant-digit radix sort on
// (index bits, bag id within the table).  A fixed grid walks the queue, so an empty queue costs one
// launch.
//
// A queued bucket is sorted by a thread-block CLUSTER of four or eight CTAs in their joint shared
// memory (the first bucket of a skewed table holds ~25,000 pairs; one CTA needs four times longer
// for it than the rest of the plan takes).  A pair's index bits and its bag id within the table are
// packed into one 32-bit word, index bits on top, so that ascending words ARE the order by (index,
// bag).  CTA c of the cluster holds positions [c * per, (c + 1) * per) of the bucket in each of two
// word buffers.  One pass: every warp counts the digits of its share of the CTA's block; the CTAs
// read each other's per-digit totals through distributed shared memory, which gives every (digit,
// CTA, warp) its first output position in the bucket; the warps then rank equal digits with ballots
// and store each word into the buffer of whichever CTA owns its new position (a remote shared-memory
// store).  Two cluster barriers per pass; keys and bag ids are rebuilt on the way out.
//
// A bucket beyond (CTAs of the cluster) * kSortBlock pairs (or more than 32 bits of index + bag) is sorted by
// the cluster's first CTA alone with passes through global memory: the bucket's pairs are first
// split into the output arrays, the passes then ping-pong between those and the bucket's own stretch
// of the pair array, which is free by then.
__global__ void __launch_bounds__(kOversizeThreads, 2)
    oversize_sort_kernel(uint2* pairs, uint32_t* kout, int32_t* vout, int key_bits, int bag_bits, int idx_bits,
                         int32_t B, const int32_t* __restrict__ queue_count, const int2* __restrict__ queue,
                         int queue_cap) {
  extern __shared__ uint32_t sort_smem[];  // two word buffers of kSortBlock, then the counters
  uint32_t* cnt = sort_smem + 2 * kSortBlock;  // [warp][digit / 2]; [warp][kMaxDigits] of 32 bits for the global passes
  int32_t* tot = reinterpret_cast<int32_t*>(cnt + kOversizeWarps * (kSortDigits / 2));  // this CTA's words per digit
  int32_t* digit_base = tot + kSortDigits;
  __shared__ int32_t warp_tot[kOversizeWarps];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int csize = static_cast<int>(cluster.num_blocks());  // 4 or 8 (chosen at launch), at most kSortCluster
  const int cid = blockIdx.x / csize, nclusters = gridDim.x / csize;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int count = min(*queue_count, queue_cap);
  for (int q = cid; q < count; q += nclusters) {  // (the same buckets for every CTA of a cluster)
    const int2 seg = queue[q];
    const int32_t n = seg.y - seg.x;
    const uint32_t first_key = pairs[seg.x].x;
    const int32_t vbase = static_cast<int32_t>(first_key >> idx_bits) * B;  // first bag of the bucket's table
    if (n <= csize * kSortBlock && key_bits + bag_bits <= 32) {
      // block length: a multiple of 32, at most kSortBlock; position / per by multiplication (exact
      // below 2^16 positions for per < 2^16)
      const int32_t per = (((n + csize - 1) / csize) + 31) & ~31;
      const uint32_t per_magic = static_cast<uint32_t>(((1ull << 32) + per - 1) / per);
      const int32_t lo = rank * per;
      const int32_t m = max(0, min(per, n - lo));  // words this CTA holds
      const uint32_t low_mask = key_bits >= 32 ? 0xffffffffu : ((1u << key_bits) - 1u);
      const uint32_t key_hi = first_key & ~low_mask;  // table and bucket bits: the same for the whole bucket
      for (int32_t i = threadIdx.x; i < m; i += kOversizeThreads) {
        const uint2 pr = pairs[seg.x + lo + i];
        sort_smem[i] = ((pr.x & low_mask) << bag_bits) | static_cast<uint32_t>(static_cast<int32_t>(pr.y) - vbase);
      }
      __syncthreads();
      const int total = key_bits + bag_bits;
      const int np = (total + kSortDigitBits - 1) / kSortDigitBits;
      const int db = np ? (total + np - 1) / np : 0;
      int32_t ca, cb;
      warp_share(0, m, w, kOversizeWarps, &ca, &cb);
      // per-warp digit counters, two 16-bit counters to a word (a CTA's block is below 2^16 words)
      uint32_t* my_cnt = cnt + w * (kSortDigits / 2);
      int side = 0;
      for (int pass = 0; pass < np; ++pass, side ^= 1) {
        const uint32_t* src = sort_smem + side * kSortBlock;
        uint32_t* dst = sort_smem + (side ^ 1) * kSortBlock;
        const int sh = pass * db, dbits = min(db, total - sh);
        const int nd = 1 << dbits;
        const uint32_t mask = static_cast<uint32_t>(nd - 1);
        for (int i = lane; i < (nd + 1) / 2; i += 32) my_cnt[i] = 0u;
        __syncwarp();
        for (int32_t p = ca + lane; p < cb; p += 32) {
          const uint32_t d = (src[p] >> sh) & mask;
          atomicAdd(&my_cnt[d >> 1], 1u << ((d & 1u) * 16));
        }
        __syncthreads();
        if (threadIdx.x < (nd + 1) / 2) {  // counts -> first place of every warp among this CTA's words of a digit
          uint32_t run = 0;  // both digits of the word at once
#pragma unroll
          for (int w2 = 0; w2 < kOversizeWarps; ++w2) {
            const uint32_t c = cnt[w2 * (kSortDigits / 2) + threadIdx.x];
            cnt[w2 * (kSortDigits / 2) + threadIdx.x] = run;
            run += c;
          }
          tot[2 * threadIdx.x] = static_cast<int32_t>(run & 0xffffu);
          tot[2 * threadIdx.x + 1] = static_cast<int32_t>(run >> 16);
        }
        cluster.sync();  // every CTA's totals are in place
        int32_t all = 0, before = 0;
        if (threadIdx.x < nd) {
#pragma unroll
          for (int c = 0; c < kSortCluster; ++c) {
            const int32_t t = c < csize ? cluster.map_shared_rank(tot, c)[threadIdx.x] : 0;
            all += t;
            if (c < rank) before += t;
          }
        }
        // words of smaller digits in the whole bucket, plus words of this digit in the CTAs in front
        const int32_t smaller = cta_exclusive_scan(all, warp_tot, threadIdx.x < ((nd + 31) & ~31));
        if (threadIdx.x < nd) digit_base[threadIdx.x] = smaller + before;
        __syncthreads();
        // (Ranking equal digits once, in the counting loop, and keeping each word's rank for this loop was
        // measured and is slower: the ballots cost more there than the conflicting shared-memory adds.)
        for (int32_t p0 = ca; p0 < cb; p0 += 32) {
          const int32_t p = p0 + lane;
          const bool valid = p < cb;
          const uint32_t x = valid ? src[p] : 0u;
          const uint32_t d = (x >> sh) & mask;
          uint32_t peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
          for (int bit = 0; bit < kSortDigitBits; ++bit) {  // (bits beyond dbits are zero in every lane: no effect)
            const uint32_t set = __ballot_sync(0xffffffffu, (d >> bit) & 1u);
            peers &= ((d >> bit) & 1u) ? set : ~set;
          }
          const int r = __popc(peers & ((1u << lane) - 1u));
          const int half = (d & 1u) * 16;
          if (valid) {
            // new position in the bucket
            const uint32_t g = static_cast<uint32_t>(digit_base[d]) + ((my_cnt[d >> 1] >> half) & 0xffffu) + r;
            const uint32_t owner = __umulhi(g, per_magic);
            cluster.map_shared_rank(dst, owner)[g - owner * static_cast<uint32_t>(per)] = x;
          }
          __syncwarp();
          if (valid && r == 0) atomicAdd(&my_cnt[d >> 1], static_cast<uint32_t>(__popc(peers)) << half);
          __syncwarp();
        }
        cluster.sync();  // every word of the pass has landed; the totals may be overwritten
      }
      const uint32_t* fin = sort_smem + side * kSortBlock;
      const uint32_t bag_mask = bag_bits >= 32 ? 0xffffffffu : ((1u << bag_bits) - 1u);
      for (int32_t i = threadIdx.x; i < m; i += kOversizeThreads) {
        const uint32_t x = fin[i];
        kout[seg.x + lo + i] = key_hi | (x >> bag_bits);
        vout[seg.x + lo + i] = vbase + static_cast<int32_t>(x & bag_mask);
      }
      __syncthreads();  // the next bucket is loaded over these buffers
      continue;
    }
    if (rank != 0) continue;
    const int vp = (bag_bits + kDigitBits - 1) / kDigitBits, kp = (key_bits + kDigitBits - 1) / kDigitBits;
    const int vd = vp ? (bag_bits + vp - 1) / vp : 0, kd = kp ? (key_bits + kp - 1) / kp : 0;
    uint32_t* scratch = reinterpret_cast<uint32_t*>(pairs + seg.x);
    uint32_t *k_src = kout + seg.x, *k_dst = scratch;
    int32_t *v_src = vout + seg.x, *v_dst = reinterpret_cast<int32_t*>(scratch + n);
    __syncthreads();  // every thread has read the bucket's first pair
    for (int32_t i = threadIdx.x; i < n; i += kOversizeThreads) {
      const uint2 pr = pairs[seg.x + i];
      k_src[i] = pr.x;
      v_src[i] = static_cast<int32_t>(pr.y);
    }
    __syncthreads();
    auto swap_sides = [&]() {
      uint32_t* kt = k_src;
      k_src = k_dst;
      k_dst = kt;
      int32_t* vt = v_src;
      v_src = v_dst;
      v_dst = vt;
    };
    for (int pass = 0; pass < vp; ++pass, swap_sides())
      radix_pass<kOversizeWarps, true>(k_src, v_src, k_dst, v_dst, n, vbase, pass * vd, min(vd, bag_bits - pass * vd),
                                       reinterpret_cast<int32_t*>(cnt), digit_base);
    for (int pass = 0; pass < kp; ++pass, swap_sides())
      radix_pass<kOversizeWarps, false>(k_src, v_src, k_dst, v_dst, n, vbase, pass * kd, min(kd, key_bits - pass * kd),
                                        reinterpret_cast<int32_t*>(cnt), digit_base);
    if (k_src != kout + seg.x) {  // an odd number of passes ends in the scratch
      for (int32_t i = threadIdx.x; i < n; i += kOversizeThreads) {
        k_dst[i] = k_src[i];
        v_dst[i] = v_src[i];
      }
      __syncthreads();
    }
  }
}

int rank_counter_shift(int bits) { return bits > kRankCounterBits ? bits - kRankCounterBits : 0; }
int rank_words(int bits) {
  const int w = (1 << (bits - rank_counter_shift(bits))) / 2;  // two 16-bit counters per word
  return w < 32 ? 32 : w;  // whole swizzle groups of 8 chunks
}

}  // namespace

bool bucket_geometry(int64_t T, int64_t N, int64_t max_rows_per_table, KeyLayout layout, const Workspace& ws,
                     BucketGeometry* g) {
  if (layout.idx_bits == 0 || N < 1 || max_rows_per_table < 1) return false;
  if (tuning(kTuneBwdSort) == 1) return false;
  const double avg = static_cast<double>(N) / static_cast<double>(T);
  double target = tuning(kTuneSortBucket);
  if (target <= 0) target = kDefaultBucketTarget;
  if (target > kBucketSortCapacity * 0.7) target = kBucketSortCapacity * 0.7;
  // widest bucket (fewest buckets) whose expected size under uniform indices stays below the target
  int shift = layout.idx_bits < kRankBits ? layout.idx_bits : kRankBits;
  while (shift > 0 && avg * static_cast<double>(1ll << shift) / static_cast<double>(max_rows_per_table) > target)
    --shift;
  const int64_t nb = ((max_rows_per_table - 1) >> shift) + 1;
  if (nb > kMaxBuckets) return false;  // tables too large (or too busy) for 4096 buckets of up to 2^14 rows
  g->shift = shift;
  g->nb = static_cast<int>(nb);
  const int64_t want = static_cast<int64_t>(avg / 8192.0) + 1;
  // the (slice, table) grid should be resident at once: 3 CTAs of the narrow scatter variant fit an SM, 2 of the wide
  const int64_t room = (nb > kFewBuckets ? 2ll : 3ll) * device_sm_count() / T;
  int64_t S = want < room ? want : room;
  if (S < 1) S = 1;
  if (S > 65535 || T > 65535) return false;
  g->slices = static_cast<int>(S);
  if (T * S * nb > ws.hist_cap || T * nb + 1 > ws.hist_cap) return false;
  return true;
}

int bucket_sort_plan(const int32_t* indices, const int32_t* offsets, int64_t T, int64_t B, int64_t N,
                     KeyLayout layout, const BucketGeometry& g, Workspace& ws, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(g.slices), static_cast<unsigned>(T));
  const int qcap = static_cast<int>(ws.queue_cap);
  int32_t* queue_count = ws.counters + 8;
  // (key, bag id) pairs between the two levels; keys_in and vals_in are adjacent in the workspace
  uint2* pairs = reinterpret_cast<uint2*>(ws.keys_in);
  const int words = rank_words(g.shift);
  const size_t rank_smem = static_cast<size_t>(words) * 4 + static_cast<size_t>(kBucketSortCapacity) * 8;
  int dev = 0;
  TBE_CUDA_TRY(cudaGetDevice(&dev));
  static std::atomic<bool> rank_opted_in[64];
  if (rank_smem > 48 * 1024 - 64 && dev < 64 && !rank_opted_in[dev].load(std::memory_order_acquire)) {
    TBE_CUDA_TRY(cudaFuncSetAttribute(bucket_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (1 << kRankCounterBits) * 2 + kBucketSortCapacity * 8));
    rank_opted_in[dev].store(true, std::memory_order_release);
  }
  // The queued-bucket sort keeps its word buffers and counters in opted-in dynamic shared memory.  Its
  // grid is as many clusters as the device keeps resident at once, each walks the queue.  A skewed
  // batch queues about one bucket per table and a bucket's sort is a chain of latencies more than of
  // work, so the clusters are eight CTAs while those fit side by side and four beyond.
  const int csize = T <= 32 ? kSortCluster : kSortCluster / 2;
  static std::atomic<int> oversize_clusters[64][2];
  int clusters = dev < 64 ? oversize_clusters[dev][csize == kSortCluster].load(std::memory_order_acquire) : 0;
  cudaLaunchAttribute sort_attr;
  sort_attr.id = cudaLaunchAttributeClusterDimension;
  sort_attr.val.clusterDim.x = static_cast<unsigned>(csize);
  sort_attr.val.clusterDim.y = 1;
  sort_attr.val.clusterDim.z = 1;
  cudaLaunchConfig_t sort_cfg = {};
  sort_cfg.blockDim = dim3(kOversizeThreads);
  sort_cfg.dynamicSmemBytes = kSortSmem;
  sort_cfg.stream = stream;
  sort_cfg.attrs = &sort_attr;
  sort_cfg.numAttrs = 1;
  if (clusters == 0) {
    TBE_CUDA_TRY(cudaFuncSetAttribute(oversize_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kSortSmem)));
    sort_cfg.gridDim = dim3(static_cast<unsigned>(csize * device_sm_count()));
    if (cudaOccupancyMaxActiveClusters(&clusters, oversize_sort_kernel, &sort_cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = device_sm_count() / csize;  // one CTA per SM
    }
    if (clusters < 1) clusters = 1;
    if (dev < 64) oversize_clusters[dev][csize == kSortCluster].store(clusters, std::memory_order_release);
  }
  const bool wide = g.nb > kFewBuckets;
  constexpr size_t kScatterSmem = kScatterTile * sizeof(uint2) + 3 * kFewBuckets * sizeof(int32_t);
  constexpr size_t kScatterSmemWide = kScatterTileWide * sizeof(uint2) + 3 * kMaxBuckets * sizeof(int32_t);
  static std::atomic<bool> wide_opted_in[64];
  if (wide && dev < 64 && !wide_opted_in[dev].load(std::memory_order_acquire)) {
    TBE_CUDA_TRY(cudaFuncSetAttribute(bucket_scatter_kernel<kMaxBuckets, kScatterTileWide>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kScatterSmemWide)));
    wide_opted_in[dev].store(true, std::memory_order_release);
  }
  {
    KernelTimer timer("bucket_count_kernel", stream);
    if (wide) {
      bucket_count_kernel<kMaxBuckets><<<grid, kCountThreads, 0, stream>>>(indices, offsets, static_cast<int32_t>(B),
                                                                          g.shift, g.nb, ws.hist, queue_count);
    } else {
      bucket_count_kernel<kFewBuckets><<<grid, kCountThreads, 0, stream>>>(indices, offsets, static_cast<int32_t>(B),
                                                                          g.shift, g.nb, ws.hist, queue_count);
    }
  }
  TBE_CHECK_LAUNCH("bucket_count_kernel");
  {
    KernelTimer timer("bucket_scatter_kernel", stream);
    if (wide) {
      bucket_scatter_kernel<kMaxBuckets, kScatterTileWide><<<grid, kScatterThreads, kScatterSmemWide, stream>>>(
          indices, offsets, static_cast<int32_t>(B), T, layout.idx_bits, g.shift, g.nb, ws.hist, ws.bucket_start, pairs);
    } else {
      bucket_scatter_kernel<kFewBuckets, kScatterTile><<<grid, kScatterThreads, kScatterSmem, stream>>>(
          indices, offsets, static_cast<int32_t>(B), T, layout.idx_bits, g.shift, g.nb, ws.hist, ws.bucket_start, pairs);
    }
  }
  TBE_CHECK_LAUNCH("bucket_scatter_kernel");
  {
    KernelTimer timer("bucket_rank_kernel", stream);
    bucket_rank_kernel<<<static_cast<unsigned>(T * g.nb), kRankThreads, rank_smem, stream>>>(
        ws.bucket_start, pairs, ws.keys, ws.vals, g.shift, rank_counter_shift(g.shift), words, queue_count, ws.oversize,
        qcap);
  }
  TBE_CHECK_LAUNCH("bucket_rank_kernel");
  {
    if (clusters > qcap) clusters = qcap;
    if (clusters < 1) clusters = 1;
    int bag_bits = 0;
    while ((1ll << bag_bits) < B) ++bag_bits;
    KernelTimer timer("oversize_sort_kernel", stream);
    sort_cfg.gridDim = dim3(static_cast<unsigned>(clusters * csize));
    TBE_CUDA_TRY(cudaLaunchKernelEx(&sort_cfg, oversize_sort_kernel, pairs, ws.keys, ws.vals, g.shift, bag_bits,
                                    layout.idx_bits, static_cast<int32_t>(B), static_cast<const int32_t*>(queue_count),
                                    static_cast<const int2*>(ws.oversize), qcap));
  }
  TBE_CHECK_LAUNCH("oversize_sort_kernel");
  return TBE_OK;
}

}  // namespace tbe
