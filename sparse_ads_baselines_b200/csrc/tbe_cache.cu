// LXU cache: a set-associative cache in HBM in front of a host-resident embedding table (sm_100a).
//
// The table lives in pinned, device-mapped host memory (every uncached access crosses the host
// link); `ways * num_sets` rows of it are kept in HBM.  Once per step, before the lookup:
//
//   1. cache_keys_kernel  : h = mix(row), a fixed bijection of the 31-bit row ids; the row's set is
//                           h % num_sets; key[p] = set * Q + h / num_sets (Q = ceil(2^31 / num_sets):
//                           sorts by set first, equal keys <=> equal rows), value[p] = p
//   2. radix sort + run starts (CUB): equal rows adjacent, the rows of one set adjacent and
//                           ascending
//   3. cache_update_kernel: one lane group per set touched this step, one lane per way holding that
//                           way's tag / last-use / use-count in registers.  First every distinct
//                           row of the set is looked up (a hit refreshes the way), then the misses
//                           claim, in ascending key order, the least-recently (LRU) or
//                           least-frequently (LFU) used way not used in this step; ties go to the
//                           lowest way.  If no way is free the row stays uncached for this step.
//   4. cache_fill_kernel  : one warp per claimed way: the dirty victim row is written back to the
//                           host table, the new row is fetched into HBM
//   5. cache_locate_kernel: every lookup position learns where its row is: a cache slot or the host
//
// The cached forward / backward read rows through that per-position location.  The policy is
// deterministic, so tags, counters and hit counts can be compared exactly with a CPU model.
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#if defined(__x86_64__)
#include <emmintrin.h>
#endif

#include "tbe_plan.cuh"

namespace tbe {
namespace {

enum Policy { kLRU = 0, kLFU = 1 };

struct CacheArgs {
  // cache state
  void* cache_rows;
  int32_t* tags;       // [num_sets * ways] row id or -1
  int32_t* last_use;   // [num_sets * ways] step of the last lookup
  int32_t* use_count;  // [num_sets * ways] lookups steps since insertion (LFU)
  uint8_t* dirty;      // [num_sets * ways]
  void* host_rows;     // device-mapped host table
  // lookups
  const int32_t* table_offsets;
  const int32_t* indices;
  const int32_t* offsets;
  // plan scratch
  uint32_t* keys_in;
  int32_t* vals_in;
  const uint32_t* keys;
  const int32_t* vals;
  const int32_t* seg_starts;
  int32_t* counters;    // [0] runs, [2] claims, [3] hit lookups, [4] hit rows, [5] uncached rows
  int32_t* entry_bag;   // bag of every position
  int32_t* run_loc;     // per run: slot or -1
  int32_t* run_row;     // per run: the row id
  int4* claims;         // {slot, old_tag, new_row, 0}
  int32_t* loc;         // per position: slot or -1 (output)
  int32_t* loc_sorted;  // per sorted entry: slot or -1
  int32_t B, T, D, N;
  int32_t num_sets, ways_log2, Q;
  FastDiv div_sets, div_q;
  int32_t now, policy;
  int32_t nvec;
};

// A bijection of the 31-bit row ids (xor-shifts and odd multiplications are each invertible modulo
// 2^31).  Rows that differ by a multiple of the table size, or by any other regular stride, would
// otherwise fall into the same set whenever that stride shares a factor with num_sets.
__device__ __forceinline__ uint32_t mix_row(uint32_t x) {
  x ^= x >> 16;
  x = (x * 0x45d9f3bu) & 0x7fffffffu;
  x ^= x >> 16;
  x = (x * 0x45d9f3bu) & 0x7fffffffu;
  x ^= x >> 16;
  return x;
}
// Sort key: set first, then the rest of the mixed id -- equal keys <=> equal rows.
__device__ __forceinline__ uint32_t cache_key(const CacheArgs& a, uint32_t row) {
  const uint32_t h = mix_row(row);
  const uint32_t q = fastdiv(h, a.div_sets);
  const uint32_t set = h - q * static_cast<uint32_t>(a.num_sets);
  return set * static_cast<uint32_t>(a.Q) + q;
}
__device__ __forceinline__ uint32_t key_set(const CacheArgs& a, uint32_t key) { return fastdiv(key, a.div_q); }
// The row a sorted entry looks up, recomputed from its index position.
__device__ __forceinline__ uint32_t row_of_position(const CacheArgs& a, int pos) {
  const int bag = __ldg(a.entry_bag + pos);
  return static_cast<uint32_t>(__ldg(a.table_offsets + bag / a.B)) + static_cast<uint32_t>(__ldg(a.indices + pos));
}

__global__ void __launch_bounds__(256) cache_keys_kernel(const CacheArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int t = static_cast<int>(bag / a.B);
    const uint32_t row0 = static_cast<uint32_t>(__ldg(a.table_offsets + t));
    const int s = __ldg(a.offsets + bag), e = __ldg(a.offsets + bag + 1);
    for (int p = s + lane; p < e; p += 32) {
      a.keys_in[p] = cache_key(a, row0 + static_cast<uint32_t>(__ldg(a.indices + p)));
      a.vals_in[p] = p;
      a.entry_bag[p] = static_cast<int32_t>(bag);
    }
  }
}

// One group of `ways` lanes per run; the group whose run is the first of its set walks all runs of
// the set.
__global__ void __launch_bounds__(256) cache_update_kernel(const CacheArgs a) {
  const int ways = 1 << a.ways_log2;
  const int lane = threadIdx.x & 31;
  const int way = lane & (ways - 1);
  const int gpw = 32 >> a.ways_log2;
  const unsigned gmask = (ways == 32) ? kFullMask : (((1u << ways) - 1u) << (lane & ~(ways - 1)));
  const int U = a.counters[0];
  const int64_t gstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5) * gpw;
  for (int64_t u0 = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * gpw +
                    (lane >> a.ways_log2);
       u0 - (lane >> a.ways_log2) < U; u0 += gstride) {
    // (the loop bound is warp-uniform; groups past the end idle)
    bool leader = false;
    uint32_t set = 0;
    if (u0 < U) {
      set = key_set(a, __ldg(a.keys + __ldg(a.seg_starts + u0)));
      leader = u0 == 0 || key_set(a, __ldg(a.keys + __ldg(a.seg_starts + u0 - 1))) != set;
    }
    if (!leader) continue;
    // runs [u0, u1) belong to this set
    int u1 = static_cast<int>(u0) + 1;
    while (u1 < U && key_set(a, __ldg(a.keys + __ldg(a.seg_starts + u1))) == set) ++u1;
    const int slot = static_cast<int>(set) * ways + way;
    int32_t tag = a.tags[slot], used = a.last_use[slot], cnt = a.use_count[slot];
    int hit_lookups = 0, hit_rows = 0, uncached = 0;
    // pass 1: hits
    for (int u = static_cast<int>(u0); u < u1; ++u) {
      const int start = __ldg(a.seg_starts + u);
      const uint32_t r2 = row_of_position(a, __ldg(a.vals + start));
      if (way == 0) a.run_row[u] = static_cast<int32_t>(r2);
      const unsigned hit = __ballot_sync(gmask, tag == static_cast<int32_t>(r2)) & gmask;
      if (hit) {
        if (tag == static_cast<int32_t>(r2)) {
          used = a.now;
          cnt += 1;
        }
        const int hway = (__ffs(hit) - 1) & (ways - 1);
        if (way == 0) {
          a.run_loc[u] = static_cast<int>(set) * ways + hway;
          const int end = (u + 1 < U) ? __ldg(a.seg_starts + u + 1) : a.N;
          hit_lookups += end - start;
          hit_rows += 1;
        }
      } else if (way == 0) {
        a.run_loc[u] = -2;  // miss, decided in pass 2
      }
    }
    __syncwarp(gmask);
    // pass 2: misses claim a way, ascending row order
    for (int u = static_cast<int>(u0); u < u1; ++u) {
      const int state = a.run_loc[u];  // written by way 0 of this group above
      if (state != -2) continue;
      const uint32_t r2 = static_cast<uint32_t>(a.run_row[u]);
      // candidate order: empty ways first, then by policy, ties to the lowest way
      const bool free_now = used < a.now || tag < 0;
      const uint32_t prio = tag < 0 ? 0u : (a.policy == kLRU ? static_cast<uint32_t>(used) + 1u
                                                             : static_cast<uint32_t>(cnt) + 1u);
      uint64_t cand = free_now ? ((static_cast<uint64_t>(prio) << 8) | static_cast<uint64_t>(way)) : ~0ull;
      for (int m = 1; m < ways; m <<= 1) {
        const uint64_t other = __shfl_xor_sync(gmask, cand, m);
        cand = other < cand ? other : cand;
      }
      if (cand == ~0ull) {
        if (way == 0) {
          a.run_loc[u] = -1;
          uncached += 1;
        }
        continue;
      }
      const int vway = static_cast<int>(cand & 0xff);
      if (way == vway) {
        const int c = atomicAdd(a.counters + 2, 1);
        a.claims[c] = make_int4(slot, tag, static_cast<int>(r2), 0);
        tag = static_cast<int32_t>(r2);
        used = a.now;
        cnt = 1;
        a.run_loc[u] = slot;
      }
      __syncwarp(gmask);
    }
    a.tags[slot] = tag;
    a.last_use[slot] = used;
    a.use_count[slot] = cnt;
    if (way == 0) {
      if (hit_lookups) atomicAdd(a.counters + 3, hit_lookups);
      if (hit_rows) atomicAdd(a.counters + 4, hit_rows);
      if (uncached) atomicAdd(a.counters + 5, uncached);
    }
  }
}

// A lane group of 2^lpr_log2 lanes (one 16-byte vector each) owns a claim; a warp therefore works on
// 32 >> lpr_log2 claims at once and every group keeps kFillBatch claims in flight: all victim rows
// (HBM) and all new rows (host link) of a batch are requested before the first store, so the host
// link sees kFillBatch * 32 lanes of outstanding reads per warp instead of one row.  Claims never
// alias: a row fetched in this step was not cached, a row evicted in this step was not looked up.
constexpr int kFillBatch = 4;

//
// Write-backs can be deferred: with a staging buffer (wb_rows, one row per claim, in HBM) the dirty
// victim is copied there instead of to the host table, wb_ids[claim] records where it belongs (-1:
// nothing to write back), and cache_writeback_kernel carries the staged rows to the host later -- on
// another stream, under the lookup that follows -- so that only the fetches stay on the critical path
// of the host link.
//
// Staged fill (mode 1 and 2): the host link is fastest for the copy engines on contiguous buffers
// (55 GB/s against 13 GB/s for SM-issued random rows in an 80 GB table), so the rows can also travel
// through staging buffers: mode 1 only copies the dirty victims of claims [c_begin, c_begin + c_count)
// into wb_rows (and their row ids into wb_ids), mode 2 only inserts the new rows of those claims from
// in_rows, where the host has gathered them in claim order.  Staging slots are indexed by
// claim - c_begin.  Mode 0 is the direct fill over all claims (c_count < 0: the count is read from the
// plan's counters).
enum FillMode { kFillDirect = 0, kFillStageVictims = 1, kFillInsertStaged = 2 };

template <int VB>
__global__ void __launch_bounds__(256) cache_fill_kernel(const CacheArgs a, int64_t row_bytes, int lpr_log2,
                                                         char* __restrict__ wb_rows, int32_t* __restrict__ wb_ids,
                                                         const char* __restrict__ in_rows, int mode, int c_begin,
                                                         int c_count) {
  const int lpr = 1 << lpr_log2;
  const int sub = threadIdx.x & (lpr - 1);
  const int64_t group = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> lpr_log2;
  const int64_t ngroups = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> lpr_log2;
  const int nclaims = c_count >= 0 ? c_count : a.counters[2];
  const bool evict = mode != kFillInsertStaged, insert = mode != kFillStageVictims;
  for (int64_t c0 = group; c0 < nclaims; c0 += ngroups * kFillBatch) {
    int4 cl[kFillBatch];
    bool live[kFillBatch], back[kFillBatch];
#pragma unroll
    for (int u = 0; u < kFillBatch; ++u) {
      const int64_t c = c0 + u * ngroups;
      live[u] = c < nclaims;
      cl[u] = live[u] ? a.claims[c_begin + c] : make_int4(0, -1, 0, 0);
      back[u] = evict && live[u] && cl[u].y >= 0 && a.dirty[cl[u].x] != 0;
    }
    for (int v = sub; v < a.nvec; v += lpr) {
      Raw<VB> old_row[kFillBatch], new_row[kFillBatch];
#pragma unroll
      for (int u = 0; u < kFillBatch; ++u) {
        char* crow = static_cast<char*>(a.cache_rows) + static_cast<int64_t>(cl[u].x) * row_bytes;
        const char* nrow = in_rows != nullptr
                               ? in_rows + (c0 + static_cast<int64_t>(u) * ngroups) * row_bytes
                               : static_cast<const char*>(a.host_rows) + static_cast<int64_t>(cl[u].z) * row_bytes;
        old_row[u] = raw_zero<VB>();
        new_row[u] = raw_zero<VB>();
        if (back[u]) old_row[u] = ld_rw<VB>(crow + static_cast<int64_t>(v) * VB);
        if (insert && live[u]) new_row[u] = ld_stream<VB>(nrow + static_cast<int64_t>(v) * VB);
      }
#pragma unroll
      for (int u = 0; u < kFillBatch; ++u) {
        char* crow = static_cast<char*>(a.cache_rows) + static_cast<int64_t>(cl[u].x) * row_bytes;
        char* back_to = wb_rows != nullptr
                            ? wb_rows + (c0 + static_cast<int64_t>(u) * ngroups) * row_bytes
                            : static_cast<char*>(a.host_rows) + static_cast<int64_t>(cl[u].y) * row_bytes;
        if (back[u]) st_row<VB>(back_to + static_cast<int64_t>(v) * VB, old_row[u]);
        if (insert && live[u]) st_row<VB>(crow + static_cast<int64_t>(v) * VB, new_row[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kFillBatch; ++u) {
      if (live[u] && sub == 0) {
        if (evict) {
          a.dirty[cl[u].x] = 0;
          if (wb_ids != nullptr) wb_ids[c0 + static_cast<int64_t>(u) * ngroups] = back[u] ? cl[u].y : -1;
        }
      }
    }
  }
}

// Staged victim rows -> host table.  A small grid is enough: the host link, not the SMs, is the limit.
template <int VB>
__global__ void __launch_bounds__(256) cache_writeback_kernel(const char* __restrict__ wb_rows,
                                                              const int32_t* __restrict__ wb_ids,
                                                              const int32_t* __restrict__ nclaims_ptr, char* host_rows,
                                                              int64_t row_bytes, int nvec, int lpr_log2) {
  const int lpr = 1 << lpr_log2;
  const int sub = threadIdx.x & (lpr - 1);
  const int64_t group = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> lpr_log2;
  const int64_t ngroups = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> lpr_log2;
  const int nclaims = *nclaims_ptr;
  for (int64_t c0 = group; c0 < nclaims; c0 += ngroups * kFillBatch) {
    int32_t id[kFillBatch];
#pragma unroll
    for (int u = 0; u < kFillBatch; ++u) {
      const int64_t c = c0 + u * ngroups;
      id[u] = c < nclaims ? __ldg(wb_ids + c) : -1;
    }
    for (int v = sub; v < nvec; v += lpr) {
      Raw<VB> r[kFillBatch];
#pragma unroll
      for (int u = 0; u < kFillBatch; ++u) {
        r[u] = raw_zero<VB>();
        if (id[u] >= 0) r[u] = ld_stream<VB>(wb_rows + (c0 + static_cast<int64_t>(u) * ngroups) * row_bytes + static_cast<int64_t>(v) * VB);
      }
#pragma unroll
      for (int u = 0; u < kFillBatch; ++u)
        if (id[u] >= 0) st_row<VB>(host_rows + static_cast<int64_t>(id[u]) * row_bytes + static_cast<int64_t>(v) * VB, r[u]);
    }
  }
}

__global__ void __launch_bounds__(256) cache_locate_kernel(const CacheArgs a) {
  const int lane = threadIdx.x & 31;
  const int U = a.counters[0];
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); u < U; u += wstride) {
    const int s = __ldg(a.seg_starts + u);
    const int e = (u + 1 < U) ? __ldg(a.seg_starts + u + 1) : a.N;
    const int where = a.run_loc[u];
    for (int i = s + lane; i < e; i += 32) {
      a.loc_sorted[i] = where;
      a.loc[__ldg(a.vals + i)] = where;
    }
  }
}

// ------------------------------------------------------------------ cached forward / backward
struct CachedRowArgs {
  const void* cache_rows;
  const void* host_rows;
  const int32_t* table_offsets;
  const int32_t* indices;
  const int32_t* offsets;
  const int32_t* loc;
  void* out;
  int32_t B, T, D, nvec, mean;
};

// One warp per bag.  Every lane first resolves one lookup of the bag to the address of its row (the
// cache slot, or the host table when the row is uncached); a row is then fetched by a group of
// 2^lpr_log2 lanes, so a warp gathers 32 >> lpr_log2 rows per step and keeps four steps in flight.
template <typename T, int VB>
__global__ void __launch_bounds__(256) cached_forward_kernel(const CachedRowArgs a, int lpr_log2) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  constexpr int kInFlight = 4;
  const int lane = threadIdx.x & 31;
  const int lpr = 1 << lpr_log2;
  const int sub = lane & (lpr - 1);
  const int slot = lane >> lpr_log2;
  const int rps = 32 >> lpr_log2;  // rows per warp step
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int t = static_cast<int>(bag / a.B);
    const int b = static_cast<int>(bag - static_cast<int64_t>(t) * a.B);
    const uint32_t row0 = static_cast<uint32_t>(__ldg(a.table_offsets + t));
    const int s = __ldg(a.offsets + bag), e = __ldg(a.offsets + bag + 1);
    char* out = static_cast<char*>(a.out) + (static_cast<int64_t>(b) * a.T + t) * row_bytes;
    for (int c = 0; c * 32 < a.nvec; ++c) {  // rows wider than 32 vectors are walked in chunks (lpr = 32 then)
      const int v = c * 32 + sub;
      const bool vact = v < a.nvec;
      acc_t acc[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) acc[k] = 0;
      for (int base = s; base < e; base += 32) {
        const int p = base + lane;
        uint64_t rowp = 0;
        if (p < e) {
          const int where = __ldg(a.loc + p);
          rowp = where >= 0 ? reinterpret_cast<uint64_t>(a.cache_rows) + static_cast<uint64_t>(where) * row_bytes
                            : reinterpret_cast<uint64_t>(a.host_rows) +
                                  static_cast<uint64_t>(row0 + static_cast<uint32_t>(__ldg(a.indices + p))) * row_bytes;
        }
        const int cnt = min(32, e - base);
        for (int j0 = 0; j0 < cnt; j0 += rps * kInFlight) {
          Raw<VB> r[kInFlight];
#pragma unroll
          for (int u = 0; u < kInFlight; ++u) {
            const int j = j0 + u * rps + slot;
            const uint32_t lo = __shfl_sync(kFullMask, static_cast<uint32_t>(rowp), j & 31);
            const uint32_t hi = __shfl_sync(kFullMask, static_cast<uint32_t>(rowp >> 32), j & 31);
            const char* row = reinterpret_cast<const char*>((static_cast<uint64_t>(hi) << 32) | lo);
            r[u] = raw_zero<VB>();
            if (j < cnt && vact) r[u] = ld_rw<VB>(row + static_cast<int64_t>(v) * VB);
          }
#pragma unroll
          for (int u = 0; u < kInFlight; ++u) accumulate<T, VB>(r[u], acc);
        }
      }
      for (int m = lpr; m < 32; m <<= 1) {  // fold the row slots of the warp together
#pragma unroll
        for (int k = 0; k < NE; ++k) acc[k] += __shfl_xor_sync(kFullMask, acc[k], m);
      }
      if (a.mean && e > s) {
#pragma unroll
        for (int k = 0; k < NE; ++k) acc[k] = acc[k] / static_cast<acc_t>(e - s);
      }
      if (slot == 0 && vact) st_row<VB>(out + static_cast<int64_t>(v) * VB, pack_rn<T, VB>(acc));
    }
  }
}

struct CachedSgdArgs {
  void* cache_rows;
  void* host_rows;
  uint8_t* dirty;
  const void* grad;
  int64_t stride_b, stride_t;
  const uint32_t* keys;
  const int32_t* vals;
  const int32_t* seg_starts;
  const int32_t* counters;
  const int32_t* entry_bag;
  const int32_t* loc_sorted;
  const int32_t* run_row;
  const int32_t* offsets;
  int2* long_list;      // runs longer than kLongCachedRun, handled by a whole CTA each
  int32_t* long_count;
  // long runs cut into parts (0 = off): a part is split_len entries, the last one up to twice that
  int32_t split_len, max_parts;
  int4* part_list;       // {first entry, end entry, list index of the run's first part, parts of the run}
  int32_t* part_run;     // at the list index of a run's first part: the run
  int32_t* part_count;
  int32_t* part_tickets; // at the list index of a run's first part: parts finished so far
  float* part_sums;      // [max_parts][D]
  int32_t B, D, N, nvec, mean;
  int32_t lpr_log2;     // lanes per row in the long-run kernel
  float lr;
};

constexpr int kLongCachedRun = 64;

// Gradient row of a bag, vector v, and 1/L of the bag for mean pooling.
template <typename T, int VB>
__device__ __forceinline__ Raw<VB> cached_grad(const CachedSgdArgs& a, int bag, int v, typename Acc<T>::type* scale) {
  using acc_t = typename Acc<T>::type;
  const int t = bag / a.B;
  const int b = bag - t * a.B;
  *scale = 1;
  if (a.mean) *scale = acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag));
  return ld_stream<VB>(static_cast<const char*>(a.grad) +
                       (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                           static_cast<int64_t>(sizeof(T)) +
                       static_cast<int64_t>(v) * VB);
}

template <typename T, int VB>
__global__ void __launch_bounds__(256) cached_sgd_kernel(const CachedSgdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int U = __ldg(a.counters);
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  for (int64_t run = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); run < U;
       run += wstride) {
    const int s = __ldg(a.seg_starts + run);
    const int e = (run + 1 < U) ? __ldg(a.seg_starts + run + 1) : a.N;
    if (e - s > kLongCachedRun) {  // a hot row: queued for the CTA-per-run kernel, cut into parts if very long
      if (lane == 0) {
        a.long_list[atomicAdd(a.long_count, 1)] = make_int2(static_cast<int>(run), 0);
        const int plen = a.split_len;
        if (plen > 0 && e - s >= 2 * plen) {
          const int nparts = (e - s) / plen;
          const int base = atomicAdd(a.part_count, nparts);  // at most N / split_len parts exist in total
          a.part_tickets[base] = 0;
          a.part_run[base] = static_cast<int>(run);
          for (int k = 0; k < nparts; ++k) {
            const int ps = s + k * plen;
            a.part_list[base + k] = make_int4(ps, k == nparts - 1 ? e : ps + plen, base, nparts);
          }
        }
      }
      continue;
    }
    const int where = __ldg(a.loc_sorted + s);
    char* w;
    if (where >= 0) {
      w = static_cast<char*>(a.cache_rows) + static_cast<int64_t>(where) * row_bytes;
      if (lane == 0) a.dirty[where] = 1;
    } else {
      w = static_cast<char*>(a.host_rows) + static_cast<int64_t>(__ldg(a.run_row + run)) * row_bytes;
    }
    for (int v = lane; v < a.nvec; v += 32) {
      acc_t acc[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) acc[k] = 0;
      for (int i = s; i < e; ++i) {
        const int bag = __ldg(a.entry_bag + __ldg(a.vals + i));
        const int t = bag / a.B;
        const int b = bag - t * a.B;
        acc_t g[NE];
        unpack<T, VB>(ld_stream<VB>(static_cast<const char*>(a.grad) +
                                    (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                                        static_cast<int64_t>(sizeof(T)) +
                                    static_cast<int64_t>(v) * VB),
                      g);
        acc_t scale = 1;
        if (a.mean) scale = acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag));
#pragma unroll
        for (int k = 0; k < NE; ++k) acc[k] += g[k] * scale;
      }
      acc_t x[NE];
      unpack<T, VB>(ld_rw<VB>(w + static_cast<int64_t>(v) * VB), x);
#pragma unroll
      for (int k = 0; k < NE; ++k) x[k] -= acc[k] * static_cast<acc_t>(a.lr);
      st_row<VB>(w + static_cast<int64_t>(v) * VB, pack_rn<T, VB>(x));
    }
  }
}

// Queued long runs.  A run is taken 256 entries at a time: every thread first turns one sorted entry
// into the address of its gradient row (and 1/L for mean pooling) and leaves it in shared memory, so
// that the row loads that follow depend on nothing but shared memory; lane groups of lpr lanes then
// sum entries g, g + G, ... with eight loads in flight each, and the groups' partial sums are folded
// in group order in shared memory.  A run shorter than two parts gets one CTA.  A longer one (the
// hottest row of a Zipf table takes a sixth of the table's lookups) was cut into parts when it was
// queued: any CTA sums a part into an fp32 partial, and the CTA that finishes a run's last outstanding
// part (a ticket per run) adds the partials in part order and updates the row.  Every order of
// summation is fixed by the sorted order and the part boundaries, never by scheduling.
template <typename T, int VB>
__global__ void __launch_bounds__(256) cached_sgd_long_kernel(const CachedSgdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  constexpr int kInFlight = 8;
  __shared__ acc_t part[256 * NE];
  __shared__ int64_t entry_off[256];
  __shared__ acc_t entry_scale[256];
  __shared__ int ticket;
  const int lpr = 1 << a.lpr_log2;
  const int sub = threadIdx.x & (lpr - 1);
  const int gid = threadIdx.x >> a.lpr_log2;
  const int G = blockDim.x >> a.lpr_log2;
  const int U = __ldg(a.counters);
  const int nlong = *a.long_count;
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);

  // sum of chunk c of the gradient rows of sorted entries [s, e); the threads of group 0 receive it
  auto sum_range = [&](int c, int s, int e, acc_t* tot) {
    const int v = c * lpr + sub;
    const bool vact = v < a.nvec;
    acc_t acc[NE];
#pragma unroll
    for (int k = 0; k < NE; ++k) acc[k] = 0;
    for (int base = s; base < e; base += 256) {
      const int m = min(256, e - base);
      __syncthreads();  // the previous block of entries has been consumed
      if (static_cast<int>(threadIdx.x) < m) {
        const int bag = __ldg(a.entry_bag + __ldg(a.vals + base + threadIdx.x));
        const int t = bag / a.B;
        const int b = bag - t * a.B;
        entry_off[threadIdx.x] = (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) *
                                 static_cast<int64_t>(sizeof(T));
        entry_scale[threadIdx.x] =
            a.mean ? acc_t(1) / static_cast<acc_t>(__ldg(a.offsets + bag + 1) - __ldg(a.offsets + bag)) : acc_t(1);
      }
      __syncthreads();
      for (int i = gid; i < m; i += G * kInFlight) {
        Raw<VB> r[kInFlight];
        acc_t sc[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const int iu = i + u * G;
          r[u] = raw_zero<VB>();
          sc[u] = 1;
          if (iu < m && vact) {
            r[u] = ld_stream<VB>(static_cast<const char*>(a.grad) + entry_off[iu] + static_cast<int64_t>(v) * VB);
            sc[u] = entry_scale[iu];
          }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          acc_t g[NE];
          unpack<T, VB>(r[u], g);
#pragma unroll
          for (int k = 0; k < NE; ++k) acc[k] += g[k] * sc[u];
        }
      }
    }
    __syncthreads();  // the previous use of `part` has been consumed
#pragma unroll
    for (int k = 0; k < NE; ++k) part[threadIdx.x * NE + k] = acc[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NE; ++k) tot[k] = 0;
    if (gid == 0 && vact) {
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int k = 0; k < NE; ++k) tot[k] += part[(g * lpr + sub) * NE + k];
      }
    }
  };
  // row -= lr * total, chunk by chunk; the row lives in the cache (marked dirty) or in the host table
  auto update_row = [&](int run, int s, auto&& chunk_total) {
    const int where = __ldg(a.loc_sorted + s);
    char* w = where >= 0 ? static_cast<char*>(a.cache_rows) + static_cast<int64_t>(where) * row_bytes
                         : static_cast<char*>(a.host_rows) + static_cast<int64_t>(__ldg(a.run_row + run)) * row_bytes;
    if (threadIdx.x == 0 && where >= 0) a.dirty[where] = 1;
    for (int c = 0; c * lpr < a.nvec; ++c) {
      const int v = c * lpr + sub;
      acc_t tot[NE];
      chunk_total(c, tot);
      if (gid == 0 && v < a.nvec) {
        acc_t x[NE];
        unpack<T, VB>(ld_rw<VB>(w + static_cast<int64_t>(v) * VB), x);
#pragma unroll
        for (int k = 0; k < NE; ++k) x[k] -= tot[k] * static_cast<acc_t>(a.lr);
        st_row<VB>(w + static_cast<int64_t>(v) * VB, pack_rn<T, VB>(x));
      }
    }
  };

  for (int li = blockIdx.x; li < nlong; li += gridDim.x) {
    const int run = a.long_list[li].x;
    const int s = __ldg(a.seg_starts + run);
    const int e = (run + 1 < U) ? __ldg(a.seg_starts + run + 1) : a.N;
    if (a.split_len > 0 && e - s >= 2 * a.split_len) continue;  // cut into parts: below
    update_row(run, s, [&](int c, acc_t* tot) { sum_range(c, s, e, tot); });
  }
  if (a.split_len <= 0) return;
  const int nparts_total = min(*a.part_count, a.max_parts);
  for (int p = blockIdx.x; p < nparts_total; p += gridDim.x) {
    const int4 pm = a.part_list[p];  // {first entry, end entry, list index of the run's first part, parts of the run}
    float* mine = a.part_sums + static_cast<int64_t>(p) * a.D;
    for (int c = 0; c * lpr < a.nvec; ++c) {
      acc_t tot[NE];
      sum_range(c, pm.x, pm.y, tot);
      const int v = c * lpr + sub;
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
    const int4 first = a.part_list[pm.z];
    const int run = a.part_run[pm.z];
    update_row(run, first.x, [&](int c, acc_t* tot) {
      const int v = c * lpr + sub;
#pragma unroll
      for (int k = 0; k < NE; ++k) tot[k] = 0;
      if (gid == 0 && v < a.nvec) {
        for (int part_i = 0; part_i < pm.w; ++part_i) {  // part order: fixed
          const float* ps = a.part_sums + static_cast<int64_t>(pm.z + part_i) * a.D + v * NE;
#pragma unroll
          for (int k = 0; k < NE; ++k) tot[k] += static_cast<acc_t>(__ldcg(ps + k));
        }
      }
    });
  }
}

template <int VB>
__global__ void __launch_bounds__(256) cache_flush_kernel(void* cache_rows, void* host_rows, const int32_t* tags,
                                                         uint8_t* dirty, int64_t slots, int64_t row_bytes, int nvec) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t slot = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < slots;
       slot += wstride) {
    const int tag = tags[slot];
    if (tag < 0 || !dirty[slot]) continue;
    const char* c = static_cast<const char*>(cache_rows) + slot * row_bytes;
    char* h = static_cast<char*>(host_rows) + static_cast<int64_t>(tag) * row_bytes;
    for (int v = lane; v < nvec; v += 32) st_row<VB>(h + v * VB, ld_rw<VB>(c + v * VB));
    __syncwarp();
    if (lane == 0) dirty[slot] = 0;
  }
}

// Scratch layout: the sort workspace of the backward followed by the cache's own arrays.
struct CacheScratch {
  Workspace ws;
  int32_t* run_loc;
  int32_t* run_row;
  int32_t* loc_sorted;
  int4* claims;
  size_t total;
};

int carve_cache(void* base, int64_t N, int64_t total_rows, CacheScratch* cs) {
  int rc = carve(base, N, total_rows, &cs->ws);
  if (rc != TBE_OK) return rc;
  char* p = static_cast<char*>(base);
  size_t off = align_up(cs->ws.total, 256);
  auto take = [&](size_t bytes) {
    void* r = p ? p + off : nullptr;
    off += align_up(bytes, 256);
    return r;
  };
  const size_t n = static_cast<size_t>(N > 0 ? N : 1);
  cs->run_loc = static_cast<int32_t*>(take(n * 4));
  cs->run_row = static_cast<int32_t*>(take(n * 4));
  cs->loc_sorted = static_cast<int32_t*>(take(n * 4));
  cs->claims = static_cast<int4*>(take(n * sizeof(int4)));
  cs->total = off;
  return TBE_OK;
}

int grid_for(int64_t warps) {
  int64_t blocks = (warps + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

int vector_bytes(const char* who, int64_t D, int dtype, const void* p0, const void* p1, const void* p2, int* vb,
                 int* nvec) {
  const RowGeom g = make_geom(D, dtype, p0, p1);
  int v = g.vb;
  if (reinterpret_cast<uintptr_t>(p2) % 16 != 0) v = 8;
  if (v == 8 && dtype != TBE_F16) return fail(TBE_ERR_INVALID_ARGUMENT, "%s: rows must be 16-byte aligned", who);
  if (v == 8 && (reinterpret_cast<uintptr_t>(p0) % 8 || reinterpret_cast<uintptr_t>(p1) % 8 ||
                 reinterpret_cast<uintptr_t>(p2) % 8))
    return fail(TBE_ERR_INVALID_ARGUMENT, "%s: rows must be 8-byte aligned", who);
  *vb = v;
  *nvec = static_cast<int>(D * elem_size(dtype) / v);
  return TBE_OK;
}

}  // namespace
}  // namespace tbe

extern "C" int64_t tbe_cache_workspace_bytes(int64_t N, int64_t total_rows) {
  if (N < 0 || total_rows <= 0) return tbe::fail(TBE_ERR_INVALID_ARGUMENT, "tbe_cache_workspace_bytes: bad sizes");
  tbe::CacheScratch cs;
  const int rc = tbe::carve_cache(nullptr, N, total_rows, &cs);
  if (rc != TBE_OK) return rc;
  return static_cast<int64_t>(cs.total);
}

namespace tbe {
namespace {

// Worker threads for the host side of the staged fill (row gather / scatter in the host table).  One
// pool per process, created on first use and never destroyed (the workers sleep between calls and must
// not be joined during static destruction); parallel_for calls are serialised.  A job is done when all
// of its items are, not when every worker has looked at it: a worker that wakes up late finds nothing
// left and the caller has long returned (waking a sleeping thread takes longer than a whole gather).
// Workers spin for a moment after a job before they go to sleep, which is how the scatter that follows
// the gather a fraction of a millisecond later finds them awake.
class HostPool {
 public:
  static HostPool& get() {
    static HostPool* pool = [] {
      HostPool* p = new HostPool();
      existing_.store(p, std::memory_order_release);
      return p;
    }();
    return *pool;
  }
  static HostPool* existing() { return existing_.load(std::memory_order_acquire); }  // null until first used
  // fn(begin, end) over [0, n) in chunks, on the workers and the calling thread; returns when all of it is done
  void parallel_for(int64_t n, const std::function<void(int64_t, int64_t)>& fn) {
    if (n <= 0) return;
    std::lock_guard<std::mutex> one_call(call_mu_);
    finish_background();
    auto job = publish(n, &fn);
    run(job.get());
    while (job->done.load(std::memory_order_acquire) < n) relax();
  }
  // The same on the workers alone (the caller too, if there are none): returns at once; wait() or
  // the next parallel_for / start waits for it.  `fn` is kept until then.
  void start(int64_t n, std::function<void(int64_t, int64_t)> fn) {
    if (n <= 0) return;
    std::lock_guard<std::mutex> one_call(call_mu_);
    finish_background();
    background_fn_ = std::move(fn);
    background_ = publish(n, &background_fn_);
    if (workers_ == 0) finish_background();
  }
  void wait() {
    std::lock_guard<std::mutex> one_call(call_mu_);
    finish_background();
  }

 private:
  struct Job {
    const std::function<void(int64_t, int64_t)>* fn = nullptr;
    int64_t n = 0, chunk = 1;
    std::atomic<int64_t> next{0}, done{0};
  };
  std::shared_ptr<Job> publish(int64_t n, const std::function<void(int64_t, int64_t)>* fn) {
    auto job = std::make_shared<Job>();
    job->fn = fn;
    job->n = n;
    const int64_t parts = 8 * (static_cast<int64_t>(workers_) + 1);
    job->chunk = (n + parts - 1) / parts;
    if (job->chunk < 64) job->chunk = 64;
    {
      std::lock_guard<std::mutex> lk(mu_);
      job_ = job;
      generation_.fetch_add(1, std::memory_order_release);
    }
    cv_work_.notify_all();
    return job;
  }
  void finish_background() {  // (call_mu_ held) helps with what is left of the background job, then waits for it
    if (!background_) return;
    run(background_.get());
    while (background_->done.load(std::memory_order_acquire) < background_->n) relax();
    background_.reset();
    background_fn_ = nullptr;
  }
  static void relax() {
#if defined(__x86_64__)
    _mm_pause();
#else
    std::this_thread::yield();
#endif
  }
  HostPool() {
    const unsigned hc = std::thread::hardware_concurrency();
    // (two cores stay free for the caller's launching thread and its autograd thread)
    workers_ = hc > 3 ? (hc - 2 < 15 ? hc - 2 : 15) : (hc > 1 ? 1 : 0);
    for (unsigned i = 0; i < workers_; ++i) std::thread([this] { loop(); }).detach();
  }
  void loop() {
    uint64_t seen = 0;
    for (;;) {
      for (int spin = 0; generation_.load(std::memory_order_acquire) == seen; ++spin) {
        if (spin < 4000) {  // ~0.2 ms: the pieces of a gather follow each other closely, the scatter soon after
          relax();
        } else {
          std::unique_lock<std::mutex> lk(mu_);
          cv_work_.wait(lk, [&] { return generation_.load(std::memory_order_acquire) != seen; });
        }
      }
      std::shared_ptr<Job> job;
      {
        std::lock_guard<std::mutex> lk(mu_);
        job = job_;
        seen = generation_.load(std::memory_order_acquire);
      }
      if (job) run(job.get());
    }
  }
  static void run(Job* job) {
    for (;;) {
      const int64_t b = job->next.fetch_add(job->chunk);
      if (b >= job->n) break;  // (a finished job's function is never called again: it may be gone)
      const int64_t e = b + job->chunk < job->n ? b + job->chunk : job->n;
      (*job->fn)(b, e);
      job->done.fetch_add(e - b, std::memory_order_release);
    }
  }
  static std::atomic<HostPool*> existing_;
  std::mutex call_mu_, mu_;
  std::condition_variable cv_work_;
  std::shared_ptr<Job> job_, background_;
  std::function<void(int64_t, int64_t)> background_fn_;
  std::atomic<uint64_t> generation_{0};
  unsigned workers_ = 0;
};

std::atomic<HostPool*> HostPool::existing_{nullptr};

// A whole row written into the host table.  The row is overwritten completely and not read again by
// this thread, so on x86-64 it goes out with streaming stores: no read-for-ownership of lines that
// are cache misses by construction (random rows of a table far larger than the caches).
inline void store_row(char* dst, const char* src, int64_t row_bytes) {
#if defined(__x86_64__)
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(row_bytes)) & 15) == 0) {
    const __m128i* s = reinterpret_cast<const __m128i*>(src);
    __m128i* d = reinterpret_cast<__m128i*>(dst);
    for (int64_t k = 0; k < row_bytes / 16; ++k) _mm_stream_si128(d + k, _mm_load_si128(s + k));
    return;
  }
#endif
  std::memcpy(dst, src, static_cast<size_t>(row_bytes));
}
inline void rows_stored() {
#if defined(__x86_64__)
  _mm_sfence();
#endif
}

// Staging for the fill through the copy engines (tbe_cache_prefetch_staged).
constexpr int kStagePieces = 4;  // the gather of a round hands its rows to the copy engine in this many pieces

struct StagedFill {
  char* host_table;    // the table's address on the host
  char* stage_dev;     // device: [rows out][rows in][int32 ids], `rows` slots each
  char* stage_host;    // pinned host memory of the same layout, then int4 claims[rows] and 16 counters
  int64_t rows;        // claims per round
};

int64_t stage_bytes_device(int64_t rows, int64_t row_bytes) { return rows * (2 * row_bytes + 4); }
int64_t stage_bytes_host(int64_t rows, int64_t row_bytes) { return rows * (2 * row_bytes + 4 + 16) + 64; }

// A side stream (and two events) per device for the device-to-host half of a staged fill, so that it
// runs beside the host-to-device half instead of in front of it.
struct StageStreams {
  cudaStream_t out = nullptr;
  cudaEvent_t staged = nullptr, arrived = nullptr, claims = nullptr;
  std::mutex in_use;  // staged fills on one device take turns (they share the stream and the events)
};
int stage_streams(StageStreams** res) {
  static StageStreams per_device[64];
  static std::mutex mu;
  int dev = 0;
  TBE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(TBE_ERR_UNSUPPORTED, "staged cache fill: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  StageStreams& s = per_device[dev];
  if (s.out == nullptr) {
    TBE_CUDA_TRY(cudaStreamCreateWithFlags(&s.out, cudaStreamNonBlocking));
    TBE_CUDA_TRY(cudaEventCreateWithFlags(&s.staged, cudaEventDisableTiming));
    TBE_CUDA_TRY(cudaEventCreateWithFlags(&s.arrived, cudaEventDisableTiming));
    TBE_CUDA_TRY(cudaEventCreateWithFlags(&s.claims, cudaEventDisableTiming));
  }
  *res = &s;
  return TBE_OK;
}

}  // namespace

void host_pool_wait() {
  if (HostPool* pool = HostPool::existing()) pool->wait();  // (never creates the threads)
}

namespace {

int cache_prefetch_impl(const char* who, void* cache_rows, int32_t* tags, int32_t* last_use, int32_t* use_count,
                        uint8_t* dirty, void* host_rows, const int32_t* table_offsets, const int32_t* indices,
                        const int32_t* offsets, int32_t* locations, int32_t* stats, int64_t T, int64_t B, int64_t D,
                        int64_t N, int64_t total_rows, int64_t num_sets, int ways, int dtype, int policy, int now,
                        void* writeback_rows, int32_t* writeback_ids, const StagedFill* staged, void* workspace,
                        int64_t workspace_bytes, void* stream_v) {
  TBE_REQUIRE((writeback_rows == nullptr) == (writeback_ids == nullptr),
              "%s: writeback_rows and writeback_ids go together", who);
  TBE_REQUIRE(cache_rows && tags && last_use && use_count && dirty && host_rows && table_offsets && offsets &&
                  locations && stats && (indices || N == 0),
              "%s: null pointer argument", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  TBE_REQUIRE(D > 0 && D % 4 == 0, "%s: D must be a positive multiple of 4", who);
  TBE_REQUIRE(ways >= 1 && ways <= 32 && (ways & (ways - 1)) == 0, "%s: ways must be a power of two <= 32", who);
  TBE_REQUIRE(num_sets >= 1 && num_sets * ways < (1ll << 31), "%s: bad num_sets", who);
  TBE_REQUIRE(policy == kLRU || policy == kLFU, "%s: policy must be 0 (LRU) or 1 (LFU)", who);
  TBE_REQUIRE(now > 0, "%s: the step counter must start at 1", who);
  const int64_t Q = ((1ll << 31) + num_sets - 1) / num_sets;  // mixed row ids span 31 bits
  TBE_REQUIRE(num_sets * Q < (1ll << 32), "%s: num_sets too large for 32-bit sort keys", who);
  TBE_REQUIRE(workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
              "%s: workspace must be non-null and 256-byte aligned", who);
  CacheScratch cs;
  rc = carve_cache(workspace, N, total_rows, &cs);
  if (rc != TBE_OK) return rc;
  if (static_cast<int64_t>(cs.total) > workspace_bytes)
    return fail(TBE_ERR_WORKSPACE_TOO_SMALL, "%s: workspace has %lld bytes, %lld needed", who,
                (long long)workspace_bytes, (long long)cs.total);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // victims of an earlier staged prefetch that are still on their way into the host table must be
  // there before this step fetches from it (by either path)
  host_pool_wait();
  TBE_CUDA_TRY(cudaMemsetAsync(cs.ws.counters, 0, 64, stream));
  if (N == 0) {
    TBE_CUDA_TRY(cudaMemsetAsync(stats, 0, 5 * sizeof(int32_t), stream));
    return TBE_OK;
  }
  int vb = 16, nvec = 0;
  rc = vector_bytes(who, D, dtype, cache_rows, host_rows, nullptr, &vb, &nvec);
  if (rc != TBE_OK) return rc;

  CacheArgs a{};
  a.cache_rows = cache_rows;
  a.tags = tags;
  a.last_use = last_use;
  a.use_count = use_count;
  a.dirty = dirty;
  a.host_rows = host_rows;
  a.table_offsets = table_offsets;
  a.indices = indices;
  a.offsets = offsets;
  a.keys_in = cs.ws.keys_in;
  a.vals_in = cs.ws.vals_in;
  a.keys = cs.ws.keys;
  a.vals = cs.ws.vals;
  a.seg_starts = cs.ws.seg_starts;
  a.counters = cs.ws.counters;
  a.entry_bag = cs.ws.entry_bag;
  a.run_loc = cs.run_loc;
  a.run_row = cs.run_row;
  a.claims = cs.claims;
  a.loc = locations;
  a.loc_sorted = cs.loc_sorted;
  a.B = static_cast<int32_t>(B);
  a.T = static_cast<int32_t>(T);
  a.D = static_cast<int32_t>(D);
  a.N = static_cast<int32_t>(N);
  a.num_sets = static_cast<int32_t>(num_sets);
  int wl = 0;
  while ((1 << wl) < ways) ++wl;
  a.ways_log2 = wl;
  a.Q = static_cast<int32_t>(Q);
  a.div_sets = make_fastdiv(static_cast<uint32_t>(num_sets));
  a.div_q = make_fastdiv(static_cast<uint32_t>(Q));
  a.now = now;
  a.policy = policy;
  a.nvec = nvec;

  {
    KernelTimer timer("cache_keys_kernel", stream);
    cache_keys_kernel<<<grid_for(T * B), 256, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("cache_keys_kernel");
  int bits = 1;
  while (bits < 32 && (1ll << bits) < num_sets * Q) ++bits;
  rc = sort_pairs(cs.ws, N, bits, stream);
  if (rc != TBE_OK) return rc;
  rc = select_run_starts(cs.ws, N, stream);
  if (rc != TBE_OK) return rc;
  {
    KernelTimer timer("cache_update_kernel", stream);
    const int gpw = 32 / ways;
    cache_update_kernel<<<grid_for((N + gpw - 1) / gpw), 256, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("cache_update_kernel");
  const int64_t row_bytes = D * elem_size(dtype);
  int fill_lpr_log2 = 0;
  while ((1 << fill_lpr_log2) < nvec && fill_lpr_log2 < 5) ++fill_lpr_log2;
  auto launch_fill = [&](char* wb_rows, int32_t* wb_ids, const char* in_rows, int mode, int c_begin, int c_count,
                         int64_t work) {
    KernelTimer timer(mode == kFillDirect ? "cache_fill_kernel"
                      : mode == kFillStageVictims ? "cache_stage_victims_kernel" : "cache_insert_staged_kernel",
                      stream);
    if (vb == 16) {
      cache_fill_kernel<16><<<grid_for(work), 256, 0, stream>>>(a, row_bytes, fill_lpr_log2, wb_rows, wb_ids, in_rows,
                                                                mode, c_begin, c_count);
    } else {
      cache_fill_kernel<8><<<grid_for(work), 256, 0, stream>>>(a, row_bytes, fill_lpr_log2, wb_rows, wb_ids, in_rows,
                                                               mode, c_begin, c_count);
    }
  };
  if (staged == nullptr) {
    launch_fill(static_cast<char*>(writeback_rows), writeback_ids, nullptr, kFillDirect, 0, -1, N);
  } else {
    // The host has to know how many claims there are: this is the one place where the call waits for
    // the stream.  Per round of up to `rows` claims: the dirty victims are staged on the device and
    // leave through the copy engine on a side stream; meanwhile the host gathers the new rows from
    // the table into pinned staging, a quarter of the round at a time, each quarter following the
    // one before through the copy engine on the caller's stream; a kernel inserts them.  The victims
    // that have arrived are scattered into the table by the workers in the background, under the
    // lookup and the update that the caller launches next: an evicted row is not looked up in the
    // step that evicted it.  The next staged prefetch, tbe_cache_flush and tbe_free_host_mapped wait
    // for that scatter.
    StageStreams* ss = nullptr;
    rc = stage_streams(&ss);
    if (rc != TBE_OK) return rc;
    std::lock_guard<std::mutex> one_fill(ss->in_use);
    const int64_t R = staged->rows;
    char* d_out = staged->stage_dev;
    char* d_in = d_out + R * row_bytes;
    int32_t* d_ids = reinterpret_cast<int32_t*>(d_in + R * row_bytes);
    char* h_out = staged->stage_host;
    char* h_in = h_out + R * row_bytes;
    int32_t* h_ids = reinterpret_cast<int32_t*>(h_in + R * row_bytes);
    int4* h_claims = reinterpret_cast<int4*>(reinterpret_cast<char*>(h_ids) + R * 4);
    int32_t* h_counters = reinterpret_cast<int32_t*>(h_claims + R);
    TBE_CUDA_TRY(cudaMemcpyAsync(h_counters, cs.ws.counters, 64, cudaMemcpyDeviceToHost, stream));
    TBE_CUDA_TRY(cudaStreamSynchronize(stream));
    const int64_t nclaims = h_counters[2];
    HostPool& pool = HostPool::get();
    char* table = staged->host_table;
    for (int64_t c0 = 0; c0 < nclaims; c0 += R) {
      const int64_t n = nclaims - c0 < R ? nclaims - c0 : R;
      launch_fill(d_out, d_ids, nullptr, kFillStageVictims, static_cast<int>(c0), static_cast<int>(n), n);
      TBE_CHECK_LAUNCH("cache_stage_victims_kernel");
      TBE_CUDA_TRY(cudaEventRecord(ss->staged, stream));
      TBE_CUDA_TRY(cudaMemcpyAsync(h_claims, a.claims + c0, n * sizeof(int4), cudaMemcpyDeviceToHost, stream));
      TBE_CUDA_TRY(cudaEventRecord(ss->claims, stream));
      TBE_CUDA_TRY(cudaEventSynchronize(ss->claims));
      // (the victims' copy is enqueued only now: it would otherwise be served before the small copy of
      // the claims, which the host is waiting for)
      TBE_CUDA_TRY(cudaStreamWaitEvent(ss->out, ss->staged, 0));
      TBE_CUDA_TRY(cudaMemcpyAsync(h_ids, d_ids, n * 4, cudaMemcpyDeviceToHost, ss->out));
      TBE_CUDA_TRY(cudaMemcpyAsync(h_out, d_out, n * row_bytes, cudaMemcpyDeviceToHost, ss->out));
      TBE_CUDA_TRY(cudaEventRecord(ss->arrived, ss->out));
      const int64_t piece = (n + kStagePieces - 1) / kStagePieces;
      for (int64_t p0 = 0; p0 < n; p0 += piece) {
        const int64_t p1 = p0 + piece < n ? p0 + piece : n;
        pool.parallel_for(p1 - p0, [&](int64_t lo, int64_t hi) {  // gather the new rows in claim order
          for (int64_t i = p0 + lo; i < p0 + hi; ++i) {
            if (i + 8 < p0 + hi) {
              const char* ahead = table + static_cast<int64_t>(h_claims[i + 8].z) * row_bytes;
              for (int64_t o = 0; o < row_bytes; o += 64) __builtin_prefetch(ahead + o, 0, 0);
            }
            std::memcpy(h_in + i * row_bytes, table + static_cast<int64_t>(h_claims[i].z) * row_bytes,
                        static_cast<size_t>(row_bytes));
          }
        });
        TBE_CUDA_TRY(cudaMemcpyAsync(d_in + p0 * row_bytes, h_in + p0 * row_bytes, (p1 - p0) * row_bytes,
                                     cudaMemcpyHostToDevice, stream));
      }
      launch_fill(nullptr, nullptr, d_in, kFillInsertStaged, static_cast<int>(c0), static_cast<int>(n), n);
      TBE_CHECK_LAUNCH("cache_insert_staged_kernel");
      TBE_CUDA_TRY(cudaEventSynchronize(ss->arrived));
      auto scatter = [table, h_out, h_ids, row_bytes](int64_t lo, int64_t hi) {  // the victims that were dirty
        for (int64_t i = lo; i < hi; ++i) {
          const int32_t row = h_ids[i];
          if (row >= 0) store_row(table + static_cast<int64_t>(row) * row_bytes, h_out + i * row_bytes, row_bytes);
        }
        rows_stored();
      };
      if (c0 + R < nclaims) {
        // another round reuses the staging buffers: finish this one first (the insert kernel must
        // have read d_in, the scatter h_out)
        pool.parallel_for(n, scatter);
        TBE_CUDA_TRY(cudaStreamSynchronize(stream));
      } else {
        pool.start(n, scatter);
      }
    }
  }
  TBE_CHECK_LAUNCH("cache_fill_kernel");
  {
    KernelTimer timer("cache_locate_kernel", stream);
    cache_locate_kernel<<<grid_for(N), 256, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("cache_locate_kernel");
  // stats: {distinct rows, rows fetched into the cache, lookups served by rows already cached,
  //         distinct rows already cached, distinct rows left uncached}
  TBE_CUDA_TRY(cudaMemcpyAsync(stats, cs.ws.counters, 4, cudaMemcpyDeviceToDevice, stream));
  TBE_CUDA_TRY(cudaMemcpyAsync(stats + 1, cs.ws.counters + 2, 16, cudaMemcpyDeviceToDevice, stream));
  return TBE_OK;
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_cache_prefetch(void* cache_rows, int32_t* tags, int32_t* last_use, int32_t* use_count,
                                  uint8_t* dirty, void* host_rows, const int32_t* table_offsets,
                                  const int32_t* indices, const int32_t* offsets, int32_t* locations,
                                  int32_t* stats, int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows,
                                  int64_t num_sets, int ways, int dtype, int policy, int now, void* writeback_rows,
                                  int32_t* writeback_ids, void* workspace, int64_t workspace_bytes,
                                  void* stream_v) {
  return tbe::cache_prefetch_impl("tbe_cache_prefetch", cache_rows, tags, last_use, use_count, dirty, host_rows,
                                  table_offsets, indices, offsets, locations, stats, T, B, D, N, total_rows, num_sets,
                                  ways, dtype, policy, now, writeback_rows, writeback_ids, nullptr, workspace,
                                  workspace_bytes, stream_v);
}

extern "C" int64_t tbe_cache_stage_bytes(int64_t stage_rows, int64_t D, int dtype, int on_host) {
  using namespace tbe;
  if (stage_rows < 1 || D < 1 || (dtype != TBE_F16 && dtype != TBE_F32 && dtype != TBE_F64))
    return fail(TBE_ERR_INVALID_ARGUMENT, "tbe_cache_stage_bytes: bad arguments");
  const int64_t row_bytes = D * elem_size(dtype);
  return on_host ? stage_bytes_host(stage_rows, row_bytes) : stage_bytes_device(stage_rows, row_bytes);
}

extern "C" int tbe_cache_prefetch_staged(void* cache_rows, int32_t* tags, int32_t* last_use, int32_t* use_count,
                                         uint8_t* dirty, void* host_rows, const int32_t* table_offsets,
                                         const int32_t* indices, const int32_t* offsets, int32_t* locations,
                                         int32_t* stats, int64_t T, int64_t B, int64_t D, int64_t N,
                                         int64_t total_rows, int64_t num_sets, int ways, int dtype, int policy,
                                         int now, void* host_rows_on_host, void* stage_device, void* stage_host,
                                         int64_t stage_rows, void* workspace, int64_t workspace_bytes,
                                         void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_cache_prefetch_staged";
  TBE_REQUIRE(host_rows_on_host && stage_device && stage_host && stage_rows >= 1 && stage_rows < (1ll << 31),
              "%s: the host address of the table, both staging buffers and a positive stage_rows are required", who);
  TBE_REQUIRE(reinterpret_cast<uintptr_t>(stage_device) % 16 == 0 && reinterpret_cast<uintptr_t>(stage_host) % 16 == 0,
              "%s: staging buffers must be 16-byte aligned", who);
  StagedFill staged;
  staged.host_table = static_cast<char*>(host_rows_on_host);
  staged.stage_dev = static_cast<char*>(stage_device);
  staged.stage_host = static_cast<char*>(stage_host);
  staged.rows = stage_rows;
  return cache_prefetch_impl(who, cache_rows, tags, last_use, use_count, dirty, host_rows, table_offsets, indices,
                             offsets, locations, stats, T, B, D, N, total_rows, num_sets, ways, dtype, policy, now,
                             nullptr, nullptr, &staged, workspace, workspace_bytes, stream_v);
}

extern "C" int tbe_cache_writeback(const void* writeback_rows, const int32_t* writeback_ids, const int32_t* stats,
                                   void* host_rows, int64_t D, int dtype, void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_cache_writeback";
  TBE_REQUIRE(writeback_rows && writeback_ids && stats && host_rows, "%s: null pointer argument", who);
  TBE_REQUIRE(D > 0 && D % 4 == 0, "%s: D must be a positive multiple of 4", who);
  int vb = 16, nvec = 0;
  int rc = vector_bytes(who, D, dtype, writeback_rows, host_rows, nullptr, &vb, &nvec);
  if (rc != TBE_OK) return rc;
  const int64_t row_bytes = D * elem_size(dtype);
  int lpr_log2 = 0;
  while ((1 << lpr_log2) < nvec && lpr_log2 < 5) ++lpr_log2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int grid = 64;  // link-bound: a few thousand threads keep it full without taking SMs from the lookup
  {
    KernelTimer timer("cache_writeback_kernel", stream);
    if (vb == 16) {
      cache_writeback_kernel<16><<<grid, 256, 0, stream>>>(static_cast<const char*>(writeback_rows), writeback_ids,
                                                           stats + 1, static_cast<char*>(host_rows), row_bytes, nvec,
                                                           lpr_log2);
    } else {
      cache_writeback_kernel<8><<<grid, 256, 0, stream>>>(static_cast<const char*>(writeback_rows), writeback_ids,
                                                          stats + 1, static_cast<char*>(host_rows), row_bytes, nvec,
                                                          lpr_log2);
    }
  }
  TBE_CHECK_LAUNCH("cache_writeback_kernel");
  return TBE_OK;
}

extern "C" int tbe_cache_forward(const void* cache_rows, const void* host_rows, const int32_t* table_offsets,
                                 const int32_t* indices, const int32_t* offsets, const int32_t* locations,
                                 void* output, int64_t T, int64_t B, int64_t D, int dtype, int pooling,
                                 void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_cache_forward";
  TBE_REQUIRE(cache_rows && host_rows && table_offsets && offsets && output, "%s: null pointer argument", who);
  TBE_REQUIRE(T > 0 && B > 0 && D > 0 && D % 4 == 0 && T * B < (1ll << 31), "%s: bad sizes", who);
  TBE_REQUIRE(pooling == TBE_POOL_SUM || pooling == TBE_POOL_MEAN, "%s: bad pooling", who);
  int vb = 16, nvec = 0;
  int rc = vector_bytes(who, D, dtype, cache_rows, host_rows, output, &vb, &nvec);
  if (rc != TBE_OK) return rc;
  CachedRowArgs a{};
  a.cache_rows = cache_rows;
  a.host_rows = host_rows;
  a.table_offsets = table_offsets;
  a.indices = indices;
  a.offsets = offsets;
  a.loc = locations;
  a.out = output;
  a.B = static_cast<int32_t>(B);
  a.T = static_cast<int32_t>(T);
  a.D = static_cast<int32_t>(D);
  a.nvec = nvec;
  a.mean = pooling == TBE_POOL_MEAN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  {
    KernelTimer timer("cached_forward_kernel", stream);
    const int grid = grid_for(T * B);
    int lpr_log2 = 0;
    while ((1 << lpr_log2) < nvec && lpr_log2 < 5) ++lpr_log2;
    if (dtype == TBE_F16 && vb == 16) cached_forward_kernel<__half, 16><<<grid, 256, 0, stream>>>(a, lpr_log2);
    else if (dtype == TBE_F16) cached_forward_kernel<__half, 8><<<grid, 256, 0, stream>>>(a, lpr_log2);
    else if (dtype == TBE_F32) cached_forward_kernel<float, 16><<<grid, 256, 0, stream>>>(a, lpr_log2);
    else return fail(TBE_ERR_UNSUPPORTED, "%s: fp16 and fp32 tables only", who);
  }
  TBE_CHECK_LAUNCH("cached_forward_kernel");
  return TBE_OK;
}

extern "C" int tbe_cache_backward_sgd(const void* grad_output, int64_t stride_b, int64_t stride_t, void* cache_rows,
                                      void* host_rows, uint8_t* dirty, const int32_t* offsets, int64_t T, int64_t B,
                                      int64_t D, int64_t N, int64_t total_rows, int64_t num_sets, int dtype,
                                      int pooling, float lr, void* workspace, int64_t workspace_bytes,
                                      void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_cache_backward_sgd";
  TBE_REQUIRE(grad_output && cache_rows && host_rows && dirty && offsets && workspace, "%s: null pointer argument", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  TBE_REQUIRE(D > 0 && D % 4 == 0 && num_sets >= 1, "%s: bad sizes", who);
  if (N == 0) return TBE_OK;
  CacheScratch cs;
  rc = carve_cache(workspace, N, total_rows, &cs);
  if (rc != TBE_OK) return rc;
  if (static_cast<int64_t>(cs.total) > workspace_bytes)
    return fail(TBE_ERR_WORKSPACE_TOO_SMALL, "%s: workspace has %lld bytes, %lld needed", who,
                (long long)workspace_bytes, (long long)cs.total);
  int vb = 16, nvec = 0;
  rc = vector_bytes(who, D, dtype, cache_rows, host_rows, grad_output, &vb, &nvec);
  if (rc != TBE_OK) return rc;
  const int es = elem_size(dtype);
  if ((stride_b * es) % vb != 0 || (stride_t * es) % vb != 0)
    return fail(TBE_ERR_INVALID_ARGUMENT, "%s: grad_output strides must keep rows %d-byte aligned", who, vb);
  CachedSgdArgs a{};
  a.cache_rows = cache_rows;
  a.host_rows = host_rows;
  a.dirty = dirty;
  a.grad = grad_output;
  a.stride_b = stride_b;
  a.stride_t = stride_t;
  a.keys = cs.ws.keys;
  a.vals = cs.ws.vals;
  a.seg_starts = cs.ws.seg_starts;
  a.counters = cs.ws.counters;
  a.entry_bag = cs.ws.entry_bag;
  a.loc_sorted = cs.loc_sorted;
  a.offsets = offsets;
  a.B = static_cast<int32_t>(B);
  a.D = static_cast<int32_t>(D);
  a.N = static_cast<int32_t>(N);
  a.nvec = nvec;
  a.mean = pooling == TBE_POOL_MEAN;
  a.run_row = cs.run_row;
  a.long_list = cs.ws.long_list;
  a.long_count = cs.ws.counters + 1;
  int lpr_log2 = 0;
  while ((1 << lpr_log2) < nvec && lpr_log2 < 5) ++lpr_log2;
  a.lpr_log2 = lpr_log2;
  a.lr = lr;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  TBE_CUDA_TRY(cudaMemsetAsync(cs.ws.counters + 1, 0, 4, stream));  // the long-run queue starts empty
  // very long runs are cut into parts; the part list, the tickets and the fp32 partial sums live where
  // the sort's input pairs were (dead since the prefetch sorted them)
  a.split_len = 0;
  {
    const size_t region =
        static_cast<size_t>(reinterpret_cast<char*>(cs.ws.seg_starts) - reinterpret_cast<char*>(cs.ws.keys_in));
    for (int64_t plen = 256; plen <= (1 << 16); plen *= 2) {
      const size_t max_parts = static_cast<size_t>(N / plen + 1);
      const size_t list_bytes = align_up(max_parts * sizeof(int4), 256), word_bytes = align_up(max_parts * sizeof(int32_t), 256);
      if (list_bytes + 2 * word_bytes + max_parts * static_cast<size_t>(D) * sizeof(float) > region) continue;
      char* base = reinterpret_cast<char*>(cs.ws.keys_in);
      a.part_list = reinterpret_cast<int4*>(base);
      a.part_tickets = reinterpret_cast<int32_t*>(base + list_bytes);
      a.part_run = reinterpret_cast<int32_t*>(base + list_bytes + word_bytes);
      a.part_sums = reinterpret_cast<float*>(base + list_bytes + 2 * word_bytes);
      a.part_count = cs.ws.counters + 9;
      a.split_len = static_cast<int32_t>(plen);
      a.max_parts = static_cast<int32_t>(max_parts);
      TBE_CUDA_TRY(cudaMemsetAsync(a.part_count, 0, 4, stream));
      break;
    }
  }
  {
    KernelTimer timer("cached_sgd_kernel", stream);
    const int grid = grid_for(N);
    if (dtype == TBE_F16 && vb == 16) cached_sgd_kernel<__half, 16><<<grid, 256, 0, stream>>>(a);
    else if (dtype == TBE_F16) cached_sgd_kernel<__half, 8><<<grid, 256, 0, stream>>>(a);
    else if (dtype == TBE_F32) cached_sgd_kernel<float, 16><<<grid, 256, 0, stream>>>(a);
    else return fail(TBE_ERR_UNSUPPORTED, "%s: fp16 and fp32 tables only", who);
  }
  TBE_CHECK_LAUNCH("cached_sgd_kernel");
  {
    KernelTimer timer("cached_sgd_long_kernel", stream);
    const int grid = device_sm_count() * 6;
    if (dtype == TBE_F16 && vb == 16) cached_sgd_long_kernel<__half, 16><<<grid, 256, 0, stream>>>(a);
    else if (dtype == TBE_F16) cached_sgd_long_kernel<__half, 8><<<grid, 256, 0, stream>>>(a);
    else cached_sgd_long_kernel<float, 16><<<grid, 256, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("cached_sgd_long_kernel");
  return TBE_OK;
}

extern "C" int tbe_cache_flush(void* cache_rows, void* host_rows, const int32_t* tags, uint8_t* dirty,
                               int64_t num_slots, int64_t D, int dtype, void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_cache_flush";
  TBE_REQUIRE(cache_rows && host_rows && tags && dirty && num_slots > 0 && D > 0 && D % 4 == 0,
              "%s: bad arguments", who);
  int vb = 16, nvec = 0;
  int rc = vector_bytes(who, D, dtype, cache_rows, host_rows, nullptr, &vb, &nvec);
  if (rc != TBE_OK) return rc;
  host_pool_wait();  // evicted rows a staged prefetch is still scattering belong to the flushed table too
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int64_t row_bytes = D * elem_size(dtype);
  {
    KernelTimer timer("cache_flush_kernel", stream);
    if (vb == 16) {
      cache_flush_kernel<16><<<grid_for(num_slots), 256, 0, stream>>>(cache_rows, host_rows, tags, dirty, num_slots,
                                                                       row_bytes, nvec);
    } else {
      cache_flush_kernel<8><<<grid_for(num_slots), 256, 0, stream>>>(cache_rows, host_rows, tags, dirty, num_slots,
                                                                      row_bytes, nvec);
    }
  }
  TBE_CHECK_LAUNCH("cache_flush_kernel");
  return TBE_OK;
}
