// Pooled embedding-bag forward (sum / mean, optional per-sample weights) for sm_100a.
//
// One warp owns one bag at a time and walks bags bag0, bag0+stride, ... (persistent
// grid).  The warp keeps a three-deep software pipeline in registers: while the rows of
// bag k are being gathered, the first 32 indices of bag k+1 and the offsets of bag k+2
// are already in flight, so the offsets -> indices -> rows dependency chain is paid once
// per warp instead of once per bag.  Indices are staged one per lane and broadcast with
// shuffles; every lane issues UNROLL independent 16-byte streaming loads per step.
// A row narrower than 32 vectors is owned by a sub-warp group, so a 256-byte row
// (D=128 fp16) is fetched by half a warp and two rows are in flight per step.
#include "tbe_common.cuh"

namespace tbe {
namespace {

struct FwdArgs {
  const void* weights;
  const int32_t* table_offsets;
  const int32_t* indices;
  const int32_t* offsets;
  const void* psw;
  void* out[TBE_MAX_PEERS];  // out[0] only unless SHARDED
  int32_t B, T, D;
  int32_t B_local, T_total, t0;
  int32_t lpr_log2, nvec, nchunks;
  int64_t out_stride_b_bytes;  // distance between the output rows of consecutive samples (unsharded)
  // tables of different width (MIXED): element offset of every table in the flat weights vector and
  // first output column of every table, both [T + 1]
  const int64_t* weight_offsets;
  const int32_t* dim_offsets;
};

template <typename T>
__device__ __forceinline__ typename Acc<T>::type to_acc(T x) {
  return static_cast<typename Acc<T>::type>(x);
}
template <>
__device__ __forceinline__ float to_acc<__half>(__half x) {
  return __half2float(x);
}

//
// MIXED: every table has its own width.  The row geometry (lanes per row, vectors, chunks), the
// table's base address and the output column are then derived per bag from dim_offsets /
// weight_offsets instead of once per launch; everything else is the same walk.
template <typename T, int VB, bool WEIGHTED, bool MEAN, bool SHARDED, int UNROLL, bool MIXED = false>
__global__ void __launch_bounds__(256) tbe_forward_kernel(const FwdArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);

  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * warps_per_block;
  int64_t bag = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  if (bag >= nbags) return;

  int lpr_log2 = a.lpr_log2;
  int rps_log2 = 5 - lpr_log2;  // log2(rows per warp step)
  int sub = lane & ((1 << lpr_log2) - 1);
  int slot = lane >> lpr_log2;
  const char* __restrict__ W = static_cast<const char*>(a.weights);
  uint32_t row_bytes = static_cast<uint32_t>(a.D) * static_cast<uint32_t>(sizeof(T));
  int nvec = a.nvec, nchunks = a.nchunks;
  const int32_t* __restrict__ offsets = a.offsets;
  const int32_t* __restrict__ indices = a.indices;
  const T* __restrict__ psw = static_cast<const T*>(a.psw);

  // pipeline state: current bag fully described, next bag's extent known
  int cur_s = __ldg(offsets + bag), cur_e = __ldg(offsets + bag + 1);
  int cur_idx = (cur_s + lane < cur_e) ? __ldg(indices + cur_s + lane) : 0;
  int64_t nbag = bag + wstride;
  int nxt_s = 0, nxt_e = 0;
  if (nbag < nbags) {
    nxt_s = __ldg(offsets + nbag);
    nxt_e = __ldg(offsets + nbag + 1);
  }

  while (true) {
    // prefetch: indices of the next bag, extent of the one after it
    const int64_t nnbag = nbag + wstride;
    int pre_idx = 0, nn_s = 0, nn_e = 0;
    if (nbag < nbags && nxt_s + lane < nxt_e) pre_idx = __ldg(indices + nxt_s + lane);
    if (nnbag < nbags) {
      nn_s = __ldg(offsets + nnbag);
      nn_e = __ldg(offsets + nnbag + 1);
    }

    const int t = static_cast<int>(bag / a.B);
    const int b = static_cast<int>(bag - static_cast<int64_t>(t) * a.B);
    uint32_t row0 = 0;
    if (!MIXED) row0 = static_cast<uint32_t>(__ldg(a.table_offsets + t));

    char* outp;
    if (MIXED) {
      const int32_t d0 = __ldg(a.dim_offsets + t);
      row_bytes = static_cast<uint32_t>(__ldg(a.dim_offsets + t + 1) - d0) * static_cast<uint32_t>(sizeof(T));
      nvec = static_cast<int>(row_bytes / VB);
      nchunks = (nvec + 31) >> 5;
      lpr_log2 = 0;
      while ((1 << lpr_log2) < nvec && lpr_log2 < 5) ++lpr_log2;
      rps_log2 = 5 - lpr_log2;
      sub = lane & ((1 << lpr_log2) - 1);
      slot = lane >> lpr_log2;
      W = static_cast<const char*>(a.weights) + __ldg(a.weight_offsets + t) * static_cast<int64_t>(sizeof(T));
      outp = static_cast<char*>(a.out[0]) + static_cast<int64_t>(b) * a.out_stride_b_bytes +
             static_cast<int64_t>(d0) * static_cast<int64_t>(sizeof(T));
    } else if (SHARDED) {
      const int dest = b / a.B_local;
      const int bl = b - dest * a.B_local;
      outp = static_cast<char*>(a.out[dest]) +
             (static_cast<int64_t>(bl) * a.T_total + a.t0 + t) * static_cast<int64_t>(row_bytes);
    } else {
      outp = static_cast<char*>(a.out[0]) + static_cast<int64_t>(b) * a.out_stride_b_bytes +
             static_cast<int64_t>(t) * static_cast<int64_t>(row_bytes);
    }

    for (int c = 0; c < nchunks; ++c) {
      const int v = (c << 5) + sub;
      const bool vact = v < nvec;
      // this lane's vector of row 0; lanes past the end of the row re-read vector 0 and never store
      const char* const Wv = W + (vact ? static_cast<int64_t>(v) * VB : 0);
      acc_t acc[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) acc[k] = 0;

      for (int base = cur_s; base < cur_e; base += 32) {
        int idx_l;
        if (base == cur_s) {
          idx_l = cur_idx;
        } else {
          idx_l = (base + lane < cur_e) ? __ldg(indices + base + lane) : 0;
        }
        acc_t w_l = 0;
        if (WEIGHTED) {
          if (base + lane < cur_e) w_l = to_acc<T>(psw[base + lane]);
        }
        const int cnt = min(32, cur_e - base);
        const int steps = (cnt + (1 << rps_log2) - 1) >> rps_log2;
        // steps in which every row slot of the warp has a row: no predicates, no zero fill
        const int full_steps = ((cnt >> rps_log2) / UNROLL) * UNROLL;
        int s = 0;
        for (; s < full_steps; s += UNROLL) {
          Raw<VB> r[UNROLL];
          acc_t w[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const int j = ((s + u) << rps_log2) + slot;
            const int idx = __shfl_sync(kFullMask, idx_l, j);
            if (WEIGHTED) w[u] = __shfl_sync(kFullMask, w_l, j);
            r[u] = ld_stream<VB>(Wv + static_cast<uint64_t>(row0 + static_cast<uint32_t>(idx)) * row_bytes);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            if (WEIGHTED) {
              acc_t e[NE];
              unpack<T, VB>(r[u], e);
#pragma unroll
              for (int k = 0; k < NE; ++k) acc[k] += e[k] * w[u];
            } else {
              accumulate<T, VB>(r[u], acc);
            }
          }
        }
        for (; s < steps; s += UNROLL) {
          Raw<VB> r[UNROLL];
          acc_t w[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const int j = ((s + u) << rps_log2) + slot;
            const int idx = __shfl_sync(kFullMask, idx_l, j & 31);
            if (WEIGHTED) w[u] = __shfl_sync(kFullMask, w_l, j & 31);
            if (j < cnt) {
              // 32-bit row id times 32-bit row size: one wide multiply-add per address
              r[u] = ld_stream<VB>(Wv + static_cast<uint64_t>(row0 + static_cast<uint32_t>(idx)) * row_bytes);
            } else {
              r[u] = raw_zero<VB>();
            }
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            if (WEIGHTED) {
              acc_t e[NE];
              unpack<T, VB>(r[u], e);
#pragma unroll
              for (int k = 0; k < NE; ++k) acc[k] += e[k] * w[u];
            } else {
              accumulate<T, VB>(r[u], acc);
            }
          }
        }
      }
      // fold the row slots of the warp together
      for (int m = 1 << lpr_log2; m < 32; m <<= 1) {
#pragma unroll
        for (int k = 0; k < NE; ++k) acc[k] += __shfl_xor_sync(kFullMask, acc[k], m);
      }
      if (MEAN) {
        const int L = cur_e - cur_s;
        if (L > 0) {
          const acc_t denom = static_cast<acc_t>(L);
#pragma unroll
          for (int k = 0; k < NE; ++k) acc[k] = acc[k] / denom;
        }
      }
      if (slot == 0 && vact) st_row<VB>(outp + static_cast<int64_t>(v) * VB, pack_rn<T, VB>(acc));
    }

    bag = nbag;
    if (bag >= nbags) break;
    cur_s = nxt_s;
    cur_e = nxt_e;
    cur_idx = pre_idx;
    nbag = nnbag;
    nxt_s = nn_s;
    nxt_e = nn_e;
  }
}

template <typename T, int VB, bool WEIGHTED, bool MEAN, bool SHARDED, int UNROLL>
int launch_fwd(const FwdArgs& a, cudaStream_t stream) {
  auto kernel = tbe_forward_kernel<T, VB, WEIGHTED, MEAN, SHARDED, UNROLL>;
  int threads = tuning(kTuneFwdThreads);
  if (threads <= 0) threads = 256;
  if (threads > 256 || threads % 32 != 0) return fail(TBE_ERR_INVALID_ARGUMENT, "fwd_threads must be a multiple of 32 <= 256");
  int per_sm = 0;
  TBE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
  if (per_sm < 1) per_sm = 1;
  // knob: blocks per SM of the persistent grid; a value above what fits makes the grid one warp per bag
  if (tuning(kTuneFwdBlocksPerSM) > 0) per_sm = tuning(kTuneFwdBlocksPerSM);
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  const int wpb = threads / 32;
  int64_t blocks = (nbags + wpb - 1) / wpb;
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  if (blocks > resident) blocks = resident;
  {
    KernelTimer timer("tbe_forward_kernel", stream);
    kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("tbe_forward_kernel");
  return TBE_OK;
}

template <typename T, int VB, bool SHARDED, int UNROLL>
int dispatch_mode(const FwdArgs& a, bool weighted, bool mean, cudaStream_t stream) {
  if (weighted) return launch_fwd<T, VB, true, false, SHARDED, UNROLL>(a, stream);
  if (mean) return launch_fwd<T, VB, false, true, SHARDED, UNROLL>(a, stream);
  return launch_fwd<T, VB, false, false, SHARDED, UNROLL>(a, stream);
}

template <bool SHARDED>
int dispatch_fwd(const FwdArgs& a, int dtype, int vb, bool weighted, bool mean, cudaStream_t stream) {
  const int unroll = tuning(kTuneFwdUnroll) > 0 ? tuning(kTuneFwdUnroll) : 4;
  if (unroll != 4 && unroll != 8 && unroll != 2) return fail(TBE_ERR_INVALID_ARGUMENT, "fwd_unroll must be 2, 4 or 8");
  switch (dtype) {
    case TBE_F16:
      if (vb == 16) {
        if (unroll == 8) return dispatch_mode<__half, 16, SHARDED, 8>(a, weighted, mean, stream);
        if (unroll == 2) return dispatch_mode<__half, 16, SHARDED, 2>(a, weighted, mean, stream);
        return dispatch_mode<__half, 16, SHARDED, 4>(a, weighted, mean, stream);
      }
      return dispatch_mode<__half, 8, SHARDED, 4>(a, weighted, mean, stream);
    case TBE_F32:
      if (unroll == 8) return dispatch_mode<float, 16, SHARDED, 8>(a, weighted, mean, stream);
      if (unroll == 2) return dispatch_mode<float, 16, SHARDED, 2>(a, weighted, mean, stream);
      return dispatch_mode<float, 16, SHARDED, 4>(a, weighted, mean, stream);
    case TBE_F64:
      return dispatch_mode<double, 16, SHARDED, 4>(a, weighted, mean, stream);
  }
  return fail(TBE_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

int forward_common(const void* weights, const int32_t* table_offsets, const int32_t* indices,
                   const int32_t* offsets, const void* psw, void* const* outs, int world,
                   int64_t T, int64_t B, int64_t D, int64_t T_total, int64_t t0, int dtype,
                   int pooling, bool sharded, int64_t out_stride_b, void* stream) {
  // `indices` may be null when every bag is empty: it is only read inside non-empty bag extents
  TBE_REQUIRE(weights && table_offsets && offsets && outs, "tbe_forward: null pointer argument");
  TBE_REQUIRE(T > 0, "tbe_forward: T must be > 0 (got %lld)", (long long)T);
  TBE_REQUIRE(B > 0, "tbe_forward: B must be > 0 (got %lld)", (long long)B);
  TBE_REQUIRE(D > 0 && D % 4 == 0, "tbe_forward: D must be a positive multiple of 4 (got %lld)", (long long)D);
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "tbe_forward: bad dtype %d", dtype);
  TBE_REQUIRE(pooling == TBE_POOL_SUM || pooling == TBE_POOL_MEAN, "tbe_forward: bad pooling %d", pooling);
  TBE_REQUIRE(!(pooling == TBE_POOL_MEAN && psw), "tbe_forward: per-sample weights need sum pooling");
  TBE_REQUIRE(B * T < (1ll << 31) && B * T_total * D / 1 > 0, "tbe_forward: B*T out of range");
  TBE_REQUIRE(world >= 1 && world <= TBE_MAX_PEERS, "tbe_forward: world must be in [1,%d]", TBE_MAX_PEERS);
  TBE_REQUIRE(B % world == 0, "tbe_forward: world (%d) must divide B (%lld)", world, (long long)B);
  TBE_REQUIRE(t0 >= 0 && t0 + T <= T_total, "tbe_forward: table columns [%lld,%lld) outside T_total=%lld",
              (long long)t0, (long long)(t0 + T), (long long)T_total);

  FwdArgs a{};
  a.weights = weights;
  a.table_offsets = table_offsets;
  a.indices = indices;
  a.offsets = offsets;
  a.psw = psw;
  const void* align_probe = nullptr;
  for (int r = 0; r < world; ++r) {
    TBE_REQUIRE(outs[r] != nullptr, "tbe_forward: output pointer %d is null", r);
    a.out[r] = outs[r];
    if (reinterpret_cast<uintptr_t>(outs[r]) % 16 != 0) align_probe = outs[r];
  }
  a.B = static_cast<int32_t>(B);
  a.T = static_cast<int32_t>(T);
  a.D = static_cast<int32_t>(D);
  a.B_local = static_cast<int32_t>(B / world);
  a.T_total = static_cast<int32_t>(T_total);
  a.t0 = static_cast<int32_t>(t0);
  if (out_stride_b <= 0) out_stride_b = T * D;
  TBE_REQUIRE(out_stride_b >= T * D, "tbe_forward: output sample stride %lld is smaller than T*D", (long long)out_stride_b);
  a.out_stride_b_bytes = out_stride_b * elem_size(dtype);
  if (a.out_stride_b_bytes % 16 != 0) align_probe = reinterpret_cast<const void*>(uintptr_t(8));
  TBE_REQUIRE(a.out_stride_b_bytes % 8 == 0, "tbe_forward: output sample stride must keep rows 8-byte aligned");
  const RowGeom g = make_geom(D, dtype, weights, align_probe);
  TBE_REQUIRE(g.vb == 16 || dtype == TBE_F16, "tbe_forward: weights/output must be 16-byte aligned");
  if (g.vb == 8) {
    TBE_REQUIRE(reinterpret_cast<uintptr_t>(weights) % 8 == 0, "tbe_forward: weights must be 8-byte aligned");
    for (int r = 0; r < world; ++r)
      TBE_REQUIRE(reinterpret_cast<uintptr_t>(outs[r]) % 8 == 0, "tbe_forward: output must be 8-byte aligned");
  }
  a.lpr_log2 = g.lpr_log2;
  a.nvec = g.nvec;
  a.nchunks = g.nchunks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool weighted = psw != nullptr;
  const bool mean = pooling == TBE_POOL_MEAN;
  return sharded ? dispatch_fwd<true>(a, dtype, g.vb, weighted, mean, s)
                 : dispatch_fwd<false>(a, dtype, g.vb, weighted, mean, s);
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_forward(const void* weights, const int32_t* table_offsets, const int32_t* indices,
                           const int32_t* offsets, const void* per_sample_weights, void* output,
                           int64_t T, int64_t B, int64_t D, int dtype, int pooling, void* stream) {
  void* outs[1] = {output};
  return tbe::forward_common(weights, table_offsets, indices, offsets, per_sample_weights, outs, 1, T, B, D,
                             T, 0, dtype, pooling, false, 0, stream);
}

extern "C" int tbe_forward_strided(const void* weights, const int32_t* table_offsets, const int32_t* indices,
                                   const int32_t* offsets, const void* per_sample_weights, void* output,
                                   int64_t out_stride_b, int64_t T, int64_t B, int64_t D, int dtype, int pooling,
                                   void* stream) {
  void* outs[1] = {output};
  return tbe::forward_common(weights, table_offsets, indices, offsets, per_sample_weights, outs, 1, T, B, D,
                             T, 0, dtype, pooling, false, out_stride_b, stream);
}

extern "C" int tbe_forward_sharded(const void* weights, const int32_t* table_offsets,
                                   const int32_t* indices, const int32_t* offsets,
                                   const void* per_sample_weights, void* const* peer_outputs, int world,
                                   int64_t T, int64_t B, int64_t D, int64_t T_total, int64_t t0,
                                   int dtype, int pooling, void* stream) {
  return tbe::forward_common(weights, table_offsets, indices, offsets, per_sample_weights, peer_outputs,
                             world, T, B, D, T_total, t0, dtype, pooling, true, 0, stream);
}

extern "C" int tbe_forward_mixed(const void* weights, const int64_t* weight_offsets, const int32_t* dim_offsets,
                                 const int32_t* indices, const int32_t* offsets, const void* per_sample_weights,
                                 void* output, int64_t T, int64_t B, int64_t total_D, int dtype, int vector_bytes,
                                 void* stream) {
  using namespace tbe;
  TBE_REQUIRE(weights && weight_offsets && dim_offsets && offsets && output, "tbe_forward_mixed: null pointer argument");
  TBE_REQUIRE(T > 0 && B > 0 && total_D > 0 && B * T < (1ll << 31), "tbe_forward_mixed: bad sizes");
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "tbe_forward_mixed: bad dtype %d", dtype);
  TBE_REQUIRE(vector_bytes == 16 || (vector_bytes == 8 && dtype == TBE_F16),
              "tbe_forward_mixed: vector_bytes must be 16 (8 is allowed for fp16 rows that are only 8-byte aligned)");
  TBE_REQUIRE(reinterpret_cast<uintptr_t>(weights) % vector_bytes == 0 &&
                  reinterpret_cast<uintptr_t>(output) % vector_bytes == 0 &&
                  (total_D * elem_size(dtype)) % vector_bytes == 0,
              "tbe_forward_mixed: weights, output and output rows must be %d-byte aligned", vector_bytes);
  FwdArgs a{};
  a.weights = weights;
  a.weight_offsets = weight_offsets;
  a.dim_offsets = dim_offsets;
  a.indices = indices;
  a.offsets = offsets;
  a.psw = per_sample_weights;
  a.out[0] = output;
  a.B = static_cast<int32_t>(B);
  a.T = static_cast<int32_t>(T);
  a.out_stride_b_bytes = total_D * elem_size(dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool weighted = per_sample_weights != nullptr;
  void (*kernel)(const FwdArgs) = nullptr;
  if (dtype == TBE_F16 && vector_bytes == 16)
    kernel = weighted ? tbe_forward_kernel<__half, 16, true, false, false, 4, true>
                      : tbe_forward_kernel<__half, 16, false, false, false, 4, true>;
  else if (dtype == TBE_F16)
    kernel = weighted ? tbe_forward_kernel<__half, 8, true, false, false, 4, true>
                      : tbe_forward_kernel<__half, 8, false, false, false, 4, true>;
  else if (dtype == TBE_F32)
    kernel = weighted ? tbe_forward_kernel<float, 16, true, false, false, 4, true>
                      : tbe_forward_kernel<float, 16, false, false, false, 4, true>;
  else
    kernel = weighted ? tbe_forward_kernel<double, 16, true, false, false, 4, true>
                      : tbe_forward_kernel<double, 16, false, false, false, 4, true>;
  int per_sm = 0;
  TBE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0));
  if (per_sm < 1) per_sm = 1;
  const int64_t nbags = B * T;
  int64_t blocks = (nbags + 7) / 8;
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  if (blocks > resident) blocks = resident;
  {
    KernelTimer timer("tbe_forward_kernel", s);
    kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
  }
  TBE_CHECK_LAUNCH("tbe_forward_kernel");
  return TBE_OK;
}
