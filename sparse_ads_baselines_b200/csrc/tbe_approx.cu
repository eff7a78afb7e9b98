// Approximate rowwise Adagrad backward, deterministic (sm_100a).
//
// "Approximate" (the reference's batched_embedding_backward_adagrad_approx_kernel_1) means every
// lookup is applied on its own with the squared gradient norm of ITS bag, instead of first summing
// the gradients of a row.  The reference applies lookups concurrently without atomics, so repeated
// rows race; here the lookups of one row are applied one after the other in ascending index
// position, which is what the reference computes whenever no row repeats.
//
// Lookups without per-sample weights take approx_backward_sorted (tbe_backward.cu): the library's own
// table-segmented sort, and runs reduced by lane groups with the per-lookup step sizes obtained from a
// prefix sum (hot rows by a whole CTA).  Per-sample weights need every lookup's index position, which
// that sort does not carry; they, and rows wider than 1 KB, take the path in this file:
//
//  1. prep kernel (a warp per bag): g2 = |grad[b][t]|^2 (times w_l^2 when weighted) stored per index
//     position, sort key and position emitted for the sort, and for weighted lookups the gradient
//     of the per-sample weight, <weights[row], grad[b][t]>, taken BEFORE any row is updated.
//  2. stable radix sort of (key, position) pairs, run starts compacted (CUB).
//  3. run kernel (a warp per run of equal rows): the row is held in fp32 registers, every lookup
//     of the run adds its g2 to the state and subtracts w_l * lr / (sqrt(state) + eps) * grad; the
//     row and the state are written once.
#include "tbe_plan.cuh"

namespace tbe {
namespace {

struct ApproxArgs {
  const void* grad;
  int64_t stride_b, stride_t;  // elements
  void* weights;
  float* state;
  const int32_t* table_offsets;
  const int32_t* indices;
  const int32_t* offsets;
  const void* psw;
  void* grad_psw;
  uint32_t* keys_in;
  int32_t* vals_in;
  int32_t* entry_bag;
  float* entry_g2;
  const uint32_t* keys;
  const int32_t* vals;
  const int32_t* seg_starts;
  const int32_t* counters;
  int32_t B, T, D, N;
  int32_t idx_bits, nvec;
  float lr, eps;
  uint64_t sr_seed, sr_offset;
};

template <typename T>
__device__ __forceinline__ float scalar_to_float(T x) {
  return static_cast<float>(x);
}
template <>
__device__ __forceinline__ float scalar_to_float<__half>(__half x) {
  return __half2float(x);
}
template <typename T>
__device__ __forceinline__ T scalar_from(typename Acc<T>::type x) {
  return static_cast<T>(x);
}
template <>
__device__ __forceinline__ __half scalar_from<__half>(float x) {
  return __float2half_rn(x);
}

template <typename A>
__device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
  return v;
}

template <typename T, int VB>
__device__ __forceinline__ const char* grad_row(const ApproxArgs& a, int bag) {
  const int t = bag / a.B;
  const int b = bag - t * a.B;
  return static_cast<const char*>(a.grad) +
         (static_cast<int64_t>(b) * a.stride_b + static_cast<int64_t>(t) * a.stride_t) * static_cast<int64_t>(sizeof(T));
}

template <typename T, int VB, bool WEIGHTED>
__global__ void __launch_bounds__(256) approx_prep_kernel(const ApproxArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  const T* psw = static_cast<const T*>(a.psw);
  for (int64_t bag = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); bag < nbags;
       bag += wstride) {
    const int t = static_cast<int>(bag / a.B);
    const uint32_t row0 = static_cast<uint32_t>(__ldg(a.table_offsets + t));
    const uint32_t key0 = a.idx_bits ? (static_cast<uint32_t>(t) << a.idx_bits) : row0;
    const char* g = grad_row<T, VB>(a, static_cast<int>(bag));
    acc_t part = 0;
    for (int v = lane; v < a.nvec; v += 32) {
      acc_t e[NE];
      unpack<T, VB>(ld_stream<VB>(g + static_cast<int64_t>(v) * VB), e);
#pragma unroll
      for (int k = 0; k < NE; ++k) part += e[k] * e[k];
    }
    const float g2 = static_cast<float>(warp_sum(part));
    const int s = __ldg(a.offsets + bag), e_ = __ldg(a.offsets + bag + 1);
    for (int p = s + lane; p < e_; p += 32) {
      float wl = 1.f;
      if (WEIGHTED) wl = scalar_to_float<T>(psw[p]);
      a.keys_in[p] = key0 + static_cast<uint32_t>(__ldg(a.indices + p));
      a.vals_in[p] = p;
      a.entry_bag[p] = static_cast<int32_t>(bag);
      a.entry_g2[p] = g2 * wl * wl;
    }
    if (WEIGHTED) {
      T* gp = static_cast<T*>(a.grad_psw);
      for (int p = s; p < e_; ++p) {  // one lookup at a time, the warp spans the row
        const char* w = static_cast<const char*>(a.weights) +
                        static_cast<int64_t>(row0 + static_cast<uint32_t>(__ldg(a.indices + p))) * row_bytes;
        acc_t dot = 0;
        for (int v = lane; v < a.nvec; v += 32) {
          acc_t we[NE], ge[NE];
          unpack<T, VB>(ld_stream<VB>(w + static_cast<int64_t>(v) * VB), we);
          unpack<T, VB>(ld_stream<VB>(g + static_cast<int64_t>(v) * VB), ge);
#pragma unroll
          for (int k = 0; k < NE; ++k) dot += we[k] * ge[k];
        }
        dot = warp_sum(dot);
        if (lane == 0) gp[p] = scalar_from<T>(dot);
      }
    }
  }
}

template <typename T, int VB, bool SR>
__device__ __forceinline__ Raw<VB> approx_pack(const typename Acc<T>::type* v, Philox* rng) {
  return pack_rn<T, VB>(v);
}
template <>
__device__ __forceinline__ Raw<16> approx_pack<__half, 16, true>(const float* v, Philox* rng) {
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
__device__ __forceinline__ Raw<8> approx_pack<__half, 8, true>(const float* v, Philox* rng) {
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

template <typename T, int VB, bool WEIGHTED, bool SR>
__global__ void __launch_bounds__(256) approx_run_kernel(const ApproxArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int U = __ldg(a.counters);
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int64_t row_bytes = static_cast<int64_t>(a.D) * sizeof(T);
  const T* psw = static_cast<const T*>(a.psw);
  Philox rng(a.sr_seed, static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x, a.sr_offset);
  for (int64_t run = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); run < U;
       run += wstride) {
    const int s = __ldg(a.seg_starts + run);
    const int e_ = (run + 1 < U) ? __ldg(a.seg_starts + run + 1) : a.N;
    const uint32_t row = key_to_row(a.table_offsets, a.idx_bits, __ldg(a.keys + s));
    char* w = static_cast<char*>(a.weights) + static_cast<int64_t>(row) * row_bytes;
    const float st0 = a.state[row];
    float st = st0;
    // the state sequence depends on the lookups only, so every lane (and every chunk of a wide row)
    // replays the same sequence
    for (int v = lane; v < a.nvec || v == lane; v += 32) {
      const bool vact = v < a.nvec;
      acc_t we[NE];
#pragma unroll
      for (int k = 0; k < NE; ++k) we[k] = 0;
      if (vact) unpack<T, VB>(ld_rw<VB>(w + static_cast<int64_t>(v) * VB), we);
      st = st0;
      for (int i = s; i < e_; ++i) {
        const int p = __ldg(a.vals + i);
        const int bag = __ldg(a.entry_bag + p);
        float wl = 1.f;
        if (WEIGHTED) wl = scalar_to_float<T>(psw[p]);
        st += __ldg(a.entry_g2 + p);
        const acc_t mult = static_cast<acc_t>(wl * (a.lr * (1.0f / (sqrtf(st) + a.eps))));
        if (vact) {
          acc_t ge[NE];
          unpack<T, VB>(ld_stream<VB>(grad_row<T, VB>(a, bag) + static_cast<int64_t>(v) * VB), ge);
#pragma unroll
          for (int k = 0; k < NE; ++k) we[k] -= mult * ge[k];
        }
      }
      if (vact) st_row<VB>(w + static_cast<int64_t>(v) * VB, approx_pack<T, VB, SR>(we, &rng));
    }
    __syncwarp();
    if (lane == 0) a.state[row] = st;
  }
}

template <typename T, int VB>
int launch_approx(ApproxArgs& a, Workspace& ws, KeyLayout layout, bool weighted, bool sr, cudaStream_t stream) {
  const int64_t nbags = static_cast<int64_t>(a.B) * a.T;
  int64_t blocks = (nbags + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  {
    KernelTimer timer("approx_prep_kernel", stream);
    if (weighted) {
      approx_prep_kernel<T, VB, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
    } else {
      approx_prep_kernel<T, VB, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
    }
  }
  TBE_CHECK_LAUNCH("approx_prep_kernel");
  int rc = sort_pairs(ws, a.N, layout.sort_bits, stream);
  if (rc != TBE_OK) return rc;
  rc = select_run_starts(ws, a.N, stream);
  if (rc != TBE_OK) return rc;
  blocks = (static_cast<int64_t>(a.N) + 7) / 8;
  if (blocks > cap) blocks = cap;
  {
    KernelTimer timer("approx_run_kernel", stream);
    if (weighted) {
      if (sr) {
        approx_run_kernel<T, VB, true, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
      } else {
        approx_run_kernel<T, VB, true, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
      }
    } else {
      if (sr) {
        approx_run_kernel<T, VB, false, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
      } else {
        approx_run_kernel<T, VB, false, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
      }
    }
  }
  TBE_CHECK_LAUNCH("approx_run_kernel");
  return TBE_OK;
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_backward_approx_rowwise_adagrad(
    const void* grad_output, int64_t stride_b, int64_t stride_t, void* weights, const int32_t* table_offsets,
    const int32_t* indices, const int32_t* offsets, const void* per_sample_weights, void* grad_per_sample_weights,
    float* optimizer_state, int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, float lr,
    float eps, int stochastic_rounding, uint64_t sr_seed, uint64_t sr_offset, int64_t max_rows_per_table,
    void* workspace, int64_t workspace_bytes, void* stream_v) {
  using namespace tbe;
  const char* who = "tbe_backward_approx_rowwise_adagrad";
  TBE_REQUIRE(grad_output && weights && table_offsets && offsets && optimizer_state && (indices || N == 0),
              "%s: null pointer argument", who);
  TBE_REQUIRE(!per_sample_weights || grad_per_sample_weights, "%s: grad_per_sample_weights is null", who);
  int rc = check_sizes(who, T, B, N, total_rows);
  if (rc != TBE_OK) return rc;
  TBE_REQUIRE(D > 0 && D % 4 == 0, "%s: D must be a positive multiple of 4 (got %lld)", who, (long long)D);
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "%s: bad dtype %d", who, dtype);
  if (!per_sample_weights) {
    // unweighted lookups run on the table-segmented sort and the lane-group run kernels
    rc = approx_backward_sorted(grad_output, stride_b, stride_t, weights, table_offsets, indices, offsets,
                                optimizer_state, T, B, D, N, total_rows, dtype, lr, eps, stochastic_rounding, sr_seed,
                                sr_offset, max_rows_per_table, workspace, workspace_bytes, stream_v);
    if (rc != TBE_ERR_UNSUPPORTED) return rc;
  }
  Workspace ws;
  rc = prepare_workspace(who, workspace, workspace_bytes, N, total_rows, &ws);
  if (rc != TBE_OK || N == 0) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const KeyLayout layout = key_layout(T, total_rows, max_rows_per_table, false);
  const int es = elem_size(dtype);
  const bool grad16 =
      reinterpret_cast<uintptr_t>(grad_output) % 16 == 0 && (stride_b * es) % 16 == 0 && (stride_t * es) % 16 == 0;
  const RowGeom g = make_geom(D, dtype, weights, grad16 ? nullptr : reinterpret_cast<const void*>(uintptr_t(8)));
  TBE_REQUIRE(g.vb == 16 || dtype == TBE_F16, "%s: weights and grad_output rows must be 16-byte aligned", who);
  if (g.vb == 8)
    TBE_REQUIRE(reinterpret_cast<uintptr_t>(grad_output) % 8 == 0 && (stride_b * es) % 8 == 0 &&
                    (stride_t * es) % 8 == 0 && reinterpret_cast<uintptr_t>(weights) % 8 == 0,
                "%s: weights and grad_output rows must be 8-byte aligned", who);
  ApproxArgs a{};
  a.grad = grad_output;
  a.stride_b = stride_b;
  a.stride_t = stride_t;
  a.weights = weights;
  a.state = optimizer_state;
  a.table_offsets = table_offsets;
  a.indices = indices;
  a.offsets = offsets;
  a.psw = per_sample_weights;
  a.grad_psw = grad_per_sample_weights;
  a.keys_in = ws.keys_in;
  a.vals_in = ws.vals_in;
  a.entry_bag = ws.entry_bag;
  a.entry_g2 = ws.entry_g2;
  a.keys = ws.keys;
  a.vals = ws.vals;
  a.seg_starts = ws.seg_starts;
  a.counters = ws.counters;
  a.B = static_cast<int32_t>(B);
  a.T = static_cast<int32_t>(T);
  a.D = static_cast<int32_t>(D);
  a.N = static_cast<int32_t>(N);
  a.idx_bits = layout.idx_bits;
  a.nvec = g.nvec;
  a.lr = lr;
  a.eps = eps;
  a.sr_seed = sr_seed;
  a.sr_offset = sr_offset;
  const bool weighted = per_sample_weights != nullptr;
  const bool sr = stochastic_rounding != 0 && dtype == TBE_F16;
  switch (dtype) {
    case TBE_F16:
      if (g.vb == 16) return launch_approx<__half, 16>(a, ws, layout, weighted, sr, stream);
      return launch_approx<__half, 8>(a, ws, layout, weighted, sr, stream);
    case TBE_F32:
      return launch_approx<float, 16>(a, ws, layout, weighted, false, stream);
    default:
      return launch_approx<double, 16>(a, ws, layout, weighted, false, stream);
  }
}
