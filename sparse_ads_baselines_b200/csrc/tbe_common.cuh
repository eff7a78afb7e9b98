// Shared device/host helpers for the TBE kernels (sm_100a).
//
// Row geometry used by every gather/scatter kernel here: a table row of D elements is
// moved as `nvec` vectors of VB bytes (16, or 8 when a fp16 row is only 8-byte
// aligned).  A row is owned by a "group" of lpr = 2^lpr_log2 lanes (lpr <= 32, the
// smallest power of two >= nvec, capped at 32); a warp therefore works on 32/lpr rows
// at once.  Rows wider than 32 vectors are walked in "chunks" of 32 vectors.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tbe_b200.h"

namespace tbe {

constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------- error plumbing
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
void count_kernel_launch(int n = 1);
void count_library_launch(int n = 1);
int tuning(int which);  // see tbe_api.cu
enum Tuning {
  kTuneFwdUnroll = 0,
  kTuneFwdThreads,
  kTuneBwdThreads,
  kTuneBwdUnroll,
  kTuneLongSegment,
  kTuneFwdBlocksPerSM,
  kTuneBwdBlocksPerSM,
  kTuneBwdVpl,
  kTuneBwdSort,     // 0: two-level bucket sort when the batch suits it, 1: always the device radix sort
  kTuneSortBucket,  // wanted mean bucket size of the two-level sort (0: default)
  kTuneSplitRuns,   // 1: never cut long runs into parts (one CTA per queued run)
  kTuneBwdStride,   // run_kernel's warps walk the tiles 1: with a fixed stride, 2: by ticket, 0: by the gradient's size
  kTuneCount
};

#define TBE_CUDA_TRY(expr)                                                            \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      return ::tbe::fail(TBE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                         cudaGetErrorString(_e), __FILE__, __LINE__);                 \
  } while (0)

#define TBE_REQUIRE(cond, ...)                                                        \
  do {                                                                                \
    if (!(cond)) return ::tbe::fail(TBE_ERR_INVALID_ARGUMENT, __VA_ARGS__);           \
  } while (0)

// Launch check that does not synchronise.
#define TBE_CHECK_LAUNCH(name)                                                        \
  do {                                                                                \
    cudaError_t _e = cudaGetLastError();                                              \
    if (_e != cudaSuccess)                                                            \
      return ::tbe::fail(TBE_ERR_CUDA, "launch of %s failed: %s", name,               \
                         cudaGetErrorString(_e));                                     \
    ::tbe::count_kernel_launch();                                                     \
  } while (0)

int device_sm_count();
int64_t device_l2_bytes();
// Waits for host-side work the library still has in flight (the staged cache fill scatters evicted
// rows into the host table in the background).
void host_pool_wait();

// Optional per-launch timing: when enabled (tbe_kernel_timing_enable), every launch site brackets
// its kernel with two CUDA events on the launch stream; tbe_kernel_timing_read sums them per name.
class KernelTimer {
 public:
  KernelTimer(const char* name, cudaStream_t stream);
  ~KernelTimer();
  KernelTimer(const KernelTimer&) = delete;
  KernelTimer& operator=(const KernelTimer&) = delete;

 private:
  const char* name_;
  cudaStream_t stream_;
  cudaEvent_t start_ = nullptr;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------- row geometry
struct RowGeom {
  int vb;        // bytes per vector (8 or 16)
  int nvec;      // vectors per row
  int lpr_log2;  // log2(lanes per row)
  int nchunks;   // ceil(nvec / 32)
};

inline int elem_size(int dtype) { return dtype == TBE_F16 ? 2 : dtype == TBE_F32 ? 4 : 8; }

// Picks the widest vector every row start is aligned to.  `base` is the weights
// pointer; rows start at base + r * D * elem_size.
inline RowGeom make_geom(int64_t D, int dtype, const void* base0, const void* base1 = nullptr) {
  RowGeom g;
  const int64_t row_bytes = D * elem_size(dtype);
  const bool a16 = (row_bytes % 16 == 0) && (reinterpret_cast<uintptr_t>(base0) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(base1) % 16 == 0);
  g.vb = a16 ? 16 : 8;
  g.nvec = static_cast<int>(row_bytes / g.vb);
  int l = 0;
  while ((1 << l) < g.nvec && l < 5) ++l;
  g.lpr_log2 = l;
  g.nchunks = (g.nvec + 31) / 32;
  return g;
}

// ---------------------------------------------------------------- raw vector moves
template <int VB>
struct Raw;
template <>
struct Raw<16> {
  uint32_t w[4];
};
template <>
struct Raw<8> {
  uint32_t w[2];
};

template <int VB>
__device__ __forceinline__ Raw<VB> raw_zero() {
  Raw<VB> r;
#pragma unroll
  for (int i = 0; i < VB / 4; ++i) r.w[i] = 0u;
  return r;
}

// Read-only streaming load: table rows and gradient rows are touched once per kernel,
// so they bypass L1 allocation.
template <int VB>
__device__ __forceinline__ Raw<VB> ld_stream(const void* p);
template <>
__device__ __forceinline__ Raw<16> ld_stream<16>(const void* p) {
  Raw<16> r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
               : "l"(p));
  return r;
}
template <>
__device__ __forceinline__ Raw<8> ld_stream<8>(const void* p) {
  Raw<8> r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(r.w[0]), "=r"(r.w[1])
               : "l"(p));
  return r;
}

// Coherent load for rows this kernel also writes (weights in the backward).
template <int VB>
__device__ __forceinline__ Raw<VB> ld_rw(const void* p);
template <>
__device__ __forceinline__ Raw<16> ld_rw<16>(const void* p) {
  Raw<16> r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
               : "l"(p)
               : "memory");
  return r;
}
template <>
__device__ __forceinline__ Raw<8> ld_rw<8>(const void* p) {
  Raw<8> r;
  asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(r.w[0]), "=r"(r.w[1])
               : "l"(p)
               : "memory");
  return r;
}

template <int VB>
__device__ __forceinline__ void st_row(void* p, const Raw<VB>& r);
template <>
__device__ __forceinline__ void st_row<16>(void* p, const Raw<16>& r) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};"
               :
               : "l"(p), "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3])
               : "memory");
}
template <>
__device__ __forceinline__ void st_row<8>(void* p, const Raw<8>& r) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" : : "l"(p), "r"(r.w[0]), "r"(r.w[1]) : "memory");
}

// L2 residency hints.  Gather/scatter kernels stream gigabytes of table rows once through L2 while
// re-reading a few tens of megabytes (pooled gradient rows, sorted ids) many times: the streamed
// rows are marked evict-first and the re-read rows evict-last so the latter stay resident.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

template <int VB>
__device__ __forceinline__ Raw<VB> ld_stream_hint(const void* p, uint64_t policy);
template <>
__device__ __forceinline__ Raw<16> ld_stream_hint<16>(const void* p, uint64_t policy) {
  Raw<16> r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
               : "l"(p), "l"(policy));
  return r;
}
template <>
__device__ __forceinline__ Raw<8> ld_stream_hint<8>(const void* p, uint64_t policy) {
  Raw<8> r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;"
               : "=r"(r.w[0]), "=r"(r.w[1])
               : "l"(p), "l"(policy));
  return r;
}

template <int VB>
__device__ __forceinline__ Raw<VB> ld_rw_hint(const void* p, uint64_t policy);
template <>
__device__ __forceinline__ Raw<16> ld_rw_hint<16>(const void* p, uint64_t policy) {
  Raw<16> r;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
               : "l"(p), "l"(policy)
               : "memory");
  return r;
}
template <>
__device__ __forceinline__ Raw<8> ld_rw_hint<8>(const void* p, uint64_t policy) {
  Raw<8> r;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;"
               : "=r"(r.w[0]), "=r"(r.w[1])
               : "l"(p), "l"(policy)
               : "memory");
  return r;
}

template <int VB>
__device__ __forceinline__ void st_row_hint(void* p, const Raw<VB>& r, uint64_t policy);
template <>
__device__ __forceinline__ void st_row_hint<16>(void* p, const Raw<16>& r, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;"
               :
               : "l"(p), "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3]), "l"(policy)
               : "memory");
}
template <>
__device__ __forceinline__ void st_row_hint<8>(void* p, const Raw<8>& r, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v2.u32 [%0], {%1,%2}, %3;"
               :
               : "l"(p), "r"(r.w[0]), "r"(r.w[1]), "l"(policy)
               : "memory");
}

// Division of a 32-bit unsigned by a run-time constant as multiply + shifts (Granlund & Montgomery,
// "Division by invariant integers using multiplication", round-up variant); exact for all n.
struct FastDiv {
  uint32_t m, s1, s2;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;  // ceil(log2 d)
  f.m = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - d)) / d + 1);
  f.s1 = l < 1 ? l : 1;
  f.s2 = l > 0 ? l - 1 : 0;
  return f;
}
__device__ __forceinline__ uint32_t fastdiv(uint32_t n, const FastDiv& f) {
  const uint32_t t1 = __umulhi(f.m, n);
  return (t1 + ((n - t1) >> f.s1)) >> f.s2;
}

// ---------------------------------------------------------------- element <-> accumulator
template <typename T>
struct Acc {
  using type = float;
};
template <>
struct Acc<double> {
  using type = double;
};

template <typename T, int VB>
struct VecTraits {
  static constexpr int N = VB / sizeof(T);  // elements per vector
  using acc_t = typename Acc<T>::type;
};

template <typename T, int VB>
__device__ __forceinline__ void unpack(const Raw<VB>& r, typename Acc<T>::type* out);

template <>
__device__ __forceinline__ void unpack<__half, 16>(const Raw<16>& r, float* out) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r.w[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void unpack<__half, 8>(const Raw<8>& r, float* out) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r.w[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void unpack<float, 16>(const Raw<16>& r, float* out) {
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = __uint_as_float(r.w[i]);
}
template <>
__device__ __forceinline__ void unpack<double, 16>(const Raw<16>& r, double* out) {
  out[0] = __hiloint2double(static_cast<int>(r.w[1]), static_cast<int>(r.w[0]));
  out[1] = __hiloint2double(static_cast<int>(r.w[3]), static_cast<int>(r.w[2]));
}

// acc[k] += element k of the vector.  For fp16 rows this is Blackwell's mixed-precision add
// (add.rn.f32.f16: fp16 operand, fp32 accumulator, one rounding): the same value as converting and
// adding, in half the instructions -- these kernels are short of issue slots, not of FLOPs.
template <typename T, int VB>
__device__ __forceinline__ void accumulate(const Raw<VB>& r, typename Acc<T>::type* acc) {
  constexpr int NE = VB / sizeof(T);
  typename Acc<T>::type e[NE];
  unpack<T, VB>(r, e);
#pragma unroll
  for (int k = 0; k < NE; ++k) acc[k] += e[k];
}
__device__ __forceinline__ void add_half2_to_floats(uint32_t packed, float& a0, float& a1) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %1, hi, %1;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "r"(packed));
}
template <>
__device__ __forceinline__ void accumulate<__half, 16>(const Raw<16>& r, float* acc) {
#pragma unroll
  for (int i = 0; i < 4; ++i) add_half2_to_floats(r.w[i], acc[2 * i], acc[2 * i + 1]);
}
template <>
__device__ __forceinline__ void accumulate<__half, 8>(const Raw<8>& r, float* acc) {
#pragma unroll
  for (int i = 0; i < 2; ++i) add_half2_to_floats(r.w[i], acc[2 * i], acc[2 * i + 1]);
}

// Round-to-nearest-even pack.
template <typename T, int VB>
__device__ __forceinline__ Raw<VB> pack_rn(const typename Acc<T>::type* in);

template <>
__device__ __forceinline__ Raw<16> pack_rn<__half, 16>(const float* in) {
  Raw<16> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    r.w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return r;
}
template <>
__device__ __forceinline__ Raw<8> pack_rn<__half, 8>(const float* in) {
  Raw<8> r;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    r.w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return r;
}
template <>
__device__ __forceinline__ Raw<16> pack_rn<float, 16>(const float* in) {
  Raw<16> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.w[i] = __float_as_uint(in[i]);
  return r;
}
template <>
__device__ __forceinline__ Raw<16> pack_rn<double, 16>(const double* in) {
  Raw<16> r;
  r.w[0] = static_cast<uint32_t>(__double2loint(in[0]));
  r.w[1] = static_cast<uint32_t>(__double2hiint(in[0]));
  r.w[2] = static_cast<uint32_t>(__double2loint(in[1]));
  r.w[3] = static_cast<uint32_t>(__double2hiint(in[1]));
  return r;
}

// Stochastic rounding to fp16: add 13 uniformly random bits below the fp16 mantissa of
// the fp32 value and truncate (the arithmetic of the reference's
// stochastic_rounding_vector, table_batched_embeddings_cuda.cu:564-578).
__device__ __forceinline__ __half sr_half(float x, uint32_t rnd) {
  return __float2half_rz(__uint_as_float(__float_as_uint(x) + (rnd >> 19)));
}

// Philox4x32-10 counter-based generator (Salmon et al., SC'11), written out here so the
// library has no curand dependency.  key = seed, counter = (offset, subsequence).
struct Philox {
  uint32_t key[2];
  uint32_t ctr[4];
  __device__ __forceinline__ Philox(uint64_t seed, uint64_t subsequence, uint64_t offset) {
    key[0] = static_cast<uint32_t>(seed);
    key[1] = static_cast<uint32_t>(seed >> 32);
    ctr[0] = static_cast<uint32_t>(offset);
    ctr[1] = static_cast<uint32_t>(offset >> 32);
    ctr[2] = static_cast<uint32_t>(subsequence);
    ctr[3] = static_cast<uint32_t>(subsequence >> 32);
  }
  __device__ __forceinline__ uint4 next() {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
    for (int round = 0; round < 10; ++round) {
      const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
      c0 = n0;
      c1 = lo1;
      c2 = n2;
      c3 = lo0;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    if (++ctr[0] == 0) ++ctr[1];
    return make_uint4(c0, c1, c2, c3);
  }
};

// Sum over the lanes of one row group (lanes differing only in bits < lpr_log2).
template <typename A>
__device__ __forceinline__ A group_sum(A v, int lpr_log2) {
  for (int m = 1; m < (1 << lpr_log2); m <<= 1) v += __shfl_xor_sync(kFullMask, v, m);
  return v;
}

}  // namespace tbe
