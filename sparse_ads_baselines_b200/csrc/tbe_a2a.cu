// All-to-all, all-gather and slot reduction of pooled rows / pooled gradients as direct peer stores
// over NVLink (sm_100a).
//
// Every rank holds src = [rows_local][world][chunk] and owns, on every peer r, a destination
// buffer dst_r = [world][rows_local][chunk]; the kernel copies src[i][r][:] to
// dst_r[rank][i][:] with plain 16-byte stores to peer-mapped addresses (no TMA, no multicast).
// With rows_local = B/W and chunk = (T/W)*D this is the gradient exchange of the table-sharded
// backward: each rank scatters its batch slice of the pooled gradient to the table owners, which
// receive [B][T/W][D] in the layout the local backward consumes, with no transpose copy on
// either side.  The caller orders the kernel against the consumers with its own barrier.
#include "tbe_common.cuh"

namespace tbe {
namespace {

struct PushArgs {
  const char* src;
  char* dst[TBE_MAX_PEERS];
  int32_t world, rank;
  int64_t rows_local;
  int64_t chunk_vecs;  // 16-byte (or VB-byte) vectors per chunk
};

template <int VB>
__global__ void __launch_bounds__(256) all2all_push_kernel(const PushArgs a) {
  const int64_t total = a.rows_local * a.world * a.chunk_vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t v = i % a.chunk_vecs;
    const int64_t rc = i / a.chunk_vecs;      // row * world + peer
    const int peer = static_cast<int>(rc % a.world);
    const int64_t row = rc / a.world;
    const Raw<VB> r = ld_stream<VB>(a.src + i * VB);
    char* d = a.dst[peer] + ((static_cast<int64_t>(a.rank) * a.rows_local + row) * a.chunk_vecs + v) * VB;
    st_row<VB>(d, r);
  }
}

// All-gather by peer stores: this rank's `vecs` vectors go to slot `rank` of every peer's buffer.
template <int VB>
__global__ void __launch_bounds__(256) allgather_push_kernel(const PushArgs a) {
  const int64_t vecs = a.chunk_vecs;
  const int64_t total = vecs * a.world;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int peer = static_cast<int>(i / vecs);
    const int64_t v = i - static_cast<int64_t>(peer) * vecs;
    const Raw<VB> r = ld_stream<VB>(a.src + v * VB);  // re-read per peer: the source stays in L2
    st_row<VB>(a.dst[peer] + (static_cast<int64_t>(a.rank) * vecs + v) * VB, r);
  }
}

struct ReduceArgs {
  const char* slots;
  char* out;
  int32_t world;
  int64_t vecs;  // vectors per slot
};

// out[i] = sum over slots r = 0 .. world-1 of slots[r][i], accumulated in fp32 (fp64 for double) in
// slot order, so the result does not depend on scheduling.
template <typename T, int VB>
__global__ void __launch_bounds__(256) reduce_slots_kernel(const ReduceArgs a) {
  using acc_t = typename Acc<T>::type;
  constexpr int NE = VB / sizeof(T);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.vecs; i += stride) {
    acc_t acc[NE];
#pragma unroll
    for (int k = 0; k < NE; ++k) acc[k] = 0;
    for (int r = 0; r < a.world; r += 4) {  // four slots in flight
      Raw<VB> v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = r + u < a.world ? ld_stream<VB>(a.slots + (static_cast<int64_t>(r + u) * a.vecs + i) * VB) : raw_zero<VB>();
#pragma unroll
      for (int u = 0; u < 4; ++u) accumulate<T, VB>(v[u], acc);
    }
    st_row<VB>(a.out + i * VB, pack_rn<T, VB>(acc));
  }
}

int64_t copy_grid(int64_t total) {
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  return blocks > cap ? cap : (blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_allgather_push(const void* src, void* const* peer_dst, int world, int rank, int64_t bytes,
                                  void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(src && peer_dst, "tbe_allgather_push: null pointer argument");
  TBE_REQUIRE(world >= 1 && world <= TBE_MAX_PEERS && rank >= 0 && rank < world,
              "tbe_allgather_push: bad world/rank %d/%d", world, rank);
  TBE_REQUIRE(bytes > 0 && bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0,
              "tbe_allgather_push: the slice must be 16-byte aligned and a multiple of 16 bytes long");
  PushArgs a{};
  a.src = static_cast<const char*>(src);
  for (int r = 0; r < world; ++r) {
    TBE_REQUIRE(peer_dst[r] != nullptr && reinterpret_cast<uintptr_t>(peer_dst[r]) % 16 == 0,
                "tbe_allgather_push: destination %d is null or misaligned", r);
    a.dst[r] = static_cast<char*>(peer_dst[r]);
  }
  a.world = world;
  a.rank = rank;
  a.chunk_vecs = bytes / 16;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  {
    KernelTimer timer("allgather_push_kernel", stream);
    allgather_push_kernel<16><<<static_cast<unsigned>(copy_grid(a.chunk_vecs * world)), 256, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("allgather_push_kernel");
  return TBE_OK;
}

extern "C" int tbe_reduce_slots(const void* slots, void* out, int world, int64_t elems_per_slot, int dtype,
                                void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(slots && out, "tbe_reduce_slots: null pointer argument");
  TBE_REQUIRE(world >= 1 && world <= TBE_MAX_PEERS, "tbe_reduce_slots: bad world %d", world);
  TBE_REQUIRE(dtype == TBE_F32 || dtype == TBE_F16 || dtype == TBE_F64, "tbe_reduce_slots: bad dtype %d", dtype);
  const int64_t bytes = elems_per_slot * elem_size(dtype);
  TBE_REQUIRE(elems_per_slot > 0 && bytes % 16 == 0 && reinterpret_cast<uintptr_t>(slots) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "tbe_reduce_slots: slots must be 16-byte aligned and a multiple of 16 bytes long");
  ReduceArgs a{static_cast<const char*>(slots), static_cast<char*>(out), world, bytes / 16};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const unsigned grid = static_cast<unsigned>(copy_grid(a.vecs));
  {
    KernelTimer timer("reduce_slots_kernel", stream);
    if (dtype == TBE_F16) {
      reduce_slots_kernel<__half, 16><<<grid, 256, 0, stream>>>(a);
    } else if (dtype == TBE_F32) {
      reduce_slots_kernel<float, 16><<<grid, 256, 0, stream>>>(a);
    } else {
      reduce_slots_kernel<double, 16><<<grid, 256, 0, stream>>>(a);
    }
  }
  TBE_CHECK_LAUNCH("reduce_slots_kernel");
  return TBE_OK;
}

extern "C" int tbe_all2all_push(const void* src, void* const* peer_dst, int world, int rank, int64_t rows_local,
                                int64_t chunk_bytes, void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(src && peer_dst, "tbe_all2all_push: null pointer argument");
  TBE_REQUIRE(world >= 1 && world <= TBE_MAX_PEERS && rank >= 0 && rank < world,
              "tbe_all2all_push: bad world/rank %d/%d", world, rank);
  TBE_REQUIRE(rows_local > 0 && chunk_bytes > 0, "tbe_all2all_push: sizes must be > 0");
  int vb = 16;
  bool ok16 = chunk_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0;
  PushArgs a{};
  a.src = static_cast<const char*>(src);
  for (int r = 0; r < world; ++r) {
    TBE_REQUIRE(peer_dst[r] != nullptr, "tbe_all2all_push: destination %d is null", r);
    a.dst[r] = static_cast<char*>(peer_dst[r]);
    if (reinterpret_cast<uintptr_t>(peer_dst[r]) % 16 != 0) ok16 = false;
  }
  if (!ok16) {
    vb = 8;
    TBE_REQUIRE(chunk_bytes % 8 == 0 && reinterpret_cast<uintptr_t>(src) % 8 == 0,
                "tbe_all2all_push: chunks must be 8-byte aligned");
    for (int r = 0; r < world; ++r)
      TBE_REQUIRE(reinterpret_cast<uintptr_t>(peer_dst[r]) % 8 == 0, "tbe_all2all_push: destination %d misaligned", r);
  }
  a.world = world;
  a.rank = rank;
  a.rows_local = rows_local;
  a.chunk_vecs = chunk_bytes / vb;
  const int64_t total = rows_local * world * a.chunk_vecs;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  {
    KernelTimer timer("all2all_push_kernel", stream);
    if (vb == 16) {
      all2all_push_kernel<16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
    } else {
      all2all_push_kernel<8><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
    }
  }
  TBE_CHECK_LAUNCH("all2all_push_kernel");
  return TBE_OK;
}
