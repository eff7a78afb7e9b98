// Cross-GPU ordering for the fused table-sharded exchange: flags in peer-mapped memory (sm_100a).
//
// The exchange kernels (tbe_forward_sharded, tbe_all2all_push) store straight into other ranks'
// buffers.  What the consumers on those ranks need is "every rank's stores of step k have landed",
// and what the producers need is "the buffer I am about to overwrite has been consumed".  Both are
// one word per (rank, peer): rank r owns a flag array int32 [world] in memory that every peer can
// write, peer j writes slot j of it.  Values only grow (step numbers), so a flag never has to be
// reset and "at least step k" is the test.
//
//   signal : one thread per peer stores `value` into slot `rank` of that peer's array with
//            st.release.sys -- ordered after everything this GPU did earlier in the stream (kernel
//            boundaries order the earlier kernels' stores before this thread, the release makes
//            them visible before the flag).
//   wait   : one thread per peer polls its local slot with ld.acquire.sys until it reaches the
//            wanted value.  The poll is BOUNDED: after `timeout_ns` of wall time the thread records
//            {TBE_ERR_TIMEOUT, peer, wanted, seen} in `status` and the kernel returns, so a rank that
//            died or never joined costs the others a timeout, not a hung GPU.  The host reads
//            `status` when it next synchronises.
//
// A kernel that polls only ever waits for kernels on OTHER GPUs (its own producer precedes it in
// stream order), so no two kernels of one GPU wait on each other.  Plain loads and stores only: no
// TMA, no multicast, no multimem.
#include "tbe_common.cuh"

namespace tbe {
namespace {

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" : : "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct SyncArgs {
  int32_t* peer_flags[TBE_MAX_PEERS];  // peer j's flag array (valid on this device); null = no signal
  const int32_t* local_flags;          // this rank's flag array; null = no wait
  int32_t* status;                     // int32 [4]: {code, peer, wanted, seen}; written on timeout only
  int32_t world, rank;
  int32_t signal_value, wait_value;
  int64_t timeout_ns;
};

// One CTA, one thread per peer: signal first, then wait.
__global__ void __launch_bounds__(32) peer_signal_wait_kernel(const SyncArgs a) {
  const int j = threadIdx.x;
  if (j >= a.world) return;
  if (a.peer_flags[j] != nullptr) {
    __threadfence_system();
    st_release_sys(a.peer_flags[j] + a.rank, a.signal_value);
  }
  if (a.local_flags == nullptr) return;
  const int32_t* slot = a.local_flags + j;
  int32_t seen = ld_acquire_sys(slot);
  if (seen - a.wait_value >= 0) return;  // (difference: correct across a wrap of the step counter)
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = static_cast<uint64_t>(a.timeout_ns);
  // the clock is read every 64 polls; the iteration cap bounds the loop even if the clock stood still
  for (uint64_t it = 0; it < (1ull << 28); ++it) {
    seen = ld_acquire_sys(slot);
    if (seen - a.wait_value >= 0) return;
    if ((it & 63u) == 63u && global_timer_ns() - t0 > limit) break;
    __nanosleep(40);
  }
  if (atomicCAS(a.status, 0, TBE_ERR_TIMEOUT) == 0) {
    a.status[1] = j;
    a.status[2] = a.wait_value;
    a.status[3] = seen;
  }
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_peer_signal_wait(void* const* peer_flags, const int32_t* local_flags, int world, int rank,
                                    int32_t signal_value, int32_t wait_value, int64_t timeout_ns, int32_t* status,
                                    void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(world >= 1 && world <= TBE_MAX_PEERS && rank >= 0 && rank < world,
              "tbe_peer_signal_wait: bad world/rank %d/%d", world, rank);
  TBE_REQUIRE(peer_flags != nullptr || local_flags != nullptr, "tbe_peer_signal_wait: nothing to signal or wait for");
  TBE_REQUIRE(local_flags == nullptr || (status != nullptr && timeout_ns > 0),
              "tbe_peer_signal_wait: a wait needs a status word and a positive timeout");
  SyncArgs a{};
  for (int j = 0; j < world; ++j) {
    a.peer_flags[j] = nullptr;
    if (peer_flags != nullptr) {
      TBE_REQUIRE(peer_flags[j] != nullptr && reinterpret_cast<uintptr_t>(peer_flags[j]) % 4 == 0,
                  "tbe_peer_signal_wait: flag pointer %d is null or misaligned", j);
      a.peer_flags[j] = static_cast<int32_t*>(peer_flags[j]);
    }
  }
  a.local_flags = local_flags;
  a.status = status;
  a.world = world;
  a.rank = rank;
  a.signal_value = signal_value;
  a.wait_value = wait_value;
  a.timeout_ns = timeout_ns;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  {
    KernelTimer timer("peer_signal_wait_kernel", stream);
    peer_signal_wait_kernel<<<1, 32, 0, stream>>>(a);
  }
  TBE_CHECK_LAUNCH("peer_signal_wait_kernel");
  return TBE_OK;
}

extern "C" int tbe_peer_status(const int32_t* status, int32_t* host_out4, void* stream_v) {
  using namespace tbe;
  TBE_REQUIRE(status && host_out4, "tbe_peer_status: null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  TBE_CUDA_TRY(cudaMemcpyAsync(host_out4, status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  TBE_CUDA_TRY(cudaStreamSynchronize(stream));
  if (host_out4[0] == TBE_ERR_TIMEOUT)
    return fail(TBE_ERR_TIMEOUT, "a bounded wait for rank %d ran out: wanted step %d, last saw %d", host_out4[1],
                host_out4[2], host_out4[3]);
  return TBE_OK;
}
