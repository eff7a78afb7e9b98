/*
 * tbe_b200.h -- C ABI of libtbe_b200.so: table-batched embedding bags (TBE) for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).  Nothing
 * here allocates device memory unless its comment says so: outputs, optimizer
 * state and scratch ("workspace") are owned by the caller.  All work is enqueued
 * on the given stream and the call returns without synchronising, unless noted.
 *
 * Return value: TBE_OK (0) or a negative tbe_status_t.  tbe_last_error_string()
 * returns a thread-local description of the last failure on the calling thread.
 *
 * Data layout shared by all calls (it is the layout of the reference's
 * table_batched_embeddings extension, table_batched_embeddings_cuda.cu:193-223):
 *   weights        [total_rows][D] row-major, dtype = tbe_dtype_t
 *   table_offsets  int32 [T]   first row of table t inside `weights`
 *   indices        int32 [N]   row ids local to their table, bags flattened [T][B][L]
 *   offsets        int32 [T*B+1] bag (t,b) owns indices[offsets[t*B+b] .. offsets[t*B+b+1])
 *   output / grad  [B][T][D]   same dtype as weights
 * Each citation "replaces <file>:<lines>" names the reference function whose
 * pybind11 binding the entry point stands in for.
 */
#ifndef TBE_B200_H_
#define TBE_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define TBE_API __attribute__((visibility("default")))
#else
#define TBE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TBE_OK = 0,
  TBE_ERR_INVALID_ARGUMENT = -1, /* shape/dtype/alignment/null-pointer contract broken */
  TBE_ERR_WORKSPACE_TOO_SMALL = -2,
  TBE_ERR_CUDA = -3,             /* a CUDA runtime call or launch failed */
  TBE_ERR_UNSUPPORTED = -4,      /* valid request this build does not implement */
  TBE_ERR_BAD_INPUT_DATA = -5,   /* tbe_check_inputs found an index/offset violation */
  TBE_ERR_TIMEOUT = -6           /* a bounded device-side wait ran out */
} tbe_status_t;

typedef enum { TBE_F32 = 0, TBE_F16 = 1, TBE_F64 = 2 } tbe_dtype_t;
typedef enum { TBE_POOL_SUM = 0, TBE_POOL_MEAN = 1 } tbe_pooling_t;

#define TBE_MAX_PEERS 16

/* ---- library ---------------------------------------------------------- */

/* Version of this ABI (bumped on any signature change). */
TBE_API int tbe_abi_version(void);
/* Thread-local text of the last error returned on this thread ("" if none). */
TBE_API const char* tbe_last_error_string(void);
/* Number of kernels of this library launched by this process so far (own kernels
 * only; CUB sort/select launches are counted separately by tbe_library_launch_count). */
TBE_API int64_t tbe_kernel_launch_count(void);
TBE_API int64_t tbe_library_launch_count(void);
/* Tuning knob for benchmarking sweeps; value 0 restores the default.  Names:
 *   fwd_unroll, fwd_threads, fwd_blocks_per_sm   forward: row loads in flight per lane, CTA size, CTAs per SM
 *   bwd_threads, bwd_blocks_per_sm               backward apply: CTA size, CTAs per SM
 *   bwd_vpl, bwd_unroll                          backward apply: 16-byte vectors per lane (1/2/4), runs in flight (1/2)
 *   long_segment                                 run length above which a run gets a CTA of its own
 *   bwd_sort                                     1: always linearize + device radix sort for the backward plan
 *   sort_bucket                                  wanted mean bucket size of the table-segmented sort
 *   split_runs                                   1: one CTA per queued long run, never several
 *   bwd_stride                                   backward apply hands out its tiles 1: with a fixed stride, 2: by a ticket
 *                                                counter (default: tickets once the pooled gradient exceeds a third of L2) */
TBE_API int tbe_set_tuning(const char* name, int value);

/* Per-launch timing for benchmarks: while enabled, every kernel launch of this library
 * (and each CUB call) is bracketed by two CUDA events on its stream.  Enabling or
 * disabling discards earlier records.  tbe_kernel_timing_read SYNCHRONISES on the
 * recorded events, writes one "name launches total_ms" line per kernel into buffer
 * (NUL-terminated), clears the records and returns the text length. */
TBE_API int tbe_kernel_timing_enable(int on);
TBE_API int64_t tbe_kernel_timing_read(char* buffer, int64_t buffer_bytes);

/* ---- forward: pooled gather ------------------------------------------- */

/* out[b][t][:] = sum_l w_l * weights[table_offsets[t] + indices[..l..]][:]  (mean: / L).
 * per_sample_weights may be NULL (w_l = 1); with TBE_POOL_MEAN it must be NULL.
 * Requires D % 4 == 0, T,B,D > 0.  Accumulates in fp32 (fp64 for TBE_F64) and
 * rounds to nearest on store.
 * replaces table_batched_embeddings_cuda.cu:253-316 (batched_embedding_forward_cuda). */
TBE_API int tbe_forward(const void* weights, const int32_t* table_offsets,
                const int32_t* indices, const int32_t* offsets,
                const void* per_sample_weights, void* output,
                int64_t T, int64_t B, int64_t D, int dtype, int pooling,
                void* stream);

/* tbe_forward into a wider output: sample b's row of table t starts at
 * output + b*out_stride_b + t*D (elements), out_stride_b >= T*D.  It lets tables of
 * different width share one [B][sum D] output, one call per width.
 * replaces table_batched_embeddings_cuda.cu:945-1004 (batched_embedding_forward_mixed_D_cuda)
 * together with the per-table loop of the mixed-D op layer. */
TBE_API int tbe_forward_strided(const void* weights, const int32_t* table_offsets,
                const int32_t* indices, const int32_t* offsets,
                const void* per_sample_weights, void* output, int64_t out_stride_b,
                int64_t T, int64_t B, int64_t D, int dtype, int pooling, void* stream);

/* Tables of different width in ONE launch: weights is a flat vector, table t's rows start at element
 * weight_offsets[t] (int64 [T+1]) and are dim_offsets[t+1] - dim_offsets[t] wide (int32 [T+1]); the
 * pooled rows go to columns [dim_offsets[t], dim_offsets[t+1]) of output [B][total_D].  Every width
 * must be a multiple of 4; vector_bytes is 16 when every table's rows, and every table's output
 * column block, start on 16-byte boundaries (always true for fp32), else 8 (fp16 only).  Sum pooling.
 * replaces table_batched_embeddings_cuda.cu:882-1004 (batched_embedding_forward_mixed_D_cuda). */
TBE_API int tbe_forward_mixed(const void* weights, const int64_t* weight_offsets, const int32_t* dim_offsets,
                              const int32_t* indices, const int32_t* offsets, const void* per_sample_weights,
                              void* output, int64_t T, int64_t B, int64_t total_D, int dtype, int vector_bytes,
                              void* stream);

/* Table-sharded forward with the all-to-all fused into the store: this rank owns
 * T local tables (global columns t0 .. t0+T of T_total) and looks up the GLOBAL
 * batch B for them; sample b belongs to rank b / (B / world) and its pooled row is
 * written straight into that rank's buffer at
 *   peer_outputs[b / B_local][(b % B_local)][t0 + t][:]     ([B_local][T_total][D])
 * where peer_outputs[r] is a device pointer valid on THIS device (peer-mapped for
 * r != own rank).  The caller orders this kernel against the consumers with its own
 * barrier.  Layout contract of sparse_embedding_cuda.cpp:471-533
 * (forward_all2all_nccl: out_j[b', r*T/W + t] = in_r[j*B/W + b', t]). */
TBE_API int tbe_forward_sharded(const void* weights, const int32_t* table_offsets,
                        const int32_t* indices, const int32_t* offsets,
                        const void* per_sample_weights,
                        void* const* peer_outputs, int world,
                        int64_t T, int64_t B, int64_t D,
                        int64_t T_total, int64_t t0,
                        int dtype, int pooling, void* stream);

/* All-to-all by direct peer stores: this rank holds src = [rows_local][world][chunk_bytes]
 * and copies src[i][r] to peer_dst[r] + ((rank * rows_local + i) * chunk_bytes), i.e. every
 * peer r ends up with dst_r = [world][rows_local][chunk_bytes].  peer_dst[r] are device
 * pointers valid on this device (peer-mapped).  With rows_local = B/W and
 * chunk_bytes = (T/W)*D*elem it is the gradient exchange of the table-sharded backward
 * (All2AllFunction.backward, sparse_embedding_cuda_ops.py:104-117) without either of
 * its transpose copies.  The caller orders it against the consumers with its own barrier.
 * replaces sparse_embedding_cuda.cpp:471-533 (forward_all2all_nccl) on the backward path. */
TBE_API int tbe_all2all_push(const void* src, void* const* peer_dst, int world, int rank,
                             int64_t rows_local, int64_t chunk_bytes, void* stream);

/* Row-wise sharding (every rank holds a slice of the rows of every table and looks up the global batch
 * with indices local to its slice; the reference's UniformShardedEmbeddingBags + ReduceScatterFunction,
 * models.py:194-209).  Forward: every rank stores its partial pooled rows for the samples of rank j
 * into slot `rank` of rank j's buffer [world][B/world][T][D] -- that is tbe_forward_sharded with
 * peer_outputs[j] advanced by rank slots, T_total = T and t0 = 0 -- and, once all slots have landed,
 * rank j sums them:  out[i] = sum_r slots[r][i], r ascending, fp32 accumulation (fp64 for TBE_F64).
 * replaces sparse_embedding_cuda.cpp:417-448 (forward_reduce_scatter: ncclReduceScatter). */
TBE_API int tbe_reduce_slots(const void* slots, void* out, int world, int64_t elems_per_slot, int dtype,
                             void* stream);
/* Backward of the same: every rank's gradient slice [B/world][T][D] (`bytes` long) goes to slot `rank`
 * of every peer's [world][B/world][T][D] = [B][T][D] buffer by direct peer stores.
 * replaces sparse_embedding_cuda.cpp:535-566 (forward_allgather: ncclAllGather). */
TBE_API int tbe_allgather_push(const void* src, void* const* peer_dst, int world, int rank, int64_t bytes,
                               void* stream);

/* Ordering between ranks for the exchange kernels above, without a collective: every rank owns a
 * flag array int32 [world] that all peers can write (peer-mapped, zero-initialised before first
 * use); rank r writes slot r of every peer's array.  One launch of one small CTA does, per peer j,
 *   signal: if peer_flags != NULL, store signal_value to peer_flags[j][rank] with release semantics at
 *           system scope -- after everything enqueued earlier on `stream`, peer stores included;
 *   wait:   if local_flags != NULL, poll local_flags[j] until it is >= wait_value (step numbers only
 *           grow).  The poll is bounded: after timeout_ns it writes {TBE_ERR_TIMEOUT, j, wait_value,
 *           last value seen} to status (device int32 [4], zero = no error; only the first timeout is
 *           kept) and returns, so a rank that died or never joined costs a timeout, never a hung GPU.
 * A barrier after a producer kernel is signal_value = wait_value = step.  Kernels launched later on
 * `stream` run after the wait returns (timed out or not): read status before trusting their results.
 * tbe_peer_status copies status to host_out4, SYNCHRONISES the stream and returns TBE_ERR_TIMEOUT
 * (with the peer and steps in the error string) if a wait ran out.
 * replaces the ncclGroupStart/ncclSend/ncclRecv/ncclGroupEnd ordering of forward_all2all_nccl
 * (sparse_embedding_cuda.cpp:488-523), which the fused exchange has no collective call to inherit. */
TBE_API int tbe_peer_signal_wait(void* const* peer_flags, const int32_t* local_flags, int world, int rank,
                                 int32_t signal_value, int32_t wait_value, int64_t timeout_ns,
                                 int32_t* status, void* stream);
TBE_API int tbe_peer_status(const int32_t* status, int32_t* host_out4, void* stream);

/* ---- backward with the optimizer fused into the write-back -------------- */

/* Scratch bytes the backward calls need for N indices over total_rows rows. */
TBE_API int64_t tbe_backward_workspace_bytes(int64_t N, int64_t total_rows);

/* The part of the backward that depends on the indices only: all N lookups sorted
 * (stable) so that lookups of one row are adjacent, with the bag id of every sorted
 * entry, left in `workspace`.  A backward call given the same workspace, the same
 * max_rows_per_table and plan_ready = 1 skips this phase, so a caller can run it on
 * another stream while the forward (or an exchange) is in flight.
 * max_rows_per_table (0 = unknown) is the largest table's row count: when known, the
 * sort only looks at ceil(log2(max_rows_per_table)) bits instead of
 * ceil(log2(total_rows)), because lookups already arrive grouped by table.
 * replaces table_batched_embeddings_cuda.cu:1471-1497,1638-1655
 * (linear_index_weight_offsets_kernel + the two cub SortPairs calls). */
TBE_API int tbe_backward_plan(const int32_t* table_offsets, const int32_t* indices,
                              const int32_t* offsets, int64_t T, int64_t B, int64_t N,
                              int64_t total_rows, int64_t max_rows_per_table,
                              void* workspace, int64_t workspace_bytes, void* stream);

/* Exact (deterministic, duplicate-summing) SGD:
 *   for every distinct row r touched: weights[r] -= lr * sum_{lookups of r} grad[b][t]
 * (mean pooling: each term divided by its bag length).  grad_output element (b,t,d)
 * is read at grad_output[b*stride_b + t*stride_t + d] (strides in elements), so the
 * transposed view the all-to-all backward produces needs no copy.  plan_ready != 0
 * means `workspace` already holds tbe_backward_plan's result for these indices.
 * replaces table_batched_embeddings_cuda.cu:383-435 (batched_embedding_backward_sgd_cuda),
 * whose per-lookup read-modify-write loses updates when a row repeats. */
TBE_API int tbe_backward_sgd(const void* grad_output, int64_t stride_b, int64_t stride_t,
                     void* weights, const int32_t* table_offsets,
                     const int32_t* indices, const int32_t* offsets,
                     int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows,
                     int dtype, int pooling, float lr,
                     int64_t max_rows_per_table, int plan_ready,
                     void* workspace, int64_t workspace_bytes, void* stream);

/* Exact rowwise Adagrad: per distinct row r with G = summed gradient,
 *   state[r] += sum_d G_d^2;  weights[r] -= lr / (sqrt(state[r]) + eps) * G.
 * stochastic_rounding applies to TBE_F16 only (13 random bits added below the fp16
 * mantissa, then round-toward-zero), seeded by (sr_seed, sr_offset).
 * replaces table_batched_embeddings_cuda.cu:1589-1705
 * (batched_embedding_backward_adagrad_exact_cuda). */
TBE_API int tbe_backward_exact_rowwise_adagrad(
    const void* grad_output, int64_t stride_b, int64_t stride_t,
    void* weights, const int32_t* table_offsets,
    const int32_t* indices, const int32_t* offsets, float* optimizer_state,
    int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows,
    int dtype, int pooling, float lr, float eps,
    int stochastic_rounding, uint64_t sr_seed, uint64_t sr_offset,
    int64_t max_rows_per_table, int plan_ready,
    void* workspace, int64_t workspace_bytes, void* stream);

/* tbe_backward_sgd for callers that cannot provide a workspace because they cannot allocate
 * device memory: a host that binds this ABI through a bare FFI and has no device allocator of
 * its own, or a serving process whose HBM is fully budgeted at start-up and which must not
 * call cudaMalloc (a device-wide synchronisation) while handling a request.  The scratch is
 * a fixed array inside the library's device image (tbe_noalloc_scratch_bytes() bytes, held by
 * every GPU that has used this entry point until the process exits); the call itself allocates
 * nothing, but CUDA loads a library's device image lazily, so the array takes its place in device
 * memory during the FIRST call on a device: make one warm-up call per device at start-up, while
 * memory is still available, not on the first request.
 * Same arguments and results as tbe_backward_sgd without plan_ready / workspace.
 *  - Limit: N <= TBE_NOALLOC_MAX_LOOKUPS; larger batches are rejected with
 *    TBE_ERR_WORKSPACE_TOO_SMALL and a message naming the limit.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the array and it keeps the previous call's contents; the
 *    words that must start at zero are cleared by every call.  Calls whose GPU work overlaps
 *    (different streams or threads on one device) race on the array: serialise them.
 * This entry point has no counterpart in the reference, which allocates its sort scratch with
 * at::empty on every call (table_batched_embeddings_cuda.cu:1618-1627,1646). */
#define TBE_NOALLOC_MAX_LOOKUPS 524288
TBE_API int64_t tbe_noalloc_scratch_bytes(void);
TBE_API int tbe_backward_sgd_noalloc(const void* grad_output, int64_t stride_b, int64_t stride_t,
                     void* weights, const int32_t* table_offsets,
                     const int32_t* indices, const int32_t* offsets,
                     int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows,
                     int dtype, int pooling, float lr, int64_t max_rows_per_table,
                     void* stream);

/* Approximate rowwise Adagrad: every lookup is applied on its own, in index order,
 * with its bag's g2 = |grad[b][t]|^2 (times w_l^2 when weighted):
 *   state[r] += g2;  weights[r] -= w_l * lr / (sqrt(state[r]) + eps) * grad[b][t].
 * grad_per_sample_weights (nullable unless per_sample_weights is given) receives
 * <weights_before_update[r], grad[b][t]> per lookup.  Lookups of one row are applied
 * in ascending index position, so the result is deterministic.
 * replaces table_batched_embeddings_cuda.cu:706-793
 * (batched_embedding_backward_adagrad_approx_cuda), whose updates race when a row repeats. */
TBE_API int tbe_backward_approx_rowwise_adagrad(
    const void* grad_output, int64_t stride_b, int64_t stride_t,
    void* weights, const int32_t* table_offsets,
    const int32_t* indices, const int32_t* offsets,
    const void* per_sample_weights, void* grad_per_sample_weights,
    float* optimizer_state,
    int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows,
    int dtype, float lr, float eps,
    int stochastic_rounding, uint64_t sr_seed, uint64_t sr_offset,
    int64_t max_rows_per_table,
    void* workspace, int64_t workspace_bytes, void* stream);

/* The integer bookkeeping of the backward on its own (what the optimizer kernels
 * consume): row ids sorted ascending, the bag id of each sorted entry, the start of
 * each run of equal row ids and the number of runs.  Outputs are device arrays of
 * N, N, N+1 and 1 int32 (the first *num_segments entries of segment_starts are set).
 * max_rows_per_table: as for tbe_backward_sgd (0 = unknown); with it the plan is
 * built by the same table-segmented sort the optimizer entry points use, which
 * requires table_offsets to ascend (table t's rows precede table t+1's).
 * replaces table_batched_embeddings_cuda.cu:1471-1497,1638-1655
 * (linear_index_weight_offsets_kernel + cub SortPairs) and the segment scan
 * at :1523-1539. */
TBE_API int tbe_sort_segments(const int32_t* table_offsets, const int32_t* indices,
                      const int32_t* offsets,
                      int64_t T, int64_t B, int64_t N, int64_t total_rows,
                      int64_t max_rows_per_table,
                      int32_t* sorted_rows, int32_t* sorted_bags,
                      int32_t* segment_starts, int32_t* num_segments,
                      void* workspace, int64_t workspace_bytes, void* stream);

/* ---- input helpers ------------------------------------------------------ */

/* lengths_out[0] = 0; lengths_out[1 + t*B + b] = length of bag (t,b) given per-table
 * begin offsets [T][B] and per-table totals [T]; the caller cumsums it.
 * replaces table_batched_embeddings_cuda.cu:1190-1213 (construct_offsets). */
TBE_API int tbe_construct_offsets(const int32_t* batch_offsets_per_table,
                          const int32_t* total_indices_per_table,
                          int32_t* lengths_out, int64_t T, int64_t B, void* stream);

/* Ragged gather of bags: destination bag g = [dst_offsets[g], dst_offsets[g+1]) receives the indices of
 * source bag src_bag[g] = [src_offsets[src_bag[g]], ...) (same length; the caller builds dst_offsets as
 * the cumulative sum of the permuted lengths).  It is the last step of the index all-to-all that turns
 * data-parallel sparse features ([T][B/W][L] per rank) into the table-sharded layout ([T/W][B][L]) the
 * lookup consumes.  The reference fabricates table-sharded indices on every rank instead of exchanging
 * them (pytorch_distributed_benchmark.py:227-231), so this has no counterpart to replace there. */
TBE_API int tbe_permute_bags(const int32_t* src_indices, const int32_t* src_offsets, const int32_t* src_bag,
                             const int32_t* dst_offsets, int32_t* dst_indices, int64_t nbags, void* stream);

/* Validates indices/offsets on the device and SYNCHRONISES the stream: offsets[0]==0,
 * non-decreasing, offsets[T*B]==N, 0 <= index < rows of its table (rows_per_table
 * int32 [T]).  Returns TBE_ERR_BAD_INPUT_DATA with the first violation in the error
 * string.  The reference has no such check (sparse_embedding_cuda_kernel.cu:212-214). */
TBE_API int tbe_check_inputs(const int32_t* indices, const int32_t* offsets,
                     const int32_t* rows_per_table,
                     int64_t T, int64_t B, int64_t N, void* stream);

/* ---- host-resident tables ------------------------------------------------ */

/* Managed allocation preferred on the host and mapped for the current device
 * (replaces CUDAManagedAllocator, table_batched_embeddings_cuda.cu:797-812), and a
 * pinned, device-mapped host allocation (not write-combined: the optimizer reads the rows back) returning both addresses
 * (replaces CUDAHostMappedAllocator, :820-838).  These DO allocate; free with the
 * matching call. */
TBE_API int tbe_alloc_managed(void** ptr, int64_t bytes);
TBE_API int tbe_free_managed(void* ptr);
TBE_API int tbe_alloc_host_mapped(void** host_ptr, void** device_ptr, int64_t bytes);
TBE_API int tbe_free_host_mapped(void* host_ptr);

/* ---- LXU cache: set-associative HBM cache in front of a host-resident table ---- */

/* The reference has no cache: its only mechanism for tables larger than HBM is
 * host-mapped memory with every lookup crossing the host link
 * (table_batched_embeddings_ops.py:159-167, table_batched_embeddings_cuda.cu:797-812).
 * These entry points have no counterpart there.
 *
 * State owned by the caller, all in device memory unless noted:
 *   cache_rows [num_sets*ways][D]  cached rows (table dtype)
 *   tags       int32 [num_sets*ways]  row id held by each way, -1 = empty (initialise to -1)
 *   last_use   int32 [num_sets*ways]  step of the last lookup (initialise to 0)
 *   use_count  int32 [num_sets*ways]  steps that looked the row up since it was inserted (0)
 *   dirty      uint8 [num_sets*ways]  row differs from the host copy (0)
 *   host_rows  [total_rows][D]  the table, in device-mapped pinned host memory
 * Placement: row r lives in set mix(r) % num_sets, where mix is a fixed bijection of the
 * 31-bit row ids (two rounds of x ^= x >> 16; x = x * 0x45d9f3b mod 2^31; then x ^= x >> 16),
 * so that rows a table size apart do not collide; "ascending order" below means ascending
 * mix(r).  Per step (now = 1, 2, ...): every distinct
 * row of the batch is looked up first (a hit refreshes last_use and use_count); then the
 * misses of a set claim, in ascending order, a way that was not used in this step --
 * an empty one first, else the one with the smallest last_use (policy 0, LRU) or the
 * smallest use_count (policy 1, LFU), ties to the lowest way; a dirty victim is written
 * back to host_rows and the new row is fetched.  A row whose set has no free way stays
 * uncached for this step and is served from host_rows.
 *
 * tbe_cache_prefetch does all of that for one batch and writes locations[p] (int32 [N]):
 * the cache slot (set*ways + way) holding the row of lookup p, or -1 = read host_rows.
 * stats (int32 [5], device): {distinct rows, rows fetched, lookups whose row was already
 * cached, distinct rows already cached, distinct rows left uncached}.  The workspace keeps
 * the sorted lookups for tbe_cache_backward_sgd of the same batch. */
TBE_API int64_t tbe_cache_workspace_bytes(int64_t N, int64_t total_rows);
TBE_API int tbe_cache_prefetch(void* cache_rows, int32_t* tags, int32_t* last_use, int32_t* use_count,
                               uint8_t* dirty, void* host_rows, const int32_t* table_offsets,
                               const int32_t* indices, const int32_t* offsets, int32_t* locations,
                               int32_t* stats, int64_t T, int64_t B, int64_t D, int64_t N,
                               int64_t total_rows, int64_t num_sets, int ways, int dtype, int policy,
                               int now, void* writeback_rows, int32_t* writeback_ids,
                               void* workspace, int64_t workspace_bytes, void* stream);
/* Deferred write-backs.  With writeback_rows / writeback_ids (both or neither; device buffers of
 * min(N, num_sets*ways) rows of the table dtype and as many int32) tbe_cache_prefetch does not write
 * dirty victims to host_rows: it stages them there, and tbe_cache_writeback -- on any stream ordered
 * after the prefetch, e.g. a side stream running under the lookup -- carries them to host_rows.  Only
 * the fetches then sit on the critical path of the host link.  The caller orders the next
 * tbe_cache_prefetch, tbe_cache_flush and any host read of the table after the write-back (an
 * evicted row is never looked up in the step that evicted it, so the lookup itself needs no order).
 * `stats` is the array the prefetch wrote (its second word is the number of staged slots). */
TBE_API int tbe_cache_writeback(const void* writeback_rows, const int32_t* writeback_ids, const int32_t* stats,
                                void* host_rows, int64_t D, int dtype, void* stream);
/* The same step with the rows travelling through the copy engines instead of SM-issued loads and
 * stores (a kernel reading random rows of an 80 GB mapped table gets ~13 GB/s out of the host link,
 * copies of contiguous pinned buffers 55 GB/s).  Per round of up to stage_rows claims: the dirty
 * victims are packed into stage_device and copied out, worker threads of the library gather the new
 * rows from the table (host_rows_on_host: the table's address on the HOST) into stage_host, one copy
 * brings them in and a kernel inserts them, and the workers scatter the victims into the table.
 *   stage_device  device buffer of tbe_cache_stage_bytes(stage_rows, D, dtype, 0) bytes
 *   stage_host    pinned host buffer of tbe_cache_stage_bytes(stage_rows, D, dtype, 1) bytes
 * Unlike every other entry point this one WAITS for the stream (it has to learn the number of
 * claims) and returns with the host table up to date for the evicted rows; host_rows stays the
 * device-mapped address, which the lookup and the update still use for rows left uncached.  Results
 * are those of tbe_cache_prefetch bit for bit. */
TBE_API int64_t tbe_cache_stage_bytes(int64_t stage_rows, int64_t D, int dtype, int on_host);
TBE_API int tbe_cache_prefetch_staged(void* cache_rows, int32_t* tags, int32_t* last_use, int32_t* use_count,
                                      uint8_t* dirty, void* host_rows, const int32_t* table_offsets,
                                      const int32_t* indices, const int32_t* offsets, int32_t* locations,
                                      int32_t* stats, int64_t T, int64_t B, int64_t D, int64_t N,
                                      int64_t total_rows, int64_t num_sets, int ways, int dtype, int policy,
                                      int now, void* host_rows_on_host, void* stage_device, void* stage_host,
                                      int64_t stage_rows, void* workspace, int64_t workspace_bytes, void* stream);
/* Pooled forward reading every row through `locations` (sum / mean, fp16 / fp32). */
TBE_API int tbe_cache_forward(const void* cache_rows, const void* host_rows,
                              const int32_t* table_offsets, const int32_t* indices,
                              const int32_t* offsets, const int32_t* locations, void* output,
                              int64_t T, int64_t B, int64_t D, int dtype, int pooling, void* stream);
/* Exact SGD on the rows of the batch tbe_cache_prefetch last prepared in `workspace`:
 * cached rows are updated in HBM and marked dirty, uncached rows are updated in host_rows. */
TBE_API int tbe_cache_backward_sgd(const void* grad_output, int64_t stride_b, int64_t stride_t,
                                   void* cache_rows, void* host_rows, uint8_t* dirty,
                                   const int32_t* offsets, int64_t T, int64_t B, int64_t D, int64_t N,
                                   int64_t total_rows, int64_t num_sets, int dtype, int pooling, float lr,
                                   void* workspace, int64_t workspace_bytes, void* stream);
/* Writes every dirty cached row back to host_rows. */
TBE_API int tbe_cache_flush(void* cache_rows, void* host_rows, const int32_t* tags, uint8_t* dirty,
                            int64_t num_slots, int64_t D, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TBE_B200_H_ */
