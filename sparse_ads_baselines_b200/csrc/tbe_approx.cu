// Approximate rowwise Adagrad backward (placeholder until the kernel lands).
#include "tbe_common.cuh"

extern "C" int tbe_backward_approx_rowwise_adagrad(
    const void* grad_output, int64_t stride_b, int64_t stride_t, void* weights, const int32_t* table_offsets,
    const int32_t* indices, const int32_t* offsets, const void* per_sample_weights, void* grad_per_sample_weights,
    float* optimizer_state, int64_t T, int64_t B, int64_t D, int64_t N, int64_t total_rows, int dtype, float lr,
    float eps, int stochastic_rounding, uint64_t sr_seed, uint64_t sr_offset, void* workspace,
    int64_t workspace_bytes, void* stream) {
  return tbe::fail(TBE_ERR_UNSUPPORTED, "tbe_backward_approx_rowwise_adagrad: not built yet");
}
