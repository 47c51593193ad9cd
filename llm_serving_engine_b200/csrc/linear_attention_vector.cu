// The matrix-memory scan with a keep factor per token, head and key channel (linear_attention_scan.cuh has the kernel).
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_linear_attention_vector)

#include "linear_attention_scan.cuh"

// The decay is a vector per token and head: token_keep float32 [tokens, heads * dim]; chunk_keep (chunked only) holds
// max_chunks * heads * dim floats.
extern "C" int lse_vector_decay_attention_scan(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                               long long ld, int q_off, int k_off, int v_off, const float* token_keep,
                                               float q_scale, float* state, const int* segment_start,
                                               const int* segment_slot, float* out, int max_segments, int heads, int dim,
                                               int vdim, int num_slots, int chunk_rows, float* chunk_state,
                                               int max_chunks, float* chunk_keep, cudaStream_t stream) {
  if (!token_keep) return LSE_ERR_BAD_ARGUMENT;
  return linear_attention_scan_launch<MODE_VECTOR>(proj, proj_dtype, n_partials, partial_stride, ld, q_off, k_off, v_off,
                                                   nullptr, state, segment_start, segment_slot, out, max_segments, heads,
                                                   dim, vdim, 0, num_slots, chunk_rows, chunk_state, max_chunks,
                                                   token_keep, nullptr, q_scale, 0, 1, chunk_keep, stream);
}

