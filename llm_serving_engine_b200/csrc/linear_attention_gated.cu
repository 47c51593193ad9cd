// The matrix-memory scan with a keep and a take factor per token and head (linear_attention_scan.cuh has the kernel):
// the gated matrix memory with its normaliser column, and the state-space scan whose B and C belong to groups of heads.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_linear_attention_gated)

#include "linear_attention_scan.cuh"

// norm_col: the state carries the normaliser's column (vdim + 1 columns); qk_share: heads that share a q and a k.
extern "C" int lse_gated_linear_attention_scan_shared(const void* proj, int proj_dtype, int n_partials,
                                                      long long partial_stride, long long ld, int q_off, int k_off,
                                                      int v_off, const float* token_keep, const float* token_take,
                                                      float q_scale, float* state, const int* segment_start,
                                                      const int* segment_slot, float* out, int max_segments, int heads,
                                                      int dim, int vdim, int num_slots, int chunk_rows,
                                                      float* chunk_state, int max_chunks, int norm_col, int qk_share,
                                                      cudaStream_t stream) {
  if (!token_keep || !token_take) return LSE_ERR_BAD_ARGUMENT;
  if (max_chunks > 12000) return LSE_ERR_TOO_LARGE;      // a chunk's factor lives in shared memory during the carry
  return linear_attention_scan_launch<MODE_GATED>(proj, proj_dtype, n_partials, partial_stride, ld, q_off, k_off, v_off,
                                                  nullptr, state, segment_start, segment_slot, out, max_segments, heads,
                                                  dim, vdim, 0, num_slots, chunk_rows, chunk_state, max_chunks,
                                                  token_keep, token_take, q_scale, norm_col, qk_share, nullptr, stream);
}

extern "C" int lse_gated_linear_attention_scan(const void* proj, int proj_dtype, int n_partials,
                                               long long partial_stride, long long ld, int q_off, int k_off, int v_off,
                                               const float* token_keep, const float* token_take, float q_scale,
                                               float* state, const int* segment_start, const int* segment_slot,
                                               float* out, int max_segments, int heads, int dim, int vdim,
                                               int num_slots, int chunk_rows, float* chunk_state, int max_chunks,
                                               cudaStream_t stream) {
  return lse_gated_linear_attention_scan_shared(proj, proj_dtype, n_partials, partial_stride, ld, q_off, k_off, v_off,
                                                token_keep, token_take, q_scale, state, segment_start, segment_slot, out,
                                                max_segments, heads, dim, vdim, num_slots, chunk_rows, chunk_state,
                                                max_chunks, 1, 1, stream);
}

