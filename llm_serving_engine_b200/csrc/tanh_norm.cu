// The tanh norm (a norm without statistics): y = tanh(alpha x) * w + b, with a learned scalar alpha, fused with the
// residual sum of a layer that norms a branch before and after it:
//     residual[t] += after(delta[t])            after(y) = tanh(alpha_a y) * w_a + b_a   (or y itself without `after`)
//     out[r]       = before(residual[rows[r]])  before(x) = tanh(alpha_b x) * w_b + b_b
// delta is the pending output of the last branch: [T, H] in float32 or bfloat16 or a float32 stack of partial sums
// (added in index order).  Everything is elementwise and float32; a value is rounded once, when `out` is bfloat16.
// The scalars are read from device memory (they are tensors of the checkpoint).
#include "common.cuh"

namespace {
template <typename TD>
__device__ __forceinline__ float tn_delta(const TD* p, int n_partials, long long partial_stride) {
  float v = 0.f;
  for (int i = 0; i < n_partials; ++i) v += to_f32<TD>(p[(size_t)i * partial_stride]);
  return v;
}

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
tanh_norm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials, long long partial_stride,
                 const float* __restrict__ after_alpha, const float* __restrict__ after_w,
                 const float* __restrict__ after_b, const float* __restrict__ before_alpha,
                 const float* __restrict__ before_w, const float* __restrict__ before_b, TO* __restrict__ out,
                 const int* __restrict__ rows, int hidden, int write_residual) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= hidden) return;
  float x = residual[(size_t)t * hidden + i];
  if (delta) {
    float y = tn_delta<TD>(delta + (size_t)t * hidden + i, n_partials, partial_stride);
    if (after_w) y = fmaf(tanhf(after_alpha[0] * y), after_w[i], after_b[i]);
    x += y;
    if (write_residual) residual[(size_t)t * hidden + i] = x;
  }
  if (out) out[(size_t)r * hidden + i] = from_f32<TO>(fmaf(tanhf(before_alpha[0] * x), before_w[i], before_b[i]));
}
}  // namespace

// residual float32 [tokens, hidden]; delta (or null) [tokens, hidden]; after_* (or null: the output is added as it
// is) and before_* float32 ([1], [hidden], [hidden]); out (or null) [n_rows, hidden]; rows int32 [n_rows] or null
// (every row, n_rows = tokens).
extern "C" int lse_tanh_norm(float* residual, const void* delta, int delta_dtype, int n_partials, long long partial_stride,
                             const float* after_alpha, const float* after_w, const float* after_b,
                             const float* before_alpha, const float* before_w, const float* before_b, void* out,
                             int out_dtype, const int* rows, int n_rows, int hidden, int write_residual,
                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || n_partials < 1 || (out && !before_w)) return LSE_ERR_BAD_ARGUMENT;
  if ((hidden + 255) / 256 > 65535) return LSE_ERR_TOO_LARGE;
  const dim3 grid(n_rows, (hidden + 255) / 256);
#define LSE_TN_CASE(TD, TO)                                                                                       \
  lse_launch(tanh_norm_kernel<TD, TO>, grid, 256, 0, stream, residual, (const TD*)delta, n_partials, partial_stride, \
             after_alpha, after_w, after_b, before_alpha, before_w, before_b, (TO*)out, rows, hidden, write_residual)
  const bool d32 = delta_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_TN_CASE(float, float);
  else if (d32 && !o32) LSE_TN_CASE(float, __nv_bfloat16);
  else if (!d32 && o32) LSE_TN_CASE(__nv_bfloat16, float);
  else LSE_TN_CASE(__nv_bfloat16, __nv_bfloat16);
#undef LSE_TN_CASE
  LSE_LAUNCH_CHECK();
}
