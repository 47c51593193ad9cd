// The tanh norm (a norm without statistics): y = tanh(alpha x) * w + b, with a learned scalar alpha, fused with the
// residual sum of a layer that norms a branch before and after it:
//     residual[t] += after(delta[t])            after(y) = tanh(alpha_a y) * w_a + b_a   (or y itself without `after`)
//     out[r]       = before(residual[rows[r]])  before(x) = tanh(alpha_b x) * w_b + b_b
// delta is the pending output of the last branch: [T, H] in float32 or bfloat16 or a float32 stack of partial sums
// (added in index order).  Everything is elementwise and float32; a value is rounded once, when `out` is bfloat16.
// The scalars are read from device memory (they are tensors of the checkpoint).
#include "common.cuh"

namespace {
// VEC consecutive elements (1, or 4 through one 16- or 8-byte access) from and to memory.
template <typename T, int VEC>
__device__ __forceinline__ void tn_load(const T* p, float (&v)[VEC]) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    const float4 w = *reinterpret_cast<const float4*>(p);
    v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
  } else if constexpr (VEC == 4) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
  } else {
    v[0] = to_f32<T>(p[0]);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void tn_store(T* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (VEC == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 w;
    w.x = *reinterpret_cast<const unsigned*>(&lo);
    w.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = w;
  } else {
    p[0] = from_f32<T>(v[0]);
  }
}

// grid (rows, tiles of 256 * VEC elements).  The pending output's partial sums are added in index order, four stacks'
// loads in flight at a time.
template <typename TD, typename TO, int VEC>
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
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (i >= hidden) return;
  float x[VEC];
  tn_load<float, VEC>(residual + (size_t)t * hidden + i, x);
  if (delta) {
    float y[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) y[e] = 0.f;
    const TD* at = delta + (size_t)t * hidden + i;
    int p = 0;
    for (; p + 4 <= n_partials; p += 4) {
      float a[VEC], b[VEC], c[VEC], d[VEC];
      tn_load<TD, VEC>(at + (size_t)p * partial_stride, a);
      tn_load<TD, VEC>(at + (size_t)(p + 1) * partial_stride, b);
      tn_load<TD, VEC>(at + (size_t)(p + 2) * partial_stride, c);
      tn_load<TD, VEC>(at + (size_t)(p + 3) * partial_stride, d);
#pragma unroll
      for (int e = 0; e < VEC; ++e) { y[e] += a[e]; y[e] += b[e]; y[e] += c[e]; y[e] += d[e]; }
    }
    for (; p < n_partials; ++p) {
      float a[VEC];
      tn_load<TD, VEC>(at + (size_t)p * partial_stride, a);
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] += a[e];
    }
    if (after_w) {
      const float alpha = after_alpha[0];
      float w[VEC], b[VEC];
      tn_load<float, VEC>(after_w + i, w);
      tn_load<float, VEC>(after_b + i, b);
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] = fmaf(tanhf(alpha * y[e]), w[e], b[e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] += y[e];
    if (write_residual) tn_store<float, VEC>(residual + (size_t)t * hidden + i, x);
  }
  if (out) {
    const float alpha = before_alpha[0];
    float w[VEC], b[VEC];
    tn_load<float, VEC>(before_w + i, w);
    tn_load<float, VEC>(before_b + i, b);
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] = fmaf(tanhf(alpha * x[e]), w[e], b[e]);
    tn_store<TO, VEC>(out + (size_t)r * hidden + i, x);
  }
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
  // four elements a thread where every row starts on a 16-byte boundary (8 for bfloat16) in every tensor
  const bool wide = hidden % 4 == 0 && partial_stride % 4 == 0 &&
                    (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)out | (uintptr_t)after_w | (uintptr_t)after_b |
                      (uintptr_t)before_w | (uintptr_t)before_b) & 15) == 0;
  const int per_block = 256 * (wide ? 4 : 1);
  if ((hidden + per_block - 1) / per_block > 65535) return LSE_ERR_TOO_LARGE;
  const dim3 grid(n_rows, (hidden + per_block - 1) / per_block);
#define LSE_TN_LAUNCH(TD, TO, VEC)                                                                                     \
  lse_launch(tanh_norm_kernel<TD, TO, VEC>, grid, 256, 0, stream, residual, (const TD*)delta, n_partials,             \
             partial_stride, after_alpha, after_w, after_b, before_alpha, before_w, before_b, (TO*)out, rows, hidden,  \
             write_residual)
#define LSE_TN_CASE(TD, TO)          \
  do {                               \
    if (wide) LSE_TN_LAUNCH(TD, TO, 4); \
    else LSE_TN_LAUNCH(TD, TO, 1);   \
  } while (0)
  const bool d32 = delta_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_TN_CASE(float, float);
  else if (d32 && !o32) LSE_TN_CASE(float, __nv_bfloat16);
  else if (!d32 && o32) LSE_TN_CASE(__nv_bfloat16, float);
  else LSE_TN_CASE(__nv_bfloat16, __nv_bfloat16);
#undef LSE_TN_CASE
#undef LSE_TN_LAUNCH
  LSE_LAUNCH_CHECK();
}
