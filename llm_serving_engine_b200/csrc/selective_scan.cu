// A selective state-space scan (the recurrence of Mamba), carried from token to token in a float32 state per request.
// Per channel c and state n, with a step size dt_t[c] > 0, A[c, n] < 0 and the token's vectors B_t, C_t [states]:
//     S_t[c, n] = exp(dt_t[c] A[c, n]) S_(t-1)[c, n] + dt_t[c] x_t[c] B_t[n]
//     y_t[c]    = sum_n S_t[c, n] C_t[n] + D[c] x_t[c],            out_t[c] = y_t[c] * silu(z_t[c]) * scale
//
//   lse_ssm_step_sizes:   dt = softplus(low W^T + b), low = the first `rank` columns of a projection's rows; W is handed
//                         over transposed ([rank, channels], float32) so that neighbouring threads read neighbours.
//   lse_selective_scan:   the recurrence over the rows of every request of the step, in order, from and into the
//                         request's slot of `state` ([slots, channels, states]).
// A thread keeps four states of one channel in registers; the lanes that share a channel add their parts of y by
// shuffles.  Tokens are staged in shared memory sixteen at a time.  Everything is float32.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_selective_scan)

namespace {
constexpr int SS_THREADS = 128;
constexpr int SS_PER_LANE = 4;     // states a thread keeps
constexpr int SS_TOKENS = 16;      // tokens staged at a time

template <typename TD>
__device__ __forceinline__ float ss_load(const TD* p, int n_partials, long long partial_stride) {
  float v = 0.f;
  for (int i = 0; i < n_partials; ++i) v += to_f32<TD>(p[(size_t)i * partial_stride]);
  return v;
}

// grid (token tiles of 16, channel tiles of 128)
template <typename TD>
__global__ void __launch_bounds__(128)
ssm_step_sizes_kernel(const TD* __restrict__ low, int n_partials, long long partial_stride, long long ld,
                      const float* __restrict__ weight_t, const float* __restrict__ bias, float* __restrict__ dt,
                      int tokens, int channels, int rank) {
  extern __shared__ float low_s[];     // [16][rank]
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * 16, n = min(16, tokens - t0);
  for (int e = threadIdx.x; e < n * rank; e += blockDim.x)
    low_s[e] = ss_load(low + (size_t)(t0 + e / rank) * ld + e % rank, n_partials, partial_stride);
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float sum[16];
#pragma unroll
  for (int t = 0; t < 16; ++t) sum[t] = 0.f;
  for (int r = 0; r < rank; ++r) {
    const float w = weight_t[(size_t)r * channels + c];
#pragma unroll
    for (int t = 0; t < 16; ++t) sum[t] = fmaf(w, t < n ? low_s[t * rank + r] : 0.f, sum[t]);
  }
  const float b = bias[c];
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    if (t < n) {
      const float z = sum[t] + b;
      dt[(size_t)(t0 + t) * channels + c] = z > 20.f ? z : log1pf(expf(z));
    }
  }
}

// LANES threads share a channel (LANES * 4 >= states); a block owns 128 / LANES channels of one request.
// x: the convolved, activated inputs [T, channels] (TX); z: columns z_off .. of the stacked projection `proj`;
// B and C: columns b_off .. and c_off .. of `low`.
template <typename TD, typename TL, typename TX, typename TO, int LANES>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt, const TD* __restrict__ proj,
                      int proj_partials, long long proj_stride, long long proj_ld, int z_off,
                      const TL* __restrict__ low, int low_partials, long long low_stride, long long low_ld, int b_off,
                      int c_off, const float* __restrict__ a_log, const float* __restrict__ skip,
                      float* __restrict__ state, const int* __restrict__ segment_start,
                      const int* __restrict__ segment_slot, TO* __restrict__ out, long long out_ld, float scale,
                      int channels, int states, int num_slots) {
  constexpr int CH = SS_THREADS / LANES;     // channels of a block
  extern __shared__ float ss_smem[];         // [16][states] B, [16][states] C, [16][CH] dt, x, z
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.x;
  const int row0 = segment_start[seg], row1 = segment_start[seg + 1];
  if (row1 <= row0) return;
  float* b_s = ss_smem;
  float* c_s = b_s + SS_TOKENS * states;
  float* dt_s = c_s + SS_TOKENS * states;
  float* x_s = dt_s + SS_TOKENS * CH;
  float* z_s = x_s + SS_TOKENS * CH;
  const int sub = threadIdx.x % LANES, local = threadIdx.x / LANES;
  const int c = blockIdx.y * CH + local;
  const bool live = c < channels;
  float* st = state + ((size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * channels + (live ? c : 0)) * states;
  float s[SS_PER_LANE], a[SS_PER_LANE];
#pragma unroll
  for (int i = 0; i < SS_PER_LANE; ++i) {
    const int n = i * LANES + sub;          // lanes of a channel read neighbouring states
    const bool has = live && n < states;
    s[i] = has ? st[n] : 0.f;
    a[i] = has ? -expf(a_log[(size_t)c * states + n]) : 0.f;
  }
  const float d_skip = live ? skip[c] : 0.f;
  for (int base = row0; base < row1; base += SS_TOKENS) {
    const int n_tok = min(SS_TOKENS, row1 - base);
    __syncthreads();
    for (int e = threadIdx.x; e < n_tok * states; e += SS_THREADS) {
      const int t = e / states, n = e % states;
      const TL* row = low + (size_t)(base + t) * low_ld;
      b_s[t * states + n] = ss_load(row + b_off + n, low_partials, low_stride);
      c_s[t * states + n] = ss_load(row + c_off + n, low_partials, low_stride);
    }
    for (int e = threadIdx.x; e < n_tok * CH; e += SS_THREADS) {
      const int t = e / CH, cc = blockIdx.y * CH + e % CH;
      const bool ok = cc < channels;
      dt_s[e] = ok ? dt[(size_t)(base + t) * channels + cc] : 0.f;
      x_s[e] = ok ? to_f32<TX>(x[(size_t)(base + t) * channels + cc]) : 0.f;
      z_s[e] = ok ? ss_load(proj + (size_t)(base + t) * proj_ld + z_off + cc, proj_partials, proj_stride) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < n_tok; ++t) {
      const float step = dt_s[t * CH + local], xv = x_s[t * CH + local];
      const float push = step * xv;
      float y = 0.f;
#pragma unroll
      for (int i = 0; i < SS_PER_LANE; ++i) {
        const int n = i * LANES + sub;
        if (n < states) {
          s[i] = fmaf(expf(step * a[i]), s[i], push * b_s[t * states + n]);
          y = fmaf(s[i], c_s[t * states + n], y);
        }
      }
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (sub == 0 && live) {
        const float zv = z_s[t * CH + local];
        y = fmaf(d_skip, xv, y);
        out[(size_t)(base + t) * out_ld + c] = from_f32<TO>(y * (zv / (1.f + expf(-zv))) * scale);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < SS_PER_LANE; ++i) {
      const int n = i * LANES + sub;
      if (n < states) st[n] = s[i];
    }
  }
}
}  // namespace

// low: rows of ld values (float32, bfloat16 or partial sums) whose first `rank` columns are the step sizes' inputs;
// weight_t float32 [rank, channels]; bias float32 [channels]; dt float32 [tokens, channels].
extern "C" int lse_ssm_step_sizes(const void* low, int low_dtype, int n_partials, long long partial_stride, long long ld,
                                  const float* weight_t, const float* bias, float* dt, int tokens, int channels, int rank,
                                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || rank <= 0 || n_partials < 1 || (channels + 127) / 128 > 65535) return LSE_ERR_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * 16 * (size_t)rank;
  if (smem > 48 * 1024) return LSE_ERR_TOO_LARGE;
  const dim3 grid((tokens + 15) / 16, (channels + 127) / 128);
  if (low_dtype == LSE_DTYPE_F32)
    lse_launch(ssm_step_sizes_kernel<float>, grid, 128, smem, stream, (const float*)low, n_partials, partial_stride, ld,
               weight_t, bias, dt, tokens, channels, rank);
  else if (low_dtype == LSE_DTYPE_BF16)
    lse_launch(ssm_step_sizes_kernel<__nv_bfloat16>, grid, 128, smem, stream, (const __nv_bfloat16*)low, n_partials,
               partial_stride, ld, weight_t, bias, dt, tokens, channels, rank);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// x [tokens, channels] (x_dtype); dt float32 [tokens, channels]; proj and low as above (their dtypes are those of the
// projections: float32 with partial sums, or the compute dtype); a_log float32 [channels, states]; skip float32
// [channels]; state float32 [slots, channels, states]; out: rows of out_ld values (out_dtype).
extern "C" int lse_selective_scan(const void* x, int x_dtype, const float* dt, const void* proj, int proj_dtype,
                                  int proj_partials, long long proj_stride, long long proj_ld, int z_off, const void* low,
                                  int low_dtype, int low_partials, long long low_stride, long long low_ld, int b_off,
                                  int c_off, const float* a_log, const float* skip, float* state,
                                  const int* segment_start, const int* segment_slot, void* out, int out_dtype,
                                  long long out_ld, float scale, int max_segments, int channels, int states,
                                  int num_slots, cudaStream_t stream) {
  if (max_segments <= 0) return 0;
  if (channels <= 0 || states <= 0 || proj_partials < 1 || low_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  if (states > 32 * SS_PER_LANE) return LSE_ERR_TOO_LARGE;
  // the data's types come in two families: everything float32, or bfloat16 activations (x, out) with projections that
  // are bfloat16 or float32
  const bool x32 = x_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  const bool p32 = proj_dtype == LSE_DTYPE_F32, l32 = low_dtype == LSE_DTYPE_F32;
  if (x32 != o32) return LSE_ERR_BAD_ARGUMENT;
  int lanes = 1;
  while (lanes * SS_PER_LANE < states) lanes <<= 1;
#define LSE_SS_LAUNCH(TD, TL, TX, TO, L)                                                                           \
  {                                                                                                                \
    constexpr int ch = SS_THREADS / L;                                                                             \
    const size_t smem = sizeof(float) * SS_TOKENS * (2 * (size_t)states + 3 * ch);                                 \
    const dim3 grid(max_segments, (channels + ch - 1) / ch);                                                       \
    lse_launch(selective_scan_kernel<TD, TL, TX, TO, L>, grid, SS_THREADS, smem, stream, (const TX*)x, dt,         \
               (const TD*)proj, proj_partials, proj_stride, proj_ld, z_off, (const TL*)low, low_partials,          \
               low_stride, low_ld, b_off, c_off, a_log, skip, state, segment_start, segment_slot, (TO*)out, out_ld, \
               scale, channels, states, num_slots);                                                                \
  }
#define LSE_SS_LANES(TD, TL, TX, TO)                      \
  switch (lanes) {                                        \
    case 1: LSE_SS_LAUNCH(TD, TL, TX, TO, 1) break;       \
    case 2: LSE_SS_LAUNCH(TD, TL, TX, TO, 2) break;       \
    case 4: LSE_SS_LAUNCH(TD, TL, TX, TO, 4) break;       \
    case 8: LSE_SS_LAUNCH(TD, TL, TX, TO, 8) break;       \
    case 16: LSE_SS_LAUNCH(TD, TL, TX, TO, 16) break;     \
    default: LSE_SS_LAUNCH(TD, TL, TX, TO, 32) break;     \
  }
  if (x32) {
    if (!p32 || !l32) return LSE_ERR_BAD_ARGUMENT;
    LSE_SS_LANES(float, float, float, float)
  } else if (p32 && l32) LSE_SS_LANES(float, float, __nv_bfloat16, __nv_bfloat16)
  else if (p32 && !l32) LSE_SS_LANES(float, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16)
  else if (!p32 && l32) LSE_SS_LANES(__nv_bfloat16, float, __nv_bfloat16, __nv_bfloat16)
  else LSE_SS_LANES(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16)
#undef LSE_SS_LANES
#undef LSE_SS_LAUNCH
  LSE_LAUNCH_CHECK();
}
