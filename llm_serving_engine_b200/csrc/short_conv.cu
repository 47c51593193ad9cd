// A short causal convolution over time on each channel of a projection, and what an attention layer does right after
// it.  For channel c with `taps` weights w[c, 0 .. taps-1] (the last one is the current token's):
//     y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]  (+ bias[c]),       u = 0 before the request's first token.
// The inputs u are columns of the layer's stacked projection (float32, bfloat16 or a float32 stack of partial sums).
// A request's last taps - 1 inputs are kept, in float32, in its state slot ([slots, taps - 1, channels], oldest
// first), so that a step can start anywhere; lse_short_conv_state moves the window on after the step's consumers
// have read the old one (stream order).
//
//   lse_short_conv_act:    y (+ bias), through SiLU or not, into a [T, channels] tensor.
//   lse_conv_qk_norm_rope: for an attention layer whose q, k and v each pass such a convolution: then one RMS norm
//       over all of q and one over all of k (not per head), a rotation of the first rot_dims values of every head
//       of q and k (value i paired with i + rot_dims / 2; angle = position * freq[i], formed in double precision;
//       cosine and sine times rot_factor), q into its tensor, k and v into the row's place in the pages, and the
//       sigmoid of one more column per head (an output gate) into a float32 tensor.
//   lse_head_gate_scale:   out[t, h, :] = attended[t, h, :] * gate[t, h] * scale into columns of a wider row.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_short_conv)

namespace {
template <typename TD>
__device__ __forceinline__ float sc_load(const TD* p, int n_partials, long long partial_stride) {
  return sum_partials<TD>(p, n_partials, partial_stride);
}

// The convolution's sum for row `r` (local index l = r - row0 in its request's rows of this step) and channel c.
// TAPS: the number of taps when the kernel was built for it (2, 3 or 4: the loops unroll), 0: any number, `taps`.
// The sum runs over the taps in ascending order from zero in every form, so all forms give the same bits.
template <typename TD, int TAPS>
__device__ __forceinline__ float sc_conv(const TD* __restrict__ proj, int n_partials, long long partial_stride,
                                         long long ld, int off, const float* __restrict__ weight,
                                         const float* __restrict__ window, int channels, int taps_rt, int r, int l, int c) {
  const int taps = TAPS ? TAPS : taps_rt;
  float y = 0.f;
  for (int j0 = 0; j0 < taps; j0 += 4) {     // four taps' inputs and weights are fetched before any is used
    float u[4], w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int j = j0 + i, back = taps - 1 - j;         // back: how many tokens before row r
      u[i] = w[i] = 0.f;
      if (j < taps) {
        w[i] = weight[(size_t)c * taps + j];
        if (l - back >= 0) u[i] = sc_load(proj + (size_t)(r - back) * ld + off + c, n_partials, partial_stride);
        else u[i] = window[(size_t)(taps - 1 + l - back) * channels + c];
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (j0 + i < taps) y = fmaf(w[i], u[i], y);
  }
  return y;
}

// grid (tiles of rows_per_block rows, tiles of 256 channels).  With TAPS known a thread walks its rows with the last
// TAPS - 1 inputs in registers (one new input a row; they are fetched afresh where a request begins inside the tile).
template <typename TD, typename TO, int TAPS>
__global__ void __launch_bounds__(256)
short_conv_act_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int off,
                      const float* __restrict__ weight, const float* __restrict__ bias, const float* __restrict__ state,
                      const int* __restrict__ segment_of_token, const int* __restrict__ segment_start,
                      const int* __restrict__ segment_slot, TO* __restrict__ out, int tokens, int rows_per_block,
                      int channels, int taps, int act, int num_slots, int num_segments) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const float b = bias ? bias[c] : 0.f;
  const int first = blockIdx.x * rows_per_block, end = min(tokens, first + rows_per_block);
  if constexpr (TAPS >= 2) {
    float w[TAPS], before[TAPS - 1];      // before[i]: the input TAPS - 1 - i rows back
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[j] = weight[(size_t)c * TAPS + j];
    int held = -1;                        // the request whose inputs `before` holds
    for (int r = first; r < end; ++r) {
      const int seg = segment_of_token[r];
      if (seg < 0) { held = -1; continue; }
      if (seg != held) {
        const int s = LSE_CHECKED(seg, 0, num_segments, 0, LSE_CHECK_SEGMENT);
        const float* window = state + (size_t)LSE_CHECKED(segment_slot[s], 0, num_slots, 0, LSE_CHECK_ROW) * (TAPS - 1) * channels;
        const int l = r - segment_start[s];
#pragma unroll
        for (int i = 0; i < TAPS - 1; ++i) {
          const int back = TAPS - 1 - i;
          before[i] = l - back >= 0 ? sc_load(proj + (size_t)(r - back) * ld + off + c, n_partials, partial_stride)
                                    : window[(size_t)(TAPS - 1 + l - back) * channels + c];
        }
        held = seg;
      }
      const float now = sc_load(proj + (size_t)r * ld + off + c, n_partials, partial_stride);
      float y = 0.f;
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) y = fmaf(w[j], before[j], y);
      y = fmaf(w[TAPS - 1], now, y) + b;
#pragma unroll
      for (int i = 0; i + 1 < TAPS - 1; ++i) before[i] = before[i + 1];
      before[TAPS - 2] = now;
      if (act == 1) y = y / (1.f + expf(-y));
      out[(size_t)r * channels + c] = from_f32<TO>(y);
    }
  } else {
    for (int r = first; r < end; ++r) {
      const int seg = segment_of_token[r];
      if (seg < 0) continue;
      const int s = LSE_CHECKED(seg, 0, num_segments, 0, LSE_CHECK_SEGMENT);
      const float* window = state + (size_t)LSE_CHECKED(segment_slot[s], 0, num_slots, 0, LSE_CHECK_ROW) * (taps - 1) * channels;
      float y = sc_conv<TD, 0>(proj, n_partials, partial_stride, ld, off, weight, window, channels, taps, r, r - segment_start[s], c) + b;
      if (act == 1) y = y / (1.f + expf(-y));
      out[(size_t)r * channels + c] = from_f32<TO>(y);
    }
  }
}

// The window after the step: entry i holds the input at position (first + count) - (taps - 1) + i.  In ascending i an
// entry only reads entries behind it, so the window moves in place.
template <typename TD>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int off,
                        float* __restrict__ state, const int* __restrict__ segment_start,
                        const int* __restrict__ segment_slot, int channels, int taps, int num_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.x;
  const int row0 = segment_start[seg], count = segment_start[seg + 1] - row0;
  if (count <= 0) return;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float* window = state + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * (taps - 1) * channels;
  for (int i = 0; i < taps - 1; ++i) {
    const int l = count - (taps - 1) + i;
    window[(size_t)i * channels + c] = l >= 0 ? sc_load(proj + (size_t)(row0 + l) * ld + off + c, n_partials, partial_stride)
                                              : window[(size_t)(i + count) * channels + c];
  }
}

// One block per row (256 to 1024 threads).  Channels: q (n_q * dk), then k (n_kv * dk), then v (n_kv * dv), consecutive columns from `off`,
// with their convolution weights stacked the same way; the gate's n_q columns start at g_off.
template <typename TD, typename TO, int TAPS>
__global__ void __launch_bounds__(1024)
conv_qk_norm_rope_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int off,
                         int g_off, const float* __restrict__ weight, const float* __restrict__ state,
                         const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                         const double* __restrict__ freq, float rot_factor, int rot_dims,
                         const int* __restrict__ positions, const int* __restrict__ segment_of_token,
                         const int* __restrict__ segment_start, const int* __restrict__ segment_slot,
                         const int* __restrict__ slot_mapping, TO* __restrict__ q_out, TO* __restrict__ k_cache,
                         TO* __restrict__ v_cache, float* __restrict__ gate_out, int n_q, int n_kv, int dk, int dv,
                         int taps, int page_size, int num_pages, int num_slots, int num_segments) {
  extern __shared__ float sc_smem[];      // [channels] convolved values, [rot_dims / 2] cosines, [rot_dims / 2] sines
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int seg = segment_of_token[r];
  if (seg < 0) return;
  const int s = LSE_CHECKED(seg, 0, num_segments, 0, LSE_CHECK_SEGMENT);
  const int q_width = n_q * dk, k_width = n_kv * dk, v_width = n_kv * dv, channels = q_width + k_width + v_width;
  const int half = rot_dims / 2;
  float* conv = sc_smem;
  float* cosines = sc_smem + channels;
  float* sines = cosines + half;
  const float* window = state + (size_t)LSE_CHECKED(segment_slot[s], 0, num_slots, 0, LSE_CHECK_ROW) * (taps - 1) * channels;
  const int l = r - segment_start[s];
  float sq_q = 0.f, sq_k = 0.f;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    const float y = sc_conv<TD, TAPS>(proj, n_partials, partial_stride, ld, off, weight, window, channels, taps, r, l, c);
    conv[c] = y;
    if (c < q_width) sq_q = fmaf(y, y, sq_q);
    else if (c < q_width + k_width) sq_k = fmaf(y, y, sq_k);
  }
  const int position = positions[r];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sine, cosine;
    sincos((double)position * freq[i], &sine, &cosine);
    cosines[i] = (float)cosine * rot_factor;
    sines[i] = (float)sine * rot_factor;
  }
  if (gate_out)
    for (int h = threadIdx.x; h < n_q; h += blockDim.x)
      gate_out[(size_t)r * n_q + h] = 1.f / (1.f + expf(-sc_load(proj + (size_t)r * ld + g_off + h, n_partials, partial_stride)));
  const float inv_q = 1.0f / sqrtf(block_sum(sq_q, scratch) / (float)q_width + eps);
  const float inv_k = 1.0f / sqrtf(block_sum(sq_k, scratch) / (float)k_width + eps);
  const int slot = LSE_CHECKED(slot_mapping[r], 0, num_pages * page_size, -1, LSE_CHECK_CACHE_SLOT);
  const int page = slot >= 0 ? slot / page_size : 0, place = slot >= 0 ? slot % page_size : 0;
  // q and k: normed over the whole projection, then rotated head by head.  A head's size is a power of two in most
  // models: a shift and a mask then take the place of the division.
  const int dk_shift = (dk & (dk - 1)) == 0 ? __ffs(dk) - 1 : -1, dv_shift = (dv & (dv - 1)) == 0 ? __ffs(dv) - 1 : -1;
  for (int c = threadIdx.x; c < q_width + k_width; c += blockDim.x) {
    const bool is_q = c < q_width;
    const int local = is_q ? c : c - q_width;
    const int head = dk_shift >= 0 ? local >> dk_shift : local / dk, i = dk_shift >= 0 ? local & (dk - 1) : local % dk;
    const float* norm = is_q ? q_norm : k_norm;
    const float inv = is_q ? inv_q : inv_k;
    float y = conv[c] * inv * norm[local];
    if (i < rot_dims) {
      const int pair = i < half ? i : i - half;
      const int other = i < half ? c + half : c - half;
      const float partner = conv[other] * inv * norm[is_q ? other : other - q_width];
      y = i < half ? y * cosines[pair] - partner * sines[pair] : y * cosines[pair] + partner * sines[pair];
    }
    if (is_q) q_out[(size_t)r * q_width + local] = from_f32<TO>(y);
    else if (slot >= 0) k_cache[(((size_t)page * n_kv + head) * page_size + place) * dk + i] = from_f32<TO>(y);
  }
  if (slot >= 0)
    for (int c = threadIdx.x; c < v_width; c += blockDim.x) {
      const int head = dv_shift >= 0 ? c >> dv_shift : c / dv, i = dv_shift >= 0 ? c & (dv - 1) : c % dv;
      v_cache[(((size_t)page * n_kv + head) * page_size + place) * dv + i] = from_f32<TO>(conv[q_width + k_width + c]);
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
head_gate_scale_kernel(const TI* __restrict__ attended, const float* __restrict__ gate, TO* __restrict__ out,
                       long long out_ld, int heads, int dv, float scale, const int* __restrict__ segment_of_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (segment_of_token && segment_of_token[t] < 0) return;
  for (int c = threadIdx.x; c < heads * dv; c += blockDim.x) {
    const float g = gate ? gate[(size_t)t * heads + c / dv] : 1.f;
    out[(size_t)t * out_ld + c] = from_f32<TO>(to_f32<TI>(attended[(size_t)t * heads * dv + c]) * g * scale);
  }
}
}  // namespace

#define LSE_SC_TYPES(CASE)                                                   \
  {                                                                          \
    const bool d32 = proj_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32; \
    if (d32 && o32) CASE(float, float);                                      \
    else if (d32 && !o32) CASE(float, __nv_bfloat16);                        \
    else if (!d32 && o32) CASE(__nv_bfloat16, float);                        \
    else CASE(__nv_bfloat16, __nv_bfloat16);                                 \
  }

// weight float32 [channels, taps]; bias float32 [channels] or null; state float32 [slots, taps - 1, channels];
// out [tokens, channels]; act: 0 none, 1 SiLU.
extern "C" int lse_short_conv_act(const void* proj, int proj_dtype, int n_partials, long long partial_stride, long long ld,
                                  int off, const float* weight, const float* bias, const float* state,
                                  const int* segment_of_token, const int* segment_start, const int* segment_slot,
                                  void* out, int out_dtype, int tokens, int channels, int taps, int act, int num_slots,
                                  int num_segments, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || taps < 1 || n_partials < 1 || (channels + 255) / 256 > 65535) return LSE_ERR_BAD_ARGUMENT;
  const int rows_per_block = tokens >= 1024 ? 16 : 1;
  const dim3 grid((tokens + rows_per_block - 1) / rows_per_block, (channels + 255) / 256);
#define LSE_SC_TAPS(TD, TO, TAPS)                                                                                   \
  lse_launch(short_conv_act_kernel<TD, TO, TAPS>, grid, 256, 0, stream, (const TD*)proj, n_partials, partial_stride, \
             ld, off, weight, bias, state, segment_of_token, segment_start, segment_slot, (TO*)out, tokens,          \
             rows_per_block, channels, taps, act, num_slots, num_segments)
#define LSE_SC_CASE(TD, TO)                          \
  do {                                               \
    if (taps == 4) LSE_SC_TAPS(TD, TO, 4);           \
    else if (taps == 3) LSE_SC_TAPS(TD, TO, 3);      \
    else if (taps == 2) LSE_SC_TAPS(TD, TO, 2);      \
    else LSE_SC_TAPS(TD, TO, 0);                     \
  } while (0)
  LSE_SC_TYPES(LSE_SC_CASE)
#undef LSE_SC_CASE
#undef LSE_SC_TAPS
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_short_conv_state(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                    long long ld, int off, float* state, const int* segment_start,
                                    const int* segment_slot, int max_segments, int channels, int taps, int num_slots,
                                    cudaStream_t stream) {
  if (max_segments <= 0 || taps <= 1) return 0;
  if (channels <= 0 || n_partials < 1 || (channels + 255) / 256 > 65535) return LSE_ERR_BAD_ARGUMENT;
  const dim3 grid(max_segments, (channels + 255) / 256);
  if (proj_dtype == LSE_DTYPE_F32)
    lse_launch(short_conv_state_kernel<float>, grid, 256, 0, stream, (const float*)proj, n_partials, partial_stride, ld,
               off, state, segment_start, segment_slot, channels, taps, num_slots);
  else if (proj_dtype == LSE_DTYPE_BF16)
    lse_launch(short_conv_state_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)proj, n_partials,
               partial_stride, ld, off, state, segment_start, segment_slot, channels, taps, num_slots);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// weight float32 [n_q dk + n_kv dk + n_kv dv, taps]; q_norm float32 [n_q dk], k_norm float32 [n_kv dk]; freq float64
// [rot_dims / 2]; q_out [tokens, n_q, dk]; k_cache [pages, n_kv, page, dk], v_cache [.., dv]; gate_out float32
// [tokens, n_q] or null.
extern "C" int lse_conv_qk_norm_rope(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                     long long ld, int off, int g_off, const float* weight, const float* state,
                                     const float* q_norm, const float* k_norm, float eps, const double* freq,
                                     float rot_factor, int rot_dims, const int* positions,
                                     const int* segment_of_token, const int* segment_start, const int* segment_slot,
                                     const int* slot_mapping, void* q_out, void* k_cache, void* v_cache, int out_dtype,
                                     float* gate_out, int tokens, int n_q, int n_kv, int dk, int dv, int taps,
                                     int page_size, int num_pages, int num_slots, int num_segments,
                                     cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n_q <= 0 || n_kv <= 0 || dk <= 0 || dv <= 0 || taps < 1 || n_partials < 1 || rot_dims < 0 || rot_dims % 2 ||
      rot_dims > dk)
    return LSE_ERR_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * ((size_t)(n_q + n_kv) * dk + (size_t)n_kv * dv + rot_dims);
  if (smem > 200 * 1024) return LSE_ERR_TOO_LARGE;
  // a thread's channels come one after the other, each a few dependent round trips: few rows get as many threads a row
  // as a block has, many rows share the SMs
  const int width = (n_q + n_kv) * dk + n_kv * dv;
  const int threads = tokens <= 64 ? min(1024, (width + 31) / 32 * 32) : min(512, (width + 31) / 32 * 32);
#define LSE_SC_TAPS(TD, TO, TAPS)                                                                                    \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(conv_qk_norm_rope_kernel<TD, TO, TAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                           (int)smem);                                                                               \
    lse_launch(conv_qk_norm_rope_kernel<TD, TO, TAPS>, tokens, threads, smem, stream, (const TD*)proj, n_partials,   \
               partial_stride, ld, off, g_off, weight, state, q_norm, k_norm, eps, freq, rot_factor, rot_dims,       \
               positions, segment_of_token, segment_start, segment_slot, slot_mapping, (TO*)q_out, (TO*)k_cache,     \
               (TO*)v_cache, gate_out, n_q, n_kv, dk, dv, taps, page_size, num_pages, num_slots, num_segments);      \
  } while (0)
#define LSE_SC_CASE(TD, TO)                          \
  do {                                               \
    if (taps == 4) LSE_SC_TAPS(TD, TO, 4);           \
    else if (taps == 3) LSE_SC_TAPS(TD, TO, 3);      \
    else LSE_SC_TAPS(TD, TO, 0);                     \
  } while (0)
  LSE_SC_TYPES(LSE_SC_CASE)
#undef LSE_SC_CASE
#undef LSE_SC_TAPS
  LSE_LAUNCH_CHECK();
}

// attended [tokens, heads, dv] (in_dtype); gate float32 [tokens, heads] or null; out: rows of out_ld values (out_dtype),
// the head's values from column 0 of the given pointer.
extern "C" int lse_head_gate_scale(const void* attended, int proj_dtype, const float* gate, void* out, int out_dtype,
                                   long long out_ld, int tokens, int heads, int dv, float scale,
                                   const int* segment_of_token, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || dv <= 0 || out_ld < (long long)heads * dv) return LSE_ERR_BAD_ARGUMENT;
#define LSE_SC_CASE(TI, TO)                                                                                   \
  lse_launch(head_gate_scale_kernel<TI, TO>, tokens, 256, 0, stream, (const TI*)attended, gate, (TO*)out, out_ld, \
             heads, dv, scale, segment_of_token)
  LSE_SC_TYPES(LSE_SC_CASE)
#undef LSE_SC_CASE
  LSE_LAUNCH_CHECK();
}
