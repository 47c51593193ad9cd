// Linear attention with a decay per head, carried from token to token in a float32 state per request:
//     S_t = decay_h * S_(t-1) + k_t v_t^T      (S is [dim][vdim] per head)
//     o_t = S_t^T q_t
// with q, k, v = act(projection) (act: SiLU, or none), and the gated norm that follows it:
//     y = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g)      over the concatenated heads.
//
// The scan kernel walks the rows of one request in order, from the state that earlier steps left in the
// request's slot, and leaves the new state there.  A block owns (request, head, a tile of state columns); a
// thread owns 32 rows of one column of S in registers, so a token costs it 32 updates and a 32-term dot
// product, and the threads that share a column (dim > 32) add their parts by shuffles.  Columns of S are
// independent of one another, which is what lets them be spread over blocks.  Tokens are staged in shared
// memory a few at a time.  Everything is float32: the projections arrive in float32, in bfloat16 or as a
// stack of float32 partial sums, and are activated in float32.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_linear_attention)

#include "linear_attention_scan.cuh"

namespace {
// out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(g[t]); g: columns g_off .. g_off + n of proj.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, const TD* __restrict__ proj, int n_partials, long long partial_stride,
                     long long ld, int g_off, const float* __restrict__ weight, TO* __restrict__ out, int n, float eps,
                     const int* __restrict__ segment_of_token) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (segment_of_token && segment_of_token[t] < 0) return;
  const float* row = o + (size_t)t * n;
  float sq = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  const TD* g = proj + (size_t)t * ld + g_off;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gate = 1.f / (1.f + expf(-la_load(g + i, n_partials, partial_stride)));
    out[(size_t)t * n + i] = from_f32<TO>(((row[i] * inv) * weight[i]) * gate);
  }
}
// What a state-space scan with one decay per head takes from its step sizes: dt = softplus(z + bias_h) (no clamp),
// keep = exp(-exp(a_log_h) dt), take = dt; z is column dt_off + h of proj.  A thread per (token, head).
template <typename TD>
__global__ void __launch_bounds__(256)
ssd_gates_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int dt_off,
                 const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ keep,
                 float* __restrict__ take, int tokens, int heads) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= tokens * heads) return;
  const int t = e / heads, h = e % heads;
  const float z = la_load(proj + (size_t)t * ld + dt_off + h, n_partials, partial_stride) + dt_bias[h];
  const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
  keep[e] = expf(-expf(a_log[h]) * dt);
  take[e] = dt;
}

// A decay per channel: keep = sigmoid(z + bias)^(1 / tau) = exp(log sigmoid(z + bias) / tau); z is column off + i of proj.
template <typename TD>
__global__ void __launch_bounds__(256)
sigmoid_power_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int off,
                     const float* __restrict__ bias, float inv_tau, float* __restrict__ keep, int tokens, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= (long long)tokens * n) return;
  const int t = (int)(e / n), i = (int)(e % n);
  float z = la_load(proj + (size_t)t * ld + off + i, n_partials, partial_stride);
  if (bias) z += bias[i];
  const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
  keep[e] = expf(log_sigmoid * inv_tau);
}

// The norm behind a scan, in `groups` equal parts of a row, each by its own root mean square:
//   a_i = o_i + skip[i / head_width] * x_i          (skip null: a = o;  x: columns x_off .. of `xsrc`)
//   gate_first:  b = a * act(g);  out = b / rms(b) * weight[i % weight_len] * scale
//   else:                         out = a / rms(a) * weight[i % weight_len] * act(g) * scale
// with act the SiLU (gate_act 1) or the sigmoid (0); g: columns g_off .. of proj.  A block owns one part of one row
// (grid: rows x parts); a thread keeps up to GGN_KEPT of the part's values (and gates) between the sum and the write.
constexpr int GGN_KEPT = 8;
template <typename TD, typename TO, bool SINGLE>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ o, const TD* __restrict__ proj, int n_partials,
                           long long partial_stride, long long ld, int g_off, const TO* __restrict__ xsrc,
                           long long x_ld, int x_off, const float* __restrict__ skip, int head_width,
                           const float* __restrict__ weight, int weight_len, TO* __restrict__ out, long long out_ld,
                           int n, int groups, float eps, float scale, int gate_first, int gate_act,
                           const int* __restrict__ segment_of_token) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, part = blockIdx.y;
  if (segment_of_token && segment_of_token[t] < 0) return;
  const int width = n / groups, lo = part * width;
  const float* row = o + (size_t)t * n;
  const TD* g = proj + (size_t)t * ld + g_off;
  auto act = [&](float z) {
    const float sg = 1.f / (1.f + expf(-z));
    return gate_act == 1 ? z * sg : sg;
  };
  auto gate = [&](int i) { return act(SINGLE ? to_f32<TD>(g[i]) : la_load(g + i, n_partials, partial_stride)); };
  auto plain = [&](int i) {
    float a = row[i];
    if (skip) a = fmaf(skip[i / head_width], to_f32<TO>(xsrc[(size_t)t * x_ld + x_off + i]), a);
    return a;
  };
  float kept[GGN_KEPT], gates[GGN_KEPT], side[GGN_KEPT];
  float sq = 0.f;
  const TO* xrow = skip ? xsrc + (size_t)t * x_ld + x_off : nullptr;
#pragma unroll
  for (int k = 0; k < GGN_KEPT; ++k) {     // every load of the thread first, so that they travel together
    const int i = lo + threadIdx.x + k * blockDim.x;
    kept[k] = gates[k] = side[k] = 0.f;
    if (i < lo + width) {
      gates[k] = SINGLE ? to_f32<TD>(g[i]) : la_load(g + i, n_partials, partial_stride);
      kept[k] = row[i];
      if (skip) side[k] = to_f32<TO>(xrow[i]);
    }
  }
#pragma unroll
  for (int k = 0; k < GGN_KEPT; ++k) {
    const int i = lo + threadIdx.x + k * blockDim.x;
    if (i < lo + width) {
      gates[k] = act(gates[k]);
      if (skip) kept[k] = fmaf(skip[i / head_width], side[k], kept[k]);
      if (gate_first) kept[k] *= gates[k];
      sq = fmaf(kept[k], kept[k], sq);
    }
  }
  for (int i = lo + threadIdx.x + GGN_KEPT * blockDim.x; i < lo + width; i += blockDim.x) {
    const float v = gate_first ? plain(i) * gate(i) : plain(i);
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
#pragma unroll
  for (int k = 0; k < GGN_KEPT; ++k) {
    const int i = lo + threadIdx.x + k * blockDim.x;
    if (i < lo + width) {
      float y = (kept[k] * inv) * weight[i % weight_len];
      if (!gate_first) y *= gates[k];
      out[(size_t)t * out_ld + i] = from_f32<TO>(y * scale);
    }
  }
  for (int i = lo + threadIdx.x + GGN_KEPT * blockDim.x; i < lo + width; i += blockDim.x) {
    const float gi = gate(i);
    float y = ((gate_first ? plain(i) * gi : plain(i)) * inv) * weight[i % weight_len];
    if (!gate_first) y *= gi;
    out[(size_t)t * out_ld + i] = from_f32<TO>(y * scale);
  }
}
// The same for narrow parts (up to 32 * GGN_WARP_KEPT columns): a warp owns a part of a row, eight parts a block, no
// barrier; the part's values and gates stay in registers.
constexpr int GGN_WARP_KEPT = 16;
template <typename TD, typename TO, bool SINGLE>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_warp_kernel(const float* __restrict__ o, const TD* __restrict__ proj, int n_partials,
                                long long partial_stride, long long ld, int g_off, const TO* __restrict__ xsrc,
                                long long x_ld, int x_off, const float* __restrict__ skip, int head_width,
                                const float* __restrict__ weight, int weight_len, TO* __restrict__ out, long long out_ld,
                                int tokens, int n, int groups, float eps, float scale, int gate_first, int gate_act,
                                const int* __restrict__ segment_of_token) {
  pdl_launch_dependents();
  pdl_wait();
  const long long item = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= (long long)tokens * groups) return;
  const int t = (int)(item / groups), part = (int)(item % groups);
  if (segment_of_token && segment_of_token[t] < 0) return;
  const int width = n / groups, lo = part * width;
  const float* row = o + (size_t)t * n + lo;
  const TD* g = proj + (size_t)t * ld + g_off + lo;
  const TO* x = skip ? xsrc + (size_t)t * x_ld + x_off + lo : nullptr;
  float kept[GGN_WARP_KEPT], gates[GGN_WARP_KEPT];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < GGN_WARP_KEPT; ++k) {     // every load of the lane first, so that they travel together
    const int c = lane + 32 * k;
    kept[k] = gates[k] = 0.f;
    if (c < width) {
      gates[k] = SINGLE ? to_f32<TD>(g[c]) : la_load(g + c, n_partials, partial_stride);
      kept[k] = row[c];
    }
  }
#pragma unroll
  for (int k = 0; k < GGN_WARP_KEPT; ++k) {
    const int c = lane + 32 * k;
    if (c < width) {
      const float z = gates[k];
      const float sg = 1.f / (1.f + expf(-z));
      gates[k] = gate_act == 1 ? z * sg : sg;
      if (skip) kept[k] = fmaf(skip[(lo + c) / head_width], to_f32<TO>(x[c]), kept[k]);
      if (gate_first) kept[k] *= gates[k];
      sq = fmaf(kept[k], kept[k], sq);
    }
  }
  const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
  const int w0 = lo % weight_len;      // the part's first weight; parts are whole multiples or whole fractions of the weight
#pragma unroll
  for (int k = 0; k < GGN_WARP_KEPT; ++k) {
    const int c = lane + 32 * k;
    if (c < width) {
      float y = (kept[k] * inv) * weight[(w0 + c) % weight_len];
      if (!gate_first) y *= gates[k];
      out[(size_t)t * out_ld + lo + c] = from_f32<TO>(y * scale);
    }
  }
}
}  // namespace

extern "C" int lse_linear_attention_scan(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                         long long ld, int q_off, int k_off, int v_off, const float* decay,
                                         float* state, const int* segment_start, const int* segment_slot, float* out,
                                         int max_segments, int heads, int dim, int vdim, int act, int num_slots,
                                         int chunk_rows, float* chunk_state, int max_chunks, cudaStream_t stream) {
  return linear_attention_scan_launch<MODE_PLAIN>(proj, proj_dtype, n_partials, partial_stride, ld, q_off, k_off, v_off,
                                                  decay, state, segment_start, segment_slot, out, max_segments, heads,
                                                  dim, vdim, act, num_slots, chunk_rows, chunk_state, max_chunks, nullptr,
                                                  nullptr, 1.0f, 0, 1, nullptr, stream);
}

extern "C" int lse_gated_rmsnorm(const float* o, const void* proj, int proj_dtype, int n_partials,
                                 long long partial_stride, long long ld, int g_off, const float* weight, void* out,
                                 int out_dtype, int tokens, int n, float eps, const int* segment_of_token,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0) return LSE_ERR_BAD_ARGUMENT;
#define LSE_GN_CASE(TD, TO)                                                                                   \
  lse_launch(gated_rmsnorm_kernel<TD, TO>, tokens, 256, 0, stream, o, (const TD*)proj, n_partials,            \
             partial_stride, ld, g_off, weight, (TO*)out, n, eps, segment_of_token);
  const bool d32 = proj_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_GN_CASE(float, float)
  else if (d32 && !o32) LSE_GN_CASE(float, __nv_bfloat16)
  else if (!d32 && o32) LSE_GN_CASE(__nv_bfloat16, float)
  else LSE_GN_CASE(__nv_bfloat16, __nv_bfloat16)
#undef LSE_GN_CASE
  LSE_LAUNCH_CHECK();
}

// keep, take float32 [tokens, heads]; proj float32 / bfloat16 rows or a float32 stack of partial sums.
extern "C" int lse_ssd_gates(const void* proj, int proj_dtype, int n_partials, long long partial_stride, long long ld,
                             int dt_off, const float* dt_bias, const float* a_log, float* keep, float* take, int tokens,
                             int heads, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)(((long long)tokens * heads + 255) / 256);
  if (proj_dtype == LSE_DTYPE_F32)
    lse_launch(ssd_gates_kernel<float>, blocks, 256, 0, stream, (const float*)proj, n_partials, partial_stride, ld, dt_off,
               dt_bias, a_log, keep, take, tokens, heads);
  else if (proj_dtype == LSE_DTYPE_BF16)
    lse_launch(ssd_gates_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)proj, n_partials,
               partial_stride, ld, dt_off, dt_bias, a_log, keep, take, tokens, heads);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// keep float32 [tokens, n] = sigmoid(proj[:, off .. off + n] + bias)^(1 / tau); bias float32 [n] or null.
extern "C" int lse_sigmoid_power(const void* proj, int proj_dtype, int n_partials, long long partial_stride, long long ld,
                                 int off, const float* bias, float tau, float* keep, int tokens, int n,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0 || n_partials < 1 || !(tau > 0.f)) return LSE_ERR_BAD_ARGUMENT;
  const long long blocks = ((long long)tokens * n + 255) / 256;
  if (blocks > 0x7fffffffLL) return LSE_ERR_TOO_LARGE;
  if (proj_dtype == LSE_DTYPE_F32)
    lse_launch(sigmoid_power_kernel<float>, (unsigned)blocks, 256, 0, stream, (const float*)proj, n_partials,
               partial_stride, ld, off, bias, 1.0f / tau, keep, tokens, n);
  else if (proj_dtype == LSE_DTYPE_BF16)
    lse_launch(sigmoid_power_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, (const __nv_bfloat16*)proj,
               n_partials, partial_stride, ld, off, bias, 1.0f / tau, keep, tokens, n);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// o float32 [tokens, n]; the gate in proj (float32 / bfloat16 / partial sums); xsrc (the output's dtype, rows x_ld apart) and
// skip float32 [n / head_width], or both null; weight float32 [weight_len], read at i % weight_len; out rows out_ld apart.
extern "C" int lse_gated_group_rmsnorm(const float* o, const void* proj, int proj_dtype, int n_partials,
                                       long long partial_stride, long long ld, int g_off, const void* xsrc, long long x_ld,
                                       int x_off, const float* skip, int head_width, const float* weight, int weight_len,
                                       void* out, int out_dtype, long long out_ld, int tokens, int n, int groups, float eps,
                                       float scale, int gate_first, int gate_act, const int* segment_of_token,
                                       cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0 || groups <= 0 || n % groups || weight_len <= 0 || n_partials < 1 || (skip && (!xsrc || head_width <= 0)))
    return LSE_ERR_BAD_ARGUMENT;
  if (groups > 65535) return LSE_ERR_TOO_LARGE;
  const int width = n / groups;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : (width > 32 ? 64 : 32));
  const dim3 grid(tokens, groups);
  const bool narrow = width <= 32 * GGN_WARP_KEPT;
  const long long warp_blocks = ((long long)tokens * groups + 7) / 8;
  if (narrow && warp_blocks > 0x7fffffffLL) return LSE_ERR_TOO_LARGE;
#define LSE_GGN_FORM(TD, TO, SINGLE)                                                                                 \
  if ((n_partials == 1) == SINGLE) {                                                                                 \
    if (narrow)                                                                                                      \
      lse_launch(gated_group_rmsnorm_warp_kernel<TD, TO, SINGLE>, (unsigned)warp_blocks, 256, 0, stream, o,           \
                 (const TD*)proj, n_partials, partial_stride, ld, g_off, (const TO*)xsrc, x_ld, x_off, skip,          \
                 head_width, weight, weight_len, (TO*)out, out_ld, tokens, n, groups, eps, scale, gate_first,         \
                 gate_act, segment_of_token);                                                                        \
    else                                                                                                             \
      lse_launch(gated_group_rmsnorm_kernel<TD, TO, SINGLE>, grid, threads, 0, stream, o, (const TD*)proj,            \
                 n_partials, partial_stride, ld, g_off, (const TO*)xsrc, x_ld, x_off, skip, head_width, weight,       \
                 weight_len, (TO*)out, out_ld, n, groups, eps, scale, gate_first, gate_act, segment_of_token);        \
  }
#define LSE_GGN_CASE(TD, TO)                                                                                         \
  {                                                                                                                  \
  LSE_GGN_FORM(TD, TO, true) else LSE_GGN_FORM(TD, TO, false)                                                        \
  }
  const bool d32 = proj_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_GGN_CASE(float, float)
  else if (d32 && !o32) LSE_GGN_CASE(float, __nv_bfloat16)
  else if (!d32 && o32) LSE_GGN_CASE(__nv_bfloat16, float)
  else LSE_GGN_CASE(__nv_bfloat16, __nv_bfloat16)
#undef LSE_GGN_CASE
#undef LSE_GGN_FORM
  LSE_LAUNCH_CHECK();
}
