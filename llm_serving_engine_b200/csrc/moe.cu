// Mixture of experts: the router and the experts' gated activation.
//
// Router (a warp per token, everything float32): the logits z_e = w_e . x over all router outputs come from a matrix
// product with float32 sums (the last `identity` outputs are identity experts, whose output is the token's input
// itself; one more column is the shared expert's gate); s = softmax(z), the `top` outputs with the
// largest s_e + correction_e are chosen (ties: the lower index), and a chosen output's weight is s_e itself, neither
// corrected nor renormalised.  The kernel leaves a dense row of weights over the real experts (zero where an expert
// was not chosen), the choices themselves, the sum of the chosen identity experts' weights, and the gate of the
// shared expert, sigmoid(w_sg . x).
//
// Activation (experts side by side in one product): the row of `gate_up` holds, expert by expert, [gate (ff values) |
// up (ff values)], then [gate | up] of the shared expert (shared_ff values each); the output row holds the experts'
// ff columns side by side, then the shared expert's:
//   g = min(gate, limit);  u = clamp(up, -limit, limit);  out = c * g * sigmoid(1.702 g) * (u + 1)
// with c the token's weight of the column's expert (the shared gate for the shared columns; 1 without weights).  The
// down product over all columns then is the weighted sum over the experts.
//
// Rows grouped by expert (many rows): every (token, chosen real expert) pair gets a row of its own in a buffer in
// which the rows of one expert are consecutive; `lse_moe_group_rows` counts, scans and places them (one block; the
// order inside an expert's range is not fixed, a row's result does not depend on it), `lse_moe_gather_rows` copies the
// tokens' inputs there, a grouped product runs per expert over its range, and `lse_moe_combine` adds, per token, its
// rows times their weights in the order of its choices, and the identity experts' share of the input.
#include "common.cuh"

namespace {
constexpr int ROUTE_THREADS = 128;   // a warp per token

// logits: float32 [tokens, ld] (or a stack of n_partials partial sums): the router's outputs, then (has_shared_gate) the
// shared expert's gate; columns beyond are padding.
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const float* __restrict__ logits, int n_partials, long long partial_stride, int ld,
                 const float* __restrict__ correction, int has_shared_gate, float* __restrict__ expert_weights,
                 float* __restrict__ identity_weight, float* __restrict__ shared_gate, int* __restrict__ chosen_out,
                 int tokens, int outputs, int identity, int top, const float* __restrict__ logit_bias, int over_chosen) {
  extern __shared__ float smem[];   // per warp: [outputs] scores, [outputs] choice scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (ROUTE_THREADS / 32) + warp;
  if (t >= tokens) return;
  float* score = smem + (size_t)warp * 2 * outputs;
  float* choice = score + outputs;
  const float* row = logits + (size_t)t * ld;
  auto logit = [&](int e) {
    float sum = 0.f;
    for (int p = 0; p < n_partials; ++p) sum += row[(size_t)p * partial_stride + e];
    return (logit_bias && e < outputs) ? sum + logit_bias[e] : sum;
  };
  const int experts = outputs - identity;
  float top_z = -INFINITY;
  for (int e = lane; e < outputs; e += 32) { const float z = logit(e); score[e] = z; top_z = fmaxf(top_z, z); }
  if (has_shared_gate && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-logit(outputs)));
  top_z = warp_max(top_z);
  float sum = 0.f;
  for (int e = lane; e < outputs; e += 32) sum += expf(score[e] - top_z);
  sum = warp_sum(sum);
  for (int e = lane; e < outputs; e += 32) {
    // over_chosen: the logits themselves are compared, and the weights are exp(z - largest) over the sum of the chosen ones
    const float s = over_chosen ? score[e] : expf(score[e] - top_z) / sum;
    score[e] = s;
    choice[e] = correction ? s + correction[e] : s;
    if (e < experts) expert_weights[(size_t)t * experts + e] = 0.f;
  }
  __syncwarp();
  float identity_sum = 0.f, chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32) {
      const float c = choice[e];
      if (c > best) { best = c; best_e = e; }   // ascending e within a lane: the first largest stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (best_e >= outputs) {   // fewer outputs than `top`: the remaining choices are none
      if (chosen_out && lane == 0)
        for (int rest = k; rest < top; ++rest) chosen_out[(size_t)t * top + rest] = -1;
      break;
    }
    const float weight = over_chosen ? expf(score[best_e] - top_z) : score[best_e];
    chosen_sum += weight;
    if (lane == 0) {
      choice[best_e] = -INFINITY;
      if (best_e < experts) expert_weights[(size_t)t * experts + best_e] = weight;
      if (chosen_out) chosen_out[(size_t)t * top + k] = best_e;
    }
    if (best_e >= experts) identity_sum += weight;
    __syncwarp();
  }
  if (over_chosen) {     // the softmax over the chosen logits only
    for (int e = lane; e < experts; e += 32) expert_weights[(size_t)t * experts + e] /= chosen_sum;
    identity_sum /= chosen_sum;
  }
  if (lane == 0) identity_weight[t] = identity_sum;
}

// A router whose scores are sigmoids, chosen within the best groups of experts (a warp per token, float32):
//   s_e = sigmoid(z_e);  c_e = s_e + correction_e  (the choice score);
//   the experts form `group_count` equal groups of neighbours; a group's score is the sum of its two largest c (of its
//   one c when a group is a single expert); only the `group_keep` best groups' experts can be chosen (group_count <= 1:
//   all experts);  the `top` largest c among them are chosen (ties: the lower index);
//   weight_e = s_e / (sum of the chosen s + 1e-20) * scale.
// Leaves what moe_route_kernel leaves: the dense row of weights, the choices, a zero identity weight, the shared gate.
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_sigmoid_kernel(const float* __restrict__ logits, int n_partials, long long partial_stride, int ld,
                         const float* __restrict__ correction, int has_shared_gate, float* __restrict__ expert_weights,
                         float* __restrict__ identity_weight, float* __restrict__ shared_gate, int* __restrict__ chosen_out,
                         int tokens, int experts, int top, int group_count, int group_keep, float scale) {
  extern __shared__ float smem[];   // per warp: [experts] scores, [experts] choice scores, [groups] group scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (ROUTE_THREADS / 32) + warp;
  if (t >= tokens) return;
  const int groups = group_count > 1 ? group_count : 1;
  float* score = smem + (size_t)warp * (2 * experts + groups);
  float* choice = score + experts;
  float* group_score = choice + experts;
  const float* row = logits + (size_t)t * ld;
  auto logit = [&](int e) {
    float sum = 0.f;
    for (int p = 0; p < n_partials; ++p) sum += row[(size_t)p * partial_stride + e];
    return sum;
  };
  for (int e = lane; e < experts; e += 32) {
    const float sg = 1.0f / (1.0f + expf(-logit(e)));
    score[e] = sg;
    choice[e] = correction ? sg + correction[e] : sg;
    expert_weights[(size_t)t * experts + e] = 0.f;
  }
  if (has_shared_gate && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-logit(experts)));
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    const int per = experts / group_count;
    for (int g = lane; g < group_count; g += 32) {
      float first = -INFINITY, second = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > first) { second = first; first = c; }
        else if (c > second) second = c;
      }
      group_score[g] = per > 1 ? first + second : first;
    }
    __syncwarp();
    // a group is kept when fewer than group_keep groups come before it (a larger score, or an equal one at a lower index)
    for (int g = lane; g < group_count; g += 32) {
      const float mine = group_score[g];
      int ahead = 0;
      for (int o = 0; o < group_count; ++o) {
        const float other = group_score[o];
        ahead += (other > mine || (other == mine && o < g)) ? 1 : 0;
      }
      if (ahead >= group_keep)
        for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  float chosen_sum = 0.f;
  int taken = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float c = choice[e];
      if (c > best) { best = c; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (best_e >= experts) {   // nothing left to choose from
      if (chosen_out && lane == 0)
        for (int rest = k; rest < top; ++rest) chosen_out[(size_t)t * top + rest] = -1;
      break;
    }
    chosen_sum += score[best_e];
    ++taken;
    if (lane == 0) {
      choice[best_e] = -INFINITY;
      expert_weights[(size_t)t * experts + best_e] = score[best_e];
      if (chosen_out) chosen_out[(size_t)t * top + k] = best_e;
    }
    __syncwarp();
  }
  const float factor = scale / (chosen_sum + 1e-20f);
  for (int e = lane; e < experts; e += 32) expert_weights[(size_t)t * experts + e] *= factor;
  if (lane == 0) identity_weight[t] = 0.f;
  (void)taken;
}

template <typename T> __device__ __forceinline__ void moe_load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void moe_load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void moe_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void moe_store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void moe_store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void moe_store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Eight columns a thread (ff and shared_ff multiples of 8, rows 16-byte aligned): the same arithmetic as the kernel below.
template <typename TI, typename TO>
__global__ void moe_gated_act8_kernel(const TI* __restrict__ gate_up, int n_partials, long long partial_stride,
                                      const float* __restrict__ expert_weights, const float* __restrict__ shared_gate,
                                      TO* __restrict__ out, int experts, int ff, int shared_ff, float limit,
                                      float shared_limit, const int* __restrict__ valid_rows, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (valid_rows && t >= *valid_rows) return;   // rows behind the last expert's range of a grouped buffer
  const int inter = experts * ff + shared_ff;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  const bool shared = i >= experts * ff;
  const float c = shared ? (shared_gate ? shared_gate[t] : 1.f)
                         : (expert_weights ? expert_weights[(size_t)t * experts + i / ff] : 1.f);
  TO* dst = out + (size_t)t * inter + i;
  float y[8];
  if (c == 0.f) {
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = 0.f;
    moe_store8<TO>(dst, y);
    return;
  }
  if (kind == 2) {      // experts without a gate: the row holds one column per output, out = c * relu(u)^2
    const TI* row = gate_up + (size_t)t * inter + i;
    float u[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) u[e] = 0.f;
    for (int p = 0; p < n_partials; ++p) {
      float b[8];
      moe_load8<TI>(row + (size_t)p * partial_stride, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) u[e] += b[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float r = fmaxf(u[e], 0.f); y[e] = c * (r * r); }
    moe_store8<TO>(dst, y);
    return;
  }
  const TI* row = gate_up + (size_t)t * 2 * inter;
  const int gate_at = shared ? 2 * experts * ff + (i - experts * ff) : (i / ff) * 2 * ff + i % ff;
  const int up_at = gate_at + (shared ? shared_ff : ff);
  float g[8], u[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) g[e] = u[e] = 0.f;
  for (int p = 0; p < n_partials; ++p) {
    float a[8], b[8];
    moe_load8<TI>(row + (size_t)p * partial_stride + gate_at, a);
    moe_load8<TI>(row + (size_t)p * partial_stride + up_at, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) { g[e] += a[e]; u[e] += b[e]; }
  }
  const float lim = shared ? shared_limit : limit;
  if (kind == 1) {      // out = c * silu(g) * u, nothing clamped
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gated = sizeof(TO) == 2 ? __fdividef(g[e], 1.0f + __expf(-g[e])) : g[e] / (1.0f + expf(-g[e]));
      y[e] = c * (gated * u[e]);
    }
    moe_store8<TO>(dst, y);
    return;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float gc = fminf(g[e], lim), uc = fminf(fmaxf(u[e], -lim), lim);
    // the result is rounded to bfloat16 far more coarsely than the fast exponential and division err
    const float gated = sizeof(TO) == 2 ? __fdividef(gc, 1.0f + __expf(-1.702f * gc)) : gc / (1.0f + expf(-1.702f * gc));
    y[e] = c * (gated * (uc + 1.0f));
  }
  moe_store8<TO>(dst, y);
}

template <typename TI, typename TO>
__global__ void moe_gated_act_kernel(const TI* __restrict__ gate_up, int n_partials, long long partial_stride,
                                     const float* __restrict__ expert_weights, const float* __restrict__ shared_gate,
                                     TO* __restrict__ out, int experts, int ff, int shared_ff, float limit,
                                     float shared_limit, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int inter = experts * ff + shared_ff;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const bool shared = i >= experts * ff;
  const float c = shared ? (shared_gate ? shared_gate[t] : 1.f)
                         : (expert_weights ? expert_weights[(size_t)t * experts + i / ff] : 1.f);
  TO* dst = out + (size_t)t * inter + i;
  if (c == 0.f) { *dst = from_f32<TO>(0.f); return; }   // an expert that the token did not choose
  if (kind == 2) {
    float u = 0.f;
    for (int p = 0; p < n_partials; ++p) u += to_f32<TI>(gate_up[(size_t)p * partial_stride + (size_t)t * inter + i]);
    u = fmaxf(u, 0.f);
    *dst = from_f32<TO>(c * (u * u));
    return;
  }
  const TI* row = gate_up + (size_t)t * 2 * inter;
  const int gate_at = shared ? 2 * experts * ff + (i - experts * ff) : (i / ff) * 2 * ff + i % ff;
  const int up_at = gate_at + (shared ? shared_ff : ff);
  float g = 0.f, u = 0.f;
  for (int p = 0; p < n_partials; ++p) {
    g += to_f32<TI>(row[(size_t)p * partial_stride + gate_at]);
    u += to_f32<TI>(row[(size_t)p * partial_stride + up_at]);
  }
  if (kind == 1) { *dst = from_f32<TO>(c * (g / (1.0f + expf(-g)) * u)); return; }
  const float lim = shared ? shared_limit : limit;
  g = fminf(g, lim);
  u = fminf(fmaxf(u, -lim), lim);
  const float act = g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
  *dst = from_f32<TO>(c * act);
}
// One block: counts[e] = rows of expert e, offsets (inclusive sums, what a grouped product takes), and for every
// (token, choice) its row in the grouped buffer (-1: an identity expert, or padding).
__global__ void __launch_bounds__(1024)
moe_group_rows_kernel(const int* __restrict__ chosen, const int* __restrict__ segment_of_token, int* __restrict__ row_of,
                      int* __restrict__ offsets, int tokens, int top, int experts) {
  extern __shared__ int group_smem[];   // [experts] counts, then [experts] first rows
  pdl_launch_dependents();
  pdl_wait();
  int* count = group_smem;
  int* first = group_smem + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  const int entries = tokens * top;
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = chosen[i];
    const bool real = e >= 0 && e < experts && (!segment_of_token || segment_of_token[i / top] >= 0);
    row_of[i] = real ? atomicAdd(&count[e], 1) : -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int e = 0; e < experts; ++e) { first[e] = running; running += count[e]; offsets[e] = running; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x)
    if (row_of[i] >= 0) row_of[i] += first[chosen[i]];
}

template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ row_of, T* __restrict__ grouped,
                                       int width, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = row_of[blockIdx.x];    // blockIdx.x = token * top + choice
  if (row < 0) return;
  const T* src = x + (size_t)(blockIdx.x / top) * width;
  T* dst = grouped + (size_t)row * width;
  if (sizeof(T) == 2 && width % 8 == 0) {
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
  }
}

// y[t] (+)= sum_k w[t, chosen[t, k]] * down[row_of[t, k]] + identity_weight[t] * x[t]   (accumulate: y holds the
// shared expert's output already; else it is overwritten)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ down, const int* __restrict__ row_of, const int* __restrict__ chosen,
                                   const float* __restrict__ expert_weights, const float* __restrict__ identity_weight,
                                   const T* __restrict__ x, float* __restrict__ y, int width, int top, int experts,
                                   int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float identity = identity_weight ? identity_weight[t] : 0.f;
  if (width % 8 == 0) {   // eight columns a thread (rows are 16-byte aligned then)
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float sum[8];
      if (accumulate) moe_load8<float>(y + (size_t)t * width + i, sum);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] = 0.f;
      }
      for (int k = 0; k < top; ++k) {
        const int row = row_of[t * top + k];
        if (row >= 0) {
          const float w = expert_weights[(size_t)t * experts + chosen[t * top + k]];
          float v[8];
          moe_load8<T>(down + (size_t)row * width + i, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) sum[e] = fmaf(w, v[e], sum[e]);
        }
      }
      if (identity != 0.f) {
        float v[8];
        moe_load8<T>(x + (size_t)t * width + i, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] = fmaf(identity, v[e], sum[e]);
      }
      moe_store8<float>(y + (size_t)t * width + i, sum);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = accumulate ? y[(size_t)t * width + i] : 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = row_of[t * top + k];
      if (row >= 0)
        sum = fmaf(expert_weights[(size_t)t * experts + chosen[t * top + k]], to_f32<T>(down[(size_t)row * width + i]), sum);
    }
    if (identity != 0.f) sum = fmaf(identity, to_f32<T>(x[(size_t)t * width + i]), sum);
    y[(size_t)t * width + i] = sum;
  }
}
}  // namespace

extern "C" int lse_moe_route_biased(const float* logits, int n_partials, long long partial_stride, int ld,
                                    const float* correction, int has_shared_gate, float* expert_weights,
                                    float* identity_weight, float* shared_gate, int* chosen, int tokens, int outputs,
                                    int identity, int top, const float* logit_bias, int over_chosen, cudaStream_t stream);

// logits float32 [tokens, ld] or n_partials partial sums partial_stride apart: column e < outputs is router output e,
// column `outputs` the shared expert's gate (has_shared_gate); correction float32 [outputs] or null.
// expert_weights float32 [tokens, outputs - identity]; identity_weight, shared_gate float32 [tokens];
// chosen int32 [tokens, top] or null (-1 where there are fewer outputs than top).
extern "C" int lse_moe_route(const float* logits, int n_partials, long long partial_stride, int ld, const float* correction,
                             int has_shared_gate, float* expert_weights, float* identity_weight, float* shared_gate,
                             int* chosen, int tokens, int outputs, int identity, int top, cudaStream_t stream) {
  return lse_moe_route_biased(logits, n_partials, partial_stride, ld, correction, has_shared_gate, expert_weights,
                              identity_weight, shared_gate, chosen, tokens, outputs, identity, top, nullptr, 0, stream);
}

// logit_bias float32 [outputs] or null: added to the router's logits.  over_chosen: the `top` largest logits are chosen
// (plus correction, if any) and the weights are the softmax over the chosen logits only.
extern "C" int lse_moe_route_biased(const float* logits, int n_partials, long long partial_stride, int ld,
                                    const float* correction, int has_shared_gate, float* expert_weights,
                                    float* identity_weight, float* shared_gate, int* chosen, int tokens, int outputs,
                                    int identity, int top, const float* logit_bias, int over_chosen,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (outputs <= 0 || identity < 0 || identity > outputs || top <= 0 || n_partials < 1 ||
      ld < outputs + (has_shared_gate ? 1 : 0))
    return LSE_ERR_BAD_ARGUMENT;
  if (outputs > 1024) return LSE_ERR_TOO_LARGE;
  const int warps = ROUTE_THREADS / 32;
  const size_t smem = sizeof(float) * 2 * (size_t)outputs * warps;
  lse_launch(moe_route_kernel, (tokens + warps - 1) / warps, ROUTE_THREADS, smem, stream, logits, n_partials,
             partial_stride, ld, correction, has_shared_gate, expert_weights, identity_weight, shared_gate, chosen, tokens,
             outputs, identity, top, logit_bias, over_chosen);
  LSE_LAUNCH_CHECK();
}

// As lse_moe_route, for sigmoid scores chosen within the best groups (see moe_route_sigmoid_kernel); no identity experts.
extern "C" int lse_moe_route_sigmoid(const float* logits, int n_partials, long long partial_stride, int ld,
                                     const float* correction, int has_shared_gate, float* expert_weights,
                                     float* identity_weight, float* shared_gate, int* chosen, int tokens, int experts,
                                     int top, int group_count, int group_keep, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || top <= 0 || n_partials < 1 || ld < experts + (has_shared_gate ? 1 : 0)) return LSE_ERR_BAD_ARGUMENT;
  if (group_count > 1 && (experts % group_count || group_keep <= 0)) return LSE_ERR_BAD_ARGUMENT;
  if (experts > 1024) return LSE_ERR_TOO_LARGE;
  const int warps = ROUTE_THREADS / 32;
  const size_t smem = sizeof(float) * (2 * (size_t)experts + (group_count > 1 ? group_count : 1)) * warps;
  lse_launch(moe_route_sigmoid_kernel, (tokens + warps - 1) / warps, ROUTE_THREADS, smem, stream, logits, n_partials,
             partial_stride, ld, correction, has_shared_gate, expert_weights, identity_weight, shared_gate, chosen, tokens,
             experts, top, group_count, group_keep, scale);
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_moe_gated_act_kind(const void* gate_up, int in_dtype, int n_partials, long long partial_stride,
                                      const float* expert_weights, const float* shared_gate, void* out, int out_dtype,
                                      int tokens, int experts, int ff, int shared_ff, float limit, float shared_limit,
                                      const int* valid_rows, int kind, cudaStream_t stream);

extern "C" int lse_moe_gated_act(const void* gate_up, int in_dtype, int n_partials, long long partial_stride,
                                 const float* expert_weights, const float* shared_gate, void* out, int out_dtype,
                                 int tokens, int experts, int ff, int shared_ff, float limit, float shared_limit,
                                 const int* valid_rows, cudaStream_t stream) {
  return lse_moe_gated_act_kind(gate_up, in_dtype, n_partials, partial_stride, expert_weights, shared_gate, out, out_dtype,
                                tokens, experts, ff, shared_ff, limit, shared_limit, valid_rows, 0, stream);
}

// kind 0: out = c * g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit);
// kind 1: out = c * silu(g) * u;
// kind 2: experts without a gate, the input row holds one column per output column: out = c * relu(u)^2.
extern "C" int lse_moe_gated_act_kind(const void* gate_up, int in_dtype, int n_partials, long long partial_stride,
                                      const float* expert_weights, const float* shared_gate, void* out, int out_dtype,
                                      int tokens, int experts, int ff, int shared_ff, float limit, float shared_limit,
                                      const int* valid_rows, int kind, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int inter = experts * ff + shared_ff;
  if (inter <= 0 || n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  if ((inter + 255) / 256 > 65535) return LSE_ERR_TOO_LARGE;
  const bool wide = ff % 8 == 0 && shared_ff % 8 == 0 && partial_stride % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0;
  const dim3 grid(tokens, wide ? (inter / 8 + 127) / 128 : (inter + 255) / 256);
  const int threads = wide ? 128 : 256;
#define LSE_MOE_ACT_CASE(TI, TO)                                                                                      \
  if (wide)                                                                                                           \
    lse_launch(moe_gated_act8_kernel<TI, TO>, grid, threads, 0, stream, (const TI*)gate_up, n_partials, partial_stride, \
               expert_weights, shared_gate, (TO*)out, experts, ff, shared_ff, limit, shared_limit, valid_rows, kind); \
  else                                                                                                                \
    lse_launch(moe_gated_act_kernel<TI, TO>, grid, threads, 0, stream, (const TI*)gate_up, n_partials, partial_stride,  \
               expert_weights, shared_gate, (TO*)out, experts, ff, shared_ff, limit, shared_limit, kind)
  if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) { LSE_MOE_ACT_CASE(float, float); }
  else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) { LSE_MOE_ACT_CASE(__nv_bfloat16, __nv_bfloat16); }
  else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) { LSE_MOE_ACT_CASE(float, __nv_bfloat16); }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_MOE_ACT_CASE
  LSE_LAUNCH_CHECK();
}

// chosen int32 [tokens, top] (what lse_moe_route left); row_of int32 [tokens, top]; offsets int32 [experts].
extern "C" int lse_moe_group_rows(const int* chosen, const int* segment_of_token, int* row_of, int* offsets, int tokens,
                                  int top, int experts, cudaStream_t stream) {
  if (tokens <= 0 || experts <= 0) return 0;
  if (top <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (experts > 4096) return LSE_ERR_TOO_LARGE;
  lse_launch(moe_group_rows_kernel, 1, 1024, sizeof(int) * 2 * (size_t)experts, stream, chosen, segment_of_token, row_of,
             offsets, tokens, top, experts);
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_moe_gather_rows(const void* x, int dtype, const int* row_of, void* grouped, int tokens, int top,
                                   int width, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (dtype == LSE_DTYPE_F32)
    lse_launch(moe_gather_rows_kernel<float>, (unsigned)tokens * top, 128, 0, stream, (const float*)x, row_of,
               (float*)grouped, width, top);
  else if (dtype == LSE_DTYPE_BF16)
    lse_launch(moe_gather_rows_kernel<__nv_bfloat16>, (unsigned)tokens * top, 128, 0, stream,
               (const __nv_bfloat16*)x, row_of, (__nv_bfloat16*)grouped, width, top);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_moe_combine(const void* down, int dtype, const int* row_of, const int* chosen, const float* expert_weights,
                               const float* identity_weight, const void* x, float* y, int tokens, int width, int top,
                               int experts, int accumulate, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == LSE_DTYPE_F32)
    lse_launch(moe_combine_kernel<float>, tokens, threads, 0, stream, (const float*)down, row_of, chosen, expert_weights,
               identity_weight, (const float*)x, y, width, top, experts, accumulate);
  else if (dtype == LSE_DTYPE_BF16)
    lse_launch(moe_combine_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (const __nv_bfloat16*)down, row_of, chosen,
               expert_weights, identity_weight, (const __nv_bfloat16*)x, y, width, top, experts, accumulate);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}
