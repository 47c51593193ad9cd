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
// A step of few rows gives a block (request, channels) and walks the request's rows in order.  A step of many rows is
// cut into chunks of chunk_rows rows that are scanned side by side, as the linear-attention scan does: a pass that
// builds every chunk's own state from zero and the sum of its step sizes (a chunk's decay is exp(A * that sum)), a
// carry from chunk to chunk, and a pass that writes the outputs from each chunk's starting state.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_selective_scan)

namespace {
constexpr int SS_THREADS = 128;
constexpr int SS_PER_LANE = 4;     // states a thread keeps (one 16-byte read of a token's B and of its C)
constexpr int SS_TOKENS = 16;      // tokens staged at a time

template <typename TD>
__device__ __forceinline__ float ss_load(const TD* p, int n_partials, long long partial_stride) {
  return sum_partials<TD>(p, n_partials, partial_stride);
}

// grid (token tiles of 16, channel tiles of 64); 256 threads: 64 channels times four parts of the rank.  A thread adds up
// its part of the rank for sixteen tokens (the tokens' inputs lie in shared memory, rank-major, so that one 16-byte
// read serves four tokens and every lane of a warp reads the same address); the four parts are then added in order.
// An output does not depend on how many rows the step has or where in a tile the row falls.
constexpr int SZ_TOKENS = 16, SZ_CHANNELS = 64, SZ_PARTS = 4;

template <typename TD>
__global__ void __launch_bounds__(SZ_CHANNELS * SZ_PARTS)
ssm_step_sizes_kernel(const TD* __restrict__ low, int n_partials, long long partial_stride, long long ld,
                      const float* __restrict__ weight_t, const float* __restrict__ bias, float* __restrict__ dt,
                      int tokens, int channels, int rank) {
  extern __shared__ float4 sz_smem[];     // [rank][16] inputs, then [3][16][64] sums of the parts after the first
  float* low_s = reinterpret_cast<float*>(sz_smem);
  float* part_s = low_s + (size_t)rank * SZ_TOKENS;
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * SZ_TOKENS, n = min(SZ_TOKENS, tokens - t0);
  for (int e = threadIdx.x; e < SZ_TOKENS * rank; e += blockDim.x) {
    const int t = e / rank, r = e % rank;
    low_s[r * SZ_TOKENS + t] = t < n ? ss_load(low + (size_t)(t0 + t) * ld + r, n_partials, partial_stride) : 0.f;
  }
  __syncthreads();
  const int cl = threadIdx.x % SZ_CHANNELS, part = threadIdx.x / SZ_CHANNELS;
  const int c = blockIdx.y * SZ_CHANNELS + cl;
  const int per = (rank + SZ_PARTS - 1) / SZ_PARTS;
  const int r0 = part * per, r1 = min(rank, r0 + per);
  float sum[SZ_TOKENS];
#pragma unroll
  for (int t = 0; t < SZ_TOKENS; ++t) sum[t] = 0.f;
  if (c < channels) {
#pragma unroll 4
    for (int r = r0; r < r1; ++r) {
      const float w = weight_t[(size_t)r * channels + c];
      const float4* in = reinterpret_cast<const float4*>(low_s + r * SZ_TOKENS);
#pragma unroll
      for (int q = 0; q < SZ_TOKENS / 4; ++q) {
        const float4 v = in[q];
        sum[4 * q] = fmaf(w, v.x, sum[4 * q]);
        sum[4 * q + 1] = fmaf(w, v.y, sum[4 * q + 1]);
        sum[4 * q + 2] = fmaf(w, v.z, sum[4 * q + 2]);
        sum[4 * q + 3] = fmaf(w, v.w, sum[4 * q + 3]);
      }
    }
  }
  if (part > 0) {
#pragma unroll
    for (int t = 0; t < SZ_TOKENS; ++t) part_s[((part - 1) * SZ_TOKENS + t) * SZ_CHANNELS + cl] = sum[t];
  }
  __syncthreads();
  if (part > 0 || c >= channels) return;
  const float b = bias[c];
#pragma unroll
  for (int t = 0; t < SZ_TOKENS; ++t) {
    if (t < n) {
      float z = sum[t];
#pragma unroll
      for (int other = 0; other < SZ_PARTS - 1; ++other) z += part_s[(other * SZ_TOKENS + t) * SZ_CHANNELS + cl];
      z += b;
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
                      int channels, int states, int num_slots, int num_segments, int chunk_rows, int phase,
                      float* __restrict__ chunk_state, float* __restrict__ chunk_dt) {
  constexpr int CH = SS_THREADS / LANES;     // channels of a block
  constexpr int SP = LANES * SS_PER_LANE;    // a token's B (or C) in shared memory: the states, then zeros up to a lane's four
  extern __shared__ __align__(16) float ss_smem[];   // [16][SP] B, [16][SP] C, [16][CH] dt, x, z
  __shared__ int item[3];
  pdl_launch_dependents();
  pdl_wait();
  int seg, row0, row1;
  if (chunk_rows == 0) {
    seg = blockIdx.x;
    row0 = segment_start[seg];
    row1 = segment_start[seg + 1];
  } else {
    if (threadIdx.x == 0) {     // which request's which rows chunk blockIdx.x is
      int before = 0, found = -1, first = 0, last = 0;
      for (int s = 0; s < num_segments && found < 0; ++s) {
        const int a = segment_start[s], b = segment_start[s + 1];
        const int chunks = (b - a + chunk_rows - 1) / chunk_rows;
        if ((int)blockIdx.x < before + chunks) {
          found = s;
          first = a + ((int)blockIdx.x - before) * chunk_rows;
          last = min(b, first + chunk_rows);
        }
        before += chunks;
      }
      item[0] = found; item[1] = first; item[2] = last;
    }
    __syncthreads();
    seg = item[0]; row0 = item[1]; row1 = item[2];
    if (seg < 0) return;
  }
  if (row1 <= row0) return;
  const bool from_zero = chunk_rows > 0 && phase == 1;      // a chunk's own state, from nothing
  const bool outputs = !from_zero;
  const bool store = !(chunk_rows > 0 && phase == 2);
  float* b_s = ss_smem;
  float* c_s = b_s + SS_TOKENS * SP;
  float* dt_s = c_s + SS_TOKENS * SP;
  float* x_s = dt_s + SS_TOKENS * CH;
  float* z_s = x_s + SS_TOKENS * CH;
  const int sub = threadIdx.x % LANES, local = threadIdx.x / LANES;
  const int c = blockIdx.y * CH + local;
  const bool live = c < channels;
  float* st = chunk_rows == 0
      ? state + ((size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * channels + (live ? c : 0)) * states
      : chunk_state + ((size_t)blockIdx.x * channels + (live ? c : 0)) * states;
  float s[SS_PER_LANE], a[SS_PER_LANE];
#pragma unroll
  for (int i = 0; i < SS_PER_LANE; ++i) {
    const int n = sub * SS_PER_LANE + i;    // a lane's four states lie side by side: one 16-byte read of B and of C a token
    const bool has = live && n < states;
    s[i] = has && !from_zero ? st[n] : 0.f;
    a[i] = has ? -expf(a_log[(size_t)c * states + n]) : 0.f;
  }
  const float d_skip = live ? skip[c] : 0.f;
  float dt_sum = 0.f;       // of the chunk's step sizes: the chunk's decay is exp(A * dt_sum)
  for (int base = row0; base < row1; base += SS_TOKENS) {
    const int n_tok = min(SS_TOKENS, row1 - base);
    __syncthreads();
    for (int e = threadIdx.x; e < n_tok * SP; e += SS_THREADS) {
      const int t = e / SP, n = e % SP;
      const TL* row = low + (size_t)(base + t) * low_ld;
      b_s[e] = n < states ? ss_load(row + b_off + n, low_partials, low_stride) : 0.f;
      if (outputs) c_s[e] = n < states ? ss_load(row + c_off + n, low_partials, low_stride) : 0.f;
    }
    for (int e = threadIdx.x; e < n_tok * CH; e += SS_THREADS) {
      const int t = e / CH, cc = blockIdx.y * CH + e % CH;
      const bool ok = cc < channels;
      dt_s[e] = ok ? dt[(size_t)(base + t) * channels + cc] : 0.f;
      x_s[e] = ok ? to_f32<TX>(x[(size_t)(base + t) * channels + cc]) : 0.f;
      if (outputs) z_s[e] = ok ? ss_load(proj + (size_t)(base + t) * proj_ld + z_off + cc, proj_partials, proj_stride) : 0.f;
    }
    __syncthreads();
    if (!outputs) {       // the pass that only builds the chunk's own state leaves the outputs' half of the work out
      for (int t = 0; t < n_tok; ++t) {
        const float step = dt_s[t * CH + local];
        const float push = step * x_s[t * CH + local];
        dt_sum += step;
        const float4 b4 = *reinterpret_cast<const float4*>(b_s + t * SP + sub * SS_PER_LANE);
        const float bv[SS_PER_LANE] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int i = 0; i < SS_PER_LANE; ++i) s[i] = fmaf(expf(step * a[i]), s[i], push * bv[i]);   // past the last state: 1 * 0 + push * 0
      }
      continue;
    }
    for (int t = 0; t < n_tok; ++t) {
      const float step = dt_s[t * CH + local], xv = x_s[t * CH + local];
      const float push = step * xv;
      float y = 0.f;
      const float4 b4 = *reinterpret_cast<const float4*>(b_s + t * SP + sub * SS_PER_LANE);
      const float4 c4 = *reinterpret_cast<const float4*>(c_s + t * SP + sub * SS_PER_LANE);
      const float bv[SS_PER_LANE] = {b4.x, b4.y, b4.z, b4.w}, cv[SS_PER_LANE] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
      for (int i = 0; i < SS_PER_LANE; ++i) {
        s[i] = fmaf(expf(step * a[i]), s[i], push * bv[i]);
        y = fmaf(s[i], cv[i], y);
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
  if (live && store) {
#pragma unroll
    for (int i = 0; i < SS_PER_LANE; ++i) {
      const int n = sub * SS_PER_LANE + i;
      if (n < states) st[n] = s[i];
    }
    if (from_zero && sub == 0) chunk_dt[(size_t)blockIdx.x * channels + c] = dt_sum;
  }
}

// Between the two passes over chunks: chunk_state[k] holds chunk k's own state (from zero) and chunk_dt[k] the sum of
// its step sizes; afterwards chunk_state[k] holds the request's state at the chunk's start, and the request's slot the
// state after its last row.  A thread carries one element (channel, state) of one request from chunk to chunk:
//     start_(k+1) = exp(A * dt_sum_k) * start_k + own_k.
__global__ void __launch_bounds__(256)
selective_scan_carry_kernel(const float* __restrict__ a_log, float* __restrict__ state,
                            const int* __restrict__ segment_start, const int* __restrict__ segment_slot,
                            float* __restrict__ chunk_state, const float* __restrict__ chunk_dt, int channels, int states,
                            int num_slots, int chunk_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.y;
  const int first = segment_start[seg], last = segment_start[seg + 1];
  if (last <= first) return;
  const int chunks = (last - first + chunk_rows - 1) / chunk_rows;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= channels * states) return;
  const int c = e / states;
  int before = 0;
  for (int s = 0; s < seg; ++s) before += (segment_start[s + 1] - segment_start[s] + chunk_rows - 1) / chunk_rows;
  const size_t per_state = (size_t)channels * states;
  const float a = -expf(a_log[e]);
  float* slot = state + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * per_state + e;
  float running = *slot;
  float* own = chunk_state + (size_t)before * per_state + e;
  const float* sums = chunk_dt + (size_t)before * channels + c;
  for (int k0 = 0; k0 < chunks; k0 += 8) {
    float mine[8], decay[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mine[i] = k0 + i < chunks ? own[(size_t)(k0 + i) * per_state] : 0.f;
      decay[i] = k0 + i < chunks ? sums[(size_t)(k0 + i) * channels] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (k0 + i < chunks) {
        own[(size_t)(k0 + i) * per_state] = running;
        running = fmaf(expf(a * decay[i]), running, mine[i]);
      }
    }
  }
  *slot = running;
}
}  // namespace

// low: rows of ld values (float32, bfloat16 or partial sums) whose first `rank` columns are the step sizes' inputs;
// weight_t float32 [rank, channels]; bias float32 [channels]; dt float32 [tokens, channels].
extern "C" int lse_ssm_step_sizes(const void* low, int low_dtype, int n_partials, long long partial_stride, long long ld,
                                  const float* weight_t, const float* bias, float* dt, int tokens, int channels, int rank,
                                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || rank <= 0 || n_partials < 1 || (channels + SZ_CHANNELS - 1) / SZ_CHANNELS > 65535) return LSE_ERR_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * SZ_TOKENS * ((size_t)rank + (SZ_PARTS - 1) * SZ_CHANNELS);
  if (smem > 160 * 1024) return LSE_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(ssm_step_sizes_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(ssm_step_sizes_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const dim3 grid((tokens + SZ_TOKENS - 1) / SZ_TOKENS, (channels + SZ_CHANNELS - 1) / SZ_CHANNELS);
  constexpr int threads = SZ_CHANNELS * SZ_PARTS;
  if (low_dtype == LSE_DTYPE_F32)
    lse_launch(ssm_step_sizes_kernel<float>, grid, threads, smem, stream, (const float*)low, n_partials, partial_stride, ld,
               weight_t, bias, dt, tokens, channels, rank);
  else if (low_dtype == LSE_DTYPE_BF16)
    lse_launch(ssm_step_sizes_kernel<__nv_bfloat16>, grid, threads, smem, stream, (const __nv_bfloat16*)low, n_partials,
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
                                  int num_slots, int chunk_rows, float* chunk_state, float* chunk_dt, int max_chunks,
                                  cudaStream_t stream) {
  if (max_segments <= 0) return 0;
  if (channels <= 0 || states <= 0 || proj_partials < 1 || low_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  if (chunk_rows < 0 || (chunk_rows > 0 && (!chunk_state || !chunk_dt || max_chunks <= 0))) return LSE_ERR_BAD_ARGUMENT;
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
    const size_t smem = sizeof(float) * SS_TOKENS * (2 * (size_t)L * SS_PER_LANE + 3 * ch);                                 \
    const dim3 grid(chunk_rows > 0 ? max_chunks : max_segments, (channels + ch - 1) / ch);                         \
    for (int phase = 1; phase <= (chunk_rows > 0 ? 2 : 1); ++phase) {                                              \
      lse_launch(selective_scan_kernel<TD, TL, TX, TO, L>, grid, SS_THREADS, smem, stream, (const TX*)x, dt,       \
                 (const TD*)proj, proj_partials, proj_stride, proj_ld, z_off, (const TL*)low, low_partials,        \
                 low_stride, low_ld, b_off, c_off, a_log, skip, state, segment_start, segment_slot, (TO*)out,      \
                 out_ld, scale, channels, states, num_slots, max_segments, chunk_rows, phase, chunk_state,         \
                 chunk_dt);                                                                                        \
      if (chunk_rows > 0 && phase == 1)                                                                            \
        lse_launch(selective_scan_carry_kernel, dim3((unsigned)((channels * states + 255) / 256), max_segments),   \
                   256, 0, stream, a_log, state, segment_start, segment_slot, chunk_state, chunk_dt, channels,     \
                   states, num_slots, chunk_rows);                                                                 \
    }                                                                                                              \
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
