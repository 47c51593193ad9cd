// The gates and the read-out of a matrix memory with exponential gates (mLSTM).  Per head and token, with the log input
// gate i_t = cap tanh(z_i / cap) and the log forget gate f_t = logsigmoid(cap tanh(z_f / cap)):
//     m_t = max(f_t + m_(t-1), i_t)                      a running maximum that keeps the exponentials in range
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,      n_t likewise with k_t alone
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// The gates kernel turns the gates' pre-activations (two columns per head of the layer's stacked projection) into the
// three numbers per token and head that the scan and the read-out need,
//     keep = exp(f_t + m_(t-1) - m_t),   take = exp(i_t - m_t),   floor = exp(-m_t),
// following each request's rows in order from the m that earlier steps left in the request's slot (zero for a new
// request) and leaving the new m there.  The scan itself is the gated form of the linear-attention scan
// (linear_attention.cu), whose extra state column carries n.  The read-out kernel divides, norms every head by its
// root mean square, and applies the norm weight and the output gate.  Everything is float32.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_mlstm)

namespace {
template <typename TD>
__device__ __forceinline__ float ml_load(const TD* p, int n_partials, long long partial_stride) {
  return sum_partials<TD>(p, n_partials, partial_stride);
}

__device__ __forceinline__ float ml_logsigmoid(float z) {
  // log(1 / (1 + exp(-z))) without overflow: min(z, 0) - log1p(exp(-|z|))
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// One block of eight warps per (request, head), 256 tokens at a time.  The recurrence of m is a chain of maps
// m -> max(m + f, i); two of them in a row are a map of the same form, (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2)),
// so a warp scans its 32 tokens' maps with shuffles, the warps' totals are chained through shared memory, and every token
// gets the m before it and its own.  keep uses exactly the m that the token before it was given, so the state's scale
// stays consistent however the rows are cut into steps; m itself may differ from one cut to another in its last bits,
// which moves nothing: it only says by what power the memory is scaled.
constexpr int MG_THREADS = 256;

template <typename TD>
__global__ void __launch_bounds__(MG_THREADS)
mlstm_gates_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int i_off,
                   int f_off, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                   float* __restrict__ state_m, const int* __restrict__ segment_start,
                   const int* __restrict__ segment_slot, float* __restrict__ keep, float* __restrict__ take,
                   float* __restrict__ floor_out, int heads, int num_slots) {
  __shared__ float total_f[MG_THREADS / 32], total_i[MG_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = segment_start[seg], row1 = segment_start[seg + 1];
  if (row1 <= row0) return;
  float* m_at = state_m + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * heads + h;
  float m = *m_at;
  const float bi = i_bias[h], bf = f_bias[h];
  for (int base = row0; base < row1; base += MG_THREADS) {
    const int r = base + threadIdx.x;
    float gi = -INFINITY, gf = 0.f;      // past the last row: the map that changes nothing
    if (r < row1) {
      const TD* row = proj + (size_t)r * ld;
      gi = cap * tanhf((ml_load(row + i_off + h, n_partials, partial_stride) + bi) / cap);
      gf = ml_logsigmoid(cap * tanhf((ml_load(row + f_off + h, n_partials, partial_stride) + bf) / cap));
    }
    float sf = gf, si = gi;              // the maps of this warp's tokens up to and with this one, in one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float uf = __shfl_up_sync(0xffffffffu, sf, o), ui = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) { si = fmaxf(ui + sf, si); sf = uf + sf; }
    }
    __syncthreads();                     // the totals of the round before have been read
    if (lane == 31) { total_f[warp] = sf; total_i[warp] = si; }
    __syncthreads();
    float m_warp = m, m_next = m;        // m before this warp's first token; m after the block's last
#pragma unroll
    for (int w = 0; w < MG_THREADS / 32; ++w) {
      m_next = fmaxf(m_next + total_f[w], total_i[w]);
      if (w + 1 == warp) m_warp = m_next;
    }
    const float m_mine = fmaxf(m_warp + sf, si);
    float m_before = __shfl_up_sync(0xffffffffu, m_mine, 1);
    if (lane == 0) m_before = m_warp;
    if (r < row1) {
      const size_t at = (size_t)r * heads + h;
      keep[at] = expf(gf + m_before - m_mine);
      take[at] = expf(gi - m_mine);
      floor_out[at] = expf(-m_mine);
    }
    m = m_next;
  }
  if (threadIdx.x == 0) *m_at = m;
}

// read [T, heads, vdim + 1]: the scan's outputs, the last column n . q.  A warp per (token, head).
template <typename TD, typename TO>
__global__ void __launch_bounds__(128)
mlstm_readout_kernel(const float* __restrict__ read, const float* __restrict__ floor_in, const TD* __restrict__ proj,
                     int n_partials, long long partial_stride, long long ld, int g_off,
                     const float* __restrict__ weight, TO* __restrict__ out, int tokens, int heads, int vdim, float eps,
                     const int* __restrict__ segment_of_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const long long pair = (long long)blockIdx.x * warps + warp;      // (token, head): a warp each, so that few rows fill the GPU too
  if (pair >= (long long)tokens * heads) return;
  const int t = (int)(pair / heads), h = (int)(pair % heads);
  if (segment_of_token && segment_of_token[t] < 0) return;
  {
    const float* row = read + ((size_t)t * heads + h) * (vdim + 1);
    const float inv_den = 1.0f / (fmaxf(fabsf(row[vdim]), floor_in[(size_t)t * heads + h]) + 1e-6f);
    float sq = 0.f;
    for (int j = lane; j < vdim; j += 32) { const float o = row[j] * inv_den; sq = fmaf(o, o, sq); }
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)vdim + eps);
    const TD* g = proj + (size_t)t * ld + g_off + h * vdim;
    for (int j = lane; j < vdim; j += 32) {
      const float gate = 1.f / (1.f + expf(-ml_load(g + j, n_partials, partial_stride)));
      out[(size_t)t * heads * vdim + h * vdim + j] =
          from_f32<TO>((((row[j] * inv_den) * inv) * weight[h * vdim + j]) * gate);
    }
  }
}
}  // namespace

// proj: the layer's stacked projection (rows of ld values, or n_partials partial sums partial_stride apart); column
// i_off + h is head h's input-gate pre-activation, f_off + h its forget gate's.  state_m float32 [slots, heads];
// keep, take, floor_out float32 [tokens, heads].
extern "C" int lse_mlstm_gates(const void* proj, int proj_dtype, int n_partials, long long partial_stride, long long ld,
                               int i_off, int f_off, const float* i_bias, const float* f_bias, float cap,
                               float* state_m, const int* segment_start, const int* segment_slot, float* keep,
                               float* take, float* floor_out, int max_segments, int heads, int num_slots,
                               cudaStream_t stream) {
  if (max_segments <= 0) return 0;
  if (heads <= 0 || heads > 65535 || !(cap > 0.f) || n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  const dim3 grid(max_segments, heads);
  if (proj_dtype == LSE_DTYPE_F32)
    lse_launch(mlstm_gates_kernel<float>, grid, MG_THREADS, 0, stream, (const float*)proj, n_partials, partial_stride, ld,
               i_off, f_off, i_bias, f_bias, cap, state_m, segment_start, segment_slot, keep, take, floor_out, heads,
               num_slots);
  else if (proj_dtype == LSE_DTYPE_BF16)
    lse_launch(mlstm_gates_kernel<__nv_bfloat16>, grid, MG_THREADS, 0, stream, (const __nv_bfloat16*)proj, n_partials,
               partial_stride, ld, i_off, f_off, i_bias, f_bias, cap, state_m, segment_start, segment_slot, keep, take,
               floor_out, heads, num_slots);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// out[t, h * vdim + j] = rms_h(read[t, h, :vdim] / den) * weight * sigmoid(gate), den = max(|read[t, h, vdim]|, floor) + 1e-6;
// the gate's pre-activation is columns g_off .. g_off + heads * vdim of proj.
extern "C" int lse_mlstm_readout(const float* read, const float* floor_in, const void* proj, int proj_dtype,
                                 int n_partials, long long partial_stride, long long ld, int g_off, const float* weight,
                                 void* out, int out_dtype, int tokens, int heads, int vdim, float eps,
                                 const int* segment_of_token, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0 || n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
#define LSE_ML_CASE(TD, TO)                                                                                          \
  lse_launch(mlstm_readout_kernel<TD, TO>, (unsigned)(((long long)tokens * heads + 3) / 4), 128, 0, stream, read,    \
             floor_in, (const TD*)proj, n_partials, partial_stride, ld, g_off, weight, (TO*)out, tokens, heads, vdim, \
             eps, segment_of_token)
  const bool d32 = proj_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_ML_CASE(float, float);
  else if (d32 && !o32) LSE_ML_CASE(float, __nv_bfloat16);
  else if (!d32 && o32) LSE_ML_CASE(__nv_bfloat16, float);
  else LSE_ML_CASE(__nv_bfloat16, __nv_bfloat16);
#undef LSE_ML_CASE
  LSE_LAUNCH_CHECK();
}
