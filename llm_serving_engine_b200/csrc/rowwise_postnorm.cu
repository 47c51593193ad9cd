// Row-wise kernels of decoders that normalise after the residual sum and take positions as learned vectors:
//   * embedding times a constant plus a learned position vector;
//   * x <- rmsnorm(alpha x + branch output [+ bias] [+ c_t x]) * w, written back as the float32 residual and, beside it,
//     in the compute dtype as the next branch's input;
//   * RMS norm of every head's query and key (one weight shared by the heads), bias, and the write of keys and values
//     into the paged cache (keys and values may have different head sizes);
//   * logits <- cap tanh(logits / cap).
// An input that comes from a matrix product may be a stack of float32 partial sums, added in index order first.
// All arithmetic is float32; a value is rounded once, when it is stored in a bfloat16 tensor.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_rowwise_postnorm)

namespace {

template <typename T> __device__ __forceinline__ void postnorm_load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void postnorm_load4<float>(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void postnorm_load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T> __device__ __forceinline__ void postnorm_store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void postnorm_store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void postnorm_store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ------------------------------------------------------------------ embedding + learned positions
template <typename T, typename TO>
__global__ void embedding_positions_kernel(const T* __restrict__ table, const T* __restrict__ pos_table,
                                           const int* __restrict__ ids, const int* __restrict__ positions, float scale,
                                           float* __restrict__ residual, TO* __restrict__ hidden_out, int hidden,
                                           int vocab, int max_positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = LSE_CHECKED(ids[t], 0, vocab, 0, LSE_CHECK_TOKEN_ID);
  int p = positions[t];
  p = p < 0 ? 0 : (p >= max_positions ? max_positions - 1 : p);   // padding rows carry position 0
  const T* src = table + (size_t)id * hidden;
  const T* pv = pos_table + (size_t)p * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = fmaf(to_f32<T>(src[i]), scale, to_f32<T>(pv[i]));
    residual[(size_t)t * hidden + i] = v;
    if (hidden_out) hidden_out[(size_t)t * hidden + i] = from_f32<TO>(v);
  }
}

// ------------------------------------------------------------------ norm after the sum
// y = alpha * residual + sum_p delta[p] + bias + row_scale[t] * x_in, x_in the row's current value in `hidden_io`
// (the compute-dtype copy of the residual; the residual itself when there is no copy);
// residual <- y / sqrt(mean(y^2) + eps) * weight;  hidden_io <- the same, rounded.
template <typename TD, typename TO>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                                          long long partial_stride, const float* __restrict__ bias,
                                          const float* __restrict__ row_scale, float alpha,
                                          const float* __restrict__ weight, TO* __restrict__ hidden_io, int hidden,
                                          float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float* res = residual + (size_t)t * hidden;
  const TD* del = delta ? delta + (size_t)t * hidden : nullptr;
  TO* hid = hidden_io ? hidden_io + (size_t)t * hidden : nullptr;
  const float extra = row_scale ? row_scale[t] : 0.f;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = res[i];
    float sum = 0.f;
    if (del)
      for (int p = 0; p < n_partials; ++p) sum += to_f32<TD>(del[(size_t)p * partial_stride + i]);
    if (bias) sum += bias[i];
    if (row_scale) sum = fmaf(extra, hid ? to_f32<TO>(hid[i]) : x, sum);
    const float y = fmaf(alpha, x, sum);
    res[i] = y;
    sq = fmaf(y, y, sq);
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float r = (res[i] * inv) * weight[i];
    res[i] = r;
    if (hid) hid[i] = from_f32<TO>(r);
  }
}

// The same for rows whose width is a multiple of 4 up to 256 * 4 * C: the row stays in registers between the sum of
// squares and the write (a thread owns C float4 pieces), the partial sums are fetched four at a time, one barrier
// pair.  Few rows (decoding) wait for round trips, not for bandwidth: this form has three of them.
template <typename TD, typename TO, int C>
__global__ void __launch_bounds__(256)
scaled_add_rmsnorm_regs_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                               long long partial_stride, const float* __restrict__ bias,
                               const float* __restrict__ row_scale, float alpha, const float* __restrict__ weight,
                               TO* __restrict__ hidden_io, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float* res = residual + (size_t)t * hidden;
  const TD* del = delta ? delta + (size_t)t * hidden : nullptr;
  TO* hid = hidden_io ? hidden_io + (size_t)t * hidden : nullptr;
  const float extra = row_scale ? row_scale[t] : 0.f;
  const int pieces = hidden / 4;
  float y[C][4];
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int piece = threadIdx.x + c * 256;
    if (piece < pieces) {
      const int i = piece * 4;
      float x[4], sum[4] = {0.f, 0.f, 0.f, 0.f};
      postnorm_load4<float>(res + i, x);
      if (del) {
        int p = 0;
        for (; p + 8 <= n_partials; p += 8) {   // eight loads in flight, added in index order
          float a[8][4];
#pragma unroll
          for (int k = 0; k < 8; ++k) postnorm_load4<TD>(del + (size_t)(p + k) * partial_stride + i, a[k]);
#pragma unroll
          for (int k = 0; k < 8; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) sum[e] += a[k][e];
        }
        for (; p + 4 <= n_partials; p += 4) {
          float a[4][4];
#pragma unroll
          for (int k = 0; k < 4; ++k) postnorm_load4<TD>(del + (size_t)(p + k) * partial_stride + i, a[k]);
#pragma unroll
          for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) sum[e] += a[k][e];
        }
        for (; p < n_partials; ++p) {
          float a[4];
          postnorm_load4<TD>(del + (size_t)p * partial_stride + i, a);
#pragma unroll
          for (int e = 0; e < 4; ++e) sum[e] += a[e];
        }
      }
      if (bias) {
        float b[4];
        postnorm_load4<float>(bias + i, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) sum[e] += b[e];
      }
      if (row_scale) {
        float h[4];
        if (hid) postnorm_load4<TO>(hid + i, h);
#pragma unroll
        for (int e = 0; e < 4; ++e) sum[e] = fmaf(extra, hid ? h[e] : x[e], sum[e]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) { y[c][e] = fmaf(alpha, x[e], sum[e]); sq = fmaf(y[c][e], y[c][e], sq); }
    }
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int piece = threadIdx.x + c * 256;
    if (piece < pieces) {
      const int i = piece * 4;
      float w[4], r[4];
      postnorm_load4<float>(weight + i, w);
#pragma unroll
      for (int e = 0; e < 4; ++e) r[e] = (y[c][e] * inv) * w[e];
      postnorm_store4<float>(res + i, r);
      if (hid) postnorm_store4<TO>(hid + i, r);
    }
  }
}

// ------------------------------------------------------------------ per-head norm of queries and keys, cache write
// A warp owns one head of one token: items 0 .. n_q-1 are query heads, then n_kv key heads, then n_kv value heads.
// The row of `proj` is [q (n_q * dk) | k (n_kv * dk) | v (n_kv * dv) | anything else].
template <typename TI, typename TO>
__global__ void head_norm_kv_write_kernel(const TI* __restrict__ proj, int n_partials, long long partial_stride,
                                          long long ld, const float* __restrict__ bias,
                                          const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                          const int* __restrict__ slot_mapping, TO* __restrict__ q_out,
                                          TO* __restrict__ k_cache, TO* __restrict__ v_cache, int tokens, int n_q,
                                          int n_kv, int dk, int dv, int page_size, int num_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int items = n_q + 2 * n_kv;
  const int warp = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= tokens * items) return;
  const int t = warp / items, item = warp % items;
  int column, width;
  const float* norm_w = nullptr;
  TO* dst = nullptr;
  if (item < n_q) {
    column = item * dk; width = dk; norm_w = q_norm;
    dst = q_out + ((size_t)t * n_q + item) * dk;
  } else {
    const int slot = LSE_CHECKED(slot_mapping[t], -1, num_pages * page_size, -1, LSE_CHECK_CACHE_SLOT);
    if (slot < 0) return;   // padding row
    const int page = slot / page_size, offset = slot % page_size;
    if (item < n_q + n_kv) {
      const int h = item - n_q;
      column = n_q * dk + h * dk; width = dk; norm_w = k_norm;
      dst = k_cache + (((size_t)page * n_kv + h) * page_size + offset) * dk;
    } else {
      const int h = item - n_q - n_kv;
      column = (n_q + n_kv) * dk + h * dv; width = dv;
      dst = v_cache + (((size_t)page * n_kv + h) * page_size + offset) * dv;
    }
  }
  const TI* src = proj + (size_t)t * ld + column;
  auto value = [&](int i) {
    float sum = 0.f;
    for (int p = 0; p < n_partials; ++p) sum += to_f32<TI>(src[(size_t)p * partial_stride + i]);
    return bias ? sum + bias[column + i] : sum;
  };
  // Four consecutive values a load when the head's width and place allow (every operand 16- or 8-byte aligned).
  const bool by_four = width % 4 == 0 && column % 4 == 0 && ld % 4 == 0 && partial_stride % 4 == 0 && width <= 512;
  if (by_four) {
    float kept[4][4];   // pieces lane, lane + 32, ... of the head
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = (lane + 32 * k) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) kept[k][e] = 0.f;
      if (i < width) {
        for (int p = 0; p < n_partials; ++p) {
          float a[4];
          postnorm_load4<TI>(src + (size_t)p * partial_stride + i, a);
#pragma unroll
          for (int e = 0; e < 4; ++e) kept[k][e] += a[e];
        }
        if (bias) {
#pragma unroll
          for (int e = 0; e < 4; ++e) kept[k][e] += bias[column + i + e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) sq = fmaf(kept[k][e], kept[k][e], sq);
      }
    }
    const float inv = norm_w ? 1.0f / sqrtf(warp_sum(sq) / (float)width + eps) : 1.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = (lane + 32 * k) * 4;
      if (i < width) {
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) r[e] = norm_w ? (kept[k][e] * inv) * norm_w[i + e] : kept[k][e];
        postnorm_store4<TO>(dst + i, r);
      }
    }
    return;
  }
  constexpr int KEPT = 8;   // values a lane keeps between the sum of squares and the write (heads up to 256 wide)
  float kept[KEPT];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < KEPT; ++k) {
    const int i = lane + 32 * k;
    kept[k] = i < width ? value(i) : 0.f;
    sq = fmaf(kept[k], kept[k], sq);
  }
  for (int i = lane + 32 * KEPT; i < width; i += 32) { const float x = value(i); sq = fmaf(x, x, sq); }
  const float inv = norm_w ? 1.0f / sqrtf(warp_sum(sq) / (float)width + eps) : 1.f;
#pragma unroll
  for (int k = 0; k < KEPT; ++k) {
    const int i = lane + 32 * k;
    if (i < width) dst[i] = from_f32<TO>(norm_w ? (kept[k] * inv) * norm_w[i] : kept[k]);
  }
  for (int i = lane + 32 * KEPT; i < width; i += 32) {
    const float x = value(i);
    dst[i] = from_f32<TO>(norm_w ? (x * inv) * norm_w[i] : x);
  }
}

// The same with a rotation behind the norm: the first rot_dims values of every query and key head are rotated in pairs
// (value i with value i + rot_dims / 2) by the angle position * freq[i], formed in double precision; cosine and sine are
// multiplied by rot_factor.  A warp owns a head of a token and passes its normed values through shared memory, so
// that a lane finds its partner's; heads up to 256 wide.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
head_norm_rope_kv_write_kernel(const TI* __restrict__ proj, int n_partials, long long partial_stride, long long ld,
                               const float* __restrict__ bias, const float* __restrict__ q_norm,
                               const float* __restrict__ k_norm, float eps, const int* __restrict__ slot_mapping,
                               const int* __restrict__ positions, const double* __restrict__ freq, float rot_factor,
                               int rot_dims, TO* __restrict__ q_out, TO* __restrict__ k_cache, TO* __restrict__ v_cache,
                               int tokens, int n_q, int n_kv, int dk, int dv, int page_size, int num_pages) {
  __shared__ float staged[4][256];
  pdl_launch_dependents();
  pdl_wait();
  const int items = n_q + 2 * n_kv;
  const int warp = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= tokens * items) return;
  const int t = warp / items, item = warp % items;
  int column, width;
  const float* norm_w = nullptr;
  TO* dst = nullptr;
  bool rotated = true;
  const int slot = LSE_CHECKED(slot_mapping[t], -1, num_pages * page_size, -1, LSE_CHECK_CACHE_SLOT);
  if (slot < 0) return;   // padding row
  if (item < n_q) {
    column = item * dk; width = dk; norm_w = q_norm;
    dst = q_out + ((size_t)t * n_q + item) * dk;
  } else {
    const int page = slot / page_size, offset = slot % page_size;
    if (item < n_q + n_kv) {
      const int h = item - n_q;
      column = n_q * dk + h * dk; width = dk; norm_w = k_norm;
      dst = k_cache + (((size_t)page * n_kv + h) * page_size + offset) * dk;
    } else {
      const int h = item - n_q - n_kv;
      column = (n_q + n_kv) * dk + h * dv; width = dv;
      dst = v_cache + (((size_t)page * n_kv + h) * page_size + offset) * dv;
      rotated = false;
    }
  }
  const TI* src = proj + (size_t)t * ld + column;
  float* mine = staged[threadIdx.x >> 5];
  float sq = 0.f;
  for (int i = lane; i < width; i += 32) {
    float sum = 0.f;
    for (int p = 0; p < n_partials; ++p) sum += to_f32<TI>(src[(size_t)p * partial_stride + i]);
    if (bias) sum += bias[column + i];
    mine[i] = sum;
    sq = fmaf(sum, sum, sq);
  }
  const float inv = norm_w ? 1.0f / sqrtf(warp_sum(sq) / (float)width + eps) : 1.f;
  __syncwarp();
  const int half = rot_dims / 2;
  const int position = positions[t];
  for (int i = lane; i < width; i += 32) {
    float x = norm_w ? (mine[i] * inv) * norm_w[i] : mine[i];
    if (rotated && i < rot_dims) {
      const int pair = i < half ? i : i - half;
      const int other = i < half ? i + half : i - half;
      const float y = norm_w ? (mine[other] * inv) * norm_w[other] : mine[other];
      double sine, cosine;
      sincos((double)position * freq[pair], &sine, &cosine);
      const float c = (float)cosine * rot_factor, s = (float)sine * rot_factor;
      x = i < half ? x * c - y * s : x * c + y * s;
    }
    dst[i] = from_f32<TO>(x);
  }
}

__global__ void softcap_kernel(float* __restrict__ values, long long count, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < count) values[i] = cap * tanhf(values[i] / cap);
}

}  // namespace

extern "C" int lse_embedding_positions(const void* table, const void* pos_table, int table_dtype, const int* ids,
                                       const int* positions, float scale, float* residual, void* hidden_out,
                                       int tokens, int hidden, int vocab, int max_positions, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (max_positions <= 0 || vocab <= 0) return LSE_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == LSE_DTYPE_F32)
    lse_launch(embedding_positions_kernel<float, float>, tokens, threads, 0, stream, (const float*)table,
               (const float*)pos_table, ids, positions, scale, residual, (float*)hidden_out, hidden, vocab, max_positions);
  else if (table_dtype == LSE_DTYPE_BF16)
    lse_launch(embedding_positions_kernel<__nv_bfloat16, __nv_bfloat16>, tokens, threads, 0, stream,
               (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, ids, positions, scale, residual,
               (__nv_bfloat16*)hidden_out, hidden, vocab, max_positions);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// hidden_io: the compute-dtype copy (type out_dtype), or null when the residual itself is what the branches read.
extern "C" int lse_scaled_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_partials,
                                      long long partial_stride, const float* bias, const float* row_scale, float alpha,
                                      const float* weight, void* hidden_io, int out_dtype, int tokens, int hidden,
                                      float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (delta && n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 2048 ? 256 : 128;
  const int pieces = hidden % 4 == 0 && partial_stride % 4 == 0 ? (hidden / 4 + 255) / 256 : 0;   // float4 pieces a thread
#define LSE_POSTNORM_ARGS(TD, TO) residual, (const TD*)delta, n_partials, partial_stride, bias, row_scale, alpha, weight, \
  (TO*)hidden_io, hidden, eps
#define LSE_POSTNORM_CASE(TD, TO)                                                                                   \
  if (pieces == 1) lse_launch(scaled_add_rmsnorm_regs_kernel<TD, TO, 1>, tokens, 256, 0, stream, LSE_POSTNORM_ARGS(TD, TO)); \
  else if (pieces == 2) lse_launch(scaled_add_rmsnorm_regs_kernel<TD, TO, 2>, tokens, 256, 0, stream, LSE_POSTNORM_ARGS(TD, TO)); \
  else if (pieces >= 3 && pieces <= 4) lse_launch(scaled_add_rmsnorm_regs_kernel<TD, TO, 4>, tokens, 256, 0, stream, LSE_POSTNORM_ARGS(TD, TO)); \
  else if (pieces >= 5 && pieces <= 8) lse_launch(scaled_add_rmsnorm_regs_kernel<TD, TO, 8>, tokens, 256, 0, stream, LSE_POSTNORM_ARGS(TD, TO)); \
  else lse_launch(scaled_add_rmsnorm_kernel<TD, TO>, tokens, threads, 0, stream, LSE_POSTNORM_ARGS(TD, TO))
  if (delta_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) { LSE_POSTNORM_CASE(float, float); }
  else if (delta_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) { LSE_POSTNORM_CASE(__nv_bfloat16, __nv_bfloat16); }
  else if (delta_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) { LSE_POSTNORM_CASE(float, __nv_bfloat16); }
  else if (delta_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_F32) { LSE_POSTNORM_CASE(__nv_bfloat16, float); }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_POSTNORM_CASE
#undef LSE_POSTNORM_ARGS
  LSE_LAUNCH_CHECK();
}

// n_kv = 0: the layer has no keys and values of its own (it reads another layer's pages); only queries are made.
extern "C" int lse_head_norm_kv_write(const void* proj, int in_dtype, int n_partials, long long partial_stride,
                                      long long ld, const float* bias, const float* q_norm, const float* k_norm,
                                      float eps, const int* slot_mapping, void* q_out, void* k_cache, void* v_cache,
                                      int out_dtype, int tokens, int n_q, int n_kv, int dk, int dv, int page_size,
                                      int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n_q <= 0 || n_kv < 0 || dk <= 0 || dv <= 0 || n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  if (n_kv > 0 && (!k_cache || !v_cache || !slot_mapping || page_size <= 0)) return LSE_ERR_BAD_ARGUMENT;
  const long long warps = (long long)tokens * (n_q + 2 * n_kv);
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return LSE_ERR_TOO_LARGE;
#define LSE_HEADNORM_CASE(TI, TO)                                                                                      \
  lse_launch(head_norm_kv_write_kernel<TI, TO>, (unsigned)blocks, threads, 0, stream, (const TI*)proj, n_partials,     \
             partial_stride, ld, bias, q_norm, k_norm, eps, slot_mapping, (TO*)q_out, (TO*)k_cache, (TO*)v_cache,      \
             tokens, n_q, n_kv, dk, dv, page_size, num_pages)
  if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) LSE_HEADNORM_CASE(float, float);
  else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) LSE_HEADNORM_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) LSE_HEADNORM_CASE(float, __nv_bfloat16);
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_HEADNORM_CASE
  LSE_LAUNCH_CHECK();
}

// As lse_head_norm_kv_write, then the first rot_dims values of every query and key head rotated (freq float64
// [rot_dims / 2], positions int32 [tokens], cosine and sine times rot_factor).  Heads up to 256 wide.
extern "C" int lse_head_norm_rope_kv_write(const void* proj, int in_dtype, int n_partials, long long partial_stride,
                                           long long ld, const float* bias, const float* q_norm, const float* k_norm,
                                           float eps, const int* slot_mapping, const int* positions, const double* freq,
                                           float rot_factor, int rot_dims, void* q_out, void* k_cache, void* v_cache,
                                           int out_dtype, int tokens, int n_q, int n_kv, int dk, int dv, int page_size,
                                           int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n_q <= 0 || n_kv <= 0 || dk <= 0 || dv <= 0 || n_partials < 1 || dk > 256 || dv > 256) return LSE_ERR_BAD_ARGUMENT;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > dk || (rot_dims > 0 && (!freq || !positions))) return LSE_ERR_BAD_ARGUMENT;
  if (!k_cache || !v_cache || !slot_mapping || page_size <= 0) return LSE_ERR_BAD_ARGUMENT;
  const long long warps = (long long)tokens * (n_q + 2 * n_kv);
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return LSE_ERR_TOO_LARGE;
#define LSE_HEADROPE_CASE(TI, TO)                                                                                      \
  lse_launch(head_norm_rope_kv_write_kernel<TI, TO>, (unsigned)blocks, threads, 0, stream, (const TI*)proj, n_partials, \
             partial_stride, ld, bias, q_norm, k_norm, eps, slot_mapping, positions, freq, rot_factor, rot_dims,       \
             (TO*)q_out, (TO*)k_cache, (TO*)v_cache, tokens, n_q, n_kv, dk, dv, page_size, num_pages)
  if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) LSE_HEADROPE_CASE(float, float);
  else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) LSE_HEADROPE_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) LSE_HEADROPE_CASE(float, __nv_bfloat16);
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_HEADROPE_CASE
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_softcap(float* values, long long count, float cap, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.f)) return LSE_ERR_BAD_ARGUMENT;
  const long long blocks = (count + 255) / 256;
  if (blocks > 0x7fffffffLL) return LSE_ERR_TOO_LARGE;
  lse_launch(softcap_kernel, (unsigned)blocks, 256, 0, stream, values, count, cap);
  LSE_LAUNCH_CHECK();
}
