// Paged attention whose scores or weights are changed on the way: general form (any head sizes up to 256, keys and
// values of different sizes, float32 or bfloat16 storage).  One block computes one query row (one token of the step)
// for up to GC query heads that share one key head.  On top of causal softmax attention over the request's pages:
//
//   * distance penalty: s_ij = (q_i . k_j) * scale - r1_h * ln(1 + r2_h * (i - j)), r1 and r2 per query head;
//   * sink: the softmax's denominator also holds exp(sink_h) (no key, no value, counted once);
//   * values of every group (`cross`): head g's weights are applied to the values of EVERY key/value head c, giving
//     O[g, c] = sum_j w_g(i, j) v_c(j) in float32.  A mixing of the heads' softmax weights,
//     w'_h = sum_g M[h, g] w_g, applied to head h's own values, is then sum_g M[h, g] O[g, kv(h)]: linear in the
//     weights, so it is taken after the softmax has been normalised (sink included) without ever holding a
//     [heads, keys] tile of weights.  `lse_head_mix_gate` does that sum and multiplies by an elementwise gate.
//
//   * window: row i reads keys j with i - j < window only (window <= 0: every key up to i); pages before the window
//     are never touched (their table entries may have been given back);
//   * cap: s <- cap * tanh(s / cap) before anything else is done with the score (cap <= 0: none);
//   * weights without a softmax (`head_bias` given): a key's weight is sigmoid(s_ij + head_bias_h), not normalised
//     over the keys; the output is the plain weighted sum of the values.  The chunks' sums are then added in order
//     (the running maximum stays 0 and the denominator is not used).
//
// Keys are walked in tiles of KT with the online-softmax recurrence, chunk by chunk (CHUNK keys, counted from key 0);
// the chunks' (max, sum, acc) are merged in order.  With few rows every chunk has a block of its own and a second
// kernel merges them with the same operations in the same order.  Chunks and tiles depend on the row's own position
// only, so a row's result is the same bit for bit whatever else is in the batch and however the prompt was cut.
//
// Cache layout: keys [page][kv head][offset in page][DK], values [page][kv head][offset in page][DV].
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_attention_scored)

namespace {
constexpr int KT = 32;        // keys per tile (one warp lane per key)
constexpr int CHUNK = 256;    // keys per chunk (a multiple of KT)
constexpr int GC = 8;         // query heads per block
constexpr int THREADS = 128;  // 4 warps
constexpr int MAX_D = 256;
constexpr int DPT = MAX_D / THREADS;  // output values per thread and head

__device__ __forceinline__ void merge_parts(float& M, float& L, float m, float l, float& wa, float& wb) {
  const float m_new = fmaxf(M, m);
  wa = expf(M - m_new);    // exp(-inf) = 0 before the first chunk; every chunk of a row has a visible key
  wb = expf(m - m_new);
  L = fmaf(l, wb, L * wa);
  M = m_new;
}

// The sink joins a finished (M, L): the factor on the outputs is returned.
__device__ __forceinline__ float add_sink(float M, float& L, float sink) {
  const float m_new = fmaxf(M, sink);
  const float wa = expf(M - m_new);
  L = fmaf(L, wa, expf(sink - m_new));
  return wa;
}

// blockIdx.z = ((chunk * n_values) + value slot) * gchunks + chunk of the group's heads   (chunk only with SPLIT).
// n_values = 1: the value head is the key head; else value slot c is value head c and the output has a row per c.
// Output element of (row t, head h, value slot c, column d): ((t * n_q + h) * n_values + c) * dv + d.
template <typename T, typename TO, bool SPLIT>
__global__ void __launch_bounds__(THREADS)
attention_scored_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        TO* __restrict__ out, const int* __restrict__ block_tables, int bt_stride,
                        const int* __restrict__ segment_of_token, const int* __restrict__ positions,
                        const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
                        int n_q, int n_kv, int dk, int dv, int n_values, int page_size, float scale, int num_pages,
                        int num_segments, float* __restrict__ partials, int max_chunks, int window, float cap,
                        const float* __restrict__ head_bias) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int kv_head = blockIdx.y;
  const int group = n_q / n_kv;
  const int gchunks = (group + GC - 1) / GC;
  int zz = blockIdx.z;
  const int g0 = (zz % gchunks) * GC;
  zz /= gchunks;
  const int value_slot = zz % n_values;
  zz /= n_values;
  const int value_head = n_values > 1 ? value_slot : kv_head;
  const int gcount = min(GC, group - g0);
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0) return;
  const int pos = positions[t];
  const int ctx = pos + 1;
  const int first_key = window > 0 ? max(0, ctx - window) : 0;   // the first key the row reads
  int chunk_lo = first_key / CHUNK, chunk_hi = pos / CHUNK;
  if (SPLIT) {
    if (zz > chunk_hi || zz < chunk_lo) return;
    chunk_lo = chunk_hi = zz;
  }
  const int* bt = block_tables + (size_t)seg * bt_stride;

  float* q_s = smem;                       // [GC][dk]
  float* k_s = q_s + GC * dk;              // [KT][dk + 1]
  float* v_s = k_s + KT * (dk + 1);        // [KT][dv]
  float* p_s = v_s + KT * dv;              // [GC][KT]
  float* corr_s = p_s + GC * KT;           // [GC]
  float* l_s = corr_s + GC;                // [GC]
  float* m_s = l_s + GC;                   // [GC]
  int* slot_s = (int*)(m_s + GC);          // [KT] page * page_size + offset of key j, -1 = masked

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first_head = kv_head * group + g0;
  for (int e = tid; e < gcount * dk; e += THREADS) {
    const int g = e / dk, d = e % dk;
    q_s[g * dk + d] = to_f32<T>(q[((size_t)t * n_q + first_head + g) * dk + d]);
  }

  float total[GC][DPT], M[GC], L[GC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    M[g] = -INFINITY;
    L[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) total[g][i] = 0.f;
  }
  // the penalty's constants of the heads this warp scores (g = warp, warp + 4)
  float pen1[GC / 4], pen2[GC / 4], hb[GC / 4];
#pragma unroll
  for (int i = 0; i < GC / 4; ++i) {
    const int g = warp + 4 * i;
    pen1[i] = (r1 && g < gcount) ? r1[first_head + g] : 0.f;
    pen2[i] = (r2 && g < gcount) ? r2[first_head + g] : 0.f;
    hb[i] = (head_bias && g < gcount) ? head_bias[first_head + g] : 0.f;
  }
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

  for (int chunk = chunk_lo; chunk <= chunk_hi; ++chunk) {
    float acc[GC][DPT];
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[g][i] = 0.f;
    float m_run[GC / 4], l_run[GC / 4];
#pragma unroll
    for (int i = 0; i < GC / 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    const int tile_end = min(ctx, (chunk + 1) * CHUNK);
    for (int base = max(chunk * CHUNK, first_key / KT * KT); base < tile_end; base += KT) {
      __syncthreads();  // previous tile fully consumed (also orders the q_s fill)
      if (tid < KT) {
        const int j = base + tid;
        int slot = -1;
        if (j < ctx && j >= first_key) {
          const int page = LSE_CHECKED(bt[j / page_size], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
          slot = page * page_size + (j % page_size);
        }
        slot_s[tid] = slot;
      }
      __syncthreads();
      for (int e = tid; e < KT * dk; e += THREADS) {
        const int j = e / dk, d = e % dk;
        const int slot = slot_s[j];
        float kv = 0.f;
        if (slot >= 0) {
          const int page = slot / page_size, offset = slot % page_size;
          kv = to_f32<T>(k_cache[(((size_t)page * n_kv + kv_head) * page_size + offset) * dk + d]);
        }
        k_s[j * (dk + 1) + d] = kv;
      }
      for (int e = tid; e < KT * dv; e += THREADS) {
        const int j = e / dv, d = e % dv;
        const int slot = slot_s[j];
        float vv = 0.f;
        if (slot >= 0) {
          const int page = slot / page_size, offset = slot % page_size;
          vv = to_f32<T>(v_cache[(((size_t)page * n_kv + value_head) * page_size + offset) * dv + d]);
        }
        v_s[j * dv + d] = vv;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < GC / 4; ++i) {
        const int g = warp + 4 * i;
        if (g < gcount) {
          const bool valid = slot_s[lane] >= 0;
          float s = 0.f;
          const float* qr = q_s + g * dk;
          const float* kr = k_s + lane * (dk + 1);
          for (int d = 0; d < dk; ++d) s = fmaf(qr[d], kr[d], s);
          s *= scale;
          if (cap > 0.f) s = cap * tanhf(s * inv_cap);
          if (r1) s -= pen1[i] * log1pf(pen2[i] * (float)(pos - (base + lane)));
          s = valid ? s : -INFINITY;
          float m_new, c, p;
          if (head_bias) {   // no softmax: the weight is the sigmoid of the score itself
            m_new = 0.f;
            c = m_run[i] == 0.f ? 1.f : 0.f;
            p = valid ? 1.0f / (1.0f + expf(-(s + hb[i]))) : 0.f;
          } else {
            m_new = fmaxf(m_run[i], warp_max(s));
            c = expf(m_run[i] - m_new);  // exp(-inf) = 0 on the first tile
            p = valid ? expf(s - m_new) : 0.f;
          }
          p_s[g * KT + lane] = p;
          float tile_sum = 0.f;  // keys in order, the same in every lane
          for (int j = 0; j < KT; ++j) tile_sum += __shfl_sync(0xffffffffu, p, j);
          l_run[i] = l_run[i] * c + tile_sum;
          m_run[i] = m_new;
          if (lane == 0) { corr_s[g] = c; l_s[g] = l_run[i]; m_s[g] = m_new; }
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < dv) {
#pragma unroll
          for (int g = 0; g < GC; ++g) {
            if (g < gcount) {
              float a = acc[g][i] * corr_s[g];
              const float* pr = p_s + g * KT;
              for (int j = 0; j < KT; ++j) a = fmaf(pr[j], v_s[j * dv + d], a);
              acc[g][i] = a;
            }
          }
        }
      }
    }
    __syncthreads();   // m_s and l_s of the chunk's last tile
    if (SPLIT) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        if (g < gcount) {
          float* dst = partials + ((((size_t)t * n_q + first_head + g) * n_values + value_slot) * max_chunks + chunk) * (dv + 2);
#pragma unroll
          for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * THREADS;
            if (d < dv) dst[d] = acc[g][i];
          }
          if (tid == 0) { dst[dv] = m_s[g]; dst[dv + 1] = l_s[g]; }
        }
      }
      return;
    }
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g < gcount) {
        float wa, wb;
        merge_parts(M[g], L[g], m_s[g], l_s[g], wa, wb);
#pragma unroll
        for (int i = 0; i < DPT; ++i) total[g][i] = fmaf(acc[g][i], wb, total[g][i] * wa);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    if (g < gcount) {
      float l = L[g];
      const float w = sink ? add_sink(M[g], l, sink[first_head + g]) : 1.f;
      if (head_bias) l = 1.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < dv)
          out[(((size_t)t * n_q + first_head + g) * n_values + value_slot) * dv + d] = from_f32<TO>(total[g][i] * w / l);
      }
    }
  }
}

// The chunks of a row, head and value slot, left by the SPLIT kernel, merged in order: grid (tokens, n_q * n_values).
template <typename TO>
__global__ void __launch_bounds__(MAX_D)
attention_scored_merge_kernel(const float* __restrict__ partials, TO* __restrict__ out,
                              const int* __restrict__ segment_of_token, const int* __restrict__ positions,
                              const float* __restrict__ sink, int n_values, int dv, int max_chunks, int num_segments,
                              int window, int unnormalised) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, item = blockIdx.y, d = threadIdx.x;
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0 || d >= dv) return;
  const int pos = positions[t];
  const float* src = partials + ((size_t)t * gridDim.y + item) * max_chunks * (dv + 2);
  float total = 0.f, M = -INFINITY, L = 0.f;
  const int first_chunk = window > 0 ? max(0, pos + 1 - window) / CHUNK : 0;
  for (int chunk = first_chunk; chunk <= pos / CHUNK; ++chunk) {
    const float* part = src + (size_t)chunk * (dv + 2);
    float wa, wb;
    merge_parts(M, L, part[dv], part[dv + 1], wa, wb);
    total = fmaf(part[d], wb, total * wa);
  }
  const float w = sink ? add_sink(M, L, sink[item / n_values]) : 1.f;
  if (unnormalised) L = 1.f;
  out[((size_t)t * gridDim.y + item) * dv + d] = from_f32<TO>(total * w / L);
}

// out[t, h, d] = gate * sum_g mix[h, g] * wide[t, g, slot(h), d], with slot(h) = h / (n_q / n_kv) when the wide rows hold
// a value slot per key/value head (n_values > 1), else wide[t, h, 0, d] (mix null: the identity);
// gate = sigmoid(sum_p gate_proj[p][t, column] + gate_bias[column]) (gate_proj null: 1).
template <typename T> __device__ __forceinline__ void scored_load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void scored_load4<float>(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void scored_load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T> __device__ __forceinline__ void scored_store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void scored_store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void scored_store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

// TW: the type of `wide` (float32, or bfloat16 from a kernel that writes its outputs rounded; then the rows are staged).
template <typename TI, typename TO, typename TW>
__global__ void head_mix_gate_kernel(const TW* __restrict__ wide, const float* __restrict__ mix,
                                     const TI* __restrict__ gate_proj, int n_partials, long long partial_stride,
                                     long long ld, const float* __restrict__ gate_bias,
                                     const int* __restrict__ segment_of_token, TO* __restrict__ out, int n_q, int n_kv,
                                     int n_values, int dv, int staged, int by_four) {
  extern __shared__ __align__(16) float mix_smem[];   // staged: the token's rows of `wide`, then the mixing table
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (segment_of_token[t] < 0) return;
  const int width = n_q * dv;
  const int row_floats = n_q * n_values * dv;
  const float* rows = sizeof(TW) == 4 ? reinterpret_cast<const float*>(wide) + (size_t)t * row_floats : nullptr;
  const float* table = mix;
  if (staged) {   // every output reads n_q of the rows: fetched once, four values a load, all loads of a thread in flight
    const TW* src = wide + (size_t)t * row_floats;
    float4* dst = reinterpret_cast<float4*>(mix_smem);
    const int pieces = row_floats / 4;
    for (int base = threadIdx.x; base < pieces; base += 4 * blockDim.x) {
      float v[4][4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (base + k * blockDim.x < pieces) scored_load4<TW>(src + 4 * (size_t)(base + k * blockDim.x), v[k]);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (base + k * blockDim.x < pieces) dst[base + k * blockDim.x] = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
    }
    if (mix) {
      float* held = mix_smem + row_floats;
      for (int e = threadIdx.x; e < n_q * n_q; e += blockDim.x) held[e] = mix[e];
      table = held;
    }
    __syncthreads();
    rows = mix_smem;
  }
  const int group = n_q / n_kv;
  if (by_four) {   // four columns of one head a thread: vector loads and stores, the index arithmetic once for four
    for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
      const int h = e / dv, d = e % dv;
      const int slot = n_values > 1 ? h / group : 0;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      if (mix) {
        for (int g = 0; g < n_q; ++g) {
          const float m = table[h * n_q + g];
          const float4 r = *reinterpret_cast<const float4*>(rows + ((size_t)g * n_values + slot) * dv + d);
          sum[0] = fmaf(m, r.x, sum[0]); sum[1] = fmaf(m, r.y, sum[1]);
          sum[2] = fmaf(m, r.z, sum[2]); sum[3] = fmaf(m, r.w, sum[3]);
        }
      } else {
        const float4 r = *reinterpret_cast<const float4*>(rows + ((size_t)h * n_values + slot) * dv + d);
        sum[0] = r.x; sum[1] = r.y; sum[2] = r.z; sum[3] = r.w;
      }
      if (gate_proj) {
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < n_partials; ++p) {
          float a[4];
          scored_load4<TI>(gate_proj + (size_t)p * partial_stride + (size_t)t * ld + e, a);
#pragma unroll
          for (int k = 0; k < 4; ++k) z[k] += a[k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (gate_bias) z[k] += gate_bias[e + k];
          sum[k] *= 1.0f / (1.0f + expf(-z[k]));
        }
      }
      scored_store4<TO>(out + (size_t)t * width + e, sum);
    }
    return;
  }
  for (int e = threadIdx.x; e < width; e += blockDim.x) {
    const int h = e / dv, d = e % dv;
    const int slot = n_values > 1 ? h / group : 0;
    float sum;
    if (mix) {
      sum = 0.f;
      for (int g = 0; g < n_q; ++g) sum = fmaf(table[h * n_q + g], rows[((size_t)g * n_values + slot) * dv + d], sum);
    } else {
      sum = rows[((size_t)h * n_values + slot) * dv + d];
    }
    if (gate_proj) {
      float z = 0.f;
      for (int p = 0; p < n_partials; ++p) z += to_f32<TI>(gate_proj[(size_t)p * partial_stride + (size_t)t * ld + e]);
      if (gate_bias) z += gate_bias[e];
      sum *= 1.0f / (1.0f + expf(-z));
    }
    out[(size_t)t * width + e] = from_f32<TO>(sum);
  }
}

size_t scored_smem_bytes(int dk, int dv) {
  return sizeof(float) * ((size_t)GC * dk + (size_t)KT * (dk + 1) + (size_t)KT * dv + GC * KT + 3 * GC) +
         sizeof(int) * KT + 16;
}

template <typename T, typename TO>
int launch_scored(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_tables,
                  int bt_stride, const int* segment_of_token, const int* positions, const float* r1, const float* r2,
                  const float* sink, int tokens, int n_q, int n_kv, int dk, int dv, int n_values, int page_size,
                  float scale, int num_pages, int num_segments, float* partials, int max_chunks, int window, float cap,
                  const float* head_bias, cudaStream_t stream) {
  const int group = n_q / n_kv;
  const int gchunks = (group + GC - 1) / GC;
  const bool split = partials != nullptr;
  const size_t smem = scored_smem_bytes(dk, dv);
  static bool configured = false;   // the largest head sizes once per instantiation (not repeated while a stream is captured)
  if (!configured) {
    const int most = (int)scored_smem_bytes(MAX_D, MAX_D);
    cudaError_t err = cudaFuncSetAttribute(attention_scored_kernel<T, TO, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(attention_scored_kernel<T, TO, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const dim3 grid(tokens, n_kv, (split ? max_chunks : 1) * n_values * gchunks);
  if (split) {
    lse_launch(attention_scored_kernel<T, TO, true>, grid, THREADS, smem, stream, (const T*)q, (const T*)k_cache,
               (const T*)v_cache, (TO*)out, block_tables, bt_stride, segment_of_token, positions, r1, r2, sink, n_q, n_kv,
               dk, dv, n_values, page_size, scale, num_pages, num_segments, partials, max_chunks, window, cap, head_bias);
    lse_launch(attention_scored_merge_kernel<TO>, dim3(tokens, n_q * n_values), ((dv + 31) / 32) * 32, 0, stream,
               (const float*)partials, (TO*)out, segment_of_token, positions, sink, n_values, dv, max_chunks,
               num_segments, window, (int)(head_bias != nullptr));
  } else {
    lse_launch(attention_scored_kernel<T, TO, false>, grid, THREADS, smem, stream, (const T*)q, (const T*)k_cache,
               (const T*)v_cache, (TO*)out, block_tables, bt_stride, segment_of_token, positions, r1, r2, sink, n_q, n_kv,
               dk, dv, n_values, page_size, scale, num_pages, num_segments, (float*)nullptr, 0, window, cap, head_bias);
  }
  return (int)cudaGetLastError();
}
}  // namespace

extern "C" int lse_attention_scored_chunk(void) { return CHUNK; }

// q [T, n_q, dk]; out [T, n_q, n_values, dv] in the cache's dtype (out_f32 = 0) or float32 (out_f32 = 1);
// cross != 0: n_values = n_kv (see the top of the file), else 1.  r1/r2 (together) and sink: float32 [n_q] or null.
// partials != null: every chunk of a row gets a block of its own; it holds tokens * n_q * n_values * max_chunks *
// (dv + 2) floats, and max_chunks chunks cover the longest context that the block tables can describe.
// window > 0: a row reads its last `window` keys only; cap > 0: scores capped by cap * tanh(s / cap); head_bias (float32
// [n_q] or null): weights sigmoid(s + head_bias_h) without a softmax (no sink then).
extern "C" int lse_attention_scored_windowed(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                             int out_f32, const int* block_tables, int bt_stride,
                                             const int* segment_of_token, const int* positions, const float* r1,
                                             const float* r2, const float* sink, int tokens, int n_q, int n_kv, int dk,
                                             int dv, int cross, int page_size, float scale, int num_pages,
                                             int num_segments, float* partials, int max_chunks, int window, float cap,
                                             const float* head_bias, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_bias && sink) return LSE_ERR_BAD_ARGUMENT;
  if (dk <= 0 || dk > MAX_D || dv <= 0 || dv > MAX_D || n_kv <= 0 || n_q % n_kv || page_size <= 0 || (!r1) != (!r2))
    return LSE_ERR_BAD_ARGUMENT;
  const int n_values = cross ? n_kv : 1;
  const int gchunks = (n_q / n_kv + GC - 1) / GC;
  if (partials && (max_chunks <= 0 || (long long)max_chunks * CHUNK < (long long)bt_stride * page_size))
    return LSE_ERR_BAD_ARGUMENT;
  if ((long long)(partials ? max_chunks : 1) * n_values * gchunks > 65535 || n_kv > 65535 || n_q * n_values > 65535)
    return LSE_ERR_TOO_LARGE;
#define LSE_SCORED_ARGS q, k_cache, v_cache, out, block_tables, bt_stride, segment_of_token, positions, r1, r2, sink, tokens, \
  n_q, n_kv, dk, dv, n_values, page_size, scale, num_pages, num_segments, partials, max_chunks, window, cap, head_bias, stream
  if (dtype == LSE_DTYPE_F32) return launch_scored<float, float>(LSE_SCORED_ARGS);
  if (dtype == LSE_DTYPE_BF16 && out_f32) return launch_scored<__nv_bfloat16, float>(LSE_SCORED_ARGS);
  if (dtype == LSE_DTYPE_BF16) return launch_scored<__nv_bfloat16, __nv_bfloat16>(LSE_SCORED_ARGS);
#undef LSE_SCORED_ARGS
  return LSE_ERR_BAD_ARGUMENT;
}

extern "C" int lse_attention_scored(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                    int out_f32, const int* block_tables, int bt_stride, const int* segment_of_token,
                                    const int* positions, const float* r1, const float* r2, const float* sink,
                                    int tokens, int n_q, int n_kv, int dk, int dv, int cross, int page_size, float scale,
                                    int num_pages, int num_segments, float* partials, int max_chunks,
                                    cudaStream_t stream) {
  return lse_attention_scored_windowed(q, k_cache, v_cache, out, dtype, out_f32, block_tables, bt_stride, segment_of_token,
                                       positions, r1, r2, sink, tokens, n_q, n_kv, dk, dv, cross, page_size, scale,
                                       num_pages, num_segments, partials, max_chunks, 0, 0.f, nullptr, stream);
}

// The second half of a launch with partials, for kernels of other files that leave partials in the same layout
// ([t][head][value slot][chunk][dv + 2]: sums, maximum, total): out [T, n_q, n_values, dv] in bfloat16 or float32.
// window, unnormalised: as the launch that left the partials had them (chunks before the window hold nothing).
extern "C" int lse_attention_scored_merge_windowed(const float* partials, void* out, int out_dtype,
                                                   const int* segment_of_token, const int* positions, const float* sink,
                                                   int tokens, int n_q, int n_values, int dv, int max_chunks,
                                                   int num_segments, int window, int unnormalised, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dv <= 0 || dv > MAX_D || n_q * n_values > 65535 || max_chunks <= 0) return LSE_ERR_BAD_ARGUMENT;
  const dim3 grid(tokens, n_q * n_values);
  const int threads = ((dv + 31) / 32) * 32;
  if (out_dtype == LSE_DTYPE_F32)
    lse_launch(attention_scored_merge_kernel<float>, grid, threads, 0, stream, partials, (float*)out, segment_of_token,
               positions, sink, n_values, dv, max_chunks, num_segments, window, unnormalised);
  else if (out_dtype == LSE_DTYPE_BF16)
    lse_launch(attention_scored_merge_kernel<__nv_bfloat16>, grid, threads, 0, stream, partials, (__nv_bfloat16*)out,
               segment_of_token, positions, sink, n_values, dv, max_chunks, num_segments, window, unnormalised);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_attention_scored_merge(const float* partials, void* out, int out_dtype, const int* segment_of_token,
                                          const int* positions, const float* sink, int tokens, int n_q, int n_values,
                                          int dv, int max_chunks, int num_segments, cudaStream_t stream) {
  return lse_attention_scored_merge_windowed(partials, out, out_dtype, segment_of_token, positions, sink, tokens, n_q,
                                             n_values, dv, max_chunks, num_segments, 0, 0, stream);
}

// wide [T, n_q, n_values, dv] (n_values = n_kv when cross, else 1) in float32, or in bfloat16 (wide_bf16; only shapes
// whose rows fit the kernel's shared memory, see lse_head_mix_gate_stages); mix float32 [n_q, n_q] or null;
// gate_proj [T, ld] (columns from the pointer on) or a float32 stack of partial sums, or null; out [T, n_q * dv].
constexpr size_t MIX_STAGE_BYTES = 160 * 1024;   // most shared memory that the mixing kernel stages a token's rows in

extern "C" int lse_head_mix_gate_stages(int n_q, int n_values, int dv) {
  return sizeof(float) * ((size_t)n_q * n_values * dv + (size_t)n_q * n_q) <= MIX_STAGE_BYTES && (n_q * n_values * dv) % 4 == 0;
}

extern "C" int lse_head_mix_gate(const void* wide, int wide_bf16, const float* mix, const void* gate_proj, int gate_dtype,
                                 int n_partials, long long partial_stride, long long ld, const float* gate_bias,
                                 const int* segment_of_token, void* out, int out_dtype, int tokens, int n_q, int n_kv,
                                 int cross, int dv, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || dv <= 0 || (gate_proj && n_partials < 1)) return LSE_ERR_BAD_ARGUMENT;
  const int n_values = cross ? n_kv : 1;
  const int threads = n_q * dv >= 1024 ? 256 : 128;
  const size_t row_bytes = sizeof(float) * ((size_t)n_q * n_values * dv + (size_t)n_q * n_q);
  const int staged = (mix != nullptr || wide_bf16) && lse_head_mix_gate_stages(n_q, n_values, dv) && (((uintptr_t)wide) & 15) == 0;
  if (wide_bf16 && !staged) return LSE_ERR_BAD_ARGUMENT;
  const int gate_bytes = gate_dtype == LSE_DTYPE_F32 ? 4 : 2;
  const int by_four = dv % 4 == 0 && (((uintptr_t)wide | (uintptr_t)out) & 15) == 0 &&
                      (!gate_proj || ((((uintptr_t)gate_proj) & (4 * gate_bytes - 1)) == 0 && ld % 4 == 0 && partial_stride % 4 == 0));
#define LSE_MIX_CONFIGURE(kernel)                                                                                   \
  {                                                                                                                 \
    static bool configured = false;   /* once per instantiation, never while a stream is captured (a first run comes first) */ \
    if (!configured && staged && row_bytes > 48 * 1024) {                                                           \
      const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MIX_STAGE_BYTES); \
      if (err != cudaSuccess) return (int)err;                                                                      \
      configured = true;                                                                                            \
    }                                                                                                               \
  }
#define LSE_MIX_CASE(TI, TO)                                                                                        \
  LSE_MIX_CONFIGURE((head_mix_gate_kernel<TI, TO, __nv_bfloat16>))                                                  \
  LSE_MIX_CONFIGURE((head_mix_gate_kernel<TI, TO, float>))                                                          \
  if (wide_bf16)                                                                                                    \
    lse_launch(head_mix_gate_kernel<TI, TO, __nv_bfloat16>, tokens, threads, row_bytes, stream,                     \
               (const __nv_bfloat16*)wide, mix, (const TI*)gate_proj, n_partials, partial_stride, ld, gate_bias,     \
               segment_of_token, (TO*)out, n_q, n_kv, n_values, dv, staged, by_four);                               \
  else                                                                                                              \
    lse_launch(head_mix_gate_kernel<TI, TO, float>, tokens, threads, staged ? row_bytes : 0, stream,                \
               (const float*)wide, mix, (const TI*)gate_proj, n_partials, partial_stride, ld, gate_bias,            \
               segment_of_token, (TO*)out, n_q, n_kv, n_values, dv, staged, by_four)
  if (gate_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) { LSE_MIX_CASE(float, float); }
  else if (gate_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) { LSE_MIX_CASE(__nv_bfloat16, __nv_bfloat16); }
  else if (gate_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) { LSE_MIX_CASE(float, __nv_bfloat16); }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_MIX_CASE
#undef LSE_MIX_CONFIGURE
  LSE_LAUNCH_CHECK();
}
