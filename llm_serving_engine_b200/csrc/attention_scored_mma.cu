// The attention of attention_scored.cu (distance penalty, sink, values of every group) on the tensor cores, for
// bfloat16 and head sizes that are multiples of 16 (keys and values of one size: 32, 48, 64, 96 or 128).
//
// One block = (tile of consecutive rows of one request, key head, value slot[, chunk of keys]).  The 64 rows of its
// score matrix are (row, query head of the group) pairs, so the keys of a key head are loaded once for all its query
// heads; keys are walked in tiles of 64 through a two-stage cp.async pipeline; causal inside the portion, all of the
// earlier context before it.  Scores (mma.sync m16n8k16, float32 accumulators), the penalty, the softmax statistics
// and the output sums are float32; the probabilities are rounded to bfloat16 for the second product.  Everything is
// kept in base two: s2 = q . k * scale * log2(e) - r1 * log2(1 + r2 * (i - j)).  The penalty depends on the head and
// the distance only, and a tile of 64 keys and a few rows has few distances: the block works them out once a tile into
// a small table (a logarithm per table entry instead of one per score).
//
// window > 0: a row reads its last `window` keys only; key tiles before the window of the tile's first row are not
// walked, and keys before it are not fetched (their pages may have been given back).  cap > 0: scores are capped by
// cap * tanh(s / cap).  head_bias: no softmax, a key's weight is sigmoid(s + head_bias_h) and the sums are not divided.
//
// With `partials` the keys of a tile of rows are cut into chunks of 256 (counted from key 0) with a block each, which
// leaves (sums, max, total) per row, head, value slot and chunk in the layout of attention_scored.cu; that file's
// merge kernel adds them up (and the sink).  This is how single decoded tokens and small portions fill the GPU.
// Shared-memory tiles are padded by 16 bytes a row (an odd number of 16-byte chunks), which keeps ldmatrix free of bank
// conflicts for every head size.
#include "common.cuh"
#include "mma_common.cuh"

LSE_CHECK_DEFINE(lse_check_attention_scored_mma)

namespace {
constexpr int BM = 64;          // (row, head-of-group) pairs per block
constexpr int BN = 64;          // keys per tile
constexpr int CHUNK = 256;      // keys per chunk when the keys are split (attention_scored.cu's)
constexpr int TABLE_STAGE = 1024;   // block-table entries a block keeps in shared memory

template <int D> __device__ __forceinline__ uint32_t padded_off(int r, int c) { return (uint32_t)(r * (D * 2 + 16) + (c << 4)); }
template <int D> constexpr int tile_bytes(int rows) { return rows * (D * 2 + 16); }

template <int DK, int DV>
__global__ void __launch_bounds__(128)
attention_scored_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                            const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ out_f32, float* __restrict__ partials,
                            const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ segment_start,
                            const int* __restrict__ segment_first_pos, int num_segments, const float* __restrict__ r1,
                            const float* __restrict__ r2, const float* __restrict__ sink, int n_q, int n_kv,
                            int n_values, int page_size, float scale_log2e, int rows_per_tile, int num_pages,
                            int max_chunks, int window, float cap, const float* __restrict__ head_bias) {
  constexpr int CHK = DK / 8, CHV = DV / 8;
  constexpr int K_BYTES = tile_bytes<DK>(BN), V_BYTES = tile_bytes<DV>(BN);
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                               // [64][DK]
  unsigned char* kv_s = smem + tile_bytes<DK>(BM);         // [2 stages][K [64][DK] | V [64][DV]]
  // the penalty of this tile's distances, a row per head of the group: entry x of head g is the penalty at distance
  // x + (position of the tile's first row - the tile's last key); a tile of 64 keys and a few rows has few distances
  float* pen_s = reinterpret_cast<float*>(kv_s + 2 * (K_BYTES + V_BYTES));
  __shared__ int bt_s[TABLE_STAGE];
  __shared__ int tile_slot[3];
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.y;
  const int group = n_q / n_kv;
  const int splits = partials ? max_chunks : 1;
  const int chunk = blockIdx.z % splits;
  const int value_slot = blockIdx.z / splits;
  const int value_head = n_values > 1 ? value_slot : kvh;

  int seg, r0, cnt;
  lse_find_tile(segment_start, num_segments, rows_per_tile, 0, blockIdx.x, tile_slot, seg, r0, cnt);
  if (seg < 0) return;
  const int nrows = min(rows_per_tile, cnt - r0);
  const int row_base = segment_start[seg] + r0;
  const int pos0 = segment_first_pos[seg] + r0;
  const int last_pos = pos0 + nrows - 1;
  const int first_key = window > 0 ? max(0, pos0 + 1 - window) : 0;   // the first key that any row of the tile reads
  int tile_lo = first_key / BN, tile_hi = (last_pos + BN) / BN;         // key tiles [tile_lo, tile_hi)
  if (partials) {
    if (chunk * CHUNK > last_pos || (chunk + 1) * CHUNK <= first_key) return;
    tile_lo = max(tile_lo, chunk * (CHUNK / BN));
    tile_hi = min(tile_hi, (chunk + 1) * (CHUNK / BN));
  }
  const int* bt = block_tables + (size_t)seg * bt_stride;
  const PageMath pm(page_size);
  const int n_pages = pm.page(last_pos) + 1;
  const bool staged = n_pages <= TABLE_STAGE;
  if (staged)
    for (int i = tid; i < n_pages; i += 128)
      bt_s[i] = i < pm.page(first_key) ? 0 : LSE_CHECKED(bt[i], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
  pdl_wait();

  for (int e = tid; e < BM * CHK; e += 128) {
    const int m = e / CHK, c = e % CHK;
    const int rl = m / group, g = m % group;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rl < nrows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row_base + rl) * n_q + kvh * group + g) * DK + c * 8);
    *reinterpret_cast<uint4*>(q_s + padded_off<DK>(m, c)) = v;
  }

  const uint32_t kv_u32 = smem_u32(kv_s);
  // A 16-key piece of a tile never straddles pages when the page size is a multiple of 16: warp w then copies piece w
  // of the 64 keys with one look at the block table; else every 16-byte chunk finds its own page.
  const bool page_pieces = (page_size % 16) == 0 && staged;
  auto load_tile = [&](int kt, int stage) {
    const uint32_t k_dst = kv_u32 + (uint32_t)stage * (K_BYTES + V_BYTES), v_dst = k_dst + K_BYTES;
    if (page_pieces) {
      const int j0 = kt * BN + warp * 16;
      const int limit = (j0 <= last_pos && j0 + 15 >= first_key) ? last_pos + 1 - j0 : 0;   // keys of the piece that exist
      const int skip = first_key - j0;       // keys of the piece before the window: not fetched
      size_t k_base = 0, v_base = 0;
      if (limit > 0) {
        const size_t page = (size_t)bt_s[pm.page(j0)];
        k_base = ((page * n_kv + kvh) * page_size + pm.offset(j0)) * DK;
        v_base = ((page * n_kv + value_head) * page_size + pm.offset(j0)) * DV;
      }
#pragma unroll
      for (int i = 0; i < CHK / 2; ++i) {
        const int n = lane + 32 * i, row = n / CHK, c = n % CHK;
        const bool valid = row < limit && row >= skip;
        cp_async16(k_dst + padded_off<DK>(warp * 16 + row, c), kc + k_base + (valid ? row * DK + c * 8 : 0), valid);
      }
#pragma unroll
      for (int i = 0; i < CHV / 2; ++i) {
        const int n = lane + 32 * i, row = n / CHV, c = n % CHV;
        const bool valid = row < limit && row >= skip;
        cp_async16(v_dst + padded_off<DV>(warp * 16 + row, c), vc + v_base + (valid ? row * DV + c * 8 : 0), valid);
      }
      return;
    }
    for (int idx = tid; idx < BN * (CHK + CHV); idx += 128) {
      const bool is_key = idx < BN * CHK;
      const int local = is_key ? idx : idx - BN * CHK;
      const int key = is_key ? local / CHK : local / CHV, c = is_key ? local % CHK : local % CHV;
      const int j = kt * BN + key;
      const bool valid = j <= last_pos && j >= first_key;
      size_t slot = 0;
      if (valid) {
        const int logical = pm.page(j);
        const int page = staged ? bt_s[logical] : LSE_CHECKED(bt[logical], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
        slot = ((size_t)page * n_kv + (is_key ? kvh : value_head)) * page_size + pm.offset(j);
      }
      if (is_key) cp_async16(k_dst + padded_off<DK>(key, c), kc + slot * DK + c * 8, valid);
      else cp_async16(v_dst + padded_off<DV>(key, c), vc + slot * DV + c * 8, valid);
    }
  };
  __syncthreads();   // q_s and bt_s are filled
  load_tile(tile_lo, 0);
  cp_async_commit();

  uint32_t qf[DK / 16][4];
  {
    const int mi = lane >> 3, r = warp * 16 + (lane & 7) + (mi & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) ldmatrix_x4(qf[ks], smem_u32(q_s + padded_off<DK>(r, ks * 2 + (mi >> 1))));
  }
  // this thread's two rows of the score matrix: their request rows, heads, positions and constants
  const int ma = warp * 16 + (lane >> 2), mb = ma + 8;
  const int rla = ma / group, ga = ma % group, rlb = mb / group, gb = mb % group;
  const int pos_a = pos0 + min(rla, nrows - 1), pos_b = pos0 + min(rlb, nrows - 1);
  const int head_a = kvh * group + ga, head_b = kvh * group + gb;
  const bool penalised = r1 != nullptr;
  const bool unnormalised = head_bias != nullptr;
  const float bias_a = unnormalised ? head_bias[head_a] * LOG2E : 0.f, bias_b = unnormalised ? head_bias[head_b] * LOG2E : 0.f;
  const float cap2 = cap * LOG2E, two_over_cap = cap > 0.f ? 2.0f / cap : 0.f;     // the cap in base two, 2 / cap in natural units
  const float scale_natural = scale_log2e * (1.0f / LOG2E);
  const int pen_width = BN + rows_per_tile;
  const float* pen_a = pen_s + ga * pen_width + rla + (BN - 1);   // minus the key's place in the tile
  const float* pen_b = pen_s + gb * pen_width + rlb + (BN - 1);

  float acc[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int kt = tile_lo; kt < tile_hi; ++kt) {
    const int stage = (kt - tile_lo) & 1;
    if (kt + 1 < tile_hi) load_tile(kt + 1, stage ^ 1);
    cp_async_commit();
    if (penalised) {
      const int nearest = pos0 - (kt * BN + BN - 1);   // distance from the tile's first row to its last key
      for (int idx = tid; idx < group * pen_width; idx += 128) {
        const int g = idx / pen_width, distance = idx % pen_width + nearest;
        const int head = kvh * group + g;
        pen_s[idx] = distance > 0 ? r1[head] * __log2f(fmaf(r2[head], (float)distance, 1.0f)) : 0.f;
      }
    }
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t ks_ = kv_u32 + (uint32_t)stage * (K_BYTES + V_BYTES);
    const uint32_t vs_ = ks_ + K_BYTES;

    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi >> 1) * 8;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
        for (int nbp = 0; nbp < BN / 16; ++nbp) {
          uint32_t b[4];
          ldmatrix_x4(b, ks_ + padded_off<DK>(nbp * 16 + key, ks * 2 + (mi & 1)));
          mma_bf16(s[2 * nbp], qf[ks], b[0], b[1]);
          mma_bf16(s[2 * nbp + 1], qf[ks], b[2], b[3]);
        }
      }
    }
    const bool diagonal = (kt + 1) * BN - 1 > pos0;   // some row of the tile ends inside these keys
    const bool windowed = window > 0 && kt * BN <= last_pos - window;   // some row of the tile starts inside or behind them
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = nb * 8 + (lane & 3) * 2 + (e & 1);
        const int j = kt * BN + key;
        const int pos = (e >> 1) ? pos_b : pos_a;
        float v = s[nb][e] * scale_log2e;
        if (cap > 0.f) {    // cap * tanh(x / cap) = cap * (1 - 2 / (exp(2 x / cap) + 1)), x the natural score
          const float t = fast_exp2(s[nb][e] * scale_natural * two_over_cap * LOG2E);
          v = cap2 * (1.0f - __fdividef(2.0f, t + 1.0f));
        }
        if (penalised) v -= ((e >> 1) ? pen_b : pen_a)[-key];
        if (diagonal && j > pos) v = -INFINITY;
        if (windowed && j <= pos - window) v = -INFINITY;
        s[nb][e] = v;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // A row that sees no key of this chunk (its position lies before it) keeps max = -inf; it is never written, and
    // its registers are kept free of NaN by taking 0 for the maximum.
    if (unnormalised) {   // sigmoid(s + b) = 1 / (1 + 2^-(s2 + b2)); a masked key (-inf) weighs 0; nothing is rescaled
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb) {
        s[nb][0] = __fdividef(1.0f, 1.0f + fast_exp2(-(s[nb][0] + bias_a)));
        s[nb][1] = __fdividef(1.0f, 1.0f + fast_exp2(-(s[nb][1] + bias_a)));
        s[nb][2] = __fdividef(1.0f, 1.0f + fast_exp2(-(s[nb][2] + bias_b)));
        s[nb][3] = __fdividef(1.0f, 1.0f + fast_exp2(-(s[nb][3] + bias_b)));
      }
      m0 = m1 = 0.f;
      l0 = l1 = 0.25f;     // four lanes add theirs: the total that the merge reads is one, and is not used
    } else {
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    const float c0 = fast_exp2(m0 - base0), c1 = fast_exp2(m1 - base1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
      s[nb][0] = fast_exp2(s[nb][0] - base0); s[nb][1] = fast_exp2(s[nb][1] - base0);
      s[nb][2] = fast_exp2(s[nb][2] - base1); s[nb][3] = fast_exp2(s[nb][3] - base1);
      sum0 += s[nb][0] + s[nb][1];
      sum1 += s[nb][2] + s[nb][3];
    }
    l0 = l0 * c0 + sum0;
    l1 = l1 * c1 + sum1;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { acc[i][0] *= c0; acc[i][1] *= c0; acc[i][2] *= c1; acc[i][3] *= c1; }
    }
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi & 1) * 8;
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                          pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int nbp = 0; nbp < DV / 16; ++nbp) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vs_ + padded_off<DV>(kk * 16 + key, nbp * 2 + (mi >> 1)));
          mma_bf16(acc[2 * nbp], pa, b[0], b[1]);
          mma_bf16(acc[2 * nbp + 1], pa, b[2], b[3]);
        }
      }
    }
    __syncthreads();   // the stage is free for the load after next
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  if (partials) {   // unnormalised sums, the maximum in natural units, the total: for the merge kernel
    constexpr float LN2 = 0.6931471805599453f;
    const bool write_a = rla < nrows && chunk * CHUNK <= pos_a && (window <= 0 || (chunk + 1) * CHUNK > pos_a + 1 - window);
    const bool write_b = rlb < nrows && chunk * CHUNK <= pos_b && (window <= 0 || (chunk + 1) * CHUNK > pos_b + 1 - window);
    float* dst_a = partials + ((((size_t)(row_base + rla) * n_q + head_a) * n_values + value_slot) * max_chunks + chunk) * (DV + 2);
    float* dst_b = partials + ((((size_t)(row_base + rlb) * n_q + head_b) * n_values + value_slot) * max_chunks + chunk) * (DV + 2);
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      if (write_a) { dst_a[d] = acc[i][0]; dst_a[d + 1] = acc[i][1]; }
      if (write_b) { dst_b[d] = acc[i][2]; dst_b[d + 1] = acc[i][3]; }
    }
    if ((lane & 3) == 0) {
      if (write_a) { dst_a[DV] = m0 * LN2; dst_a[DV + 1] = l0; }
      if (write_b) { dst_b[DV] = m1 * LN2; dst_b[DV + 1] = l1; }
    }
    return;
  }
  float w0 = 1.f, w1 = 1.f;
  if (sink) {   // exp(sink) joins the total; the sums are rescaled when the sink is the new maximum
    const float sa = sink[head_a] * LOG2E, sb = sink[head_b] * LOG2E;
    const float na = fmaxf(m0, sa), nb = fmaxf(m1, sb);
    w0 = fast_exp2(m0 - na); w1 = fast_exp2(m1 - nb);
    l0 = l0 * w0 + fast_exp2(sa - na);
    l1 = l1 * w1 + fast_exp2(sb - nb);
  }
  const float inv0 = unnormalised ? 1.f : w0 / l0, inv1 = unnormalised ? 1.f : w1 / l1;
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) {
    const int d = i * 8 + (lane & 3) * 2;
    if (rla < nrows) {
      const size_t at = (((size_t)(row_base + rla) * n_q + head_a) * n_values + value_slot) * DV + d;
      if (out_f32) { out_f32[at] = acc[i][0] * inv0; out_f32[at + 1] = acc[i][1] * inv0; }
      else *reinterpret_cast<__nv_bfloat162*>(out + at) = __floats2bfloat162_rn(acc[i][0] * inv0, acc[i][1] * inv0);
    }
    if (rlb < nrows) {
      const size_t at = (((size_t)(row_base + rlb) * n_q + head_b) * n_values + value_slot) * DV + d;
      if (out_f32) { out_f32[at] = acc[i][2] * inv1; out_f32[at + 1] = acc[i][3] * inv1; }
      else *reinterpret_cast<__nv_bfloat162*>(out + at) = __floats2bfloat162_rn(acc[i][2] * inv1, acc[i][3] * inv1);
    }
  }
}

template <int D>
int launch_scored_mma(const void* q, const void* kc, const void* vc, void* out, int out_is_f32, float* partials,
                      const int* block_tables, int bt_stride, const int* segment_start, const int* segment_first_pos,
                      int num_segments, const float* r1, const float* r2, const float* sink, int tokens, int n_q, int n_kv,
                      int n_values, int page_size, float scale, int num_pages, int max_chunks, int window, float cap,
                      const float* head_bias, cudaStream_t stream) {
  const int group = n_q / n_kv;
  const int rows_per_tile = BM / group;
  const size_t tiles_bytes = (size_t)tile_bytes<D>(BM) + 2 * (size_t)(tile_bytes<D>(BN) + tile_bytes<D>(BN));
  const size_t smem = tiles_bytes + sizeof(float) * (size_t)group * (BN + rows_per_tile);
  static bool configured = false;
  if (!configured) {   // room for the largest penalty table (64 heads a group) once
    cudaError_t err = cudaFuncSetAttribute(attention_scored_mma_kernel<D, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(tiles_bytes + sizeof(float) * BM * (BN + 1)));
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int tiles = (tokens + rows_per_tile - 1) / rows_per_tile + num_segments;   // every request may end with a partial tile
  const long long depth = (long long)n_values * (partials ? max_chunks : 1);
  if (depth > 65535 || n_kv > 65535) return LSE_ERR_TOO_LARGE;
  dim3 grid(tiles, n_kv, (unsigned)depth);
  lse_launch(attention_scored_mma_kernel<D, D>, grid, 128, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
             (const __nv_bfloat16*)vc, out_is_f32 ? (__nv_bfloat16*)nullptr : (__nv_bfloat16*)out,
             out_is_f32 ? (float*)out : (float*)nullptr, partials, block_tables, bt_stride, segment_start, segment_first_pos,
             num_segments, r1, r2, sink, n_q, n_kv, n_values, page_size, scale * LOG2E, rows_per_tile, num_pages, max_chunks,
             window, cap, head_bias);
  return (int)cudaGetLastError();
}
}  // namespace

// Whether the tensor-core kernel takes this shape (else the caller uses the general kernel).
extern "C" int lse_attention_scored_mma_supported(int dk, int dv, int n_q, int n_kv) {
  if (dk != dv || (dk != 32 && dk != 48 && dk != 64 && dk != 96 && dk != 128)) return 0;
  if (n_kv <= 0 || n_q % n_kv) return 0;
  return (n_q / n_kv) <= BM ? 1 : 0;
}

// The arguments of lse_attention_scored, with the step's rows described by segments (segment_start int32 [S + 1],
// segment_first_pos int32 [S]) instead of row by row.  Without `partials` the result goes to `out` (bfloat16, or
// float32 when out_f32); with them the caller runs lse_attention_scored_merge afterwards.
extern "C" int lse_attention_scored_mma_windowed(const void* q, const void* k_cache, const void* v_cache, void* out,
                                                 int out_f32, const int* block_tables, int bt_stride,
                                                 const int* segment_start, const int* segment_first_pos, int num_segments,
                                                 const float* r1, const float* r2, const float* sink, int tokens, int n_q,
                                                 int n_kv, int dk, int dv, int cross, int page_size, float scale,
                                                 int num_pages, float* partials, int max_chunks, int window, float cap,
                                                 const float* head_bias, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_bias && sink) return LSE_ERR_BAD_ARGUMENT;
  if (!lse_attention_scored_mma_supported(dk, dv, n_q, n_kv) || page_size <= 0 || (!r1) != (!r2)) return LSE_ERR_BAD_ARGUMENT;
  if (partials && (max_chunks <= 0 || (long long)max_chunks * CHUNK < (long long)bt_stride * page_size))
    return LSE_ERR_BAD_ARGUMENT;
  const int n_values = cross ? n_kv : 1;
#define LSE_SCORED_MMA_ARGS q, k_cache, v_cache, out, out_f32, partials, block_tables, bt_stride, segment_start, \
  segment_first_pos, num_segments, r1, r2, sink, tokens, n_q, n_kv, n_values, page_size, scale, num_pages, max_chunks, \
  window, cap, head_bias, stream
  switch (dk) {
    case 32: return launch_scored_mma<32>(LSE_SCORED_MMA_ARGS);
    case 48: return launch_scored_mma<48>(LSE_SCORED_MMA_ARGS);
    case 64: return launch_scored_mma<64>(LSE_SCORED_MMA_ARGS);
    case 96: return launch_scored_mma<96>(LSE_SCORED_MMA_ARGS);
    default: return launch_scored_mma<128>(LSE_SCORED_MMA_ARGS);
  }
#undef LSE_SCORED_MMA_ARGS
}

extern "C" int lse_attention_scored_mma(const void* q, const void* k_cache, const void* v_cache, void* out, int out_f32,
                                        const int* block_tables, int bt_stride, const int* segment_start,
                                        const int* segment_first_pos, int num_segments, const float* r1, const float* r2,
                                        const float* sink, int tokens, int n_q, int n_kv, int dk, int dv, int cross,
                                        int page_size, float scale, int num_pages, float* partials, int max_chunks,
                                        cudaStream_t stream) {
  return lse_attention_scored_mma_windowed(q, k_cache, v_cache, out, out_f32, block_tables, bt_stride, segment_start,
                                           segment_first_pos, num_segments, r1, r2, sink, tokens, n_q, n_kv, dk, dv, cross,
                                           page_size, scale, num_pages, partials, max_chunks, 0, 0.f, nullptr, stream);
}
