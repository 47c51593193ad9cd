// The matrix-memory scan shared by linear_attention.cu (one decay per head), linear_attention_gated.cu (a keep and a
// take factor per token and head) and linear_attention_vector.cu (a keep factor per token, head and key channel): each
// file builds the forms of one mode.  The including file defines its LSE_CHECK_DEFINE reader first.
#pragma once
namespace {
constexpr int LA_THREADS = 128;
constexpr int LA_DPT = 32;       // rows of the state that a thread keeps

template <typename TD>
__device__ __forceinline__ float la_load(const TD* p, int n_partials, long long partial_stride) {
  float v = 0.f;
  for (int i = 0; i < n_partials; ++i) v += to_f32<TD>(p[(size_t)i * partial_stride]);
  return v;
}
__device__ __forceinline__ float la_act(float z, int act) { return act == 1 ? z / (1.f + expf(-z)) : z; }

// proj: rows of `ld` values; q of head h at q_off + h * dim, k at k_off + h * dim, v at v_off + h * vdim.
// PARTS threads share a column (PARTS * 32 >= dim), CW = 32 / PARTS columns a warp, 4 * CW a block.
//
// A block's work item is a run of consecutive rows of one request:
//   chunk_rows == 0: all rows of request blockIdx.x, from and into the request's state slot (few rows, decoding);
//   chunk_rows  > 0: the rows of every request are cut into chunks of chunk_rows rows, numbered request by request,
//     and blockIdx.x is a chunk.  phase 1: from a zero state, no outputs, the chunk's own state goes to
//     chunk_state[chunk].  phase 2: from chunk_state[chunk] (which linear_attention_carry_kernel has turned into the
//     state at the chunk's start), outputs written, the state is not stored.
// Chunks are what lets a long prompt use the whole GPU: a request's rows are walked in order only within a chunk.
// OUTPUTS false: the pass that only builds a chunk's own state (phase 1) leaves the output's half of the work out.
//
// GATED: the decay and the weight of the new outer product are numbers per token and head instead of one decay per head,
//     S_t = keep[t, h] * S_(t-1) + take[t, h] * k_t v_t^T,
// and the state has one more column, whose "value" is one for every token: it carries n_t = keep n_(t-1) + take k_t, so
// that the output's last column is n_t . q_t (the normaliser of a gated matrix memory).  State and output rows then hold
// vdim + 1 columns a head (norm_col; without it the state has vdim columns, as for a state-space scan whose decay and
// step size are numbers per token and head).  q is multiplied by q_scale in every form.
//
// MODE 2: the decay is a vector per token and head, one factor per row of the state (per key channel),
//     S_t = diag(keep[t, h, :]) S_(t-1) + k_t v_t^T,      token_keep float32 [tokens, heads * dim].
//
// qk_share: this many neighbouring heads read the same q and k columns (head h reads q at q_off + (h / qk_share) * dim):
// the groups of a state-space scan, whose B and C are shared by the heads of a group.  1: a q and a k per head.
constexpr int MODE_PLAIN = 0, MODE_GATED = 1, MODE_VECTOR = 2;
template <typename TD, int PARTS, bool OUTPUTS, int MODE>
__global__ void __launch_bounds__(LA_THREADS, 4)     // four blocks an SM (measured faster than three blocks without the few spills)
linear_attention_scan_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld,
                             int q_off, int k_off, int v_off, const float* __restrict__ decay,
                             float* __restrict__ state, const int* __restrict__ segment_start,
                             const int* __restrict__ segment_slot, float* __restrict__ out, int heads, int dim,
                             int vdim, int act, int num_slots, int num_segments, int chunk_rows, int phase,
                             float* __restrict__ chunk_state, const float* __restrict__ token_keep,
                             const float* __restrict__ token_take, float q_scale, int norm_col, int qk_share) {
  constexpr bool GATED = MODE == MODE_GATED;
  constexpr bool VECTOR = MODE == MODE_VECTOR;
  constexpr int CW = 32 / PARTS;
  constexpr int CB = 4 * CW;
  constexpr int PADDED = LA_DPT + 4;                // a part's 32 values, 16-byte aligned and four banks apart from the next part's
  constexpr int QS = PARTS * PADDED;                // a token's q (or k) in shared memory
  constexpr int LA_TT = PARTS <= 2 ? 16 : (PARTS == 4 ? 8 : 4);   // tokens staged at a time: eight values of q and of k a thread
  constexpr int QK_LOADS = LA_TT * PARTS * LA_DPT / LA_THREADS;   // values of q (and of k) a thread stages per tile
  constexpr int V_LOADS = (LA_TT * CB + LA_THREADS - 1) / LA_THREADS;
  __shared__ __align__(16) float q_s[LA_TT * QS], k_s[LA_TT * QS], v_s[LA_TT * CB];
  __shared__ __align__(16) float a_s[VECTOR ? LA_TT * QS : 4];
  __shared__ float keep_s[LA_TT];
  __shared__ int item[3];
  const int vs = vdim + (GATED && norm_col ? 1 : 0);     // columns of a head's state and of its output
  const int hq = (int)blockIdx.y / qk_share;
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, col0 = blockIdx.z * CB;
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
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane / CW, cb = warp * CW + lane % CW, col = col0 + cb;
  const float decay_h = MODE == MODE_PLAIN ? decay[h] : 1.f;
  float* st = chunk_rows == 0
      ? state + ((size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * heads + h) * dim * vs
      : chunk_state + ((size_t)blockIdx.x * heads + h) * dim * vs;
  const bool from_zero = chunk_rows > 0 && phase == 1;
  const bool store = !(chunk_rows > 0 && phase == 2);
  float s[LA_DPT];
#pragma unroll
  for (int i = 0; i < LA_DPT; ++i) {
    const int d = part * LA_DPT + i;
    s[i] = (!from_zero && d < dim && col < vs) ? st[(size_t)d * vs + col] : 0.f;
  }
  float qv[QK_LOADS], kv[QK_LOADS], vv_in[V_LOADS], take[QK_LOADS], av[VECTOR ? QK_LOADS : 1];
  auto fetch = [&](int base) {      // a tile's q, k and v into registers, all loads in flight together
    const int n = min(LA_TT, row1 - base);
#pragma unroll
    for (int i = 0; i < QK_LOADS; ++i) {
      const int e = threadIdx.x + i * LA_THREADS;
      const int t = e / (PARTS * LA_DPT), d = e % (PARTS * LA_DPT);
      qv[i] = kv[i] = take[i] = 0.f;
      if (VECTOR) av[i] = 0.f;
      if (t < n && d < dim) {
        const TD* row = proj + (size_t)(base + t) * ld + hq * dim + d;
        qv[i] = la_load(row + q_off, n_partials, partial_stride);
        kv[i] = la_load(row + k_off, n_partials, partial_stride);
        if (GATED) take[i] = token_take[(size_t)(base + t) * heads + h];
        if (VECTOR) av[i] = token_keep[((size_t)(base + t) * heads + h) * dim + d];
      }
    }
#pragma unroll
    for (int i = 0; i < V_LOADS; ++i) {
      const int e = threadIdx.x + i * LA_THREADS;
      const int t = e / CB, c = e % CB;
      vv_in[i] = 0.f;
      if (e < LA_TT * CB && t < n && col0 + c < vdim)
        vv_in[i] = la_load(proj + (size_t)(base + t) * ld + v_off + h * vdim + col0 + c, n_partials, partial_stride);
      else if (GATED && norm_col && e < LA_TT * CB && t < n && col0 + c == vdim)
        vv_in[i] = 1.f;      // the normaliser's column
    }
  };
  fetch(row0);
  for (int base = row0; base < row1; base += LA_TT) {
    const int n = min(LA_TT, row1 - base);
    __syncthreads();      // the tile before has been used
#pragma unroll
    for (int i = 0; i < QK_LOADS; ++i) {
      const int e = threadIdx.x + i * LA_THREADS;
      const int t = e / (PARTS * LA_DPT), d = e % (PARTS * LA_DPT);
      const int at = t * QS + (d / LA_DPT) * PADDED + d % LA_DPT;
      q_s[at] = la_act(qv[i], act) * q_scale;
      k_s[at] = GATED ? la_act(kv[i], act) * take[i] : la_act(kv[i], act);
      if (VECTOR) a_s[at] = av[i];
    }
    if (GATED && threadIdx.x < LA_TT)
      keep_s[threadIdx.x] = (int)threadIdx.x < n ? token_keep[(size_t)(base + threadIdx.x) * heads + h] : 1.f;
#pragma unroll
    for (int i = 0; i < V_LOADS; ++i) {
      const int e = threadIdx.x + i * LA_THREADS;
      if (e < LA_TT * CB) v_s[e] = (GATED && norm_col && col0 + e % CB == vdim) ? vv_in[i] : la_act(vv_in[i], act);
    }
    __syncthreads();
    if (base + LA_TT < row1) fetch(base + LA_TT);    // the next tile travels while this one is worked on
    for (int t = 0; t < n; ++t) {
      const float4* qr = reinterpret_cast<const float4*>(q_s + t * QS + part * PADDED);
      const float4* kr = reinterpret_cast<const float4*>(k_s + t * QS + part * PADDED);
      const float4* ar = reinterpret_cast<const float4*>(a_s + (VECTOR ? t * QS + part * PADDED : 0));
      const float vv = v_s[t * CB + cb];
      const float dk = GATED ? keep_s[t] : decay_h;
      float o[4] = {0.f, 0.f, 0.f, 0.f};     // four short chains instead of one of 32 dependent additions
#pragma unroll
      for (int i = 0; i < LA_DPT / 4; ++i) {
        const float4 kq = kr[i], qq = OUTPUTS ? qr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 aa = VECTOR ? ar[i] : make_float4(dk, dk, dk, dk);
        s[4 * i + 0] = fmaf(aa.x, s[4 * i + 0], kq.x * vv);
        s[4 * i + 1] = fmaf(aa.y, s[4 * i + 1], kq.y * vv);
        s[4 * i + 2] = fmaf(aa.z, s[4 * i + 2], kq.z * vv);
        s[4 * i + 3] = fmaf(aa.w, s[4 * i + 3], kq.w * vv);
        if (OUTPUTS) {
          o[0] = fmaf(s[4 * i + 0], qq.x, o[0]); o[1] = fmaf(s[4 * i + 1], qq.y, o[1]);
          o[2] = fmaf(s[4 * i + 2], qq.z, o[2]); o[3] = fmaf(s[4 * i + 3], qq.w, o[3]);
        }
      }
      if (OUTPUTS) {
        float total = (o[0] + o[1]) + (o[2] + o[3]);
#pragma unroll
        for (int off = CW; off < 32; off <<= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (part == 0 && col < vs) out[(size_t)(base + t) * heads * vs + h * vs + col] = total;
      }
    }
  }
  if (store) {
#pragma unroll
    for (int i = 0; i < LA_DPT; ++i) {
      const int d = part * LA_DPT + i;
      if (d < dim && col < vs) st[(size_t)d * vs + col] = s[i];
    }
  }
}

// Between the two phases: chunk_state[c] holds chunk c's own state (from zero); it becomes the state at the chunk's
// start, S_start(c + 1) = decay^rows(c) * S_start(c) + own(c), beginning with the request's slot, which receives the
// state after the request's last chunk.  One thread per element of (request, head, dim, vdim).
__global__ void __launch_bounds__(256)
linear_attention_carry_kernel(const float* __restrict__ decay, float* __restrict__ state,
                              const int* __restrict__ segment_start, const int* __restrict__ segment_slot,
                              float* __restrict__ chunk_state, int heads, int dim, int vdim, int num_slots,
                              int chunk_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.y;
  const int a = segment_start[seg], b = segment_start[seg + 1];
  if (b <= a) return;
  const size_t per_state = (size_t)heads * dim * vdim;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_state) return;
  int before = 0;
  for (int s = 0; s < seg; ++s) before += (segment_start[s + 1] - segment_start[s] + chunk_rows - 1) / chunk_rows;
  const int h = (int)(e / ((size_t)dim * vdim));
  const float dk = decay[h];
  float full = 1.f;
  for (int i = 0; i < chunk_rows; ++i) full *= dk;
  float* slot = state + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * per_state + e;
  float running = *slot;
  const int chunks = (b - a + chunk_rows - 1) / chunk_rows;
  float last_power = 1.f;
  for (int i = 0; i < b - a - (chunks - 1) * chunk_rows; ++i) last_power *= dk;
  float* own = chunk_state + (size_t)before * per_state + e;
  for (int c0 = 0; c0 < chunks; c0 += 8) {      // eight chunks' states are fetched together, then carried in order
    float mine[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) mine[i] = c0 + i < chunks ? own[(size_t)(c0 + i) * per_state] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c0 + i < chunks) {
        own[(size_t)(c0 + i) * per_state] = running;
        running = fmaf(c0 + i == chunks - 1 ? last_power : full, running, mine[i]);
      }
    }
  }
  *slot = running;
}

// The carry for the gated form: a chunk's decay is the product of its tokens' keep factors.  A block owns 256 elements
// of one head's state of one request; its warps first multiply up every chunk's factors (shared memory, one number a
// chunk), then every thread carries its element from chunk to chunk as above.  vs = columns of the state.
__global__ void __launch_bounds__(256)
linear_attention_gated_carry_kernel(const float* __restrict__ token_keep, float* __restrict__ state,
                                    const int* __restrict__ segment_start, const int* __restrict__ segment_slot,
                                    float* __restrict__ chunk_state, int heads, int dim, int vs, int num_slots,
                                    int chunk_rows) {
  extern __shared__ float chunk_keep[];     // [chunks of this request]
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.z, h = blockIdx.y;
  const int a = segment_start[seg], b = segment_start[seg + 1];
  if (b <= a) return;
  const int chunks = (b - a + chunk_rows - 1) / chunk_rows;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = warp; c < chunks; c += 8) {
    const int r0 = a + c * chunk_rows, r1 = min(b, r0 + chunk_rows);
    float product = 1.f;
    for (int r = r0 + lane; r < r1; r += 32) product *= token_keep[(size_t)r * heads + h];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) product *= __shfl_xor_sync(0xffffffffu, product, o);
    if (lane == 0) chunk_keep[c] = product;
  }
  __syncthreads();
  const int per_head = dim * vs;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_head) return;
  int before = 0;
  for (int s = 0; s < seg; ++s) before += (segment_start[s + 1] - segment_start[s] + chunk_rows - 1) / chunk_rows;
  const size_t per_state = (size_t)heads * per_head;
  const size_t at = (size_t)h * per_head + e;
  float* slot = state + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * per_state + at;
  float running = *slot;
  float* own = chunk_state + (size_t)before * per_state + at;
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float mine[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) mine[i] = c0 + i < chunks ? own[(size_t)(c0 + i) * per_state] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c0 + i < chunks) {
        own[(size_t)(c0 + i) * per_state] = running;
        running = fmaf(chunk_keep[c0 + i], running, mine[i]);
      }
    }
  }
  *slot = running;
}

// The vector form's carry.  First every chunk's factors, one per row of the state: the product of its tokens' keep
// vectors, chunk_keep[chunk][head][dim] (a block per chunk and head, a thread per row).
__global__ void __launch_bounds__(256)
linear_attention_chunk_keep_kernel(const float* __restrict__ token_keep, const int* __restrict__ segment_start,
                                   float* __restrict__ chunk_keep, int heads, int dim, int num_segments, int chunk_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y;
  int before = 0, first = 0, last = 0;
  bool found = false;
  for (int s = 0; s < num_segments && !found; ++s) {
    const int a = segment_start[s], b = segment_start[s + 1];
    const int chunks = (b - a + chunk_rows - 1) / chunk_rows;
    if ((int)blockIdx.x < before + chunks) {
      found = true;
      first = a + ((int)blockIdx.x - before) * chunk_rows;
      last = min(b, first + chunk_rows);
    }
    before += chunks;
  }
  if (!found) return;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float product = 1.f;
    for (int r = first; r < last; ++r) product *= token_keep[((size_t)r * heads + h) * dim + d];
    chunk_keep[((size_t)blockIdx.x * heads + h) * dim + d] = product;
  }
}

// Then, as above, every element carried from chunk to chunk with its row's factor.
__global__ void __launch_bounds__(256)
linear_attention_vector_carry_kernel(const float* __restrict__ chunk_keep, float* __restrict__ state,
                                     const int* __restrict__ segment_start, const int* __restrict__ segment_slot,
                                     float* __restrict__ chunk_state, int heads, int dim, int vs, int num_slots,
                                     int chunk_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.z, h = blockIdx.y;
  const int a = segment_start[seg], b = segment_start[seg + 1];
  if (b <= a) return;
  const int chunks = (b - a + chunk_rows - 1) / chunk_rows;
  const int per_head = dim * vs;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_head) return;
  const int d = e / vs;
  int before = 0;
  for (int s = 0; s < seg; ++s) before += (segment_start[s + 1] - segment_start[s] + chunk_rows - 1) / chunk_rows;
  const size_t per_state = (size_t)heads * per_head;
  const size_t at = (size_t)h * per_head + e;
  float* slot = state + (size_t)LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW) * per_state + at;
  float running = *slot;
  float* own = chunk_state + (size_t)before * per_state + at;
  const float* factor = chunk_keep + ((size_t)before * heads + h) * dim + d;
  for (int c = 0; c < chunks; ++c) {
    const float mine = own[(size_t)c * per_state];
    own[(size_t)c * per_state] = running;
    running = fmaf(factor[(size_t)c * heads * dim], running, mine);
  }
  *slot = running;
}


// chunk_rows == 0: one block row per request of the step (max_segments), empty requests leave at once.
// chunk_rows > 0: three launches over chunks of chunk_rows rows; chunk_state holds max_chunks states
// [heads][dim][columns] (max_chunks >= tokens / chunk_rows + max_segments bounds the number of chunks).
// token_keep, token_take (float32 [tokens, heads], or both null): the gated form, whose states and outputs have
// vdim + 1 columns a head; decay is not read then.
template <int MODE>
static int linear_attention_scan_launch(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                        long long ld, int q_off, int k_off, int v_off, const float* decay,
                                        float* state, const int* segment_start, const int* segment_slot, float* out,
                                        int max_segments, int heads, int dim, int vdim, int act, int num_slots,
                                        int chunk_rows, float* chunk_state, int max_chunks, const float* token_keep,
                                        const float* token_take, float q_scale, int norm_col, int qk_share,
                                        float* chunk_keep, cudaStream_t stream) {
  if (max_segments <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 8 * LA_DPT || heads > 65535) return LSE_ERR_BAD_ARGUMENT;
  if (qk_share <= 0 || heads % qk_share) return LSE_ERR_BAD_ARGUMENT;
  if (chunk_rows < 0 || (chunk_rows > 0 && (chunk_state == nullptr || max_chunks <= 0))) return LSE_ERR_BAD_ARGUMENT;
  if (MODE == MODE_VECTOR && chunk_rows > 0 && chunk_keep == nullptr) return LSE_ERR_BAD_ARGUMENT;
  const int vs = vdim + (MODE == MODE_GATED && norm_col ? 1 : 0);
  int parts = 1;
  while (parts * LA_DPT < dim) parts <<= 1;
#define LSE_LA_CASE(TD, P)                                                                                       \
  {                                                                                                              \
    const int cb = 4 * (32 / P);                                                                                 \
    dim3 grid(chunk_rows ? max_chunks : max_segments, heads, (vs + cb - 1) / cb);                                \
    for (int phase = 1; phase <= (chunk_rows ? 2 : 1); ++phase) {                                                \
      if (chunk_rows && phase == 1)                                                                              \
        lse_launch(linear_attention_scan_kernel<TD, P, false, MODE>, grid, LA_THREADS, 0, stream,                \
                   (const TD*)proj, n_partials, partial_stride, ld, q_off, k_off, v_off, decay, state,           \
                   segment_start, segment_slot, out, heads, dim, vdim, act, num_slots, max_segments, chunk_rows, \
                   phase, chunk_state, token_keep, token_take, q_scale, norm_col, qk_share);                     \
      else                                                                                                       \
        lse_launch(linear_attention_scan_kernel<TD, P, true, MODE>, grid, LA_THREADS, 0, stream,                 \
                   (const TD*)proj, n_partials, partial_stride, ld, q_off, k_off, v_off, decay, state,           \
                   segment_start, segment_slot, out, heads, dim, vdim, act, num_slots, max_segments, chunk_rows, \
                   phase, chunk_state, token_keep, token_take, q_scale, norm_col, qk_share);                     \
      if (chunk_rows && phase == 1) {                                                                            \
        const size_t per_state = (size_t)heads * dim * vs;                                                       \
        if (MODE == MODE_GATED)                                                                                  \
          lse_launch(linear_attention_gated_carry_kernel, dim3((unsigned)((dim * vs + 255) / 256), heads,        \
                                                               max_segments),                                   \
                     256, sizeof(float) * (size_t)max_chunks, stream, token_keep, state, segment_start,          \
                     segment_slot, chunk_state, heads, dim, vs, num_slots, chunk_rows);                          \
        else if (MODE == MODE_VECTOR) {                                                                          \
          lse_launch(linear_attention_chunk_keep_kernel, dim3(max_chunks, heads), dim >= 128 ? 128 : 64, 0,      \
                     stream, token_keep, segment_start, chunk_keep, heads, dim, max_segments, chunk_rows);       \
          lse_launch(linear_attention_vector_carry_kernel, dim3((unsigned)((dim * vs + 255) / 256), heads,       \
                                                                max_segments),                                  \
                     256, 0, stream, (const float*)chunk_keep, state, segment_start, segment_slot, chunk_state,  \
                     heads, dim, vs, num_slots, chunk_rows);                                                     \
        } else                                                                                                   \
          lse_launch(linear_attention_carry_kernel, dim3((unsigned)((per_state + 255) / 256), max_segments),     \
                     256, 0, stream, decay, state, segment_start, segment_slot, chunk_state, heads, dim, vdim,   \
                     num_slots, chunk_rows);                                                                     \
      }                                                                                                          \
    }                                                                                                            \
  }
#define LSE_LA_PARTS(TD)                                  \
  switch (parts) {                                        \
    case 1: LSE_LA_CASE(TD, 1) break;                     \
    case 2: LSE_LA_CASE(TD, 2) break;                     \
    case 4: LSE_LA_CASE(TD, 4) break;                     \
    default: LSE_LA_CASE(TD, 8) break;                    \
  }
  if (proj_dtype == LSE_DTYPE_F32) { LSE_LA_PARTS(float) }
  else if (proj_dtype == LSE_DTYPE_BF16) { LSE_LA_PARTS(__nv_bfloat16) }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_LA_PARTS
#undef LSE_LA_CASE
  LSE_LAUNCH_CHECK();
}

}  // namespace
