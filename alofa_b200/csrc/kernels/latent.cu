// Kernels of latent attention, sandwich norms and routed feed-forwards that
// take every size and both dtypes (T = float: the true 32-bit path; T = bf16:
// activations and cache rows in bfloat16).  Everything that the model states
// in 32-bit is fp32 here in both: positions and angles, norms, scores and
// softmax weights, router scores, the residual sum.  No tensor cores, no
// approximate intrinsics; for every output element the order of additions is
// fixed by the problem sizes alone, never by which other rows share the launch.
//
// Latent attention keeps ONE row per token in a paged cache: a normed latent c
// (kv_rank numbers) followed by a rotated key part (rot numbers) that all heads
// share.  With W_uk the per-head map from c to unrotated keys, the score of
// query head h against token j is
//   (q_h . (W_uk_h c_j) + qr_h . kr_j) * scale = ((W_uk_h^T q_h) . c_j + qr_h . kr_j) * scale,
// so the query is carried into the latent space once ("absorbed", a product per
// head) and every head attends to the same rows [c_j | kr_j]; values are
// W_uv_h applied to sum_j p_j c_j, so the cache row's first kv_rank numbers
// also serve as the value.  The softmax denominator has one more term,
// exp(sink_h), that belongs to no key.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Interleaved rotary encoding: the pair (x[2i], x[2i+1]), i < dims/2, at
// position p turns by the angle p * f_i, f_i given as fp32.  Angle, cosine and
// sine are fp32 (the precise library functions).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void turn(float u, float v, float angle, float& a, float& b, float mag = 1.0f) {
  float s, c;
  sincosf(angle, &s, &c);
  s *= mag;  // a factor on cosine and sine alike (1: none), as scaled rotary encodings have
  c *= mag;
  a = u * c - v * s;
  b = v * c + u * s;
}
// Which two numbers pair i of a rotated part of `dims` numbers joins: neighbours (2i, 2i + 1), or (halves) i and i + dims / 2.
__device__ __forceinline__ void pair_of(int i, int dims, int halves, int& lo, int& hi) {
  lo = halves ? i : 2 * i;
  hi = halves ? i + dims / 2 : 2 * i + 1;
}

// ---------------------------------------------------------------------------
// After the stacked down-projection [c_q raw | c raw | key part raw] (fp32):
//   cq[t]          = rmsnorm(first q_rank) * wq            (compute dtype)
//   cache[slot, :kv_rank] = rmsnorm(next kv_rank) * wkv
//   cache[slot, kv_rank:] = the last rot numbers, the first rot_dims of them turned
// One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(T* __restrict__ cq, T* __restrict__ cache, const float* __restrict__ lat,
                                                             const float* __restrict__ wq, const float* __restrict__ wkv,
                                                             const float* __restrict__ freq, const int* __restrict__ positions,
                                                             const int* __restrict__ slot_map, int q_rank, int kv_rank, int rot, int rot_dims,
                                                             float eps, int ld, int halves, float mag) {
  __shared__ float scratch[32];
  pdl_begin();
  const int t = blockIdx.x;
  const float* row = lat + (size_t)t * ld;
  float ss = 0.f;
  if (q_rank > 0) {  // a design without a query latent has q_rank 0
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    ss = block_sum(ss, scratch);
    const float fq = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq[(size_t)t * q_rank + c] = from_f<T>(row[c] * fq * wq[c]);
  }
  if (!cache) return;
  const int slot = slot_map[t];
  if (slot < 0) return;
  const float* kv = row + q_rank;
  ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) ss = fmaf(kv[c], kv[c], ss);
  ss = block_sum(ss, scratch);
  const float fk = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  T* out = cache + (size_t)slot * (kv_rank + rot);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) out[c] = from_f<T>(kv[c] * fk * wkv[c]);
  const float p = (float)positions[t];
  const float* kr = kv + kv_rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    float a, b;
    int lo, hi;
    pair_of(i, rot_dims, halves, lo, hi);
    turn(kr[lo], kr[hi], p * freq[i], a, b, mag);
    out[kv_rank + lo] = from_f<T>(a);
    out[kv_rank + hi] = from_f<T>(b);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) out[kv_rank + c] = from_f<T>(kr[c]);
}

ALOFA_API int alofa_latent_prepare(void* cq, void* cache, const float* lat, const float* wq, const float* wkv, const float* freq,
                                   const int* positions, const int* slot_map, int n_tokens, int q_rank, int kv_rank, int rot, int rot_dims,
                                   float eps, int ld, int halves, float mag, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (q_rank < 0 || kv_rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || ld < q_rank + kv_rank + rot) return ALOFA_ERR_ARGUMENT;
  if (is_bf16)
    launch_dep(latent_prepare_kernel<bf16>, n_tokens, 256, 0, stream, (bf16*)cq, (bf16*)cache, lat, wq, wkv, freq, positions, slot_map, q_rank, kv_rank,
               rot, rot_dims, eps, ld, halves, mag);
  else
    launch_dep(latent_prepare_kernel<float>, n_tokens, 256, 0, stream, (float*)cq, (float*)cache, lat, wq, wkv, freq, positions, slot_map, q_rank,
               kv_rank, rot, rot_dims, eps, ld, halves, mag);
  return launch_status();
}

// ---------------------------------------------------------------------------
// The rotated part of the queries: q [T, H, dim + rot] -> qa [T, H, kv_rank + rot]
// at columns kv_rank.. (the first kv_rank columns are the absorbed unrotated
// part, written by the batched product).  One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_query_turn_kernel(T* __restrict__ qa, const T* __restrict__ q, const float* __restrict__ freq,
                                         const int* __restrict__ positions, int heads, int dim, int rot, int rot_dims, int kv_rank, int halves,
                                         float mag) {
  pdl_begin();
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  const int half = rot_dims / 2;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    const T* src = q + ((size_t)t * heads + h) * (dim + rot) + dim;
    T* dst = qa + ((size_t)t * heads + h) * (kv_rank + rot) + kv_rank;
    float a, b;
    int lo, hi;
    pair_of(i, rot_dims, halves, lo, hi);
    turn(to_f(src[lo]), to_f(src[hi]), p * freq[i], a, b, mag);
    dst[lo] = from_f<T>(a);
    dst[hi] = from_f<T>(b);
  }
  const int rest = rot - rot_dims;
  for (int e = threadIdx.x; e < heads * rest; e += blockDim.x) {
    const int h = e / rest, c = rot_dims + (e - h * rest);
    qa[((size_t)t * heads + h) * (kv_rank + rot) + kv_rank + c] = q[((size_t)t * heads + h) * (dim + rot) + dim + c];
  }
}

ALOFA_API int alofa_latent_query_turn(void* qa, const void* q, const float* freq, const int* positions, int n_tokens, int heads, int dim, int rot,
                                      int rot_dims, int kv_rank, int halves, float mag, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0 || rot <= 0) return ALOFA_OK;
  if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return ALOFA_ERR_ARGUMENT;
  if (is_bf16)
    launch_dep(latent_query_turn_kernel<bf16>, n_tokens, 128, 0, stream, (bf16*)qa, (const bf16*)q, freq, positions, heads, dim, rot, rot_dims, kv_rank, halves, mag);
  else
    launch_dep(latent_query_turn_kernel<float>, n_tokens, 128, 0, stream, (float*)qa, (const float*)q, freq, positions, heads, dim, rot, rot_dims, kv_rank, halves, mag);
  return launch_status();
}

// In-place turn of q [T, heads, hd] and k [T, kv_heads, hd] views (row strides given): the same
// encoding for mixers that hold whole heads.
template <typename T>
__global__ void rotary_interleaved_kernel(T* __restrict__ x, const float* __restrict__ freq, const int* __restrict__ positions, int heads, int hd,
                                          int row_stride, int rot_dims) {
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  const int half = rot_dims / 2;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    T* v = x + (size_t)t * row_stride + (size_t)h * hd;
    float a, b;
    turn(to_f(v[2 * i]), to_f(v[2 * i + 1]), p * freq[i], a, b);
    v[2 * i] = from_f<T>(a);
    v[2 * i + 1] = from_f<T>(b);
  }
}

ALOFA_API int alofa_rotary_interleaved(void* x, const float* freq, const int* positions, int n_tokens, int heads, int hd, int row_stride,
                                       int rot_dims, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0 || heads <= 0 || rot_dims <= 0) return ALOFA_OK;
  if (rot_dims > hd || (rot_dims & 1)) return ALOFA_ERR_ARGUMENT;
  if (is_bf16)
    rotary_interleaved_kernel<bf16><<<n_tokens, 128, 0, stream>>>((bf16*)x, freq, positions, heads, hd, row_stride, rot_dims);
  else
    rotary_interleaved_kernel<float><<<n_tokens, 128, 0, stream>>>((float*)x, freq, positions, heads, hd, row_stride, rot_dims);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Batched product with strides: for batch b, out_b[m, n] = act(sum_k x_b[m, k] * w_b[n, k] + bias_b[n]),
//   x_b = x + b * x_batch (row stride ldx), w_b = w + b * w_batch (row stride ldw),
//   out_b = out + b * out_batch (row stride ldo), bias_b = bias + b * bias_batch.
// With tile_batch (one entry per tile of tile_rows rows of M, a multiple of 64) there is one x and one out,
// and tile i multiplies by the weight of batch tile_batch[i] (negative: the
// tile is empty): rows sorted by expert, each expert's rows padded to whole tiles.
// 64x64 tile, 16-deep slices, every output summed by one thread over k ascending.
// ---------------------------------------------------------------------------
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_batched_kernel(TO* __restrict__ out, const TA* __restrict__ x, const TW* __restrict__ w,
                                                           const float* __restrict__ bias, const int* __restrict__ tile_batch, int M, int N, int K,
                                                           long long ldx, long long x_batch, long long ldw, long long w_batch, long long ldo,
                                                           long long out_batch, long long bias_batch, int act, int tile_rows) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  pdl_begin();
  int b = blockIdx.z;
  if (tile_batch) {
    b = tile_batch[blockIdx.y * 64 / tile_rows];  // tile_rows is a multiple of this kernel's 64 rows
    if (b < 0) return;
    w += (size_t)b * w_batch;
    if (bias) bias += (size_t)b * bias_batch;
  } else {
    x += (size_t)b * x_batch;
    w += (size_t)b * w_batch;
    out += (size_t)b * out_batch;
    if (bias) bias += (size_t)b * bias_batch;
  }
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + 256 * i;
      const int r = e >> 4, k = e & 15;
      const int gm = m0 + r, gk = k0 + k, gn = n0 + r;
      xs[k][r] = (gm < M && gk < K) ? to_f(x[(size_t)gm * ldx + gk]) : 0.f;
      ws[k][r] = (gn < N && gk < K) ? to_f(w[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty + 16 * i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      out[(size_t)gm * ldo + gn] = from_f<TO>(activate(v, act));
    }
  }
}

template <typename TA, typename TW, typename TO>
static int gemm_batched_launch(void* out, const void* x, const void* w, const float* bias, const int* tile_batch, int batches, int M, int N, int K,
                               long long ldx, long long x_batch, long long ldw, long long w_batch, long long ldo, long long out_batch,
                               long long bias_batch, int act, int tile_rows, cudaStream_t stream) {
  dim3 grid((N + 63) / 64, (M + 63) / 64, tile_batch ? 1 : batches);
  launch_dep(gemm_batched_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (TO*)out, (const TA*)x, (const TW*)w, bias, tile_batch, M, N, K, ldx,
             x_batch, ldw, w_batch, ldo, out_batch, bias_batch, act, tile_rows);
  return launch_status();
}

// dtype flags: 0 = fp32, 1 = bf16.  x and w share a dtype flag pair as in alofa_gemm_generic.
ALOFA_API int alofa_gemm_batched(void* out, const void* x, const void* w, const float* bias, const int* tile_batch, int batches, int M, int N, int K,
                                 long long ldx, long long x_batch, long long ldw, long long w_batch, long long ldo, long long out_batch,
                                 long long bias_batch, int act, int tile_rows, int x_bf16, int w_bf16, int out_bf16, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batches <= 0) return ALOFA_OK;
  if (K <= 0 || (M + 63) / 64 > 65535 || batches > 65535 || (tile_batch && (tile_rows <= 0 || tile_rows % 64))) return ALOFA_ERR_ARGUMENT;
  const int key = (x_bf16 ? 4 : 0) | (w_bf16 ? 2 : 0) | (out_bf16 ? 1 : 0);
#define ALOFA_BATCHED(TA, TW, TO) \
  return gemm_batched_launch<TA, TW, TO>(out, x, w, bias, tile_batch, batches, M, N, K, ldx, x_batch, ldw, w_batch, ldo, out_batch, bias_batch, act, tile_rows, stream)
  switch (key) {
    case 0: ALOFA_BATCHED(float, float, float);
    case 1: ALOFA_BATCHED(float, float, bf16);
    case 2: ALOFA_BATCHED(float, bf16, float);
    case 3: ALOFA_BATCHED(float, bf16, bf16);
    case 4: ALOFA_BATCHED(bf16, float, float);
    case 5: ALOFA_BATCHED(bf16, float, bf16);
    case 6: ALOFA_BATCHED(bf16, bf16, float);
    default: ALOFA_BATCHED(bf16, bf16, bf16);
  }
#undef ALOFA_BATCHED
}

// out = act(x + bias) elementwise: x fp32 [rows, n], out in the compute dtype.
template <typename T>
__global__ void activate_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ bias, long long count, int n, int act) {
  pdl_begin();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i];
    if (bias) v += bias[i % n];
    out[i] = from_f<T>(activate(v, act));
  }
}

ALOFA_API int alofa_activate(void* out, const float* x, const float* bias, long long rows, int n, int act, int out_bf16, cudaStream_t stream) {
  const long long count = rows * n;
  if (count <= 0) return ALOFA_OK;
  const int blocks = (int)((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
  if (out_bf16) launch_dep(activate_kernel<bf16>, blocks, 256, 0, stream, (bf16*)out, x, bias, count, n, act);
  else launch_dep(activate_kernel<float>, blocks, 256, 0, stream, (float*)out, x, bias, count, n, act);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Latent attention over the paged cache of rows [c | kr] (width D = kv_rank + rot).
//   qa  [T, H, D]        absorbed queries (compute dtype)
//   out [T, H, kv_rank]  sum_j p_j c_j per head (compute dtype)
// The query at position P of request r sees rows max(0, P - window + 1) .. P
// (window <= 0: all) through block_table[r][j / page_size].  One block takes
// one token and up to 8 heads, a warp per head: all heads read the same rows,
// so a chunk of 32 rows is brought into shared memory once for the block.  Per
// chunk (boundaries at multiples of 32 of the row index, whatever the step
// holds): lane j scores row j, the warp takes maximum and sum in butterfly
// order, and each lane keeps the output columns lane, lane + 32, ... of its
// head, rescaled as in streaming softmax.  The sink enters as the initial
// state (maximum = sink, sum = 1, output = 0): a term exp(sink) with no row.
// ---------------------------------------------------------------------------
constexpr int LA_HEADS = 8;    // heads (warps) per block
constexpr int LA_CHUNK = 32;   // rows per chunk
constexpr int LA_MAX_COLS = 32;  // output columns per lane: kv_rank <= 1024

template <typename T>
__global__ void __launch_bounds__(LA_HEADS * 32) latent_attention_kernel(T* __restrict__ out, const T* __restrict__ qa, const T* __restrict__ cache,
                                                                         const float* __restrict__ sink, const int* __restrict__ positions,
                                                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                                                         int max_blocks, int page_size, int heads, int kv_rank, int rot, int window,
                                                                         float scale) {
  extern __shared__ float smem[];
  const int D = kv_rank + rot, pitch = D + 1;
  float* qs = smem;                       // [LA_HEADS][D]
  float* rows = qs + LA_HEADS * D;        // [LA_CHUNK][pitch]
  float* ps = rows + LA_CHUNK * pitch;    // [LA_HEADS][LA_CHUNK]
  pdl_begin();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * LA_HEADS + warp;
  const bool live = h < heads;
  const int P = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * max_blocks;
  if (live)
    for (int d = lane; d < D; d += 32) qs[warp * D + d] = to_f(qa[((size_t)t * heads + h) * D + d]);
  int first = 0;
  if (window > 0 && P - window + 1 > 0) first = P - window + 1;
  float m = live && sink ? sink[h] : -INFINITY, l = live && sink ? 1.f : 0.f;
  float acc[LA_MAX_COLS];
#pragma unroll
  for (int i = 0; i < LA_MAX_COLS; ++i) acc[i] = 0.f;
  const int n_cols = (kv_rank + 31) / 32;
  for (int c0 = (first / LA_CHUNK) * LA_CHUNK; c0 <= P; c0 += LA_CHUNK) {
    __syncthreads();  // the chunk before is read out (and, the first time, qs is written)
    const int n_in = min(LA_CHUNK, P - c0 + 1);
    for (int e = threadIdx.x; e < n_in * D; e += blockDim.x) {
      const int j = e / D, d = e - j * D;
      const int key = c0 + j;
      if (key < first) {  // before the window: its page may have been given back, and its table entry then names no page
        rows[j * pitch + d] = 0.f;
        continue;
      }
      const int slot = table[key / page_size] * page_size + key % page_size;
      rows[j * pitch + d] = to_f(cache[(size_t)slot * D + d]);
    }
    __syncthreads();
    if (!live) continue;
    const int j = c0 + lane;
    const bool visible = lane < n_in && j >= first;
    float s = -INFINITY;
    if (visible) {
      float dot = 0.f;
      const float* q = qs + warp * D;
      const float* r = rows + lane * pitch;
      for (int d = 0; d < D; ++d) dot = fmaf(q[d], r[d], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = visible ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
    ps[warp * LA_CHUNK + lane] = p;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < LA_MAX_COLS; ++i) {
      if (i >= n_cols) break;
      const int c = lane + 32 * i;
      float a = acc[i] * corr;
      if (c < kv_rank)
        for (int jj = 0; jj < n_in; ++jj) a = fmaf(ps[warp * LA_CHUNK + jj], rows[jj * pitch + c], a);
      acc[i] = a;
    }
  }
  if (!live) return;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < LA_MAX_COLS; ++i) {
    if (i >= n_cols) break;
    const int c = lane + 32 * i;
    if (c < kv_rank) out[((size_t)t * heads + h) * kv_rank + c] = from_f<T>(acc[i] * inv);
  }
}

ALOFA_API int alofa_latent_attention(void* out, const void* qa, const void* cache, const float* sink, const int* positions, const int* seq_of_token,
                                     const int* block_table, int max_blocks, int page_size, int n_tokens, int heads, int kv_rank, int rot,
                                     int window, float scale, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (heads <= 0 || kv_rank <= 0 || kv_rank > 32 * LA_MAX_COLS || rot < 0 || page_size <= 0) return ALOFA_ERR_ARGUMENT;
  const int D = kv_rank + rot;
  const size_t smem = ((size_t)LA_HEADS * D + (size_t)LA_CHUNK * (D + 1) + LA_HEADS * LA_CHUNK) * sizeof(float);
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
  dim3 grid(n_tokens, (heads + LA_HEADS - 1) / LA_HEADS);
  if (is_bf16) {
    static size_t set = 0;
    if (smem > set) {
      if (cudaFuncSetAttribute(latent_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set = smem;
    }
    launch_dep(latent_attention_kernel<bf16>, grid, dim3(LA_HEADS * 32), smem, stream, (bf16*)out, (const bf16*)qa, (const bf16*)cache, sink, positions,
               seq_of_token, block_table, max_blocks, page_size, heads, kv_rank, rot, window, scale);
  } else {
    static size_t set = 0;
    if (smem > set) {
      if (cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set = smem;
    }
    launch_dep(latent_attention_kernel<float>, grid, dim3(LA_HEADS * 32), smem, stream, (float*)out, (const float*)qa, (const float*)cache, sink,
               positions, seq_of_token, block_table, max_blocks, page_size, heads, kv_rank, rot, window, scale);
  }
  return launch_status();
}

// ---------------------------------------------------------------------------
// Sandwich norms.  h (fp32 stream) += rmsnorm(y) * w_post; and, when x is given,
// x = rmsnorm(h) * w_next of the updated row (the norm ahead of the next
// sublayer; without w_next the updated row itself) in the compute dtype.  One
// block per row, fp32 throughout.
// ---------------------------------------------------------------------------
// y may still be owed: `splits` planes of partial sums (plane z at y + z * plane) that a product left for this kernel
// to add, in split order, and a bias on top - the same additions in the same order as the kernel that would
// otherwise have added them up.  splits 0: y is the finished output.
struct OwedSums {
  int splits;
  long long plane;
  const float* bias;
};

__device__ __forceinline__ float owed_value(const float* __restrict__ y, const OwedSums& o, size_t at, int c) {
  if (o.splits == 0) return y[at];
  float a = 0.f;
  for (int z = 0; z < o.splits; ++z) a += y[(size_t)z * o.plane + at];
  if (o.bias) a += o.bias[c];
  return a;
}

__device__ __forceinline__ float4 owed_value4(const float* __restrict__ y, const OwedSums& o, size_t at, int c) {
  if (o.splits == 0) return *reinterpret_cast<const float4*>(y + at);
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < o.splits; ++z) {
    const float4 v = *reinterpret_cast<const float4*>(y + (size_t)z * o.plane + at);
    a.x += v.x, a.y += v.y, a.z += v.z, a.w += v.w;
  }
  if (o.bias) {
    const float4 b = *reinterpret_cast<const float4*>(o.bias + c);
    a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
  }
  return a;
}

template <typename T>
__global__ void __launch_bounds__(256) sandwich_norm_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ w_post,
                                                            float eps_post, T* __restrict__ x, const float* __restrict__ w_next, float eps_next,
                                                            int hidden, OwedSums owed) {
  __shared__ float scratch[32];
  pdl_begin();
  const size_t r = (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = owed_value(y, owed, r + c, c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float f = 1.0f / sqrtf(ss / (float)hidden + eps_post);
  float s2 = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = h[r + c] + owed_value(y, owed, r + c, c) * f * w_post[c];
    h[r + c] = v;
    s2 = fmaf(v, v, s2);
  }
  if (!x) return;
  if (!w_next) {  // no norm ahead of the next sublayer: it reads the row itself
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) x[r + c] = from_f<T>(h[r + c]);
    return;
  }
  s2 = block_sum(s2, scratch);
  const float g = 1.0f / sqrtf(s2 / (float)hidden + eps_next);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) x[r + c] = from_f<T>(h[r + c] * g * w_next[c]);
}

// The same with the row in registers (hidden a multiple of 4, at most 4 * 256 * CHUNKS): every element
// of y and h is read once, 16 bytes a thread, and h and x are written once.  The sums run over the same
// elements per thread and the same block reduction as above only when the sizes agree, so a size goes
// one way or the other for every row of every step.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(256) sandwich_norm_rows_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ w_post,
                                                                 float eps_post, T* __restrict__ x, const float* __restrict__ w_next, float eps_next,
                                                                 int hidden, OwedSums owed) {
  __shared__ float scratch[32];
  pdl_begin();
  const size_t r = (size_t)blockIdx.x * hidden;
  const int quads = hidden >> 2;
  float4 yv[CHUNKS], hv[CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = threadIdx.x + 256 * i;
    if (c < quads) {
      yv[i] = owed_value4(y, owed, r + 4 * (size_t)c, 4 * c);
      hv[i] = reinterpret_cast<const float4*>(h + r)[c];
      ss = fmaf(yv[i].x, yv[i].x, fmaf(yv[i].y, yv[i].y, fmaf(yv[i].z, yv[i].z, fmaf(yv[i].w, yv[i].w, ss))));
    }
  }
  ss = block_sum(ss, scratch);
  const float f = 1.0f / sqrtf(ss / (float)hidden + eps_post);
  float s2 = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = threadIdx.x + 256 * i;
    if (c < quads) {
      const float4 w = reinterpret_cast<const float4*>(w_post)[c];
      hv[i] = make_float4(hv[i].x + yv[i].x * f * w.x, hv[i].y + yv[i].y * f * w.y, hv[i].z + yv[i].z * f * w.z, hv[i].w + yv[i].w * f * w.w);
      reinterpret_cast<float4*>(h + r)[c] = hv[i];
      s2 = fmaf(hv[i].x, hv[i].x, fmaf(hv[i].y, hv[i].y, fmaf(hv[i].z, hv[i].z, fmaf(hv[i].w, hv[i].w, s2))));
    }
  }
  if (!x) return;
  float g = 1.0f;
  if (w_next) {
    s2 = block_sum(s2, scratch);
    g = 1.0f / sqrtf(s2 / (float)hidden + eps_next);
  }
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = threadIdx.x + 256 * i;
    if (c < quads) {
      const float4 w = w_next ? reinterpret_cast<const float4*>(w_next)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
      T* o = x + r + 4 * (size_t)c;
      o[0] = from_f<T>(hv[i].x * g * w.x);
      o[1] = from_f<T>(hv[i].y * g * w.y);
      o[2] = from_f<T>(hv[i].z * g * w.z);
      o[3] = from_f<T>(hv[i].w * g * w.w);
    }
  }
}

template <typename T>
static void sandwich_norm_launch(float* h, const float* y, const float* w_post, float eps_post, T* x, const float* w_next, float eps_next, int rows,
                                 int hidden, OwedSums owed, cudaStream_t stream) {
  const bool aligned = (hidden & 3) == 0 && !(((uintptr_t)h | (uintptr_t)y | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)owed.bias) & 15) && (owed.plane & 3) == 0;
  if (aligned && hidden <= 4 * 256 * 2)
    launch_dep(sandwich_norm_rows_kernel<T, 2>, rows, 256, 0, stream, h, y, w_post, eps_post, x, w_next, eps_next, hidden, owed);
  else if (aligned && hidden <= 4 * 256 * 8)
    launch_dep(sandwich_norm_rows_kernel<T, 8>, rows, 256, 0, stream, h, y, w_post, eps_post, x, w_next, eps_next, hidden, owed);
  else
    launch_dep(sandwich_norm_kernel<T>, rows, 256, 0, stream, h, y, w_post, eps_post, x, w_next, eps_next, hidden, owed);
}

// splits > 0: y holds that many planes of partial sums [rows, hidden] (plane z at y + z * plane floats) still to be added
// up, with y_bias (may be null) on top; splits 0: y is the sublayer's finished output.
ALOFA_API int alofa_sandwich_norm(float* h, const float* y, const float* w_post, float eps_post, void* x, const float* w_next, float eps_next,
                                  int rows, int hidden, int x_bf16, int splits, long long plane, const float* y_bias, cudaStream_t stream) {
  if (rows <= 0) return ALOFA_OK;
  if (splits < 0 || (splits > 0 && plane < (long long)rows * hidden)) return ALOFA_ERR_ARGUMENT;
  OwedSums owed;
  owed.splits = splits;
  owed.plane = plane;
  owed.bias = splits > 0 ? y_bias : nullptr;
  if (x_bf16) sandwich_norm_launch<bf16>(h, y, w_post, eps_post, (bf16*)x, w_next, eps_next, rows, hidden, owed, stream);
  else sandwich_norm_launch<float>(h, y, w_post, eps_post, (float*)x, w_next, eps_next, rows, hidden, owed, stream);
  return launch_status();
}

// out [T, 2 * hidden] = [a | b] in the compute dtype, from two fp32 matrices.
template <typename T>
__global__ void concat_rows_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int hidden) {
  pdl_begin();
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    out[t * 2 * hidden + c] = from_f<T>(a[t * hidden + c]);
    out[t * 2 * hidden + hidden + c] = from_f<T>(b[t * hidden + c]);
  }
}

// out = a, elementwise, from fp32 into the compute dtype: the rows a sublayer reads when no norm stands ahead of it.
template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ a, long long count) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = from_f<T>(a[i]);
}

ALOFA_API int alofa_cast_rows(void* out, const float* a, long long count, int out_bf16, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  if (out_bf16) launch_dep(cast_rows_kernel<bf16>, (unsigned)((count + 255) / 256), 256, 0, stream, (bf16*)out, a, count);
  else launch_dep(cast_rows_kernel<float>, (unsigned)((count + 255) / 256), 256, 0, stream, (float*)out, a, count);
  return launch_status();
}

ALOFA_API int alofa_concat_rows(void* out, const float* a, const float* b, int rows, int hidden, int out_bf16, cudaStream_t stream) {
  if (rows <= 0) return ALOFA_OK;
  if (out_bf16) launch_dep(concat_rows_kernel<bf16>, rows, 256, 0, stream, (bf16*)out, a, b, hidden);
  else launch_dep(concat_rows_kernel<float>, rows, 256, 0, stream, (float*)out, a, b, hidden);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Routed feed-forward.
// route: z [T, E (+1)] fp32 router logits (the last column, when gated, is the
// shared expert's gate).  score = sigmoid(z) or softmax over the experts; the
// `top` largest are chosen (ties: the lower index), their scores are the
// weights, optionally divided by their sum.  One warp per token.
// ---------------------------------------------------------------------------
__global__ void moe_route_kernel(int* __restrict__ choice, float* __restrict__ weight, float* __restrict__ gate, const float* __restrict__ z, int T,
                                 int E, int top, int cols, int softmax, int renormalize) {
  extern __shared__ float sc[];  // [warps][E]
  pdl_begin();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* s = sc + warp * E;
  const float* zr = z + (size_t)t * cols;
  if (softmax) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      s[e] = expf(zr[e] - mx);
      sum += s[e];
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) s[e] /= sum;
  } else {
    for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-zr[e]));
  }
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best) best = s[e], arg = e;  // ascending e: the first of equals
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
    }
    if (arg >= E) arg = k, best = 0.f;  // scores that are no numbers: some expert, weight zero
    if (lane == 0) {
      choice[(size_t)t * top + k] = arg;
      weight[(size_t)t * top + k] = best;
      s[arg] = -INFINITY;
    }
    total += best;
    __syncwarp();
  }
  if (renormalize && lane < top) weight[(size_t)t * top + lane] /= total;
  if (gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-zr[E]));
}

// The router's product and the choice in one kernel: z = x Wr^T in fp32 (x in the compute dtype, Wr fp32
// [E (+1), hidden]).  A block takes up to eight tokens, whose rows it keeps in shared memory; a warp takes
// the experts warp, warp + 8, ... and, for each, sums all the block's tokens at once: every lane reads its
// share of the expert's weights once and multiplies it into each token's row, then the warp adds the
// lanes' shares in butterfly order.  The order of additions of a (token, expert) sum depends on the depth
// alone.  The logits stay in shared memory; then a warp per token takes scores and choice as above.
template <typename T, int TT>
__global__ void __launch_bounds__(256) moe_router_kernel(int* __restrict__ choice, float* __restrict__ weight, float* __restrict__ gate,
                                                         const T* __restrict__ x, const float* __restrict__ wr, int T_, int E, int top, int hidden,
                                                         int gated, int softmax, int renormalize, const float* __restrict__ correction,
                                                         float renorm_eps, int groups, int keep, float route_scale) {
  extern __shared__ __align__(16) uint8_t router_smem[];
  const int cols = E + (gated ? 1 : 0);
  float* z = reinterpret_cast<float*>(router_smem);      // [TT][cols]
  float* gsc = z + TT * cols;                            // [TT][groups]: the groups' scores
  T* xs = reinterpret_cast<T*>(z + ((TT * (cols + groups) + 3) & ~3));  // [TT][hidden], on a 16-byte boundary
  pdl_begin();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT;
  const int live = min(TT, T_ - t0);
  if ((hidden * sizeof(T)) % 16 == 0) {  // rows start on 16-byte boundaries: 16 bytes a thread
    constexpr int PER = 16 / sizeof(T);
    const int chunks = hidden / PER;
    for (int e = threadIdx.x; e < TT * chunks; e += 256) {
      const int r = e / chunks, c = e - r * chunks;
      reinterpret_cast<uint4*>(xs)[e] = r < live ? reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * hidden)[c] : make_uint4(0, 0, 0, 0);
    }
  } else {
    for (int r = 0; r < TT; ++r)
      for (int c = threadIdx.x; c < hidden; c += 256) xs[r * hidden + c] = r < live ? x[(size_t)(t0 + r) * hidden + c] : from_f<T>(0.f);
  }
  __syncthreads();
  for (int e = warp; e < cols; e += 8) {
    const float* w = wr + (size_t)e * hidden;
    float dot[TT];
#pragma unroll
    for (int r = 0; r < TT; ++r) dot[r] = 0.f;
    if ((hidden & 3) == 0) {
      // four depth entries a lane and several loads in flight: with one scalar load at a time a warp spent
      // its time waiting for the weights (190 us a call at 64 experts, whatever the number of tokens)
#pragma unroll 4
      for (int c = lane * 4; c < hidden; c += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + c);
#pragma unroll
        for (int r = 0; r < TT; ++r) {
          const T* xr = xs + r * hidden + c;
          dot[r] = fmaf(to_f(xr[3]), wv.w, fmaf(to_f(xr[2]), wv.z, fmaf(to_f(xr[1]), wv.y, fmaf(to_f(xr[0]), wv.x, dot[r]))));
        }
      }
    } else {
      for (int c = lane; c < hidden; c += 32) {
        const float wv = w[c];
#pragma unroll
        for (int r = 0; r < TT; ++r) dot[r] = fmaf(to_f(xs[r * hidden + c]), wv, dot[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < TT; ++r) {
      const float v = warp_sum(dot[r]);
      if (lane == 0) z[r * cols + e] = v;
    }
  }
  __syncthreads();
  for (int r = warp; r < live; r += 8) {
    const int t = t0 + r;
    float* s = z + r * cols;
    const float zg = gated ? s[E] : 0.f;
    if (softmax) {
      float mx = -INFINITY;
      for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
      mx = warp_max(mx);
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) {
        s[e] = expf(s[e] - mx);
        sum += s[e];
      }
      sum = warp_sum(sum);
      for (int e = lane; e < E; e += 32) s[e] /= sum;
    } else {
      for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
    }
    __syncwarp();
    if (groups > 1) {
      // experts form `groups` equal groups of neighbours; a group's score is the sum of its two largest choice
      // scores (score + correction); only experts of the `keep` best groups can be chosen (ties: the lower group)
      const int per = E / groups;
      float* gs = gsc + r * groups;
      for (int g = lane; g < groups; g += 32) {
        float a = -INFINITY, b = -INFINITY;  // the largest and the second
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = correction ? s[e] + correction[e] : s[e];
          if (v > a) b = a, a = v;
          else if (v > b) b = v;
        }
        gs[g] = per > 1 ? a + b : a;
      }
      __syncwarp();
      for (int g = lane; g < groups; g += 32) {
        const float mine = gs[g];
        int ahead = 0;
        for (int o = 0; o < groups; ++o) ahead += (gs[o] > mine || (gs[o] == mine && o < g)) ? 1 : 0;
        if (ahead >= keep)
          for (int e = g * per; e < (g + 1) * per; ++e) s[e] = -INFINITY;  // never the largest: score + correction stays -inf
      }
      __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      // the choice goes by score + correction (when given), the weight is the score itself
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float v = correction ? s[e] + correction[e] : s[e];
        if (v > best) best = v, arg = e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
      if (arg >= E) arg = k, best = 0.f;
      else if (correction) best = s[arg];
      __syncwarp();
      if (lane == 0) {
        choice[(size_t)t * top + k] = arg;
        weight[(size_t)t * top + k] = best;
        s[arg] = -INFINITY;
      }
      total += best;
      __syncwarp();
    }
    if (renormalize && lane < top) weight[(size_t)t * top + lane] = weight[(size_t)t * top + lane] / (total + renorm_eps) * route_scale;
    else if (route_scale != 1.0f && lane < top) weight[(size_t)t * top + lane] *= route_scale;
    if (gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-zg));
  }
}

template <typename T, int TT>
static int moe_router_launch(int* choice, float* weight, float* gate, const void* x, const float* wr, int T_, int E, int top, int hidden, int softmax,
                             int renormalize, const float* correction, float renorm_eps, int groups, int keep, float route_scale, cudaStream_t stream) {
  const int cols = E + (gate ? 1 : 0);
  const size_t smem = ((size_t)TT * (cols + groups) + 4) * sizeof(float) + (size_t)TT * hidden * sizeof(T);
  static size_t set = 0;
  if (smem > set) {
    if (cudaFuncSetAttribute(moe_router_kernel<T, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
    set = smem;
  }
  launch_dep(moe_router_kernel<T, TT>, (T_ + TT - 1) / TT, 256, smem, stream, choice, weight, gate, (const T*)x, wr, T_, E, top, hidden, gate ? 1 : 0, softmax,
             renormalize, correction, renorm_eps, groups, keep, route_scale);
  return launch_status();
}

// correction (optional, fp32 [E]): added to the scores for the choice only.  renorm_eps: added to the sum the weights are divided by.
// groups > 1: the experts form that many equal groups of neighbours, of which only the `keep` best (by the sum of their two largest
// choice scores) can be chosen.  route_scale: a factor on the weights.
ALOFA_API int alofa_moe_router(int* choice, float* weight, float* gate, const void* x, const float* wr, int T, int E, int top, int hidden, int softmax,
                               int renormalize, int x_bf16, const float* correction, float renorm_eps, int groups, int keep, float route_scale,
                               cudaStream_t stream) {
  if (T <= 0) return ALOFA_OK;
  if (E <= 0 || top <= 0 || top > E || top > 32) return ALOFA_ERR_ARGUMENT;
  if (groups < 1) groups = 1;
  if (groups > 1 && (E % groups || keep < 1 || keep > groups || keep * (E / groups) < top)) return ALOFA_ERR_ARGUMENT;
  const size_t row = (size_t)hidden * (x_bf16 ? 2 : 4) + (size_t)(E + groups + 1) * 4;
  const size_t room = 200 * 1024;
  // few tokens: two to a block, so that a decode step's tokens are spread over more than a handful of SMs
  if (8 * row <= room && T > 512)
    return x_bf16 ? moe_router_launch<bf16, 8>(choice, weight, gate, x, wr, T, E, top, hidden, softmax, renormalize, correction, renorm_eps, groups, keep, route_scale, stream)
                  : moe_router_launch<float, 8>(choice, weight, gate, x, wr, T, E, top, hidden, softmax, renormalize, correction, renorm_eps, groups, keep, route_scale, stream);
  if (2 * row <= room)
    return x_bf16 ? moe_router_launch<bf16, 2>(choice, weight, gate, x, wr, T, E, top, hidden, softmax, renormalize, correction, renorm_eps, groups, keep, route_scale, stream)
                  : moe_router_launch<float, 2>(choice, weight, gate, x, wr, T, E, top, hidden, softmax, renormalize, correction, renorm_eps, groups, keep, route_scale, stream);
  return ALOFA_ERR_ARGUMENT;
}

ALOFA_API int alofa_moe_route(int* choice, float* weight, float* gate, const float* z, int T, int E, int top, int cols, int softmax, int renormalize,
                              cudaStream_t stream) {
  if (T <= 0) return ALOFA_OK;
  if (E <= 0 || top <= 0 || top > E || top > 32 || cols < E + (gate ? 1 : 0) || (size_t)8 * E * 4 > 48 * 1024) return ALOFA_ERR_ARGUMENT;
  launch_dep(moe_route_kernel, (T + 7) / 8, 256, (size_t)8 * E * sizeof(float), stream, choice, weight, gate, z, T, E, top, cols, softmax, renormalize);
  return launch_status();
}

// sort: the pairs (token, k) in the order of their expert, each expert's rows
// padded to whole tiles of `tile` rows.  dest[pair] = row of the sorted matrix;
// tile_expert[i] = expert of tile i, -1 for tiles past the end.  One block;
// thread e walks all pairs in order and numbers those of expert e, so the
// order within an expert is the order of the pairs.
__global__ void moe_sort_kernel(int* __restrict__ dest, int* __restrict__ tile_expert, const int* __restrict__ choice, int pairs, int E, int tile,
                                int max_tiles) {
  extern __shared__ int counts[];  // [E] counts, then [E] first rows
  pdl_begin();
  int* first = counts + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int n = 0;
    for (int i = 0; i < pairs; ++i) n += choice[i] == e;
    counts[e] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      first[e] = at;
      const int tiles = (counts[e] + tile - 1) / tile;
      for (int i = 0; i < tiles; ++i) tile_expert[at / tile + i] = e;
      at += tiles * tile;
    }
    for (int i = at / tile; i < max_tiles; ++i) tile_expert[i] = -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int at = first[e];
    for (int i = 0; i < pairs; ++i)
      if (choice[i] == e) dest[i] = at++;
  }
  for (int i = threadIdx.x; i < pairs; i += blockDim.x)
    if (choice[i] >= E) dest[i] = -1;  // a choice that is no expert with weights (an identity expert): no row
}

// The same result faster, for as many experts as shared memory holds a count per thread for: thread i
// takes the pairs [i * share, (i + 1) * share), counts them per expert, the counts of each expert are
// summed over the threads in thread order (so the order within an expert stays the order of the pairs),
// and every thread numbers its pairs from there.
constexpr int SORT_THREADS = 256;
__global__ void __launch_bounds__(SORT_THREADS) moe_sort_counted_kernel(int* __restrict__ dest, int* __restrict__ tile_expert, const int* __restrict__ choice,
                                                                        int pairs, int E, int tile, int max_tiles) {
  extern __shared__ int counted[];  // [E][SORT_THREADS] counts, then offsets; then [E] first rows
  pdl_begin();
  int* first = counted + E * SORT_THREADS;
  const int tid = threadIdx.x;
  const int share = (pairs + SORT_THREADS - 1) / SORT_THREADS;
  const int lo = min(pairs, tid * share), hi = min(pairs, lo + share);
  for (int e = 0; e < E; ++e) counted[e * SORT_THREADS + tid] = 0;
  for (int i = lo; i < hi; ++i)
    if (choice[i] < E) counted[choice[i] * SORT_THREADS + tid] += 1;
  __syncthreads();
  // an exclusive sum over the threads, per expert: a warp takes experts in turn, a lane eight threads' counts
  const int warp = tid >> 5, lane = tid & 31;
  for (int e = warp; e < E; e += SORT_THREADS / 32) {
    int* row = counted + e * SORT_THREADS;
    int v[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = row[lane * 8 + j];
      sum += v[j];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int at = incl - sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[lane * 8 + j] = at;
      at += v[j];
    }
    if (lane == 31) first[e] = incl;  // the expert's count, for now
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      const int n = first[e], tiles = (n + tile - 1) / tile;
      first[e] = at;
      for (int i = 0; i < tiles; ++i) tile_expert[at / tile + i] = e;
      at += tiles * tile;
    }
    for (int i = at / tile; i < max_tiles; ++i) tile_expert[i] = -1;
  }
  __syncthreads();
  for (int i = lo; i < hi; ++i) {
    const int e = choice[i];
    dest[i] = e < E ? first[e] + counted[e * SORT_THREADS + tid]++ : -1;  // no row for a choice that is no expert with weights
  }
}

ALOFA_API int alofa_moe_sort(int* dest, int* tile_expert, const int* choice, int pairs, int E, int tile, int max_tiles, cudaStream_t stream) {
  if (pairs <= 0) return ALOFA_OK;
  if (E <= 0 || tile <= 0 || (size_t)2 * E * 4 > 48 * 1024 || max_tiles < (pairs + tile - 1) / tile) return ALOFA_ERR_ARGUMENT;
  const size_t counted = ((size_t)E * SORT_THREADS + E) * sizeof(int);
  if (counted <= 200 * 1024) {
    static size_t set = 0;
    if (counted > set) {
      if (cudaFuncSetAttribute(moe_sort_counted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)counted) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set = counted;
    }
    launch_dep(moe_sort_counted_kernel, 1, SORT_THREADS, counted, stream, dest, tile_expert, choice, pairs, E, tile, max_tiles);
    return launch_status();
  }
  launch_dep(moe_sort_kernel, 1, 256, (size_t)2 * E * sizeof(int), stream, dest, tile_expert, choice, pairs, E, tile, max_tiles);
  return launch_status();
}

// scatter: xs[dest[pair]] = x[token] * (weight[pair] if the weight multiplies the input) in the compute dtype.
template <typename T>
__global__ void moe_scatter_kernel(T* __restrict__ xs, const T* __restrict__ x, const float* __restrict__ weight, const int* __restrict__ dest, int top,
                                   int hidden) {
  pdl_begin();
  const int pair = blockIdx.x, t = pair / top;
  const float w = weight ? weight[pair] : 1.0f;
  if (dest[pair] < 0) return;
  const size_t to = (size_t)dest[pair] * hidden, from = (size_t)t * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) xs[to + c] = weight ? from_f<T>(to_f(x[from + c]) * w) : x[from + c];
}

ALOFA_API int alofa_moe_scatter(void* xs, const void* x, const float* weight, const int* dest, int pairs, int top, int hidden, int is_bf16,
                                cudaStream_t stream) {
  if (pairs <= 0) return ALOFA_OK;
  if (is_bf16) launch_dep(moe_scatter_kernel<bf16>, pairs, 128, 0, stream, (bf16*)xs, (const bf16*)x, weight, dest, top, hidden);
  else launch_dep(moe_scatter_kernel<float>, pairs, 128, 0, stream, (float*)xs, (const float*)x, weight, dest, top, hidden);
  return launch_status();
}

// combine: y[t] = sum_k (weight[t, k] if the weight multiplies the output) * ys[dest[t, k]] + gate[t] * shared[t]  (fp32; k ascending).
// A pair without a row (dest < 0: an identity expert) contributes the token's own input x[t]; with `add` the sum is added to y.
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ y, const float* __restrict__ ys, const int* __restrict__ dest, const float* __restrict__ weight,
                                   const float* __restrict__ shared, const float* __restrict__ gate, int top, int hidden, const T* __restrict__ x, int add) {
  pdl_begin();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = dest[(size_t)t * top + k];
      const float e = row >= 0 ? ys[(size_t)row * hidden + c] : (x ? to_f(x[(size_t)t * hidden + c]) : 0.f);
      v += weight ? weight[(size_t)t * top + k] * e : e;
    }
    if (shared) v += (gate ? gate[t] : 1.0f) * shared[(size_t)t * hidden + c];
    if (add) y[(size_t)t * hidden + c] += v;
    else y[(size_t)t * hidden + c] = v;
  }
}

ALOFA_API int alofa_moe_combine(float* y, const float* ys, const int* dest, const float* weight, const float* shared, const float* gate, int T, int top,
                                int hidden, const void* x, int x_bf16, int add, cudaStream_t stream) {
  if (T <= 0) return ALOFA_OK;
  if (x_bf16) launch_dep(moe_combine_kernel<bf16>, T, 256, 0, stream, y, ys, dest, weight, shared, gate, top, hidden, (const bf16*)x, add);
  else launch_dep(moe_combine_kernel<float>, T, 256, 0, stream, y, ys, dest, weight, shared, gate, top, hidden, (const float*)x, add);
  return launch_status();
}

// mid[r, c] = silu(gu[r, c]) * gu[r, ff + c]: the gated activation of rows that hold [gate | up] side by side (fp32 sums in, compute dtype out).
template <typename T>
__global__ void gate_up_kernel(T* __restrict__ mid, const float* __restrict__ gu, long long count, int ff) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long r = i / ff;
  const int c = (int)(i - r * ff);
  const float g = gu[r * 2 * ff + c], u = gu[r * 2 * ff + ff + c];
  mid[i] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

ALOFA_API int alofa_gate_up(void* mid, const float* gu, long long rows, int ff, int out_bf16, cudaStream_t stream) {
  const long long count = rows * ff;
  if (count <= 0) return ALOFA_OK;
  if (out_bf16) launch_dep(gate_up_kernel<bf16>, (unsigned)((count + 255) / 256), 256, 0, stream, (bf16*)mid, gu, count, ff);
  else launch_dep(gate_up_kernel<float>, (unsigned)((count + 255) / 256), 256, 0, stream, (float*)mid, gu, count, ff);
  return launch_status();
}
