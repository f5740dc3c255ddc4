// Latent attention on tensor cores for bfloat16, built per latent size
// (-DKV_RANK=..., -DROT=...): prompt portions and decode tokens of a step.
//
// Every head of a token attends to the same cached rows [c | kr] (width D =
// KV_RANK + ROT), so heads are packed on the row axis: row r of a request's
// portion is (token r / heads, head r % heads), and a CTA owns 64 consecutive
// rows, which lie contiguously in the absorbed-query matrix qa [T, heads, D].  A
// decode token alone gives `heads` rows, a prompt portion many tiles.  Keys come
// in blocks of 32 rows of the paged cache (cp.async, a ring of blocks); the same
// block in shared memory is the key operand (all D columns) and the value
// operand (its first KV_RANK columns).  Eight warps: warp = (row group of 16
// rows, half of the value columns).  The two warps of a row group share the
// group's scores S = Q K^T (mma.sync m16n8k16, fp32 sums over D): each takes 16
// of the block's 32 keys, they exchange the rows' maxima through shared memory
// behind a two-warp barrier, take the streaming softmax in fp32 in registers
// (exp2 of scores scaled by scale * log2 e), round the weights to bfloat16 -
// one warp's 16 keys are exactly one A fragment of the second product -,
// exchange fragments and sums, and each adds P V for its half of the columns
// into fp32 accumulators in registers (KV_RANK / 4 per thread).  The sink enters as the initial state of a row:
// maximum = sink, sum = 1, nothing added to the output.
//
// Causal bound and window go by the row's own position; keys past the request's
// length are never fetched (their rows in shared memory are zeroed).
//
// Decode steps split each request's key blocks over grid.z CTAs (a request alone
// is one CTA per 64 rows, far fewer than there are SMs): every split leaves its
// normalised output, maximum and sum in fp32, the sink enters in split 0 only,
// and a second kernel merges the splits in split order.
#include "common.cuh"

#ifndef KV_RANK
#define KV_RANK 64
#endif
#ifndef ROT
#define ROT 16
#endif

namespace {

constexpr int D = KV_RANK + ROT;
constexpr int PITCH = D + 8;          // elements per row in shared memory: 16 bytes of padding keep ldmatrix off bank conflicts
constexpr int BN = 32;                // keys per block
// Two shapes of the CTA.  Wide: four row groups (64 rows), eight warps, three key blocks in flight: prompt
// portions, and decode tokens of more than 16 heads.  Narrow: one row group (16 rows), two warps, two key
// blocks in flight, two CTAs to an SM: decode tokens of up to 16 heads, whose rows would fill a quarter of
// the wide tile while its other warps only fetched.
constexpr int MIN_CTAS_WIDE = KV_RANK <= 256 ? 2 : 1;  // the output accumulators are KV_RANK / 4 registers a thread
constexpr int HALF = KV_RANK / 2;     // value columns per warp
constexpr int NT = HALF / 8;          // n-tiles of the output per warp
static_assert(KV_RANK % 32 == 0 && D % 16 == 0, "latent sizes this kernel takes");

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src)); }
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
constexpr int XCHG_BYTES = 2 * 16 * 4 + 2 * 16 * 4 + 2 * 32 * 16;  // per row group
// the two warps of row group `rg` meet (named barriers 1..4; barrier 0 is the block's)
__device__ __forceinline__ void pair_sync(int rg) { asm volatile("bar.sync %0, 64;" ::"r"(rg + 1) : "memory"); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int GROUPS, int STAGES>
__global__ void __launch_bounds__(GROUPS * 64, GROUPS == 1 ? 2 : MIN_CTAS_WIDE)
latent_attention_bf16_kernel(bf16* __restrict__ out, const bf16* __restrict__ qa, const bf16* __restrict__ cache, const float* __restrict__ sink,
                             const int* __restrict__ q_start, const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_blocks,
                             int page_size, int heads, int window, float scale_log2, float* __restrict__ part_o, float* __restrict__ part_ml,
                             int blocks_per_split, int total_rows) {
  constexpr int BM = 16 * GROUPS, THREADS = 64 * GROUPS;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);      // [BM][PITCH]
  bf16* Ks = Qs + BM * PITCH;                        // [STAGES][BN][PITCH]
  // what the two warps of a row group hand one another per key block: maxima and sums of their 16 keys per row, their weight fragments
  uint8_t* xchg = reinterpret_cast<uint8_t*>(Ks + (size_t)STAGES * BN * PITCH) + (size_t)((threadIdx.x >> 5) % GROUPS) * XCHG_BYTES;
  float* x_max = reinterpret_cast<float*>(xchg);           // [2][16]
  float* x_sum = x_max + 32;                                // [2][16]
  uint4* x_frag = reinterpret_cast<uint4*>(x_sum + 32);     // [2][32]
  pdl_begin();
  const int seq = blockIdx.y, tile = blockIdx.x;
  const int t0 = q_start[seq], q_len = q_start[seq + 1] - t0;
  const int rows = q_len * heads, r0 = tile * BM;
  if (r0 >= rows) return;
  const int n_keys = kv_len[seq];            // rows of this request in the cache after this step
  const int pos0 = n_keys - q_len;           // position of the portion's first token
  const int* table = block_table + (size_t)seq * max_blocks;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp % GROUPS, ch = warp / GROUPS, g = lane >> 2, t = lane & 3;

  // the query tile: 64 consecutive rows of qa
  {
    const bf16* src = qa + ((size_t)t0 * heads + r0) * D;
    const int live = min(BM, rows - r0);
    constexpr int CHUNKS = D / 8;
    for (int e = tid; e < BM * CHUNKS; e += THREADS) {
      const int r = e / CHUNKS, c = e - r * CHUNKS;
      if (r < live) cp16(smem_addr(Qs + r * PITCH + c * 8), src + (size_t)r * D + c * 8);
      else *reinterpret_cast<uint4*>(Qs + r * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  // keys this tile needs: up to the position of its last row, from the window's start of its first row
  const int last_row = min(r0 + BM, rows) - 1;
  const int key_hi = pos0 + last_row / heads;  // inclusive
  int key_lo = 0;
  if (window > 0) key_lo = max(0, pos0 + r0 / heads - window + 1);
  int b_lo = key_lo / BN, b_hi = key_hi / BN;
  const bool split = gridDim.z > 1;
  if (split) {  // this CTA's share of the key blocks (it may be empty)
    b_lo = max(b_lo, (int)blockIdx.z * blocks_per_split);
    b_hi = min(b_hi, ((int)blockIdx.z + 1) * blocks_per_split - 1);
  }

  // A block's rows are dealt to the threads, THREADS / BN threads to a row: a thread finds its row's slot
  // once (one division, one block-table entry) and copies every (THREADS / BN)-th 16-byte chunk of the row.
  auto fetch = [&](int b, int buf) {
    constexpr int CHUNKS = D / 8, PER_ROW = THREADS / BN;
    const int j = tid / PER_ROW, c0 = tid - j * PER_ROW;
    bf16* dst = Ks + ((size_t)buf * BN + j) * PITCH;
    const int key = b * BN + j;
    if (key >= key_lo && key <= key_hi) {  // rows before the window may lie in a page that was given back: its table entry names no page
      const int page = key / page_size;
      const bf16* src = cache + ((size_t)table[page] * page_size + (key - page * page_size)) * D;
#pragma unroll 4
      for (int c = c0; c < CHUNKS; c += PER_ROW) cp16(smem_addr(dst + c * 8), src + c * 8);
    } else {
      for (int c = c0; c < CHUNKS; c += PER_ROW) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    }
  };
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (b_lo + st <= b_hi) fetch(b_lo + st, st);
    cp_commit();
  }

  // this thread's two rows of its group: g and g + 8
  int pos[2], first[2];
  float m[2], l[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + rg * 16 + g + 8 * i;
    const bool live = r < rows;
    pos[i] = live ? pos0 + r / heads : -1;
    first[i] = (window > 0 && live) ? max(0, pos[i] - window + 1) : 0;
    const bool sunk = live && sink != nullptr && blockIdx.z == 0;
    m[i] = sunk ? sink[r % heads] * 1.4426950408889634f : -INFINITY;
    l[i] = sunk ? 1.f : 0.f;
  }
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int k = 0; k < 4; ++k) o[j][k] = 0.f;

  const uint32_t q_base = smem_addr(Qs + (rg * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8);
  for (int b = b_lo; b <= b_hi; ++b) {
    const int buf = (b - b_lo) % STAGES;
    if (b + STAGES - 1 <= b_hi) fetch(b + STAGES - 1, (b - b_lo + STAGES - 1) % STAGES);  // into the buffer of the block before this one, read out
    cp_commit();
    cp_wait<STAGES - 1>();
    __syncthreads();
    const bf16* Kb = Ks + (size_t)buf * BN * PITCH;
    if (r0 + rg * 16 >= rows) {  // a row group without a live row (a decode token's heads fill a part of the tile): it only helps to fetch
      __syncthreads();
      continue;
    }
    // S = Q K^T for 16 rows x this warp's 16 keys of the block (the group's other warp takes the other 16)
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) s[j][k] = 0.f;
    const uint32_t k_base = smem_addr(Kb + (ch * 16 + (lane & 7) + (lane >> 4) * 8) * PITCH + ((lane >> 3) & 1) * 8);
#pragma unroll 4
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t a[4], kb[4];
      ldsm4(a, q_base + k0 * 2);
      ldsm4(kb, k_base + k0 * 2);
      mma16816(s[0], a, kb[0], kb[1]);
      mma16816(s[1], a, kb[2], kb[3]);
    }
    // mask; the rows' maxima over the warp's keys, then over the group's (in units of log2)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = k >> 1;
        const int key = b * BN + ch * 16 + j * 8 + 2 * t + (k & 1);
        const float v = (key <= pos[i] && key >= first[i]) ? s[j][k] * scale_log2 : -INFINITY;
        s[j][k] = v;
        mx[i] = fmaxf(mx[i], v);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      if (t == 0) x_max[ch * 16 + g + 8 * i] = mx[i];
    }
    pair_sync(rg);
    float corr[2], sum[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float m_new = fmaxf(m[i], fmaxf(mx[i], x_max[(ch ^ 1) * 16 + g + 8 * i]));
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[i] = exp2f(m[i] - m_use);  // m = -inf: 0
      m[i] = m_new;
      sum[i] = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][2 * i] = exp2f(s[j][2 * i] - m_use);
        s[j][2 * i + 1] = exp2f(s[j][2 * i + 1] - m_use);
        sum[i] += s[j][2 * i] + s[j][2 * i + 1];
      }
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      if (t == 0) x_sum[ch * 16 + g + 8 * i] = sum[i];
    }
    // the weights of the warp's 16 keys, rounded, are one A fragment of the second product: both warps need both
    uint4 mine;
    mine.x = pack2(s[0][0], s[0][1]);
    mine.y = pack2(s[0][2], s[0][3]);
    mine.z = pack2(s[1][0], s[1][1]);
    mine.w = pack2(s[1][2], s[1][3]);
    x_frag[ch * 32 + lane] = mine;
    pair_sync(rg);
    const uint4 other = x_frag[(ch ^ 1) * 32 + lane];
#pragma unroll
    for (int i = 0; i < 2; ++i) l[i] = l[i] * corr[i] + (x_sum[g + 8 * i] + x_sum[16 + g + 8 * i]);  // keys 0-15 first, in both warps
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
    // O += P V over this warp's half of the value columns, all 32 keys
    const uint32_t v_base = smem_addr(Kb + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + ch * HALF + (lane >> 4) * 8);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const uint4 f = kk == ch ? mine : other;
      const uint32_t p[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t v[4];
        ldsm4_t(v, v_base + (kk * 16 * PITCH + j * 8) * 2);
        mma16816(o[j], p, v[0], v[1]);
        mma16816(o[j + 1], p, v[2], v[3]);
      }
    }
    __syncthreads();  // the block is read out: its buffer may be refilled
  }
  cp_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + rg * 16 + g + 8 * i;
    if (r >= rows) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    if (split) {
      const size_t row = (size_t)blockIdx.z * total_rows + (size_t)t0 * heads + r;
      float* dst = part_o + row * KV_RANK + ch * HALF + 2 * t;
#pragma unroll
      for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
      if (ch == 0 && t == 0) *reinterpret_cast<float2*>(part_ml + row * 2) = make_float2(m[i], l[i]);
      continue;
    }
    bf16* dst = out + ((size_t)t0 * heads + r) * KV_RANK + ch * HALF + 2 * t;
#pragma unroll
    for (int j = 0; j < NT; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8) = pack2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
  }
}

// out[row] = sum_z w_z o_z / sum_z w_z with w_z = l_z 2^(m_z - max m), splits in ascending order.
__global__ void latent_attention_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                              int total_rows) {
  pdl_begin();
  const size_t row = blockIdx.x;
  float top = -INFINITY;
  for (int z = 0; z < splits; ++z) top = fmaxf(top, part_ml[((size_t)z * total_rows + row) * 2]);
  for (int c = threadIdx.x; c < KV_RANK; c += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)z * total_rows + row) * 2);
      const float w = ml.y > 0.f ? ml.y * exp2f(ml.x - top) : 0.f;
      num = fmaf(w, part_o[((size_t)z * total_rows + row) * KV_RANK + c], num);
      den += w;
    }
    out[row * KV_RANK + c] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
  }
}

}  // namespace

// qa [T, heads, D], out [T, heads, KV_RANK], cache [slots, D]: bfloat16.  max_q_len: the longest portion of the
// step (or, for a recorded step, the longest it may hold).
ALOFA_API int alofa_latent_attention_bf16(void* out, const void* qa, const void* cache, const float* sink, const int* q_start, const int* kv_len,
                                          const int* block_table, int max_blocks, int page_size, int n_seqs, int max_q_len, int heads, int window,
                                          float scale, float* part_o, float* part_ml, int splits, int blocks_per_split, int total_rows,
                                          cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return ALOFA_OK;
  if (heads <= 0 || page_size <= 0) return ALOFA_ERR_ARGUMENT;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!part_o || !part_ml || blocks_per_split <= 0 || total_rows <= 0 || splits > 65535)) return ALOFA_ERR_ARGUMENT;
  const bool narrow = (long long)max_q_len * heads <= 16;
  const int bm = narrow ? 16 : 64, stages = narrow ? 2 : 3;
  const size_t smem = (size_t)(bm + stages * BN) * PITCH * sizeof(bf16) + (size_t)(narrow ? 1 : 4) * XCHG_BYTES;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(latent_attention_bf16_kernel<4, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((64 + 3 * BN) * PITCH * sizeof(bf16) + 4 * XCHG_BYTES)) != cudaSuccess ||
        cudaFuncSetAttribute(latent_attention_bf16_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((16 + 2 * BN) * PITCH * sizeof(bf16) + XCHG_BYTES)) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    set = true;
  }
  const long long tiles = ((long long)max_q_len * heads + bm - 1) / bm;
  if (tiles > 2147483647LL || n_seqs > 65535) return ALOFA_ERR_ARGUMENT;
  if (narrow)
    launch_dep(latent_attention_bf16_kernel<1, 2>, dim3((unsigned)tiles, n_seqs, splits), dim3(64), smem, stream, (bf16*)out, (const bf16*)qa, (const bf16*)cache,
               sink, q_start, kv_len, block_table, max_blocks, page_size, heads, window, scale * 1.4426950408889634f, part_o, part_ml, blocks_per_split,
               total_rows);
  else
    launch_dep(latent_attention_bf16_kernel<4, 3>, dim3((unsigned)tiles, n_seqs, splits), dim3(256), smem, stream, (bf16*)out, (const bf16*)qa, (const bf16*)cache,
               sink, q_start, kv_len, block_table, max_blocks, page_size, heads, window, scale * 1.4426950408889634f, part_o, part_ml, blocks_per_split,
               total_rows);
  if (splits > 1) launch_dep(latent_attention_merge_kernel, dim3(total_rows), dim3(128), 0, stream, (bf16*)out, part_o, part_ml, splits, total_rows);
  return launch_status();
}

ALOFA_API int alofa_latent_attention_bf16_sizes(int* kv_rank, int* rot) {
  *kv_rank = KV_RANK;
  *rot = ROT;
  return (int)((64 + 3 * BN) * PITCH * sizeof(bf16) + 4 * XCHG_BYTES);
}
