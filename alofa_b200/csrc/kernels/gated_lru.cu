// The real-gated linear recurrent unit: a recurrence element by element whose decay and input gate
// are made from the (convolved) input of the current token by block-diagonal maps,
//
//   r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)       per block b of the channels
//   log a = -c * r * softplus(lam),  a = exp(log a)
//   S_t = a * S_(t-1) + sqrt(1 - a^2) * i * u
//
// and whose output is S_t times the activated other branch.  Everything here is fp32 (the gates'
// sums too: plain multiply-adds in a fixed order over the block's inputs), in prompts and decoding
// alike, so that a position's value does not depend on how the prompt was cut or on what else is
// in the batch.
#include "common.cuh"

__device__ __forceinline__ float lru_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float lru_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// lru_gates: u [T, W] fp32; wa, wi [B][bs][bs] fp32 stored [block][in][out] (the transposes of the
// checkpoint's [out, in], so that the threads of a warp read neighbouring numbers); ba, bi [W];
// lam [W] and c: log a = -c * r * softplus(lam).  Writes a [T, W] and the driven input
// b = sqrt(1 - a^2) * i * u [T, W].  A block takes TT tokens, one block of the channels and
// LRU_OT of its outputs, a thread per output; the tokens' inputs lie in shared memory.
// ---------------------------------------------------------------------------
constexpr int LRU_TT = 8;       // tokens a block of the kernel for a handful of tokens takes
constexpr int LRU_TT_LONG = 32; // and of this kernel over prompt portions: every weight is read once for so many tokens
constexpr int LRU_OT = 128;

template <int TT>
__global__ void __launch_bounds__(LRU_OT) lru_gates_kernel(float* __restrict__ a_out, float* __restrict__ b_out, const float* __restrict__ u, const float* __restrict__ wa,
                                                           const float* __restrict__ wi, const float* __restrict__ ba, const float* __restrict__ bi,
                                                           const float* __restrict__ lam, float decay_scale, int n_tokens, int W, int bs) {
  extern __shared__ __align__(16) float lru_us[];  // [TT][bs]
  pdl_begin();
  const int t0 = blockIdx.x * TT, blk = blockIdx.y, o = blockIdx.z * LRU_OT + threadIdx.x;
  const int live = min(TT, n_tokens - t0);
  for (int e = threadIdx.x; e < TT * bs; e += LRU_OT) {
    const int r = e / bs, c = e - r * bs;
    lru_us[e] = r < live ? u[(size_t)(t0 + r) * W + blk * bs + c] : 0.f;
  }
  __syncthreads();
  if (o >= bs) return;
  float sa[TT], si[TT];
#pragma unroll
  for (int r = 0; r < TT; ++r) sa[r] = si[r] = 0.f;
  const float* pa = wa + (size_t)blk * bs * bs + o;
  const float* pi = wi + (size_t)blk * bs * bs + o;
  if ((bs & 3) == 0) {
    // four inputs at a time: a token's four come in one 16-byte load from shared memory (one a thread per input made the
    // load/store unit, not the multiply-adds, the limit); every sum still takes its inputs in ascending order
#pragma unroll 2
    for (int k = 0; k < bs; k += 4) {
      float va[4], vi[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) va[j] = pa[(size_t)(k + j) * bs], vi[j] = pi[(size_t)(k + j) * bs];
#pragma unroll
      for (int r = 0; r < TT; ++r) {
        const float4 x = *reinterpret_cast<const float4*>(lru_us + r * bs + k);
        sa[r] = fmaf(va[3], x.w, fmaf(va[2], x.z, fmaf(va[1], x.y, fmaf(va[0], x.x, sa[r]))));
        si[r] = fmaf(vi[3], x.w, fmaf(vi[2], x.z, fmaf(vi[1], x.y, fmaf(vi[0], x.x, si[r]))));
      }
    }
  } else {
#pragma unroll 4
    for (int k = 0; k < bs; ++k) {
      const float va = pa[(size_t)k * bs], vi = pi[(size_t)k * bs];
#pragma unroll
      for (int r = 0; r < TT; ++r) {
        const float x = lru_us[r * bs + k];
        sa[r] = fmaf(va, x, sa[r]);
        si[r] = fmaf(vi, x, si[r]);
      }
    }
  }
  const int ch = blk * bs + o;
  const float bias_a = ba[ch], bias_i = bi[ch], rt = -decay_scale * lru_softplus(lam[ch]);
#pragma unroll
  for (int r = 0; r < TT; ++r) {
    if (r >= live) break;
    const float gate_r = lru_sigmoid(sa[r] + bias_a), gate_i = lru_sigmoid(si[r] + bias_i);
    const float log_a = rt * gate_r;  // never positive
    const float a = expf(log_a);
    const float keep = sqrtf(-expm1f(2.0f * log_a));  // sqrt(1 - a^2) without the cancellation near a = 1
    const size_t at = (size_t)(t0 + r) * W + ch;
    a_out[at] = a;
    b_out[at] = keep * gate_i * lru_us[r * bs + o];
  }
}

// The same over prompt portions as a register-tiled product: a block of 256 threads takes 64 tokens and 128 outputs of one
// block of the channels, a thread 4 tokens x 8 outputs of both gates (64 sums in registers); the inputs' and the weights'
// tiles of 16 depth entries go through shared memory, so that 64 multiply-adds stand against five 16-byte loads.  Every
// sum still takes its inputs in ascending order with the same multiply-adds as the kernel above: the same bits.
constexpr int LRU_TILE_T = 64, LRU_TILE_O = 128, LRU_TILE_K = 16;

__global__ void __launch_bounds__(256) lru_gates_tiled_kernel(float* __restrict__ a_out, float* __restrict__ b_out, const float* __restrict__ u, const float* __restrict__ wa,
                                                              const float* __restrict__ wi, const float* __restrict__ ba, const float* __restrict__ bi,
                                                              const float* __restrict__ lam, float decay_scale, int n_tokens, int W, int bs) {
  __shared__ __align__(16) float us[LRU_TILE_K][LRU_TILE_T];   // inputs, [depth][token]
  __shared__ __align__(16) float was[LRU_TILE_K][LRU_TILE_O];  // weights of the decay's gate, [depth][output]
  __shared__ __align__(16) float wis[LRU_TILE_K][LRU_TILE_O];
  pdl_begin();
  const int t0 = blockIdx.x * LRU_TILE_T, blk = blockIdx.y, o0 = blockIdx.z * LRU_TILE_O;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // tx: outputs 4 tx .. 4 tx + 3 and the same 64 further on (no two lanes of a load on one bank), ty: 4 tokens
  float sa[4][8], si[4][8];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) sa[r][c] = si[r][c] = 0.f;
  const float* wab = wa + (size_t)blk * bs * bs;
  const float* wib = wi + (size_t)blk * bs * bs;
  for (int k0 = 0; k0 < bs; k0 += LRU_TILE_K) {
    // inputs: 64 tokens x 16 depth entries, a thread four neighbouring depth entries of one token
    {
      const int r = threadIdx.x >> 2, kk = (threadIdx.x & 3) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + r < n_tokens && k0 + kk < bs) v = *reinterpret_cast<const float4*>(u + (size_t)(t0 + r) * W + blk * bs + k0 + kk);  // bs is a multiple of four
      us[kk][r] = v.x, us[kk + 1][r] = v.y, us[kk + 2][r] = v.z, us[kk + 3][r] = v.w;
    }
    // weights: 16 depth entries x 128 outputs of both gates, 16 bytes a thread and round
#pragma unroll
    for (int e = threadIdx.x; e < LRU_TILE_K * LRU_TILE_O / 4; e += 256) {
      const int kk = e / (LRU_TILE_O / 4), c = (e - kk * (LRU_TILE_O / 4)) * 4;
      float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vi = va;
      if (k0 + kk < bs && o0 + c < bs) {
        va = *reinterpret_cast<const float4*>(wab + (size_t)(k0 + kk) * bs + o0 + c);
        vi = *reinterpret_cast<const float4*>(wib + (size_t)(k0 + kk) * bs + o0 + c);
      }
      *reinterpret_cast<float4*>(&was[kk][c]) = va;
      *reinterpret_cast<float4*>(&wis[kk][c]) = vi;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LRU_TILE_K; ++kk) {
      const float4 x = *reinterpret_cast<const float4*>(&us[kk][ty * 4]);
      const float4 a0 = *reinterpret_cast<const float4*>(&was[kk][tx * 4]), a1 = *reinterpret_cast<const float4*>(&was[kk][64 + tx * 4]);
      const float4 i0 = *reinterpret_cast<const float4*>(&wis[kk][tx * 4]), i1 = *reinterpret_cast<const float4*>(&wis[kk][64 + tx * 4]);
      const float xs[4] = {x.x, x.y, x.z, x.w};
      const float as[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float is[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          sa[r][c] = fmaf(as[c], xs[r], sa[r][c]);
          si[r][c] = fmaf(is[c], xs[r], si[r][c]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int o = o0 + (c < 4 ? tx * 4 + c : 64 + tx * 4 + c - 4);
    if (o >= bs) continue;
    const int ch = blk * bs + o;
    const float bias_a = ba[ch], bias_i = bi[ch], rt = -decay_scale * lru_softplus(lam[ch]);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int t = t0 + ty * 4 + r;
      if (t >= n_tokens) break;
      const float gate_r = lru_sigmoid(sa[r][c] + bias_a), gate_i = lru_sigmoid(si[r][c] + bias_i);
      const float log_a = rt * gate_r;
      const size_t at = (size_t)t * W + ch;
      a_out[at] = expf(log_a);
      b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * gate_i * u[at];
    }
  }
}

// The same for a handful of tokens (decode steps), where the kernel above would leave most of the device idle and every
// thread waiting for its own weights: wa_rows, wi_rows [B][out][in] as the checkpoint has them; a warp takes an output
// channel at a time, its lanes share the block's inputs four neighbours each (16-byte loads of the weights' rows), and
// the lanes' shares are added in butterfly order.  The order of a sum's additions depends on the block's size alone.
constexpr int LRU_ROWS_OUT = 8;  // outputs a CTA of eight warps takes: one a warp, so that a decode step's few tokens still spread over every SM
                                 // (with 32, eight tokens of 1,280 channels ran on 40 blocks, each warp waiting for its weights four times in turn: 23 us cold)

__global__ void __launch_bounds__(256) lru_gates_rows_kernel(float* __restrict__ a_out, float* __restrict__ b_out, const float* __restrict__ u,
                                                             const float* __restrict__ wa, const float* __restrict__ wi, const float* __restrict__ ba,
                                                             const float* __restrict__ bi, const float* __restrict__ lam, float decay_scale, int n_tokens, int W, int bs) {
  extern __shared__ __align__(16) float lru_rows_us[];  // [LRU_TT][bs]
  pdl_begin();
  const int t0 = blockIdx.x * LRU_TT, blk = blockIdx.y, o0 = blockIdx.z * LRU_ROWS_OUT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int live = min(LRU_TT, n_tokens - t0);
  for (int e = threadIdx.x; e < LRU_TT * bs; e += 256) {
    const int r = e / bs, c = e - r * bs;
    lru_rows_us[e] = r < live ? u[(size_t)(t0 + r) * W + blk * bs + c] : 0.f;
  }
  __syncthreads();
  for (int o = o0 + warp; o < min(o0 + LRU_ROWS_OUT, bs); o += 8) {
    const float4* pa = reinterpret_cast<const float4*>(wa + ((size_t)blk * bs + o) * bs);
    const float4* pi = reinterpret_cast<const float4*>(wi + ((size_t)blk * bs + o) * bs);
    float sa[LRU_TT], si[LRU_TT];
#pragma unroll
    for (int r = 0; r < LRU_TT; ++r) sa[r] = si[r] = 0.f;
    for (int c = lane; c < bs / 4; c += 32) {
      const float4 va = pa[c], vi = pi[c];
#pragma unroll
      for (int r = 0; r < LRU_TT; ++r) {
        const float4 x = reinterpret_cast<const float4*>(lru_rows_us + r * bs)[c];
        sa[r] = fmaf(va.w, x.w, fmaf(va.z, x.z, fmaf(va.y, x.y, fmaf(va.x, x.x, sa[r]))));
        si[r] = fmaf(vi.w, x.w, fmaf(vi.z, x.z, fmaf(vi.y, x.y, fmaf(vi.x, x.x, si[r]))));
      }
    }
    const int ch = blk * bs + o;
    const float bias_a = ba[ch], bias_i = bi[ch], rt = -decay_scale * lru_softplus(lam[ch]);
#pragma unroll
    for (int r = 0; r < LRU_TT; ++r) {
      const float za = warp_sum(sa[r]), zi = warp_sum(si[r]);
      if (lane == 0 && r < live) {
        const float gate_r = lru_sigmoid(za + bias_a), gate_i = lru_sigmoid(zi + bias_i);
        const float log_a = rt * gate_r;
        const size_t at = (size_t)(t0 + r) * W + ch;
        a_out[at] = expf(log_a);
        b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * gate_i * lru_rows_us[r * bs + o];
      }
    }
  }
}

// wa, wi: [B][in][out]; wa_rows, wi_rows: the same matrices as [B][out][in] (may be null: then every step takes the first kernel).
ALOFA_API int alofa_lru_gates(float* a_out, float* b_out, const float* u, const float* wa, const float* wi, const float* wa_rows, const float* wi_rows, const float* ba,
                              const float* bi, const float* lam, float decay_scale, int n_tokens, int W, int blocks, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (W <= 0 || blocks <= 0 || W % blocks) return ALOFA_ERR_ARGUMENT;
  const int bs = W / blocks;
  const size_t smem = (size_t)LRU_TT * bs * sizeof(float);
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
  if (wa_rows && wi_rows && n_tokens <= 128 && bs % 4 == 0 && W % 4 == 0) {
    static size_t set_rows = 48 * 1024;
    if (smem > set_rows) {
      if (cudaFuncSetAttribute(lru_gates_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set_rows = smem;
    }
    launch_dep(lru_gates_rows_kernel, dim3((n_tokens + LRU_TT - 1) / LRU_TT, blocks, (bs + LRU_ROWS_OUT - 1) / LRU_ROWS_OUT), 256, smem, stream, a_out, b_out, u, wa_rows,
               wi_rows, ba, bi, lam, decay_scale, n_tokens, W, bs);
    return launch_status();
  }
  // prompt portions: the register-tiled kernel where blocks and rows lie on 16-byte boundaries
  if (n_tokens >= 256 && bs % 4 == 0 && W % 4 == 0 && !(((uintptr_t)u | (uintptr_t)wa | (uintptr_t)wi) & 15)) {
    launch_dep(lru_gates_tiled_kernel, dim3((n_tokens + LRU_TILE_T - 1) / LRU_TILE_T, blocks, (bs + LRU_TILE_O - 1) / LRU_TILE_O), 256, 0, stream, a_out, b_out, u, wa, wi,
               ba, bi, lam, decay_scale, n_tokens, W, bs);
    return launch_status();
  }
  // else 32 tokens a block where their inputs fit in shared memory (with 8 every block pulled its 2 x bs x 128 weights
  // from L2 for 8 tokens' worth of arithmetic, and L2 set the pace: 460 us for 4,096 tokens of 2,560 channels in blocks of 256)
  const size_t smem_long = (size_t)LRU_TT_LONG * bs * sizeof(float);
  if (n_tokens >= 8 * LRU_TT_LONG && smem_long <= 200 * 1024) {
    static size_t set_long = 48 * 1024;
    if (smem_long > set_long) {
      if (cudaFuncSetAttribute(lru_gates_kernel<LRU_TT_LONG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_long) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set_long = smem_long;
    }
    launch_dep(lru_gates_kernel<LRU_TT_LONG>, dim3((n_tokens + LRU_TT_LONG - 1) / LRU_TT_LONG, blocks, (bs + LRU_OT - 1) / LRU_OT), LRU_OT, smem_long, stream, a_out, b_out,
               u, wa, wi, ba, bi, lam, decay_scale, n_tokens, W, bs);
    return launch_status();
  }
  static size_t set = 48 * 1024;
  if (smem > set) {
    if (cudaFuncSetAttribute(lru_gates_kernel<LRU_TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
    set = smem;
  }
  launch_dep(lru_gates_kernel<LRU_TT>, dim3((n_tokens + LRU_TT - 1) / LRU_TT, blocks, (bs + LRU_OT - 1) / LRU_OT), LRU_OT, smem, stream, a_out, b_out, u, wa, wi, ba, bi, lam,
             decay_scale, n_tokens, W, bs);
  return launch_status();
}

// ---------------------------------------------------------------------------
// lru_scan: S_t = a_t S_(t-1) + b_t over each request's tokens of the step in order, out[t] = S_t *
// act(y[t]) with y the other branch's fp32 sums at column y_off of rows of ldy numbers (act: a code
// of the activations in common.cuh).  A block takes 32 channels (a lane each) of one request; its
// warps share the request's tokens of the step, a stretch of consecutive tokens each.  The
// recurrence is linear in the state, so a stretch is the map S -> A S + B with A the product of its
// decays and B its result from a zero state: every warp finds its stretch's (A, B), the stretches
// before it give its starting state (in order, from the request's stored state), and it then walks
// its stretch and writes the outputs.  A warp reads LRU_AHEAD tokens' inputs before it uses the
// first, so that the loads do not wait on one another.  Decode steps are launched with one warp a
// block, which walks its (one) token from the stored state.
// ---------------------------------------------------------------------------
constexpr int LRU_AHEAD = 8;
constexpr int LRU_MAX_WARPS = 32;

template <typename TO>
__global__ void __launch_bounds__(LRU_MAX_WARPS * 32) lru_scan_kernel(TO* __restrict__ out, const float* __restrict__ a_in, const float* __restrict__ b_in,
                                                                       const float* __restrict__ y, int ldy, int y_off, int act, float* __restrict__ state,
                                                                       long long slot_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                                                       int width) {
  __shared__ float seg_a[LRU_MAX_WARPS][32], seg_b[LRU_MAX_WARPS][32];
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + lane, s = blockIdx.y;
  const bool live = c < width;
  const int t0 = q_start[s], t1 = q_start[s + 1];
  if (t0 >= t1) return;  // the whole block
  const int per = (t1 - t0 + warps - 1) / warps;
  const int lo = min(t0 + warp * per, t1), hi = min(lo + per, t1);
  const int cc = live ? c : 0;
  if (warps > 1) {
    float A = 1.f, B = 0.f;
    for (int t = lo; t < hi; t += LRU_AHEAD) {
      float as[LRU_AHEAD], bs[LRU_AHEAD];
#pragma unroll
      for (int i = 0; i < LRU_AHEAD; ++i) {
        const size_t at = (size_t)min(t + i, hi - 1) * width + cc;
        as[i] = a_in[at];
        bs[i] = b_in[at];
      }
#pragma unroll
      for (int i = 0; i < LRU_AHEAD; ++i) {
        if (t + i >= hi) break;
        B = fmaf(as[i], B, bs[i]);
        A *= as[i];
      }
    }
    seg_a[warp][lane] = A;
    seg_b[warp][lane] = B;
    __syncthreads();
  }
  if (lo >= hi || !live) return;
  float* st = state + (long long)state_slots[s] * slot_stride + c;
  float S = *st;
  for (int w = 0; w < warp; ++w) S = fmaf(seg_a[w][lane], S, seg_b[w][lane]);
  for (int t = lo; t < hi; t += LRU_AHEAD) {
    float as[LRU_AHEAD], bs[LRU_AHEAD], ys[LRU_AHEAD];
#pragma unroll
    for (int i = 0; i < LRU_AHEAD; ++i) {
      const size_t row = (size_t)min(t + i, hi - 1);
      as[i] = a_in[row * width + c];
      bs[i] = b_in[row * width + c];
      ys[i] = y[row * ldy + y_off + c];
    }
#pragma unroll
    for (int i = 0; i < LRU_AHEAD; ++i) {
      if (t + i >= hi) break;
      S = fmaf(as[i], S, bs[i]);
      out[(size_t)(t + i) * width + c] = from_f<TO>(S * activate(ys[i], act));
    }
  }
  if (hi == t1) *st = S;  // the stretch that ends the request's tokens leaves the state
}

// n_tokens: rows of the step.  With as many rows as requests every request has one token.
ALOFA_API int alofa_lru_scan(void* out, const float* a, const float* b, const float* y, int ldy, int y_off, int act, float* state, long long slot_stride,
                             const int* q_start, const int* state_slots, int n_seqs, int n_tokens, int width, int out_bf16, cudaStream_t stream) {
  if (n_seqs <= 0) return ALOFA_OK;
  if (width <= 0) return ALOFA_ERR_ARGUMENT;
  const dim3 grid((width + 31) / 32, n_seqs);
  // stretches of 16 tokens or more: shorter ones cost more in the (A, B) pass than they save
  int warps = 1;
  while (warps < LRU_MAX_WARPS && (long long)n_tokens >= (long long)n_seqs * warps * 2 * 16) warps *= 2;
  if (out_bf16) launch_dep(lru_scan_kernel<bf16>, grid, warps * 32, 0, stream, (bf16*)out, a, b, y, ldy, y_off, act, state, slot_stride, q_start, state_slots, width);
  else launch_dep(lru_scan_kernel<float>, grid, warps * 32, 0, stream, (float*)out, a, b, y, ldy, y_off, act, state, slot_stride, q_start, state_slots, width);
  return launch_status();
}
