// Two recurrences with a state of fixed size per request, both fp32 throughout and walked token by
// token in prompts and decoding alike, so that a position's value does not depend on how the
// prompt was cut or on what else is in the batch (the order of additions is fixed by the sizes).
//
// min_gru: element by element, S_t = (1 - z_t) S_(t-1) + z_t c_t with z = sigmoid(.), the candidate
//   c = x + 1/2 where x >= 0 and sigmoid(x) where x < 0; the output is S_t * silu(gate).
//
// The gated delta rule over a matrix state per head (N key channels x P value channels), with one
// decay per head and key channel:
//   S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
// so the read-out sees the token's own write.  A value channel's column of S never meets another
// column: o_t[p] = (g S[:, p]) . q + u[p] (k . q), and u[p] needs (g S[:, p]) . k.  Both dot
// products of the decayed column are taken in one round of exchanges between the threads that
// share the column; k . q comes ready from delta_prepare.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// min_gru: u [T, ld] fp32 holds the projections' sums (biases added) at columns z_off, x_off, g_off;
// out [T, width] in the compute dtype; state [slots][>= width] fp32.  A block takes 32 channels (a
// lane each) of one request; its warps share the request's tokens of the step, a stretch of
// consecutive tokens each.  The recurrence is linear in the state, so a stretch is the map
// S -> A S + B with A = prod (1 - z_t) and B its result from a zero state: every warp finds its
// stretch's (A, B), the stretches before it give its starting state (in order, from the request's
// stored state), and it then walks its stretch and writes the outputs.  A warp reads GRU_AHEAD
// tokens' inputs before it uses the first, so that the loads do not wait on one another.  Decode
// steps are launched with one warp a block, which walks its (one) token from the stored state.
// ---------------------------------------------------------------------------
constexpr int GRU_AHEAD = 8;
constexpr int GRU_MAX_WARPS = 16;

__device__ __forceinline__ float gru_candidate(float x) { return x >= 0.f ? x + 0.5f : sigmoid_f(x); }

template <typename TO>
__global__ void __launch_bounds__(GRU_MAX_WARPS * 32) min_gru_kernel(TO* __restrict__ out, const float* __restrict__ u, int ld, int z_off, int x_off, int g_off,
                                                                      float* __restrict__ state, long long slot_stride, const int* __restrict__ q_start,
                                                                      const int* __restrict__ state_slots, int width) {
  __shared__ float seg_a[GRU_MAX_WARPS][32], seg_b[GRU_MAX_WARPS][32];
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + lane, s = blockIdx.y;
  const bool live = c < width;
  const int t0 = q_start[s], t1 = q_start[s + 1];
  if (t0 >= t1) return;  // the whole block
  const int per = (t1 - t0 + warps - 1) / warps;
  const int a = min(t0 + warp * per, t1), b = min(a + per, t1);
  const float* col = u + (live ? c : 0);
  if (warps > 1) {
    float A = 1.f, B = 0.f;
    for (int t = a; t < b; t += GRU_AHEAD) {
      float zs[GRU_AHEAD], xs[GRU_AHEAD];
#pragma unroll
      for (int i = 0; i < GRU_AHEAD; ++i) {
        const float* row = col + (size_t)min(t + i, b - 1) * ld;
        zs[i] = row[z_off];
        xs[i] = row[x_off];
      }
#pragma unroll
      for (int i = 0; i < GRU_AHEAD; ++i) {
        if (t + i >= b) break;
        const float z = sigmoid_f(zs[i]);
        B = (1.0f - z) * B + z * gru_candidate(xs[i]);
        A *= 1.0f - z;
      }
    }
    seg_a[warp][lane] = A;
    seg_b[warp][lane] = B;
    __syncthreads();
  }
  if (a >= b || !live) return;
  float* st = state + (long long)state_slots[s] * slot_stride + c;
  float S = *st;
  for (int w = 0; w < warp; ++w) S = seg_a[w][lane] * S + seg_b[w][lane];
  for (int t = a; t < b; t += GRU_AHEAD) {
    float zs[GRU_AHEAD], xs[GRU_AHEAD], gs[GRU_AHEAD];
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      const float* row = col + (size_t)min(t + i, b - 1) * ld;
      zs[i] = row[z_off];
      xs[i] = row[x_off];
      gs[i] = row[g_off];
    }
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      if (t + i >= b) break;
      const float z = sigmoid_f(zs[i]);
      S = (1.0f - z) * S + z * gru_candidate(xs[i]);
      out[(size_t)(t + i) * width + c] = from_f<TO>(S * (gs[i] / (1.0f + expf(-gs[i]))));
    }
  }
  if (b == t1) *st = S;  // the stretch that ends the request's tokens leaves the state
}

// n_tokens: rows of the step.  With as many rows as requests every request has one token.
ALOFA_API int alofa_min_gru(void* out, const float* u, int ld, int z_off, int x_off, int g_off, float* state, long long slot_stride, const int* q_start,
                            const int* state_slots, int n_seqs, int n_tokens, int width, int out_bf16, cudaStream_t stream) {
  if (n_seqs <= 0) return ALOFA_OK;
  if (width <= 0) return ALOFA_ERR_ARGUMENT;
  const dim3 grid((width + 31) / 32, n_seqs);
  // stretches of 16 tokens or more: shorter ones cost more in the (A, B) pass than they save
  int warps = 1;
  while (warps < GRU_MAX_WARPS && (long long)n_tokens >= (long long)n_seqs * warps * 2 * 16) warps *= 2;
  if (out_bf16) launch_dep(min_gru_kernel<bf16>, grid, warps * 32, 0, stream, (bf16*)out, u, ld, z_off, x_off, g_off, state, slot_stride, q_start, state_slots, width);
  else launch_dep(min_gru_kernel<float>, grid, warps * 32, 0, stream, (float*)out, u, ld, z_off, x_off, g_off, state, slot_stride, q_start, state_slots, width);
  return launch_status();
}

// ---------------------------------------------------------------------------
// delta_prepare: what the recurrence reads, once per token.  conv [T, ldc] fp32 holds the
// convolved and activated [q: G * N | k: G * N | v: H * P]; dz [T, ldz] the decays' logits (H * N of them);
// u [T, ldu] the gate logit of each head at column b_off.
//   qn = q / sqrt(sum(q^2) + unit_eps) * q_scale,  kn = k / sqrt(sum(k^2) + unit_eps)   per group
//   kq[t, g] = kn . qn
//   g[t, h, n] = exp(-exp(A_log[h]) * softplus(dz[t, h, n] + dt_bias[h, n]))
//   beta[t, h] = sigmoid(u[t, b_off + h])
// One block per token, a warp per group in turn.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ g,
                                                            float* __restrict__ beta, const float* __restrict__ conv, int ldc, const float* __restrict__ dz, int ldz,
                                                            const float* __restrict__ u, int ldu, int b_off, const float* __restrict__ dt_bias,
                                                            const float* __restrict__ A_log, int H, int G, int N, float unit_eps, float q_scale) {
  pdl_begin();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const float* row = conv + (size_t)t * ldc;
  for (int grp = warp; grp < G; grp += nwarp) {
    const float* q = row + (size_t)grp * N;
    const float* k = row + (size_t)(G + grp) * N;
    float sq = 0.f, sk = 0.f;
    for (int n = lane; n < N; n += 32) {
      sq = fmaf(q[n], q[n], sq);
      sk = fmaf(k[n], k[n], sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.0f / sqrtf(sk + unit_eps);
    float dot = 0.f;
    for (int n = lane; n < N; n += 32) {
      const float a = q[n] * rq, b = k[n] * rk;
      qn[((size_t)t * G + grp) * N + n] = a;
      kn[((size_t)t * G + grp) * N + n] = b;
      dot = fmaf(a, b, dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) kq[(size_t)t * G + grp] = dot;
  }
  for (int e = threadIdx.x; e < H * N; e += blockDim.x) {
    const int h = e / N;
    g[(size_t)t * H * N + e] = expf(-expf(A_log[h]) * softplus_f(dz[(size_t)t * ldz + e] + dt_bias[e]));
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(size_t)t * H + h] = sigmoid_f(u[(size_t)t * ldu + b_off + h]);
}

ALOFA_API int alofa_delta_prepare(float* qn, float* kn, float* kq, float* g, float* beta, const float* conv, int ldc, const float* dz, int ldz, const float* u, int ldu,
                                  int b_off, const float* dt_bias, const float* A_log, int n_tokens, int H, int G, int N, float unit_eps, float q_scale,
                                  cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (H <= 0 || G <= 0 || H % G || N <= 0) return ALOFA_ERR_ARGUMENT;
  launch_dep(delta_prepare_kernel, n_tokens, 256, 0, stream, qn, kn, kq, g, beta, conv, ldc, dz, ldz, u, ldu, b_off, dt_bias, A_log, H, G, N, unit_eps, q_scale);
  return launch_status();
}

// ---------------------------------------------------------------------------
// delta_scan: a block takes one (head, request) and PC value channels and walks the request's
// tokens of the step in order.  The NS threads that share a value channel (neighbours in a warp)
// each hold R key channels of its column in registers, four neighbours at a time: channels 4 ns ..
// 4 ns + 3, then those 4 NS further on, ... (a token's keys, queries and decays are then R / 4 loads of
// 16 bytes each, and the NS threads' loads lie side by side in shared memory).  The state lies
// in memory as [head][value channel][key channel].  Keys, queries, decays, values, beta and k . q
// of TC tokens at a time come into shared memory by asynchronous copies, the next ones while
// these are worked on.
// ---------------------------------------------------------------------------
struct DeltaArgs {
  float* y;                              // [T, H * P]
  const float* v; int ldv, v_off;        // values: v[t * ldv + v_off + h * P + p]
  const float* kn; const float* qn;      // [T, G, N]
  const float* kq;                       // [T, G]
  const float* g;                        // [T, H, N]
  const float* beta;                     // [T, H]
  float* state; long long slot_stride;
  const int* q_start; const int* state_slots;
  int H, G, N, P, NS, PC, TC, vec;
};

__device__ __forceinline__ void delta_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_cp_done() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int R>
__global__ void __launch_bounds__(256) delta_scan_kernel(const DeltaArgs a) {
  extern __shared__ __align__(16) float delta_smem[];
  const int N = a.N, P = a.P, NS = a.NS, PC = a.PC, TC = a.TC;
  const int NW = NS * R;                       // key channels a stage holds per token (zeros past N)
  const int per_stage = TC * (3 * NW + PC + 4);  // k, q, g, v, then beta and k.q (two words, padded to four)
  const int h = blockIdx.x, s = blockIdx.y, p0 = blockIdx.z * PC;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int pl = tid / NS, ns = tid - pl * NS;
  const int p = p0 + pl;
  const bool live_p = pl < PC && p < P;
  const int grp = h / (a.H / a.G);
  for (int e = tid; e < 2 * per_stage; e += nthreads) delta_smem[e] = 0.f;  // the rows' tails that no copy writes stay zero
  pdl_begin();
  const int t0 = a.q_start[s], t1 = a.q_start[s + 1];
  float* S = a.state + (long long)a.state_slots[s] * a.slot_stride + ((size_t)h * P + (live_p ? p : 0)) * N;
  float st[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int n = (j >> 2) * 4 * NS + 4 * ns + (j & 3);
    st[j] = (live_p && n < N) ? S[n] : 0.f;
  }
  __syncthreads();

  auto fetch = [&](int which, int c0) {
    float* ks = delta_smem + which * per_stage;
    float* qs = ks + TC * NW;
    float* gs = qs + TC * NW;
    float* vs = gs + TC * NW;
    float* bs = vs + TC * PC;
    const int live = min(TC, t1 - c0);
    if (a.vec) {
      const int n4 = N >> 2;
      for (int e = tid; e < live * n4; e += nthreads) {
        const int tt = e / n4, c = (e - tt * n4) * 4;
        const size_t t = c0 + tt;
        delta_cp16(ks + tt * NW + c, a.kn + (t * a.G + grp) * N + c);
        delta_cp16(qs + tt * NW + c, a.qn + (t * a.G + grp) * N + c);
        delta_cp16(gs + tt * NW + c, a.g + (t * a.H + h) * N + c);
      }
      const int p4 = PC >> 2;
      for (int e = tid; e < live * p4; e += nthreads) {
        const int tt = e / p4, c = (e - tt * p4) * 4;
        if (p0 + c < P) delta_cp16(vs + tt * PC + c, a.v + (size_t)(c0 + tt) * a.ldv + a.v_off + h * P + p0 + c);
      }
    } else {
      for (int e = tid; e < live * N; e += nthreads) {
        const int tt = e / N, c = e - tt * N;
        const size_t t = c0 + tt;
        delta_cp4(ks + tt * NW + c, a.kn + (t * a.G + grp) * N + c);
        delta_cp4(qs + tt * NW + c, a.qn + (t * a.G + grp) * N + c);
        delta_cp4(gs + tt * NW + c, a.g + (t * a.H + h) * N + c);
      }
      for (int e = tid; e < live * PC; e += nthreads) {
        const int tt = e / PC, c = e - tt * PC;
        if (p0 + c < P) delta_cp4(vs + tt * PC + c, a.v + (size_t)(c0 + tt) * a.ldv + a.v_off + h * P + p0 + c);
      }
    }
    for (int tt = tid; tt < live; tt += nthreads) {
      delta_cp4(bs + 4 * tt, a.beta + (size_t)(c0 + tt) * a.H + h);
      delta_cp4(bs + 4 * tt + 1, a.kq + (size_t)(c0 + tt) * a.G + grp);
    }
  };

  if (t0 < t1) fetch(0, t0);
  int which = 0;
  for (int c0 = t0; c0 < t1; c0 += TC, which ^= 1) {
    delta_cp_done();
    __syncthreads();  // this stage has arrived for everyone, and everyone is done with the other
    if (c0 + TC < t1) fetch(which ^ 1, c0 + TC);
    const int live = min(TC, t1 - c0);
    const float* ks = delta_smem + which * per_stage;
    const float* qs = ks + TC * NW;
    const float* gs = qs + TC * NW;
    const float* vs = gs + TC * NW;
    const float* bs = vs + TC * PC;
    for (int tt = 0; tt < live; ++tt) {
      const float4* kr = reinterpret_cast<const float4*>(ks + tt * NW) + ns;
      const float4* qr = reinterpret_cast<const float4*>(qs + tt * NW) + ns;
      const float4* gr = reinterpret_cast<const float4*>(gs + tt * NW) + ns;
      float kk[R];
      float r0 = 0.f, r1 = 0.f, w0 = 0.f, w1 = 0.f;
#pragma unroll
      for (int j4 = 0; j4 < R / 4; ++j4) {
        const float4 k4 = kr[j4 * NS], q4 = qr[j4 * NS], g4 = gr[j4 * NS];
        const int j = 4 * j4;
        kk[j] = k4.x, kk[j + 1] = k4.y, kk[j + 2] = k4.z, kk[j + 3] = k4.w;
        st[j] *= g4.x, st[j + 1] *= g4.y, st[j + 2] *= g4.z, st[j + 3] *= g4.w;
        r0 = fmaf(st[j], k4.x, r0);
        w0 = fmaf(st[j], q4.x, w0);
        r1 = fmaf(st[j + 1], k4.y, r1);
        w1 = fmaf(st[j + 1], q4.y, w1);
        r0 = fmaf(st[j + 2], k4.z, r0);
        w0 = fmaf(st[j + 2], q4.z, w0);
        r1 = fmaf(st[j + 3], k4.w, r1);
        w1 = fmaf(st[j + 3], q4.w, w1);
      }
      float r = r0 + r1, w = w0 + w1;
      for (int o = NS >> 1; o > 0; o >>= 1) {
        r += __shfl_xor_sync(0xffffffffu, r, o);
        w += __shfl_xor_sync(0xffffffffu, w, o);
      }
      const float vv = pl < PC ? vs[tt * PC + pl] : 0.f;
      const float uu = bs[4 * tt] * (vv - r);
#pragma unroll
      for (int j = 0; j < R; ++j) st[j] = fmaf(kk[j], uu, st[j]);
      if (ns == 0 && live_p) a.y[(size_t)(c0 + tt) * a.H * P + h * P + p] = fmaf(uu, bs[4 * tt + 1], w);
    }
  }
  if (live_p && t0 < t1) {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int n = (j >> 2) * 4 * NS + 4 * ns + (j & 3);
      if (n < N) S[n] = st[j];
    }
  }
}

template <int R>
static int delta_scan_launch(const DeltaArgs& a, int n_seqs, int threads, size_t smem, cudaStream_t stream) {
  static size_t set = 48 * 1024;
  if (smem > set) {
    if (cudaFuncSetAttribute(delta_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
    set = smem;
  }
  launch_dep(delta_scan_kernel<R>, dim3(a.H, n_seqs, (a.P + a.PC - 1) / a.PC), threads, smem, stream, a);
  return launch_status();
}

// spread: how many blocks the scan should have at least, if the value channels allow it.
ALOFA_API int alofa_delta_scan(float* y, const float* v, int ldv, int v_off, const float* kn, const float* qn, const float* kq, const float* g, const float* beta,
                               float* state, long long slot_stride, const int* q_start, const int* state_slots, int n_tokens, int n_seqs, int H, int G, int N, int P,
                               int spread, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return ALOFA_OK;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 1024 || P <= 0) return ALOFA_ERR_ARGUMENT;
  int R = N <= 64 ? 8 : (N <= 256 ? 16 : 32);
  // Prompt portions of few requests and heads wait on each token's chain of dependent instructions, not on
  // throughput: half the channels a thread (twice the threads to a value channel, one more level of exchange)
  // shortens it (4 heads of 128 x 256, one request of 2,048 tokens: 717 -> 610 us).  With blocks of 16 value
  // channels enough to fill the device it does not pay (8 such heads: the prompt step 4.06 -> 4.28 ms).
  if (R == 16 && N <= 128 && n_tokens >= 8 * n_seqs && (long long)H * n_seqs * ((P + 15) / 16) < spread) R = 8;
  int NS = 1;
  while (NS * R < N) NS *= 2;
  if (NS > 32) return ALOFA_ERR_ARGUMENT;
  int PC = 256 / NS;  // value channels per block, one per group of NS threads
  while (PC > 4 && PC / 2 >= P) PC /= 2;
  while (PC > 4 && PC * NS > 32 && (long long)H * n_seqs * ((P + PC - 1) / PC) < spread) PC /= 2;
  while (PC * NS < 32) PC *= 2;
  if (PC < 4) PC = 4;
  const int threads = (PC * NS + 31) / 32 * 32;
  const bool vec = N % 4 == 0 && P % 4 == 0 && PC % 4 == 0 && ldv % 4 == 0 && v_off % 4 == 0 && ((uintptr_t)v % 16 == 0) && ((uintptr_t)kn % 16 == 0) &&
                   ((uintptr_t)qn % 16 == 0) && ((uintptr_t)g % 16 == 0);
  int TC = 16;
  while (TC > 2 && (size_t)2 * TC * (3 * NS * R + PC + 4) * sizeof(float) > 160 * 1024) TC /= 2;
  const size_t smem = (size_t)2 * TC * (3 * NS * R + PC + 4) * sizeof(float);
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
  DeltaArgs a = {y, v, ldv, v_off, kn, qn, kq, g, beta, state, slot_stride, q_start, state_slots, H, G, N, P, NS, PC, TC, vec ? 1 : 0};
  if (R == 8) return delta_scan_launch<8>(a, n_seqs, threads, smem, stream);
  if (R == 16) return delta_scan_launch<16>(a, n_seqs, threads, smem, stream);
  return delta_scan_launch<32>(a, n_seqs, threads, smem, stream);
}
