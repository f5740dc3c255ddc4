// Kernels of mixers that carry a state of fixed size from token to token: a short causal
// convolution per channel, and a linear recurrence over a matrix state per head,
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S is N x P: N key channels, P value channels)
//   y_t = S_t^T q_t (+ D v_t)
//
// which covers both a state-space layer with one scalar decay per head and token
// (a_t = exp(-exp(A_log) dt_t) on every row, k_t = dt_t B_t, q_t = C_t) and gated linear attention with
// one decay per key channel (a_t = sigmoid(z_t)^(1/tau)).  Beside them the norms such mixers end
// with, an embedding with a scale and a sinusoidal position vector, and the sum of several
// branches' normed outputs into the residual stream.
//
// Everything here is fp32: decays and their logarithms, softplus and exponentials, step sizes, the
// state, the sums; inputs are the fp32 sums of the projections.  A sequence's tokens are taken one
// after the other in both prompts and decoding, so a position's result does not depend on how the
// prompt was cut into steps or on what else is in the batch: for every output element the order of
// additions is fixed by the sizes alone.
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------
// Embedding: out[t, c] = table[id_t, c] * scale + pos(p_t, c), where (freq given) entry 2i of the
// position vector is sin(p f_i) and entry 2i + 1 is cos(p f_i); the angle is an fp32 product.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_scaled_kernel(float* __restrict__ out, const TW* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ src,
                                    const int* __restrict__ fed, const int* __restrict__ positions, const float* __restrict__ freq, int hidden, int vocab,
                                    float scale, int* status) {
  pdl_begin();
  const int t = blockIdx.x;
  int id = ids[t];
  if (src && src[t] >= 0) id = fed[src[t]];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && status) atomicExch(status, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  const float p = (float)positions[t];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = ok ? to_f(row[c]) * scale : 0.f;
    if (freq && ok) {
      const float ang = p * freq[c >> 1];
      v += (c & 1) ? cosf(ang) : sinf(ang);
    }
    out[(size_t)t * hidden + c] = v;
  }
}

ALOFA_API int alofa_embed_scaled(float* out, const void* table, const int* ids, const int* src, const int* fed, const int* positions, const float* freq,
                                 int n_tokens, int hidden, int vocab, float scale, int table_bf16, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (table_bf16) launch_dep(embed_scaled_kernel<bf16>, n_tokens, 256, 0, stream, out, (const bf16*)table, ids, src, fed, positions, freq, hidden, vocab, scale, status);
  else launch_dep(embed_scaled_kernel<float>, n_tokens, 256, 0, stream, out, (const float*)table, ids, src, fed, positions, freq, hidden, vocab, scale, status);
  return launch_status();
}

// out += x, elementwise (fp32).
__global__ void add_rows_kernel(float* __restrict__ out, const float* __restrict__ x, long long count) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] += x[i];
}

ALOFA_API int alofa_add_rows(float* out, const float* x, long long count, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  launch_dep(add_rows_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, out, x, count);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Causal convolution per channel with an activation (act 1: silu, 0: none): for channel c of the token at place j of its
// request, out = act(bias[c] + sum_l w[c, taps - 1 - l] * in(j - l)), l = 0 .. taps - 1 (the last
// column of w belongs to the token itself).  Inputs before the step's first token come from the
// request's state, which holds its last taps - 1 inputs (the newest last; zeros before a request's
// start).  u [T, ld] fp32, the channels at columns offset ..; out [T, channels] fp32.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) causal_conv_kernel(float* __restrict__ out, const float* __restrict__ u, int ld, int offset, const float* __restrict__ w,
                                                          const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                                                          const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                                          const int* __restrict__ seq_of_token, int channels, int taps, int act) {
  pdl_begin();
  const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= channels) return;
  const int s = seq_of_token[t];
  const int j = t - q_start[s];
  const float* st = state + (long long)state_slots[s] * slot_stride;
  float acc = bias ? bias[c] : 0.f;
  for (int l = taps - 1; l >= 0; --l) {  // the oldest input first
    const int jj = j - l;
    const float v = jj >= 0 ? u[(size_t)(t - l) * ld + offset + c] : st[(size_t)(taps - 1 + jj) * channels + c];
    acc = fmaf(w[(size_t)c * taps + taps - 1 - l], v, acc);
  }
  out[(size_t)t * channels + c] = act ? silu_f(acc) : acc;
}

// The state after the step: the last taps - 1 inputs of each request.  One thread per (request,
// channel) moves its own column: entry i becomes input number count - (taps - 1) + i of the step,
// or, where that is before the step's first token, the old entry i + count (always a later entry
// than the one being written, so ascending order reads every old value before it is overwritten).
__global__ void __launch_bounds__(256) conv_state_kernel(float* __restrict__ state, long long slot_stride, const float* __restrict__ u, int ld, int offset,
                                                         const int* __restrict__ q_start, const int* __restrict__ state_slots, int channels, int taps) {
  pdl_begin();
  const int s = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= channels) return;
  const int t0 = q_start[s], count = q_start[s + 1] - t0;
  float* st = state + (long long)state_slots[s] * slot_stride;
  for (int i = 0; i < taps - 1; ++i) {
    const int idx = count - (taps - 1) + i;
    st[(size_t)i * channels + c] = idx >= 0 ? u[(size_t)(t0 + idx) * ld + offset + c] : st[(size_t)(i + count) * channels + c];
  }
}

ALOFA_API int alofa_causal_conv(float* out, const float* u, int ld, int offset, const float* w, const float* bias, float* state, long long slot_stride,
                                const int* q_start, const int* state_slots, const int* seq_of_token, int n_tokens, int n_seqs, int channels, int taps,
                                int act, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (channels <= 0 || taps <= 0) return ALOFA_ERR_ARGUMENT;
  launch_dep(causal_conv_kernel, dim3(n_tokens, (channels + 255) / 256), 256, 0, stream, out, u, ld, offset, w, bias, (const float*)state, slot_stride, q_start,
             state_slots, seq_of_token, channels, taps, act);
  if (taps > 1)
    launch_dep(conv_state_kernel, dim3(n_seqs, (channels + 255) / 256), 256, 0, stream, state, slot_stride, u, ld, offset, q_start, state_slots, channels, taps);
  return launch_status();
}

// ---------------------------------------------------------------------------
// The recurrence, in two kernels.
//
// scan_decays: what the recurrence multiplies by, once per token, in fp32 with the precise library functions:
//   mode 0 (one decay per head and token): dt = softplus(dec[t, h] + dt_bias[h]) and a = exp(-exp(A_log[h]) * dt)
//   mode 1 (one decay per key channel):    a[n] = exp(log_sigmoid(dec[t, h, n]) / tau) = sigmoid(.)^(1/tau)
//
// linear_scan: one block takes one (request, head) and a range of value channels and walks the
// request's tokens of this step in order.  A thread holds, for two value channels, 4 * J key
// channels of the state in registers (the state lies in memory as [head][value channel][key
// channel]; a thread's key channels are the 16-byte groups ns, ns + NS, ...).  The NS threads that
// share value channels are neighbours in a warp and add their shares of y in butterfly order, four
// tokens' sums at a time so that the exchanges of one token overlap the arithmetic of the next.
// Keys, queries, decays and values of 16 tokens at a time (fewer for very wide keys) come into shared
// memory by asynchronous copies, the next ones while these are worked on.
//
//   mode 0: k_t = dt_t * b[t, g, :], q_t = c[t, g, :], y_t += D[h] * v_t      (g = h / (H / G))
//   mode 1: k_t = b[t, h, :],        q_t = c[t, h, :] * q_scale
// ---------------------------------------------------------------------------
__global__ void scan_decays_kernel(float* __restrict__ a_out, float* __restrict__ dt_out, const float* __restrict__ dec, int ldd, int d_off,
                                   const float* __restrict__ dt_bias, const float* __restrict__ A_log, float tau_inv, long long count, int cols, int mode) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long t = i / cols;
  const int c = (int)(i - t * cols);
  const float z = dec[t * ldd + d_off + c];
  if (mode == 0) {
    const float dt = softplus_f(z + (dt_bias ? dt_bias[c] : 0.f));
    dt_out[i] = dt;
    a_out[i] = expf(-expf(A_log[c]) * dt);
  } else {
    a_out[i] = expf(-softplus_f(-z) * tau_inv);
  }
}

struct ScanArgs {
  float* y;                             // [T, H * P]
  const float* v; int ldv, v_off;       // values:  v[t * ldv + v_off + h * P + p]
  const float* k; int ldk, k_off;       // keys:    k[t * ldk + k_off + g * N + n]
  const float* q; int ldq, q_off;       // queries: q[t * ldq + q_off + g * N + n]
  const float* a;                       // decays: mode 0 [T, H], mode 1 [T, H * N]
  const float* dt;                      // mode 0: step sizes [T, H]
  const float* D;
  float q_scale;
  float* state; long long slot_stride;  // state of slot s at state + s * slot_stride, [H][P][N]
  const int* q_start; const int* state_slots;
  int H, G, N, P, NS, PC, vec, TC;      // vec: every row and offset is a multiple of 4 floats (16-byte copies); TC: tokens a stage holds
};


__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_done() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int J, int MODE>
__global__ void __launch_bounds__(512) linear_scan_kernel(const ScanArgs a) {
  extern __shared__ __align__(16) float scan_smem[];
  constexpr int R = 4 * J;
  const int N = a.N, P = a.P, NS = a.NS, PC = a.PC;
  const int NW = NS * R;  // key channels a stage holds per token (zeros past N)
  const int SCAN_TC = a.TC;
  const int per_stage = SCAN_TC * (2 * NW + (MODE ? NW : 2) + PC);
  const int h = blockIdx.x, s = blockIdx.y, p0 = blockIdx.z * PC;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int pl = tid / NS, ns = tid - pl * NS;
  const int pa = p0 + 2 * pl, pb = pa + 1;
  const bool in_a = 2 * pl < PC && pa < P, in_b = 2 * pl + 1 < PC && pb < P;
  const int g = h / (a.H / a.G);
  // the tails of the rows that no copy writes stay zero: keys and queries of zero leave state and sums alone
  for (int e = tid; e < 2 * per_stage; e += nthreads) scan_smem[e] = 0.f;
  pdl_begin();
  const int t0 = a.q_start[s], t1 = a.q_start[s + 1];
  float* S = a.state + (long long)a.state_slots[s] * a.slot_stride + (size_t)h * P * N;
  float sa[R], sb[R];
#pragma unroll
  for (int j = 0; j < J; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = (j * NS + ns) * 4 + e;
      sa[j * 4 + e] = (in_a && n < N) ? S[(size_t)pa * N + n] : 0.f;
      sb[j * 4 + e] = (in_b && n < N) ? S[(size_t)pb * N + n] : 0.f;
    }
  const float dskip = (MODE == 0 && a.D) ? a.D[h] : 0.f;
  __syncthreads();

  auto stage_at = [&](int which) { return scan_smem + which * per_stage; };
  auto fetch = [&](int which, int c0) {
    float* ks = stage_at(which);
    float* qs = ks + SCAN_TC * NW;
    float* as = qs + SCAN_TC * NW;
    float* vs = as + SCAN_TC * (MODE ? NW : 2);
    const int live = min(SCAN_TC, t1 - c0);
    if (a.vec) {
      const int n4 = N >> 2;
      for (int e = tid; e < live * n4; e += nthreads) {
        const int tt = e / n4, c = (e - tt * n4) * 4;
        const size_t t = c0 + tt;
        cp_async_16(ks + tt * NW + c, a.k + t * a.ldk + a.k_off + g * N + c);
        cp_async_16(qs + tt * NW + c, a.q + t * a.ldq + a.q_off + g * N + c);
        if (MODE) cp_async_16(as + tt * NW + c, a.a + t * ((size_t)a.H * N) + h * N + c);
      }
      const int p4 = PC >> 2;
      for (int e = tid; e < live * p4; e += nthreads) {
        const int tt = e / p4, c = (e - tt * p4) * 4;
        if (p0 + c < P) cp_async_16(vs + tt * PC + c, a.v + (size_t)(c0 + tt) * a.ldv + a.v_off + h * P + p0 + c);
      }
    } else {
      for (int e = tid; e < live * N; e += nthreads) {
        const int tt = e / N, c = e - tt * N;
        const size_t t = c0 + tt;
        cp_async_4(ks + tt * NW + c, a.k + t * a.ldk + a.k_off + g * N + c);
        cp_async_4(qs + tt * NW + c, a.q + t * a.ldq + a.q_off + g * N + c);
        if (MODE) cp_async_4(as + tt * NW + c, a.a + t * ((size_t)a.H * N) + h * N + c);
      }
      for (int e = tid; e < live * PC; e += nthreads) {
        const int tt = e / PC, c = e - tt * PC;
        if (p0 + c < P) cp_async_4(vs + tt * PC + c, a.v + (size_t)(c0 + tt) * a.ldv + a.v_off + h * P + p0 + c);
      }
    }
    if (!MODE)
      for (int tt = tid; tt < live; tt += nthreads) {
        cp_async_4(as + 2 * tt, a.a + (size_t)(c0 + tt) * a.H + h);
        cp_async_4(as + 2 * tt + 1, a.dt + (size_t)(c0 + tt) * a.H + h);
      }
  };

  if (t0 < t1) fetch(0, t0);
  int which = 0;
  for (int c0 = t0; c0 < t1; c0 += SCAN_TC, which ^= 1) {
    cp_async_done();
    __syncthreads();  // this stage has arrived for everyone, and everyone is done with the other
    if (c0 + SCAN_TC < t1) fetch(which ^ 1, c0 + SCAN_TC);
    const int live = min(SCAN_TC, t1 - c0);
    const float* ks = stage_at(which);
    const float* qs = ks + SCAN_TC * NW;
    const float* as = qs + SCAN_TC * NW;
    const float* vs = as + SCAN_TC * (MODE ? NW : 2);
    for (int tt0 = 0; tt0 < live; tt0 += 4) {
      float ya[4], yb[4], xa[4], xb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int tt = tt0 + u;
        ya[u] = yb[u] = xa[u] = xb[u] = 0.f;
        if (tt < live) {
          xa[u] = 2 * pl < PC ? vs[tt * PC + 2 * pl] : 0.f;
          xb[u] = 2 * pl + 1 < PC ? vs[tt * PC + 2 * pl + 1] : 0.f;
          float dec = 0.f, ka = xa[u], kb = xb[u];
          if (MODE == 0) {
            dec = as[2 * tt];
            ka *= as[2 * tt + 1];
            kb *= as[2 * tt + 1];
          }
#pragma unroll
          for (int j = 0; j < J; ++j) {
            const int at = tt * NW + (j * NS + ns) * 4;
            const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + at);
            float4 a4 = make_float4(dec, dec, dec, dec);
            if (MODE) a4 = *reinterpret_cast<const float4*>(as + at);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              sa[j * 4 + e] = fmaf(aa[e], sa[j * 4 + e], kk[e] * ka);
              sb[j * 4 + e] = fmaf(aa[e], sb[j * 4 + e], kk[e] * kb);
              ya[u] = fmaf(sa[j * 4 + e], qq[e], ya[u]);
              yb[u] = fmaf(sb[j * 4 + e], qq[e], yb[u]);
            }
          }
        }
      }
      for (int o = NS >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          ya[u] += __shfl_xor_sync(0xffffffffu, ya[u], o);
          yb[u] += __shfl_xor_sync(0xffffffffu, yb[u], o);
        }
      }
      if (ns == 0) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (tt0 + u < live) {
            float* yr = a.y + (size_t)(c0 + tt0 + u) * a.H * P + h * P;
            if (in_a) yr[pa] = ya[u] * a.q_scale + dskip * xa[u];
            if (in_b) yr[pb] = yb[u] * a.q_scale + dskip * xb[u];
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < J; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = (j * NS + ns) * 4 + e;
      if (in_a && n < N) S[(size_t)pa * N + n] = sa[j * 4 + e];
      if (in_b && n < N) S[(size_t)pb * N + n] = sb[j * 4 + e];
    }
}

template <int J, int MODE>
static int linear_scan_launch(const ScanArgs& a, int n_seqs, int threads, size_t smem, cudaStream_t stream) {
  static size_t set = 48 * 1024;
  if (smem > set) {
    if (cudaFuncSetAttribute(linear_scan_kernel<J, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
    set = smem;
  }
  launch_dep(linear_scan_kernel<J, MODE>, dim3(a.H, n_seqs, (a.P + a.PC - 1) / a.PC), threads, smem, stream, a);
  return launch_status();
}

// work: fp32 scratch of n_tokens * (mode 0: 2 * H; mode 1: H * N) numbers for the decays.  spread: how many blocks the scan
// should have at least, if the value channels allow it (a prompt of one request has few (request, head) pairs; its value
// channels are dealt to more blocks).
ALOFA_API int alofa_linear_scan(float* y, const float* v, int ldv, int v_off, const float* b, int ldb, int b_off, const float* c, int ldc, int c_off,
                                const float* dec, int ldd, int d_off, const float* dt_bias, const float* A_log, const float* D, float tau_inv, float q_scale,
                                float* state, long long slot_stride, const int* q_start, const int* state_slots, int n_tokens, int n_seqs, int H, int G, int N,
                                int P, int mode, int spread, float* work, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return ALOFA_OK;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 1024 || P <= 0 || !work || (mode == 0 && !A_log)) return ALOFA_ERR_ARGUMENT;
  const int cols = mode ? H * N : H;
  const long long count = (long long)n_tokens * cols;
  float* a_out = work;
  float* dt_out = mode ? nullptr : work + count;
  launch_dep(scan_decays_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, a_out, dt_out, dec, ldd, d_off, dt_bias, A_log, tau_inv, count, cols, mode);
  // Key channels a thread holds (4 * J), measured on 32 heads of 128 x 64: decode steps (64 requests, a token each) are fastest
  // with 16 and 32 value channels a block (53 us against 67 with 8 and 16: fewer, longer loads of the state); prompts (2,048
  // tokens of one request) with 8 and 16 value channels a block (0.62 ms against 0.71: more warps to hide each other's waits).
  const bool prompt_like = n_tokens > 4 * n_seqs;
  const int J = N <= 32 ? 1 : (N <= 64 ? 2 : (N <= 256 ? (prompt_like ? 2 : 4) : (N <= 512 ? 4 : 8)));
  const int R = 4 * J;
  int NS = 1;
  while (NS * R < N) NS *= 2;
  if (NS > 32) return ALOFA_ERR_ARGUMENT;
  const bool vec = N % 4 == 0 && ldv % 4 == 0 && v_off % 4 == 0 && P % 4 == 0 && ldb % 4 == 0 && b_off % 4 == 0 && ldc % 4 == 0 && c_off % 4 == 0 &&
                   ((uintptr_t)v % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 16 == 0) && ((uintptr_t)work % 16 == 0);
  int PC = 2 * (512 / NS);  // value channels per block: two a thread
  while (PC > 4 && PC / 2 >= P) PC /= 2;
  if (PC > (prompt_like ? 16 : 32)) PC = prompt_like ? 16 : 32;  // more blocks of fewer warps (see above)
  while (PC > 8 && (long long)H * n_seqs * ((P + PC - 1) / PC) < spread) PC /= 2;
  if (PC < 4) PC = 4;
  const int threads = ((PC / 2) * NS + 31) / 32 * 32;
  int TC = 16;  // tokens a stage holds: fewer when the keys are so wide that two stages of 16 do not fit
  while (TC > 4 && (size_t)2 * TC * (2 * NS * R + (mode ? NS * R : 2) + PC) * sizeof(float) > 160 * 1024) TC /= 2;
  ScanArgs a = {y, v, ldv, v_off, b, ldb, b_off, c, ldc, c_off, a_out, dt_out, D, q_scale, state, slot_stride, q_start, state_slots, H, G, N, P, NS, PC, vec ? 1 : 0, TC};
  const size_t smem = (size_t)2 * TC * (2 * NS * R + (mode ? NS * R : 2) + PC) * sizeof(float);
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
#define SCAN_CASE(JJ) \
  if (J == JJ) return mode ? linear_scan_launch<JJ, 1>(a, n_seqs, threads, smem, stream) : linear_scan_launch<JJ, 0>(a, n_seqs, threads, smem, stream);
  SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8)
#undef SCAN_CASE
  return ALOFA_ERR_ARGUMENT;
}

// ---------------------------------------------------------------------------
// The norm such a mixer ends with: rows y [T, width] in `groups` equal parts, each part divided by
// its own root mean square (eps inside the root), times w[c % wlen], and a gate silu(g[t, c]) that
// multiplies either before the norm (gate_first: the gated values are what is normed) or after it.
// One block per (token, part): as many threads as the part has groups of four numbers, up to 256.
// ---------------------------------------------------------------------------
// gate_first: bit 0 = the gate multiplies before the norm; bit 1 = the gate is sigmoid(g), not silu(g)
__device__ __forceinline__ float gate_of(float z, int sigmoid) { return sigmoid ? 1.0f / (1.0f + expf(-z)) : silu_f(z); }

template <typename TO>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ gate, int ldg,
                                                               int g_off, const float* __restrict__ w, int wlen, int width, int groups, float eps,
                                                               int gate_first) {
  __shared__ float scratch[32];
  pdl_begin();
  const int t = blockIdx.x, grp = blockIdx.y;
  const int part = width / groups, lo = grp * part;
  const float* yr = y + (size_t)t * width;
  const float* gr = gate ? gate + (size_t)t * ldg + g_off : nullptr;
  float ss = 0.f;
  for (int c = lo + threadIdx.x; c < lo + part; c += blockDim.x) {
    float v = yr[c];
    if (gr && (gate_first & 1)) v *= gate_of(gr[c], gate_first & 2);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)part + eps);
  for (int c = lo + threadIdx.x; c < lo + part; c += blockDim.x) {
    float v = yr[c];
    if (gr) v *= gate_of(gr[c], gate_first & 2);  // before or after the norm, the gate is a factor of the result
    out[(size_t)t * width + c] = from_f<TO>(v * r * w[c % wlen]);
  }
}

ALOFA_API int alofa_gated_group_norm(void* out, const float* y, const float* gate, int ldg, int g_off, const float* w, int wlen, int n_tokens, int width,
                                     int groups, float eps, int gate_first, int out_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (groups <= 0 || groups > 65535 || width % groups || wlen <= 0) return ALOFA_ERR_ARGUMENT;
  const int part = width / groups;
  const int threads = part >= 1024 ? 256 : (part >= 256 ? 128 : (part >= 64 ? 64 : 32));
  const dim3 grid(n_tokens, groups);
  if (out_bf16) launch_dep(gated_group_norm_kernel<bf16>, grid, threads, 0, stream, (bf16*)out, y, gate, ldg, g_off, w, wlen, width, groups, eps, gate_first);
  else launch_dep(gated_group_norm_kernel<float>, grid, threads, 0, stream, (float*)out, y, gate, ldg, g_off, w, wlen, width, groups, eps, gate_first);
  return launch_status();
}

// ---------------------------------------------------------------------------
// h += scale * (rmsnorm(ya) * wa + rmsnorm(yb) * wb): the outputs of branches that ran side by
// side, each normed over the model width with its own plain weight, into the fp32 residual stream
// (yb may be absent).  One block per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) branch_norm_add_kernel(float* __restrict__ h, const float* __restrict__ ya, const float* __restrict__ wa,
                                                              const float* __restrict__ yb, const float* __restrict__ wb, int hidden, float eps,
                                                              float scale) {
  __shared__ float scratch[32];
  pdl_begin();
  const size_t row = (size_t)blockIdx.x * hidden;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < hidden; c += 256) {
    const float va = ya[row + c];
    sa = fmaf(va, va, sa);
    if (yb) {
      const float vb = yb[row + c];
      sb = fmaf(vb, vb, sb);
    }
  }
  sa = block_sum(sa, scratch);
  const float ra = 1.0f / sqrtf(sa / (float)hidden + eps);
  float rb = 0.f;
  if (yb) {
    sb = block_sum(sb, scratch);
    rb = 1.0f / sqrtf(sb / (float)hidden + eps);
  }
  for (int c = threadIdx.x; c < hidden; c += 256) {
    float v = ya[row + c] * ra * wa[c];
    if (yb) v += yb[row + c] * rb * wb[c];
    h[row + c] += scale * v;
  }
}

ALOFA_API int alofa_branch_norm_add(float* h, const float* ya, const float* wa, const float* yb, const float* wb, int rows, int hidden, float eps, float scale,
                                    cudaStream_t stream) {
  if (rows <= 0) return ALOFA_OK;
  launch_dep(branch_norm_add_kernel, rows, 256, 0, stream, h, ya, wa, yb, wb, hidden, eps, scale);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Queries, keys and values of softmax attention from the fp32 sums of one stacked projection, a row of ld
// numbers that starts [q: H * maps * d | k: G * maps * d | v: G * dv] (v_from_k: no v columns, the values
// are the keys as projected, before their norm).  With maps > 1 a head has several queries and a key head
// several keys, side by side ([map 1, map 2] per head): softmax maps of their own over the same values.
// q and k divided by their root mean square over d per head and map (qk_norm), times a weight of d
// numbers (q_w, k_w; may be absent); q times 1 + coef * ln(floor((p + 1) / every) + 1) at position p
// (coef != 0); the first rot_dims numbers turned in neighbouring pairs; q to its own buffer, k and v to
// the token's cache slot.  A warp per (token, head and map).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const float* __restrict__ qkv, int ld,
                                                          const int* __restrict__ positions, const int* __restrict__ slot_map, int H, int G, int d, int dv, int maps,
                                                          int qk_norm, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps, float coef, int every,
                                                          int n_tokens, const float* __restrict__ freq, int rot_dims, float mag, int v_from_k, int v_copies,
                                                          int splits, long long plane, const float* __restrict__ bias, float* __restrict__ extra_out, int extra_at,
                                                          int extra_n) {
  pdl_begin();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HQ = H * maps, GK = G * maps;
  const int per = HQ + GK + G + (extra_out ? 1 : 0);
  const long long unit = (long long)blockIdx.x * 8 + warp;
  if (unit >= (long long)n_tokens * per) return;
  const int t = (int)(unit / per), u = (int)(unit - (long long)t * per);
  const float* row = qkv + (size_t)t * ld;
  // column `col` of the token's row: the finished sum, or (splits > 0) the planes of partial sums a product left owed,
  // added in split order with the bias on top, as the kernel that settles them would have
  auto at = [&](int col) -> float {
    if (splits == 0) return row[col];
    float a = 0.f;
    for (int z = 0; z < splits; ++z) a += row[(size_t)z * plane + col];
    if (bias) a += bias[col];
    return a;
  };
  if (u < HQ + GK) {
    const int x0 = u * d;  // the unit's first column
    float mul = 1.f;
    if (qk_norm) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) {
        const float v = at(x0 + c);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      mul = 1.0f / sqrtf(ss / (float)d + eps);
    }
    T* to;
    const float* w;
    if (u < HQ) {
      if (coef != 0.f) mul *= 1.0f + coef * logf((float)((positions[t] + 1) / every) + 1.0f);
      // head h's map m goes where the heads of its key head's group lie side by side: [key head][map][head of the group]
      const int h = u / maps, m = u - h * maps, hg = H / G;
      const int g = h / hg, hh = h - g * hg;
      to = q_out + ((size_t)t * HQ + (size_t)(g * maps + m) * hg + hh) * d;
      w = q_w;
    } else {
      to = k_cache + ((size_t)slot_map[t] * GK + (u - HQ)) * d;
      w = k_w;
    }
    if (rot_dims > 0) {
      // neighbouring pairs (2i, 2i + 1), i < rot_dims / 2, turned by the angle p * freq[i] (an fp32 product, precise sine and cosine),
      // cosine and sine times mag
      const float p = (float)positions[t];
      for (int i = lane; i < rot_dims / 2; i += 32) {
        float sn, cs;
        sincosf(p * freq[i], &sn, &cs);
        sn *= mag;
        cs *= mag;
        float a = at(x0 + 2 * i) * mul, b = at(x0 + 2 * i + 1) * mul;
        if (w) a *= w[2 * i], b *= w[2 * i + 1];
        to[2 * i] = from_f<T>(a * cs - b * sn);
        to[2 * i + 1] = from_f<T>(b * cs + a * sn);
      }
    }
    if (w) for (int c = rot_dims + lane; c < d; c += 32) to[c] = from_f<T>(at(x0 + c) * mul * w[c]);
    else for (int c = rot_dims + lane; c < d; c += 32) to[c] = from_f<T>(at(x0 + c) * mul);
  } else if (u < HQ + GK + G) {
    const int gi = u - HQ - GK;
    // the values: their own columns, or (v_from_k) the keys as projected, before their norm
    const int x0 = v_from_k ? HQ * d + gi * d : (HQ + GK) * d + gi * dv;
    // v_copies > 1: the value head is written that many times side by side, one for each of the key head's keys
    T* to = v_cache + ((size_t)slot_map[t] * G + gi) * v_copies * dv;
    for (int c = lane; c < dv; c += 32) {
      const T v = from_f<T>(at(x0 + c));
      for (int k = 0; k < v_copies; ++k) to[(size_t)k * dv + c] = v;
    }
  } else {
    // what follows q, k and v in the row (a gate's logits): finished, for the kernels after the attention
    for (int c = lane; c < extra_n; c += 32) extra_out[(size_t)t * extra_n + c] = at(extra_at + c);
  }
}

// splits > 0: qkv holds that many planes of partial sums (plane z at qkv + z * plane floats) still to be added up, with bias
// (may be null) on top.  extra_out (may be null): the extra_n columns from extra_at on are written there, finished, [T, extra_n].
ALOFA_API int alofa_qkv_prepare(void* q_out, void* k_cache, void* v_cache, const float* qkv, int ld, const int* positions, const int* slot_map, int n_tokens, int H, int G,
                                int d, int dv, int maps, int qk_norm, const float* q_w, const float* k_w, float eps, float coef, int every, const float* freq,
                                int rot_dims, float mag, int v_from_k, int v_copies, int is_bf16, int splits, long long plane, const float* bias, float* extra_out,
                                int extra_at, int extra_n, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || maps <= 0 || (coef != 0.f && every <= 0) || rot_dims < 0 || rot_dims > d || (rot_dims & 1) || (rot_dims && !freq) ||
      (v_from_k && (maps != 1 || dv != d)) || v_copies < 1 || ld < (H + G) * maps * d + (v_from_k ? 0 : G * dv) || splits < 0 ||
      (splits > 0 && plane < (long long)n_tokens * ld) || (extra_out && (extra_n <= 0 || extra_at < 0 || extra_at + extra_n > ld)))
    return ALOFA_ERR_ARGUMENT;
  if (splits == 0) bias = nullptr;
  const long long units = (long long)n_tokens * ((H + G) * maps + G + (extra_out ? 1 : 0));
  const unsigned blocks = (unsigned)((units + 7) / 8);
  if (is_bf16)
    launch_dep(qkv_prepare_kernel<bf16>, blocks, 256, 0, stream, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, qkv, ld, positions, slot_map, H, G, d, dv, maps, qk_norm,
               q_w, k_w, eps, coef, every, n_tokens, freq, rot_dims, mag, v_from_k, v_copies, splits, plane, bias, extra_out, extra_at, extra_n);
  else
    launch_dep(qkv_prepare_kernel<float>, blocks, 256, 0, stream, (float*)q_out, (float*)k_cache, (float*)v_cache, qkv, ld, positions, slot_map, H, G, d, dv, maps,
               qk_norm, q_w, k_w, eps, coef, every, n_tokens, freq, rot_dims, mag, v_from_k, v_copies, splits, plane, bias, extra_out, extra_at, extra_n);
  return launch_status();
}

// ---------------------------------------------------------------------------
// heads_finish: what some attentions do to a head's output before the output projection, one warp per
// (token, head), fp32.  a [T, H * maps, dv] fp32 holds the attention outputs in the order qkv_prepare
// gave the queries ([key head][map][head of the group]); the tensor-core attention kernels leave them in bfloat16.
//   maps 1: o = a
//   maps 2: o = a_1 - lambda * a_2, then o / sqrt(mean(o^2) + eps) * post   (two softmax maps over the same values)
//   gate:   o *= sigmoid(gate[t, g_off + h])   (fp32 sums of a projection, row stride ldg)
// out [T, H * dv] in the compute dtype, heads in their own order.
// ---------------------------------------------------------------------------
template <typename T, typename TA>
__global__ void __launch_bounds__(256) heads_finish_kernel(T* __restrict__ out, const TA* __restrict__ a, const float* __restrict__ gate, int ldg, int g_off,
                                                           int H, int G, int dv, int maps, float lambda, float eps, float post, long long units) {
  pdl_begin();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 8 + warp;
  if (unit >= units) return;
  const long long t = unit / H;
  const int h = (int)(unit - t * H), hg = H / G;
  const int g = h / hg, hh = h - g * hg;
  const TA* a1 = a + ((size_t)t * H * maps + (size_t)(g * maps) * hg + hh) * dv;
  T* o = out + ((size_t)t * H + h) * dv;
  float f = 1.f;
  if (gate) f = 1.0f / (1.0f + expf(-gate[t * ldg + g_off + h]));
  if (maps == 1) {
    for (int c = lane; c < dv; c += 32) o[c] = from_f<T>(to_f(a1[c]) * f);
    return;
  }
  const TA* a2 = a1 + (size_t)hg * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float v = to_f(a1[c]) - lambda * to_f(a2[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = post / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) o[c] = from_f<T>((to_f(a1[c]) - lambda * to_f(a2[c])) * r * f);
}

// a_bf16: the maps' outputs are bfloat16 (out then is too), else fp32.
ALOFA_API int alofa_heads_finish(void* out, const void* a, const float* gate, int ldg, int g_off, int n_tokens, int H, int G, int dv, int maps, float lambda, float eps,
                                 float post, int is_bf16, int a_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (H <= 0 || G <= 0 || H % G || dv <= 0 || maps < 1 || maps > 2) return ALOFA_ERR_ARGUMENT;
  const long long units = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((units + 7) / 8);
  if (a_bf16 && !is_bf16) return ALOFA_ERR_ARGUMENT;
  if (a_bf16) launch_dep(heads_finish_kernel<bf16, bf16>, blocks, 256, 0, stream, (bf16*)out, (const bf16*)a, gate, ldg, g_off, H, G, dv, maps, lambda, eps, post, units);
  else if (is_bf16) launch_dep(heads_finish_kernel<bf16, float>, blocks, 256, 0, stream, (bf16*)out, (const float*)a, gate, ldg, g_off, H, G, dv, maps, lambda, eps, post, units);
  else launch_dep(heads_finish_kernel<float, float>, blocks, 256, 0, stream, (float*)out, (const float*)a, gate, ldg, g_off, H, G, dv, maps, lambda, eps, post, units);
  return launch_status();
}
