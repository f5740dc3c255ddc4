// Several residual streams side by side ("hyper-connections"), and small sums of rows around them.
//
// A model may keep S copies x_1 .. x_S of the residual stream, [S][T][W] fp32.  A sublayer reads
//   u = sum_s in[s] x_s                      (then its norm: u / sqrt(mean(u^2) + eps) * w)
// and, with its output y, all streams move at once from the old ones:
//   x_t <- sum_s mix[s][t] x_s + out[t] y    (mix is indexed [from][to])
// hyper_connect does the write of one sublayer, the read (with the norm) of the next, and the
// streams' sum, any subset of the three, in one pass over the row: one block per token, the
// row's u in shared memory between the sum of squares and the scaling.  Everything is fp32 and the
// order of additions is fixed by the sizes (s ascending; the block's reduction).
#include "common.cuh"

constexpr int HYPER_MAX_STREAMS = 8;

struct HyperArgs {
  float* streams; long long plane;  // stream s at streams + s * plane, rows of `width`
  const float* y;                   // [T, W] the sublayer output to write in, or null
  const float* mix; const float* out_w;  // [S, S], [S]
  const float* in_w;                // [S] of the sublayer that reads next, or null
  const float* norm_w; float eps;   // that sublayer's norm
  void* x_out;                      // [T, W] its normed input (compute dtype), or null
  float* sum_out;                   // [T, W] the streams' sum, or null
  int S, width;
};

template <typename TO>
__global__ void __launch_bounds__(256) hyper_connect_kernel(const HyperArgs a) {
  extern __shared__ float hyper_u[];
  __shared__ float scratch[32];
  __shared__ float mix_s[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], out_s[HYPER_MAX_STREAMS], in_s[HYPER_MAX_STREAMS];
  const int S = a.S, W = a.width;
  if (threadIdx.x < S * S) mix_s[threadIdx.x] = a.y ? a.mix[threadIdx.x] : 0.f;  // weights: not written by any kernel of the step
  if (threadIdx.x < S) {
    out_s[threadIdx.x] = a.y ? a.out_w[threadIdx.x] : 0.f;
    in_s[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 0.f;
  }
  pdl_begin();
  __syncthreads();
  const size_t row = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float x[HYPER_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s) x[s] = s < S ? a.streams[(size_t)s * a.plane + row + c] : 0.f;
    if (a.y) {
      const float yv = a.y[row + c];
      float nx[HYPER_MAX_STREAMS];
#pragma unroll
      for (int t = 0; t < HYPER_MAX_STREAMS; ++t) {
        float v = 0.f;
        if (t < S) {
#pragma unroll
          for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
            if (s < S) v = fmaf(mix_s[s * S + t], x[s], v);
          v = fmaf(out_s[t], yv, v);
          a.streams[(size_t)t * a.plane + row + c] = v;
        }
        nx[t] = v;
      }
#pragma unroll
      for (int t = 0; t < HYPER_MAX_STREAMS; ++t) x[t] = nx[t];
    }
    if (a.sum_out) {
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
        if (s < S) v += x[s];
      a.sum_out[row + c] = v;
    }
    if (a.x_out) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
        if (s < S) u = fmaf(in_s[s], x[s], u);
      hyper_u[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!a.x_out) return;
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)W + a.eps);
  TO* xo = (TO*)a.x_out + row;
  for (int c = threadIdx.x; c < W; c += blockDim.x) xo[c] = from_f<TO>(hyper_u[c] * r * a.norm_w[c]);
}

ALOFA_API int alofa_hyper_connect(float* streams, long long plane, const float* y, const float* mix, const float* out_w, const float* in_w, const float* norm_w,
                                  float eps, void* x_out, float* sum_out, int n_tokens, int S, int width, int out_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (S <= 0 || S > HYPER_MAX_STREAMS || width <= 0 || (x_out && (!in_w || !norm_w)) || (y && (!mix || !out_w))) return ALOFA_ERR_ARGUMENT;
  const size_t smem = x_out ? (size_t)width * sizeof(float) : 0;
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
  HyperArgs a = {streams, plane, y, mix, out_w, in_w, norm_w, eps, x_out, sum_out, S, width};
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  if (out_bf16) {
    static size_t set = 48 * 1024;
    if (smem > set) {
      if (cudaFuncSetAttribute(hyper_connect_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set = smem;
    }
    launch_dep(hyper_connect_kernel<bf16>, n_tokens, threads, smem, stream, a);
  } else {
    static size_t set = 48 * 1024;
    if (smem > set) {
      if (cudaFuncSetAttribute(hyper_connect_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ALOFA_ERR_LAUNCH;
      set = smem;
    }
    launch_dep(hyper_connect_kernel<float>, n_tokens, threads, smem, stream, a);
  }
  return launch_status();
}

// Every stream starts as the embedding output: streams[s] = h for s < S.
__global__ void streams_fill_kernel(float* __restrict__ streams, long long plane, const float* __restrict__ h, long long count, int S) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const float v = h[i];
  for (int s = 0; s < S; ++s) streams[(size_t)s * plane + i] = v;
}

ALOFA_API int alofa_streams_fill(float* streams, long long plane, const float* h, long long count, int S, cudaStream_t stream) {
  if (count <= 0 || S <= 0) return ALOFA_OK;
  launch_dep(streams_fill_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, streams, plane, h, count, S);
  return launch_status();
}

// out (+)= sa * ya + sb * yb, elementwise fp32 (yb may be absent): the outputs of branches that ran side by side, each with its own factor.
__global__ void scaled_sum_kernel(float* __restrict__ out, const float* __restrict__ ya, float sa, const float* __restrict__ yb, float sb, long long count,
                                  int accumulate) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float v = sa * ya[i];
  if (yb) v = fmaf(sb, yb[i], v);
  out[i] = accumulate ? out[i] + v : v;
}

ALOFA_API int alofa_scaled_sum(float* out, const float* ya, float sa, const float* yb, float sb, long long count, int accumulate, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  launch_dep(scaled_sum_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, out, ya, sa, yb, sb, count, accumulate);
  return launch_status();
}

// x *= scale (fp32): logits that the design multiplies by a constant.
__global__ void scale_rows_kernel(float* __restrict__ x, float scale, long long count) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) x[i] *= scale;
}

ALOFA_API int alofa_scale_rows(float* x, float scale, long long count, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  launch_dep(scale_rows_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, x, scale, count);
  return launch_status();
}

// x = cap * tanh(x / cap) (fp32): logits that the design bounds.
__global__ void softcap_rows_kernel(float* __restrict__ x, float cap, long long count) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) x[i] = cap * tanhf(x[i] / cap);
}

ALOFA_API int alofa_softcap_rows(float* x, float cap, long long count, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  if (!(cap > 0.f)) return ALOFA_ERR_ARGUMENT;
  launch_dep(softcap_rows_kernel, (unsigned)((count + 255) / 256), 256, 0, stream, x, cap, count);
  return launch_status();
}

// o[t, h, :] *= sigmoid(g[t, g_off + h]): one gate per head from fp32 sums of a projection (row stride ldg); o in the compute dtype.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, const float* __restrict__ g, int ldg, int g_off, int heads, int vdim, long long count) {
  pdl_begin();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long th = i / vdim;
  const long long t = th / heads;
  const int h = (int)(th - t * heads);
  const float z = g[t * ldg + g_off + h];
  o[i] = from_f<T>(to_f(o[i]) / (1.0f + expf(-z)));
}

ALOFA_API int alofa_head_gate(void* o, const float* g, int ldg, int g_off, int n_tokens, int heads, int vdim, int is_bf16, cudaStream_t stream) {
  const long long count = (long long)n_tokens * heads * vdim;
  if (count <= 0) return ALOFA_OK;
  if (is_bf16) launch_dep(head_gate_kernel<bf16>, (unsigned)((count + 255) / 256), 256, 0, stream, (bf16*)o, g, ldg, g_off, heads, vdim, count);
  else launch_dep(head_gate_kernel<float>, (unsigned)((count + 255) / 256), 256, 0, stream, (float*)o, g, ldg, g_off, heads, vdim, count);
  return launch_status();
}
