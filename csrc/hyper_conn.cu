// Hyper-connected residual streams with a one-number RMS norm, the xIELU activation and the gated group norm.
//
// A model with S residual streams keeps X [tokens, S, W] in fp32. Around a sublayer with output y:
//
//   write   x_t <- sum_s mix[s, t] x_s + out[t] * (ls (.) y)            (all streams at once from the old ones)
//   read    u = sum_s in[s] x_s ;  h = u / sqrt(mean(u^2) + eps) * g     (g one number; h in the GEMM dtype)
//
// b200_hc_step does the write of one sublayer and the read of the next in one pass over X (one CTA per token), like the
// sandwich norm does for a single stream. S = 1 with mix = out = in = 1 is the plain pre-norm residual sum. The entry form
// turns an embedding row into the S equal streams (normed with its own number first), the exit form only reads.
#include "common.cuh"
#include "../include/b200_ops.h"

#define B200_DISPATCH_T(dtype, ...)                                   \
  if (dtype == B200_DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else if (dtype == B200_DT_FP16) { using T = __half; __VA_ARGS__; }   \
  else if (dtype == B200_DT_FP32) { using T = float; __VA_ARGS__; }    \
  else return B200_ERR_UNSUPPORTED;

namespace b200 {

constexpr int kMaxStreams = 16;

// mode 0: write (y fp32) then read; 1: entry (y = embedding rows in dtype TE, normed by g_entry, copied to every stream)
// then read; 2: read only.
// SS: the stream count at compile time (1 .. 4: the streams of an element stay in registers), 0: any count up to kMaxStreams
template <typename TH, typename TE, int SS>
__global__ void __launch_bounds__(256)
hc_step_kernel(const void* __restrict__ y_, const float* __restrict__ ls, float* __restrict__ X, const float* __restrict__ mix,
               const float* __restrict__ outc, const float* __restrict__ g_entry, const float* __restrict__ in_next,
               const float* __restrict__ g_next, TH* __restrict__ h, float* __restrict__ xsum, int S_, int W, float eps, int mode) {
  constexpr int NS = SS ? SS : kMaxStreams;
  const int S = SS ? SS : S_;
  extern __shared__ float u_s[];                 // [W]
  __shared__ float red[32];
  __shared__ float cm[kMaxStreams * kMaxStreams], co[kMaxStreams], ci[kMaxStreams];
  const long long t = blockIdx.x;
  float* xr = X + t * (long long)S * W;
  if (threadIdx.x < S * S && mode == 0) cm[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    co[threadIdx.x] = mode == 0 ? outc[threadIdx.x] : 0.f;
    ci[threadIdx.x] = in_next ? in_next[threadIdx.x] : 1.f;
  }
  float entry_scale = 0.f;
  if (mode == 1) {
    const TE* e = reinterpret_cast<const TE*>(y_) + t * W;
    float ss = 0.f;
    for (int w = threadIdx.x; w < W; w += blockDim.x) { const float v = to_f32<TE>(e[w]); ss += v * v; }
    ss = block_sum(ss, red);
    entry_scale = rsqrtf(ss / W + eps) * g_entry[0];
  }
  __syncthreads();
  float ss = 0.f;
  for (int w = threadIdx.x; w < W; w += blockDim.x) {
    float xo[NS], xn[NS];
    if (mode == 1) {
      const float v = to_f32<TE>(reinterpret_cast<const TE*>(y_)[t * W + w]) * entry_scale;
#pragma unroll
      for (int s = 0; s < S; ++s) { xn[s] = v; xr[(long long)s * W + w] = v; }
    } else {
#pragma unroll
      for (int s = 0; s < S; ++s) xo[s] = xr[(long long)s * W + w];
      if (mode == 0) {
        const float yv = reinterpret_cast<const float*>(y_)[t * W + w] * (ls ? ls[w] : 1.f);
#pragma unroll
        for (int to = 0; to < S; ++to) {
          float a = co[to] * yv;
#pragma unroll
          for (int s = 0; s < S; ++s) a = fmaf(cm[s * S + to], xo[s], a);
          xn[to] = a;
          xr[(long long)to * W + w] = a;
        }
      } else {
#pragma unroll
        for (int s = 0; s < S; ++s) xn[s] = xo[s];
      }
    }
    float u = 0.f, sm = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) { u = fmaf(ci[s], xn[s], u); sm += xn[s]; }
    if (xsum) xsum[t * W + w] = sm;
    u_s[w] = u;
    ss += u * u;
  }
  if (h == nullptr) return;
  ss = block_sum(ss, red);
  const float sc = rsqrtf(ss / W + eps) * g_next[0];
  for (int w = threadIdx.x; w < W; w += blockDim.x) h[t * W + w] = from_f32<TH>(u_s[w] * sc);
}

// xIELU with raw parameters pq = (p, q): z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (e^z - 1 - z) + z / 2
template <typename T, int V>
__global__ void xielu_kernel(const T* __restrict__ z, T* __restrict__ y, long long n, const float* __restrict__ pq) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (i >= n) return;
  const float p = pq[0], q = pq[1];
  const float ap = p > 20.f ? p : log1pf(expf(p));
  const float aq = 0.5f + (q > 20.f ? q : log1pf(expf(q)));
  T in[V], ov[V];
  if (V > 1) *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(z + i);
  else in[0] = z[i];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const float v = to_f32<T>(in[j]);
    // 16-bit outputs take the fast exponential (its error is far below their rounding); fp32 keeps expm1f, whose result
    // stays accurate where exp(v) - 1 cancels
    const float em1 = sizeof(T) == 4 ? expm1f(fminf(v, 0.f)) : __expf(fminf(v, 0.f)) - 1.f;
    ov[j] = from_f32<T>(v > 0.f ? ap * v * v + 0.5f * v : aq * (em1 - v) + 0.5f * v);
  }
  if (V > 1) *reinterpret_cast<uint4*>(y + i) = *reinterpret_cast<const uint4*>(ov);
  else y[i] = ov[0];
}

// out[t, g, :] = o[t, g, :] / sqrt(mean_g(o^2) + eps) * w[:] * sigmoid(gate[t, g, :])   (groups of GS columns; w [GS] shared)
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ld_gate, const float* __restrict__ w,
                        T* __restrict__ out, int NG, int GS, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int g = blockIdx.y;
  const float* orow = o + (t * NG + g) * (long long)GS;
  float ss = 0.f;
  for (int c = threadIdx.x; c < GS; c += blockDim.x) { const float v = orow[c]; ss += v * v; }
  ss = block_sum(ss, red);
  const float sc = rsqrtf(ss / GS + eps);
  for (int c = threadIdx.x; c < GS; c += blockDim.x) {
    float v = orow[c] * sc * w[c];
    if (gate) v *= 1.f / (1.f + expf(-gate[t * ld_gate + (long long)g * GS + c]));
    out[(t * NG + g) * (long long)GS + c] = from_f32<T>(v);
  }
}
}  // namespace b200

B200_API int b200_hc_step(const void* y, const float* ls, float* X, const float* mix, const float* outc, const float* g_entry,
                          const float* in_next, const float* g_next, void* h, float* xsum, long long tokens, int S, int W,
                          float eps, int mode, int h_dtype, int e_dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (S < 1 || S > kMaxStreams || W <= 0 || mode < 0 || mode > 2) return B200_ERR_BAD_SHAPE;
  if ((size_t)W * 4 > 200 * 1024) return B200_ERR_TOO_LARGE;
  const size_t smem = (size_t)W * 4;
  cudaStream_t st = (cudaStream_t)stream;
#define HC_LAUNCH_S(TH, TE, SS)                                                                                            \
  do {                                                                                                                     \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(hc_step_kernel<TH, TE, SS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    hc_step_kernel<TH, TE, SS><<<(unsigned)tokens, 256, smem, st>>>(y, ls, X, mix, outc, g_entry, in_next, g_next, (TH*)h, xsum, S, W, eps, mode); \
  } while (0)
#define HC_LAUNCH(TH, TE)                                                                                                  \
  do {                                                                                                                     \
    if (S == 1) HC_LAUNCH_S(TH, TE, 1); else if (S == 2) HC_LAUNCH_S(TH, TE, 2); else if (S == 3) HC_LAUNCH_S(TH, TE, 3);  \
    else if (S == 4) HC_LAUNCH_S(TH, TE, 4); else HC_LAUNCH_S(TH, TE, 0);                                                  \
  } while (0)
  if (h_dtype == B200_DT_FP32) {
    if (e_dtype == B200_DT_FP32) HC_LAUNCH(float, float); else if (e_dtype == B200_DT_BF16) HC_LAUNCH(float, __nv_bfloat16); else HC_LAUNCH(float, __half);
  } else if (h_dtype == B200_DT_BF16) {
    if (e_dtype == B200_DT_FP32) HC_LAUNCH(__nv_bfloat16, float); else if (e_dtype == B200_DT_BF16) HC_LAUNCH(__nv_bfloat16, __nv_bfloat16); else return B200_ERR_UNSUPPORTED;
  } else {
    if (e_dtype == B200_DT_FP32) HC_LAUNCH(__half, float); else if (e_dtype == B200_DT_FP16) HC_LAUNCH(__half, __half); else return B200_ERR_UNSUPPORTED;
  }
#undef HC_LAUNCH
#undef HC_LAUNCH_S
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_xielu(const void* z, void* y, long long n, const float* pq, int dtype, void* stream) {
  using namespace b200;
  if (n <= 0) return 0;
  const int V = dtype == B200_DT_FP32 ? 4 : 8;
  const bool vec = n % V == 0 && !((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(y)) & 15);
  const unsigned grid = (unsigned)(((vec ? n / V : n) + 255) / 256);
  if (vec) { B200_DISPATCH_T(dtype, xielu_kernel<T, 16 / sizeof(T)><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)y, n, pq)); }
  else { B200_DISPATCH_T(dtype, xielu_kernel<T, 1><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)y, n, pq)); }
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_gated_group_norm(const float* o, const float* gate, long long ld_gate, const float* w, void* out, long long tokens,
                                   int NG, int GS, float eps, int dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (NG <= 0 || GS <= 0 || NG > 65535) return B200_ERR_BAD_SHAPE;
  dim3 grid((unsigned)tokens, NG);
  B200_DISPATCH_T(dtype, gated_group_norm_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(o, gate, ld_gate, w, (T*)out, NG, GS, eps));
  B200_LAUNCH_CHECK();
  return 0;
}
