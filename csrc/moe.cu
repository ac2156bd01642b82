// Mixture-of-experts routing and combination around the grouped GEMMs.
//
//   b200_moe_route     router logits z = W_r h (+ bias) in fp32 (h may be 16-bit, W_r 16-bit or fp32), the `top` largest
//                      experts per token and their weights. mode 0: softmax over the chosen logits only; mode 1: softmax
//                      over all experts, chosen probabilities kept as they are; mode 2: mode 1 renormalised to sum 1.
//                      One warp per token; ties go to the lower expert index.
//   b200_moe_route_grouped   router with group-limited choice: s = sigmoid(W_r h) (or softmax over the experts); the choice is made on
//                      s + correction, only among the experts of the `keep` groups (of `groups` equal runs of neighbours)
//                      whose `group_top` largest choice scores sum highest; the weights are s of the chosen experts, as
//                      they are or renormalised to sum 1. Rows of W_r past the experts are per-token gates: their sigmoid
//                      goes to gate_out (the gate of a shared expert). One warp per token; ties go to the lower index.
//   b200_moe_dispatch  the expert-sorted, tile-padded row layout of the assignments (a stable counting sort in one launch).
//   b200_moe_combine   out[t] = sum_k p[t, k] * y[dest[t * top + k]] (+ gate[t] * shared[t]) in fp32 (y: the expert-sorted
//                      rows the grouped GEMM wrote), a fixed order of additions per token.
#include "common.cuh"
#include "../include/b200_ops.h"

namespace b200 {

template <typename T> __device__ __forceinline__ void route_load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void route_load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void route_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(q[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

// z[r] = W_r[r, :] . h for r < rows, by one warp, fp32 accumulation. Rows are taken eight at a time so that eight rows' loads
// are in flight per lane (a row after the other waits a memory round trip per 32 columns); 16-byte loads where the width
// and the pointers allow, lane-strided scalar loads otherwise. Lane 0 writes z.
template <typename TH, typename TW>
__device__ __forceinline__ void route_logits(const TH* __restrict__ hr, const TW* __restrict__ wr, int W, int rows, int lane,
                                             float* __restrict__ z) {
  constexpr int EB = 8;
  const bool vec = W % 8 == 0 && ((reinterpret_cast<uintptr_t>(hr) | reinterpret_cast<uintptr_t>(wr)) & 15) == 0;
  for (int e0 = 0; e0 < rows; e0 += EB) {
    float acc[EB];
    const TW* wrow[EB];
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      acc[j] = 0.f;
      wrow[j] = wr + (long long)min(e0 + j, rows - 1) * W;      // rows past the last repeat it: every load is unconditional
    }
    if (vec) {
      for (int c = lane * 8; c < W; c += 256) {
        float hv[8];
        route_load8<TH>(hr + c, hv);
#pragma unroll
        for (int j = 0; j < EB; ++j) {
          float wv[8];
          route_load8<TW>(wrow[j] + c, wv);
#pragma unroll
          for (int x = 0; x < 8; ++x) acc[j] = fmaf(hv[x], wv[x], acc[j]);
        }
      }
    } else {
      for (int i = lane; i < W; i += 32) {
        const float hv = to_f32<TH>(hr[i]);
#pragma unroll
        for (int j = 0; j < EB; ++j) acc[j] = fmaf(hv, to_f32<TW>(wrow[j][i]), acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      const float a = warp_sum(acc[j]);
      if (lane == 0 && e0 + j < rows) z[e0 + j] = a;
    }
  }
}

template <typename TH, typename TW>
__global__ void __launch_bounds__(128)
moe_route_kernel(const TH* __restrict__ h, const TW* __restrict__ wr, const float* __restrict__ bias, long long* __restrict__ top_i,
                 float* __restrict__ top_p, float* __restrict__ logits_out, long long tokens, int W, int E, int top, int mode) {
  extern __shared__ float zbuf[];                     // [warps, E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* z = zbuf + warp * E;
  const TH* hr = h + t * W;
  route_logits<TH, TW>(hr, wr, W, E, lane, z);
  __syncwarp();
  if (lane != 0) return;
  for (int e = 0; e < E; ++e) {
    z[e] += bias ? bias[e] : 0.f;
    if (logits_out) logits_out[t * E + e] = z[e];
  }
  float zmax = -INFINITY, zsum = 0.f;
  if (mode != 0) {
    for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, z[e]);
    for (int e = 0; e < E; ++e) zsum += expf(z[e] - zmax);
  }
  float first = 0.f, psum = 0.f;
  for (int k = 0; k < top; ++k) {
    int best = 0;
    float bv = z[0];
    for (int e = 1; e < E; ++e)
      if (z[e] > bv) { best = e; bv = z[e]; }
    z[best] = -INFINITY;                               // taken
    top_i[t * top + k] = best;
    if (k == 0) first = bv;
    const float pv = mode == 0 ? expf(bv - first) : expf(bv - zmax) / zsum;
    top_p[t * top + k] = pv;
    psum += pv;
  }
  if (mode == 0 || mode == 2)
    for (int k = 0; k < top; ++k) top_p[t * top + k] /= psum;
}

template <typename TH, typename TW>
__global__ void __launch_bounds__(128)
moe_route_grouped_kernel(const TH* __restrict__ h, const TW* __restrict__ wr, const float* __restrict__ corr,
                         long long* __restrict__ top_i, float* __restrict__ top_p, float* __restrict__ gate_out, long long tokens,
                         int W, int E, int X, int top, int groups, int keep, int group_top, int renorm, int softmax) {
  extern __shared__ float zbuf[];                     // per warp: s [E + X], choice [E], group score [groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* s = zbuf + warp * (2 * E + X + groups);
  float* choice = s + E + X;
  float* gs = choice + E;
  const TH* hr = h + t * W;
  route_logits<TH, TW>(hr, wr, W, E + X, lane, s);
  __syncwarp();
  if (lane != 0) return;
  for (int e = softmax ? E : 0; e < E + X; ++e) s[e] = 1.f / (1.f + expf(-s[e]));
  if (softmax) {                                       // scores are the softmax of the logits over all experts
    float zmax = -INFINITY, zsum = 0.f;
    for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, s[e]);
    for (int e = 0; e < E; ++e) { s[e] = expf(s[e] - zmax); zsum += s[e]; }
    for (int e = 0; e < E; ++e) s[e] /= zsum;
  }
  for (int x = 0; x < X; ++x) gate_out[t * X + x] = s[E + x];
  for (int e = 0; e < E; ++e) choice[e] = s[e] + (corr ? corr[e] : 0.f);
  const int per = E / groups;
  if (keep < groups) {
    for (int g = 0; g < groups; ++g) {                 // sum of the group's `group_top` largest choice scores
      float sum = 0.f;
      int last = -1;
      float lastv = INFINITY;
      for (int k = 0; k < group_top && k < per; ++k) {   // k-th largest in (value desc, index asc) order
        int best = -1;
        float bv = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = choice[e];
          const bool after = v < lastv || (v == lastv && e > last);
          if (after && (best < 0 || v > bv)) { best = e; bv = v; }
        }
        if (best < 0) break;
        sum += bv;
        last = best;
        lastv = bv;
      }
      gs[g] = sum;
    }
    for (int k = 0; k < keep; ++k) {                   // the `keep` best groups, marked by a score of +inf
      int best = -1;
      float bv = -INFINITY;
      for (int g = 0; g < groups; ++g)
        if (gs[g] != INFINITY && (best < 0 || gs[g] > bv)) { best = g; bv = gs[g]; }
      gs[best] = INFINITY;
    }
    for (int e = 0; e < E; ++e)
      if (gs[e / per] != INFINITY) choice[e] = -INFINITY;
  }
  float psum = 0.f;
  for (int k = 0; k < top; ++k) {
    int best = 0;
    float bv = choice[0];
    for (int e = 1; e < E; ++e)
      if (choice[e] > bv) { best = e; bv = choice[e]; }
    choice[best] = -INFINITY;                          // taken
    top_i[t * top + k] = best;
    top_p[t * top + k] = s[best];
    psum += s[best];
  }
  if (renorm)
    for (int k = 0; k < top; ++k) top_p[t * top + k] /= psum;
}

// Expert-sorted, tile-padded row layout of R = tokens * top assignments: dest[r] = first row of expert e's segment (segments
// are padded to whole tiles) + the number of earlier assignments to e (a stable counting sort), tile_map[t] = expert of row
// tile t or -1, counts[e], tok[r] = r / top. Every CTA counts all assignments (shared-memory atomics over a 16-bit copy of the
// expert ids) and takes the prefix sums itself, so no CTA waits for another; then each warp places one expert's
// assignments in order with ballots. CTA 0 also writes counts, tile_map and tok.
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const long long* __restrict__ top_i, long long* __restrict__ dest, long long* __restrict__ tok,
                    int* __restrict__ tile_map, long long* __restrict__ counts, int R, int E, int top, int tile, int n_tiles) {
  extern __shared__ __align__(16) unsigned char dsm[];
  int* cnt = reinterpret_cast<int*>(dsm);                          // [E]
  int* seg = cnt + E;                                              // [E + 1] first row of each expert's segment
  unsigned short* ids = reinterpret_cast<unsigned short*>(seg + E + 1);   // [R]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int r = tid; r < R; r += blockDim.x) {
    const long long e = top_i[r];
    const bool ok = e >= 0 && e < E;
    ids[r] = ok ? (unsigned short)e : (unsigned short)0xffff;
    if (ok) atomicAdd(&cnt[(int)e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      seg[e] = at;
      at += (cnt[e] + tile - 1) / tile * tile;
    }
    seg[E] = at;
  }
  __syncthreads();
  const int e = blockIdx.x * (blockDim.x >> 5) + warp;
  if (e < E) {
    int run = seg[e];
    for (int r0 = 0; r0 < R; r0 += 32) {
      const int r = r0 + lane;
      const bool mine = r < R && ids[r] == (unsigned short)e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) dest[r] = run + __popc(m & ((1u << lane) - 1u));
      run += __popc(m);
    }
  }
  if (blockIdx.x != 0) return;
  for (int x = tid; x < E; x += blockDim.x) counts[x] = cnt[x];
  for (int r = tid; r < R; r += blockDim.x) tok[r] = r / top;
  for (int t = tid; t < n_tiles; t += blockDim.x) {
    const int row = t * tile;
    int lo = 0, hi = E;                                            // the last expert whose segment starts at or before row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seg[mid] <= row) lo = mid; else hi = mid;
    }
    // empty experts have empty segments: step over them to the one that holds the row
    while (lo + 1 < E && seg[lo + 1] <= row) ++lo;
    tile_map[t] = row < seg[E] ? lo : -1;
  }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const long long* __restrict__ dest, const float* __restrict__ p,
                                   const T* __restrict__ shared, const float* __restrict__ gate, float* __restrict__ out,
                                   long long tokens, int W, int top) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * W) return;
  const long long t = idx / W;
  const int c = (int)(idx - t * W);
  float a = 0.f;
  for (int k = 0; k < top; ++k) a = fmaf(p[t * top + k], to_f32<T>(y[dest[t * top + k] * W + c]), a);
  if (shared) a = fmaf(gate ? gate[t] : 1.f, to_f32<T>(shared[idx]), a);
  out[idx] = a;
}

}  // namespace b200

using namespace b200;

B200_API int b200_moe_route(const void* h, const void* wr, const float* bias, long long* top_i, float* top_p, float* logits_out,
                            long long tokens, int W, int E, int top, int mode, int h_dtype, int w_dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens <= 0) return 0;
  if (W <= 0 || E <= 0 || top <= 0 || top > E || E > 2048) return B200_ERR_BAD_SHAPE;
  const int warps = 4;
  const unsigned grid = (unsigned)((tokens + warps - 1) / warps);
  const size_t smem = (size_t)warps * E * sizeof(float);
  typedef __nv_bfloat16 bf;
#define RT(TH, TW)                                                                                                          \
  moe_route_kernel<TH, TW><<<grid, warps * 32, smem, st>>>((const TH*)h, (const TW*)wr, bias, top_i, top_p, logits_out, tokens, W, \
                                                          E, top, mode)
  if (h_dtype == B200_DT_BF16 && w_dtype == B200_DT_BF16) RT(bf, bf);
  else if (h_dtype == B200_DT_BF16 && w_dtype == B200_DT_FP32) RT(bf, float);
  else if (h_dtype == B200_DT_FP32 && w_dtype == B200_DT_FP32) RT(float, float);
  else if (h_dtype == B200_DT_FP32 && w_dtype == B200_DT_BF16) RT(float, bf);
  else return B200_ERR_UNSUPPORTED;
#undef RT
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_moe_route_grouped(const void* h, const void* wr, const float* corr, long long* top_i, float* top_p,
                                    float* gate_out, long long tokens, int W, int E, int X, int top, int groups, int keep,
                                    int group_top, int renorm, int softmax, int h_dtype, int w_dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens <= 0) return 0;
  if (W <= 0 || E <= 0 || X < 0 || top <= 0 || top > E || E > 2048 || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      group_top <= 0 || top > keep * (E / groups) || (X > 0 && !gate_out))
    return B200_ERR_BAD_SHAPE;
  const int warps = 4;
  const unsigned grid = (unsigned)((tokens + warps - 1) / warps);
  const size_t smem = (size_t)warps * (2 * E + X + groups) * sizeof(float);
  typedef __nv_bfloat16 bf;
#define RG(TH, TW)                                                                                                          \
  moe_route_grouped_kernel<TH, TW><<<grid, warps * 32, smem, st>>>((const TH*)h, (const TW*)wr, corr, top_i, top_p, gate_out,    \
                                                                  tokens, W, E, X, top, groups, keep, group_top, renorm, softmax)
  if (h_dtype == B200_DT_BF16 && w_dtype == B200_DT_BF16) RG(bf, bf);
  else if (h_dtype == B200_DT_BF16 && w_dtype == B200_DT_FP32) RG(bf, float);
  else if (h_dtype == B200_DT_FP32 && w_dtype == B200_DT_FP32) RG(float, float);
  else if (h_dtype == B200_DT_FP32 && w_dtype == B200_DT_BF16) RG(float, bf);
  else return B200_ERR_UNSUPPORTED;
#undef RG
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_moe_dispatch(const long long* top_i, long long* dest, long long* tok, int* tile_map, long long* counts,
                               long long assignments, int E, int top, int tile, int n_tiles, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (assignments <= 0) return 0;
  if (E <= 0 || E >= 0xffff || top <= 0 || tile <= 0 || n_tiles <= 0) return B200_ERR_BAD_SHAPE;
  const size_t smem = (size_t)(2 * E + 1) * sizeof(int) + (size_t)assignments * sizeof(unsigned short);
  if (smem > 200 * 1024) return B200_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int warps = 8;
  moe_dispatch_kernel<<<(E + warps - 1) / warps, warps * 32, smem, st>>>(top_i, dest, tok, tile_map, counts, (int)assignments, E,
                                                                        top, tile, n_tiles);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_moe_combine(const void* y, const long long* dest, const float* p, const void* shared, const float* gate,
                              float* out, long long tokens, int W, int top, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens <= 0) return 0;
  const unsigned grid = (unsigned)((tokens * W + 255) / 256);
  if (dtype == B200_DT_BF16)
    moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)y, dest, p, (const __nv_bfloat16*)shared, gate, out, tokens, W, top);
  else if (dtype == B200_DT_FP16)
    moe_combine_kernel<__half><<<grid, 256, 0, st>>>((const __half*)y, dest, p, (const __half*)shared, gate, out, tokens, W, top);
  else if (dtype == B200_DT_FP32)
    moe_combine_kernel<float><<<grid, 256, 0, st>>>((const float*)y, dest, p, (const float*)shared, gate, out, tokens, W, top);
  else return B200_ERR_UNSUPPORTED;
  B200_LAUNCH_CHECK();
  return 0;
}
