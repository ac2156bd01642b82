// Multi-map attention over the paged KV cache: M attention maps per head (each with its own query and key rows, all over the
// same values), a sliding window that keeps the first tokens of the sequence, and an optional differential combination.
//
//   keys    cache K [blocks, G * M, block_size, D]   (key head g, map m at row g * M + m; normed and rotated when stored)
//   values  cache V [blocks, G,     block_size, Dv]  (Dv need not equal D)
//   token t (position p of cache row slot[t]) sees key j of its row if j <= p and (p - j < window or j < keep_first);
//   window <= 0 means every j <= p.
//   a_m = softmax_j(scale q_{h,m} . k_{g,m,j}) V_g        g = h / (H / G)
//   M = 2, combine:  o = a_0 - lambda a_1 ;  o <- o / sqrt(mean(o^2) + eps) * post      (differential attention)
//   otherwise:       o = a_0 (M = 1)
//
// b200_qknorm_rope_store   per-(head, map) RMS norm with a weight over D, rotary on the first `rot` dims in the split layout
//                          (dim i pairs with i + rot/2), q -> q_out in the cache dtype, k and v -> their pages.
// b200_multimap_attn       one warp per (token, head): fp32 arithmetic over a 16-bit or 32-bit cache; prompt pieces and
//                          decoded tokens take the same path.
#include "common.cuh"
#include "../include/b200_ops.h"

#define B200_DISPATCH_T(dtype, ...)                                   \
  if (dtype == B200_DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else if (dtype == B200_DT_FP16) { using T = __half; __VA_ARGS__; }   \
  else if (dtype == B200_DT_FP32) { using T = float; __VA_ARGS__; }    \
  else return B200_ERR_UNSUPPORTED;

namespace b200 {

// proj fp32 [tokens, ld]: q rows (QR = H * M of D) at column 0, then (has_kv) k rows (KR = G * M of D) and v (G * Dv).
template <typename T>
__global__ void __launch_bounds__(128)
qknorm_rope_store_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ wq, const float* __restrict__ wk,
                         const float* __restrict__ cs, const float* __restrict__ sn, const int* __restrict__ pos,
                         const int* __restrict__ slot, const int* __restrict__ table, int max_blocks, T* __restrict__ q_out,
                         T* __restrict__ ck, T* __restrict__ cv, int QR, int KR, int G, int D, int Dv, int rot, int block_size,
                         float eps, int has_kv) {
  extern __shared__ float sh[];                          // [warps, D]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int p = pos[t];
  const float* row = proj + (long long)t * ld;
  const float* c = cs + (long long)p * (rot / 2);
  const float* s = sn + (long long)p * (rot / 2);
  float* buf = sh + warp * D;
  long long kbase = 0, vbase = 0;
  if (has_kv) {
    const int blk = table[(long long)slot[t] * max_blocks + p / block_size];
    const int off = p % block_size;
    kbase = ((long long)blk * KR * block_size + off) * D;            // + r * block_size * D
    vbase = ((long long)blk * G * block_size + off) * Dv;            // + g * block_size * Dv
  }
  const int rows = QR + (has_kv ? KR : 0);
  const int hr = rot / 2;
  for (int r = warp; r < rows; r += nw) {
    const float* x = row + (long long)r * D;
    const float* w = r < QR ? wq : wk;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { const float v = x[d]; ss += v * v; }
    ss = warp_sum(ss);
    const float sc = rsqrtf(ss / D + eps);
    __syncwarp();
    for (int d = lane; d < D; d += 32) buf[d] = x[d] * sc * w[d];
    __syncwarp();
    T* dst = r < QR ? q_out + ((long long)t * QR + r) * D : ck + kbase + (long long)(r - QR) * block_size * D;
    for (int d = lane; d < D; d += 32) {
      float v = buf[d];
      if (d < hr) v = buf[d] * c[d] - buf[d + hr] * s[d];
      else if (d < rot) v = buf[d] * c[d - hr] + buf[d - hr] * s[d - hr];
      dst[d] = from_f32<T>(v);
    }
  }
  if (has_kv) {
    const float* vsrc = row + (long long)(QR + KR) * D;
    for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) {
      const int g = i / Dv, d = i % Dv;
      cv[vbase + (long long)g * block_size * Dv + d] = from_f32<T>(vsrc[i]);
    }
  }
}

constexpr int kMaxDv = 256;
constexpr int kAcc = kMaxDv / 32;
constexpr int kMaxMaps = 2;

template <typename T>
__device__ __forceinline__ float dot_qk(const float* __restrict__ q, const T* __restrict__ k, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(q[d], to_f32<T>(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_qk<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int D) {
  float acc = 0.f;
  if ((D & 7) == 0) {
    for (int d = 0; d < D; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        acc = fmaf(q[d + 2 * j], f.x, acc);
        acc = fmaf(q[d + 2 * j + 1], f.y, acc);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(128)
multimap_attn_kernel(const T* __restrict__ q, const T* __restrict__ ck, const T* __restrict__ cv, const int* __restrict__ pos,
                     const int* __restrict__ slot, const int* __restrict__ table, int max_blocks, T* __restrict__ out, int tokens,
                     int H, int G, int M, int D, int Dv, int block_size, float scale, int window, int keep_first, int combine,
                     float lambda, float post, float eps) {
  extern __shared__ float qs[];                          // [warps, D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long item = (long long)blockIdx.x * nw + warp;          // (token, head)
  if (item >= (long long)tokens * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const int g = h / (H / G);
  const int p = pos[t];
  const int* trow = table + (long long)slot[t] * max_blocks;
  int lo = 0;
  if (window > 0 && p + 1 - window > 0) lo = p + 1 - window;
  const int n1 = min(max(keep_first, 0), lo);            // kept first tokens that the window no longer covers
  const int total = n1 + (p + 1 - lo);
  float* myq = qs + warp * D;
  float res[kAcc];
#pragma unroll
  for (int i = 0; i < kAcc; ++i) res[i] = 0.f;
  for (int m = 0; m < M; ++m) {
    const T* qr = q + (((long long)t * H + h) * M + m) * D;
    __syncwarp();
    for (int d = lane; d < D; d += 32) myq[d] = to_f32<T>(qr[d]);
    __syncwarp();
    float mx = -INFINITY, l = 0.f;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) acc[i] = 0.f;
    const int kh = g * M + m;
    for (int i0 = 0; i0 < total; i0 += 32) {
      const int i = i0 + lane;
      const bool valid = i < total;
      long long voff = 0;
      float sc = -INFINITY;
      if (valid) {
        const int kp = i < n1 ? i : lo + (i - n1);
        const int blk = trow[kp / block_size];
        const int off = kp % block_size;
        sc = dot_qk<T>(myq, ck + (((long long)blk * G * M + kh) * block_size + off) * D, D) * scale;
        voff = (((long long)blk * G + g) * block_size + off) * Dv;
      }
      const float m_new = fmaxf(mx, warp_max(sc));
      const float pj = valid ? expf(sc - m_new) : 0.f;
      const float resc = (mx == -INFINITY) ? 0.f : expf(mx - m_new);
      l = l * resc + warp_sum(pj);
      mx = m_new;
#pragma unroll
      for (int a = 0; a < kAcc; ++a) acc[a] *= resc;
      const int nk = min(32, total - i0);
      for (int j = 0; j < nk; ++j) {
        const float w = __shfl_sync(0xffffffffu, pj, j);
        const long long ro = __shfl_sync(0xffffffffu, voff, j);
        const T* vr = cv + ro;
#pragma unroll
        for (int a = 0; a < kAcc; ++a) {
          const int d = lane + 32 * a;
          if (d < Dv) acc[a] = fmaf(w, to_f32<T>(vr[d]), acc[a]);
        }
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float coef = (m == 0) ? 1.f : -lambda;
#pragma unroll
    for (int a = 0; a < kAcc; ++a) res[a] = fmaf(coef, acc[a] * inv, res[a]);
  }
  float mult = 1.f;
  if (combine) {
    float ss = 0.f;
#pragma unroll
    for (int a = 0; a < kAcc; ++a) ss += (lane + 32 * a < Dv) ? res[a] * res[a] : 0.f;
    ss = warp_sum(ss);
    mult = rsqrtf(ss / Dv + eps) * post;
  }
  T* orow = out + ((long long)t * H + h) * Dv;
#pragma unroll
  for (int a = 0; a < kAcc; ++a) {
    const int d = lane + 32 * a;
    if (d < Dv) orow[d] = from_f32<T>(res[a] * mult);
  }
}
}  // namespace b200

B200_API int b200_qknorm_rope_store(const float* proj, long long ld, const float* wq, const float* wk, const float* cos_t,
                                    const float* sin_t, const int* pos, const int* slot, const int* table, int max_blocks,
                                    void* q_out, void* ck, void* cv, int tokens, int H, int G, int M, int D, int Dv, int rot,
                                    int block_size, float eps, int has_kv, int dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || M <= 0 || D <= 0 || rot < 0 || rot > D || (rot & 1) || block_size <= 0) return B200_ERR_BAD_SHAPE;
  const size_t smem = 4 * (size_t)D * 4;
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_T(dtype, qknorm_rope_store_kernel<T><<<tokens, 128, smem, (cudaStream_t)stream>>>(
      proj, ld, wq, wk, cos_t, sin_t, pos, slot, table, max_blocks, (T*)q_out, (T*)ck, (T*)cv, H * M, G * M, G, D, Dv, rot,
      block_size, eps, has_kv));
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_multimap_attn(const void* q, const void* ck, const void* cv, const int* pos, const int* slot, const int* table,
                                int max_blocks, void* out, int tokens, int H, int G, int M, int D, int Dv, int block_size,
                                float scale, int window, int keep_first, int combine, float lambda, float post, float eps,
                                int dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || M < 1 || M > kMaxMaps || D <= 0 || Dv <= 0 || block_size <= 0) return B200_ERR_BAD_SHAPE;
  if (Dv > kMaxDv) return B200_ERR_TOO_LARGE;
  if (combine && M != 2) return B200_ERR_UNSUPPORTED;
  const int nw = 4;
  const size_t smem = (size_t)nw * D * 4;
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)(((long long)tokens * H + nw - 1) / nw);
  B200_DISPATCH_T(dtype, multimap_attn_kernel<T><<<grid, nw * 32, smem, (cudaStream_t)stream>>>(
      (const T*)q, (const T*)ck, (const T*)cv, pos, slot, table, max_blocks, (T*)out, tokens, H, G, M, D, Dv, block_size, scale,
      window, keep_first, combine, lambda, post, eps));
  B200_LAUNCH_CHECK();
  return 0;
}
