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
// b200_multimap_attn       per-token attention in fp32 arithmetic over a 16-bit or 32-bit cache; prompt pieces and decoded
//                          tokens take the same path: a vector kernel (16-byte row chunks, the heads of a KV group share the
//                          K/V reads, `nsplit` key ranges + a merge kernel for few tokens with many keys) and a scalar one
//                          (a warp per (token, head)) for row sizes that are not whole chunks.
#include "common.cuh"
#include "mma_sync.cuh"
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
// Vector variant (D and Dv whole 16-byte chunks, at most 32 chunks each): a CTA owns one token, up to HB query heads of one
// KV group, ONE map and one range of the visible keys (blockIdx.z = range * M + map). A lane is (key sub-index, chunk): the
// CP lanes of a group read the key row of the map and the value row of one key with one 16-byte load each; scores are
// reduced over the group's lanes and every lane keeps its own running (max, sum, acc) per head — nothing crosses groups
// inside the loop. Groups are merged by shuffles at the end, the four warps through shared memory. With one map and one
// range the result is written directly; otherwise (max, sum, acc) go to `part` [tokens, H, M, nsplit, Dv + 2] and
// multimap_attn_merge_kernel merges ranges and maps.
// VC: value chunks per lane (2 when the value rows are wider than the key rows: a group then has only as many lanes as a key
// row has chunks, covers twice the keys per instruction, and every lane accumulates chunks c and c + CP of the values)
template <typename T, int HB, int VC>
__global__ void __launch_bounds__(128, 4)               // four CTAs per SM: a decode batch of 64 x 4 groups x 2 maps is one wave
multimap_attn_vec_kernel(const T* __restrict__ q, const T* __restrict__ ck, const T* __restrict__ cv, const int* __restrict__ pos,
                         const int* __restrict__ slot, const int* __restrict__ table, int max_blocks, T* __restrict__ out,
                         float* __restrict__ part, int H, int G, int M, int D, int Dv, int bs_log2, float scale, int window,
                         int keep_first, int nsplit, int CP, int CPK, int CPV) {
  constexpr int E = 16 / sizeof(T);
  extern __shared__ float sm[];                          // [4 warps][HB][Dv + 2]
  const int t = blockIdx.x;
  const int rep = H / G;
  const int passes = (rep + HB - 1) / HB;
  const int g = blockIdx.y / passes;
  const int h0 = g * rep + (blockIdx.y % passes) * HB;
  const int nh = min(HB, g * rep + rep - h0);
  const int split = blockIdx.z / M, m = blockIdx.z % M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KPI = 32 / CP;
  const int kk = lane / CP, c = lane % CP;
  const bool liveK = c < CPK;
  bool liveV[VC];
#pragma unroll
  for (int x = 0; x < VC; ++x) liveV[x] = c + x * CP < CPV;
  const int p = pos[t];
  const int* trow = table + (long long)slot[t] * max_blocks;
  int lo = 0;
  if (window > 0 && p + 1 - window > 0) lo = p + 1 - window;
  const int n1 = min(max(keep_first, 0), lo);
  const int total = n1 + (p + 1 - lo);
  int i_lo = 0, i_hi = total;
  if (nsplit > 1) {
    const int chunk = ((total + nsplit - 1) / nsplit + 31) / 32 * 32;
    i_lo = split * chunk;
    i_hi = min(total, i_lo + chunk);
  }
  // scores are kept in units of log 2 (scale * log2(e) is folded into q): one ex2 per exponential; the merge kernel reads
  // the recorded maxima in the same units
  const float sl2 = scale * 1.4426950408889634f;
  float qv[HB][E], acc[HB][VC][E], mx[HB], l[HB];
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    mx[hh] = -INFINITY;
    l[hh] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
#pragma unroll
      for (int x = 0; x < VC; ++x) acc[hh][x][e] = 0.f;
      qv[hh][e] = (liveK && hh < nh) ? to_f32<T>(q[(((long long)t * H + h0 + hh) * M + m) * D + c * E + e]) * sl2 : 0.f;
    }
  }
  const int bs_mask = (1 << bs_log2) - 1;
  const int stride = 4 * KPI;
  constexpr int U = HB >= 4 ? 2 : 4;
  for (int ib = i_lo; ib < i_hi; ib += stride * U) {
    uint4 kr[U], vr[U][VC];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = ib + u * stride + warp * KPI + kk;
      valid[u] = i < i_hi;
      kr[u] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int x = 0; x < VC; ++x) vr[u][x] = make_uint4(0, 0, 0, 0);
      if (valid[u]) {
        const int kp = i < n1 ? i : lo + (i - n1);
        const long long blk = trow[kp >> bs_log2];
        const int off = kp & bs_mask;
        if (liveK) kr[u] = *reinterpret_cast<const uint4*>(ck + ((((blk * G + g) * M + m) << bs_log2) + off) * D + c * E);
#pragma unroll
        for (int x = 0; x < VC; ++x)
          if (liveV[x]) vr[u][x] = *reinterpret_cast<const uint4*>(cv + ((((blk * G) + g) << bs_log2) + off) * Dv + (c + x * CP) * E);
      }
    }
    // the U keys of a lane are scored first; the running maximum moves once per batch of U keys, so the accumulators are
    // rescaled once per batch
    float vf[U][VC][E], sc[U][HB];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[E];
      const T* kp_ = reinterpret_cast<const T*>(&kr[u]);
#pragma unroll
      for (int e = 0; e < E; ++e) kf[e] = to_f32<T>(kp_[e]);
#pragma unroll
      for (int x = 0; x < VC; ++x) {
        const T* vp = reinterpret_cast<const T*>(&vr[u][x]);
#pragma unroll
        for (int e = 0; e < E; ++e) vf[u][x][e] = to_f32<T>(vp[e]);
      }
#pragma unroll
      for (int hh = 0; hh < HB; ++hh) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) s = fmaf(qv[hh][e], kf[e], s);
        for (int o = CP >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        sc[u][hh] = valid[u] ? s : -INFINITY;
      }
    }
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) {
      float mn = mx[hh];
#pragma unroll
      for (int u = 0; u < U; ++u) mn = fmaxf(mn, sc[u][hh]);
      const float ms = mn == -INFINITY ? 0.f : mn;       // no key of this lane yet: every term below is 2^(-inf) = 0
      const float r = ex2_approx(mx[hh] - ms);
      mx[hh] = mn;
      l[hh] *= r;
#pragma unroll
      for (int x = 0; x < VC; ++x)
#pragma unroll
        for (int e = 0; e < E; ++e) acc[hh][x][e] *= r;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float pj = ex2_approx(sc[u][hh] - ms);
        l[hh] += pj;
#pragma unroll
        for (int x = 0; x < VC; ++x)
#pragma unroll
          for (int e = 0; e < E; ++e) acc[hh][x][e] = fmaf(pj, vf[u][x][e], acc[hh][x][e]);
      }
    }
  }
  const int LDW = Dv + 2;
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    for (int o = CP; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mx[hh], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[hh], o);
      const float mn = fmaxf(mx[hh], m2);
      const float e1 = mx[hh] == -INFINITY ? 0.f : exp2f(mx[hh] - mn);
      const float e2 = m2 == -INFINITY ? 0.f : exp2f(m2 - mn);
      l[hh] = l[hh] * e1 + l2 * e2;
#pragma unroll
      for (int x = 0; x < VC; ++x)
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float a2 = __shfl_xor_sync(0xffffffffu, acc[hh][x][e], o);
          acc[hh][x][e] = acc[hh][x][e] * e1 + a2 * e2;
        }
      mx[hh] = mn;
    }
    if (kk == 0) {
      float* w = sm + (warp * HB + hh) * LDW;
      if (c == 0) { w[0] = mx[hh]; w[1] = l[hh]; }
#pragma unroll
      for (int x = 0; x < VC; ++x)
        if (liveV[x]) {
#pragma unroll
          for (int e = 0; e < E; ++e) w[2 + (c + x * CP) * E + e] = acc[hh][x][e];
        }
    }
  }
  __syncthreads();
  const bool direct = M == 1 && nsplit == 1;
  for (int i = threadIdx.x; i < nh * Dv; i += blockDim.x) {
    const int hh = i / Dv, d = i % Dv;
    const int h = h0 + hh;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm[(w * HB + hh) * LDW]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* ws = sm + (w * HB + hh) * LDW;
      if (ws[0] != -INFINITY) {
        const float e = exp2f(ws[0] - mt);
        lt += ws[1] * e;
        at += ws[2 + d] * e;
      }
    }
    if (direct) {
      out[((long long)t * H + h) * Dv + d] = from_f32<T>(lt > 0.f ? at / lt : 0.f);
    } else {
      float* pr = part + ((((long long)t * H + h) * M + m) * nsplit + split) * LDW;
      if (d == 0) { pr[0] = mt; pr[1] = lt; }
      pr[2 + d] = at;
    }
  }
}

// one warp per (token, head): merges the key ranges of every map, then the combination and the norm
template <typename T>
__global__ void __launch_bounds__(128)
multimap_attn_merge_kernel(const float* __restrict__ part, T* __restrict__ out, long long items, int M, int Dv, int nsplit,
                           int combine, float lambda, float post, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;            // (token, head)
  if (item >= items) return;
  const int LDW = Dv + 2;
  float res[kAcc];
#pragma unroll
  for (int a = 0; a < kAcc; ++a) res[a] = 0.f;
  for (int m = 0; m < M; ++m) {
    const float* pr = part + (item * M + m) * nsplit * LDW;
    float mt = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mt = fmaxf(mt, pr[s * LDW]);
    float lt = 0.f, at[kAcc];
#pragma unroll
    for (int a = 0; a < kAcc; ++a) at[a] = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = pr[s * LDW];
      if (ms == -INFINITY) continue;
      const float e = exp2f(ms - mt);                    // the recorded maxima are in units of log 2
      lt += pr[s * LDW + 1] * e;
#pragma unroll
      for (int a = 0; a < kAcc; ++a) {
        const int d = lane + 32 * a;
        if (d < Dv) at[a] += pr[s * LDW + 2 + d] * e;
      }
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    const float coef = m == 0 ? 1.f : -lambda;
#pragma unroll
    for (int a = 0; a < kAcc; ++a) res[a] = fmaf(coef, at[a] * inv, res[a]);
  }
  float mult = 1.f;
  if (combine) {
    float ss = 0.f;
#pragma unroll
    for (int a = 0; a < kAcc; ++a) ss += (lane + 32 * a < Dv) ? res[a] * res[a] : 0.f;
    ss = warp_sum(ss);
    mult = rsqrtf(ss / Dv + eps) * post;
  }
#pragma unroll
  for (int a = 0; a < kAcc; ++a) {
    const int d = lane + 32 * a;
    if (d < Dv) out[item * Dv + d] = from_f32<T>(res[a] * mult);
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
                                int max_blocks, void* out, float* part, int tokens, int H, int G, int M, int D, int Dv,
                                int block_size, float scale, int window, int keep_first, int nsplit, int combine, float lambda,
                                float post, float eps, int dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || M < 1 || M > kMaxMaps || D <= 0 || Dv <= 0 || block_size <= 0 || nsplit < 1) return B200_ERR_BAD_SHAPE;
  if (Dv > kMaxDv) return B200_ERR_TOO_LARGE;
  if (combine && M != 2) return B200_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int rep = H / G;
  {
    // vector kernel: key and value rows of whole 16-byte chunks, at most 32 of them, pages of a power-of-two size
    const int E = dtype == B200_DT_FP32 ? 4 : 8;
    const int CPK = D / E, CPV = Dv / E;
    int bs_log2 = 0;
    while ((1 << bs_log2) < block_size) ++bs_log2;
    if (D % E == 0 && Dv % E == 0 && CPK <= 32 && CPV <= 32 && (1 << bs_log2) == block_size && (part || (M == 1 && nsplit == 1)) &&
        !((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(ck) | reinterpret_cast<uintptr_t>(cv)) & 15)) {
      // lanes per key: the chunks of a key row, or of half a value row if that is more (a lane then holds two value chunks)
      int CP = 1;
      while (CP < CPK || 2 * CP < CPV) CP <<= 1;
      const int VC = CPV > CP ? 2 : 1;
      const int HB = rep >= 4 ? 4 : (rep >= 2 ? 2 : 1);
      const int passes = (rep + HB - 1) / HB;
      const bool direct = M == 1 && nsplit == 1;
      if ((long long)G * passes > 65535 || nsplit * M > 65535) return B200_ERR_TOO_LARGE;
      if (!direct && !part) return B200_ERR_BAD_SHAPE;
      dim3 grid(tokens, G * passes, nsplit * M);
      const size_t smem = (size_t)4 * HB * (Dv + 2) * sizeof(float);
#define MMV2(T, HBV, VCV)                                                                                                    \
  multimap_attn_vec_kernel<T, HBV, VCV><<<grid, 128, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, pos, slot, table,   \
      max_blocks, (T*)out, part, H, G, M, D, Dv, bs_log2, scale, window, keep_first, nsplit, CP, CPK, CPV)
#define MMV(T, HBV)                                                                                                          \
  do { if (VC == 2) MMV2(T, HBV, 2); else MMV2(T, HBV, 1); } while (0)
#define MMV_T(T)                                                                                                             \
  do {                                                                                                                       \
    if (HB == 4) MMV(T, 4); else if (HB == 2) MMV(T, 2); else MMV(T, 1);                                                     \
    if (!direct)                                                                                                             \
      multimap_attn_merge_kernel<T><<<(unsigned)(((long long)tokens * H + 3) / 4), 128, 0, st>>>(                             \
          part, (T*)out, (long long)tokens * H, M, Dv, nsplit, combine, lambda, post, eps);                                  \
  } while (0)
      if (dtype == B200_DT_BF16) MMV_T(__nv_bfloat16);
      else if (dtype == B200_DT_FP16) MMV_T(__half);
      else if (dtype == B200_DT_FP32) MMV_T(float);
      else return B200_ERR_UNSUPPORTED;
#undef MMV_T
#undef MMV
#undef MMV2
      B200_LAUNCH_CHECK();
      return 0;
    }
  }
  const int nw = 4;
  const size_t smem = (size_t)nw * D * 4;
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)(((long long)tokens * H + nw - 1) / nw);
  B200_DISPATCH_T(dtype, multimap_attn_kernel<T><<<grid, nw * 32, smem, st>>>(
      (const T*)q, (const T*)ck, (const T*)cv, pos, slot, table, max_blocks, (T*)out, tokens, H, G, M, D, Dv, block_size, scale,
      window, keep_first, combine, lambda, post, eps));
  B200_LAUNCH_CHECK();
  return 0;
}
