// Talking-heads attention over the paged key cache, for the ragged serving step: the heads' scores are mixed by a learned
// [H, H] matrix BEFORE the softmax, a logarithmic distance penalty is taken off every score, keys double as values, and only
// the last `window` positions are visible.
//
//   raw_g(i, j)  = scale * q_g(i) . k_kv(g)(j) - r1_g * log(1 + r2_g * (i - j))            0 <= i - j < window
//   s_h(i, j)    = sum_g talk[h, g] raw_g(i, j)
//   p_h(i, .)    = softmax_j s_h(i, .)
//   out_h(i)     = (sum_j p_h(i, j) k_kv(h)(j)) * sigmoid(gate_h(i))                        (gate optional)
//
// Because the mixing couples all heads of a (query, key) pair, a CTA owns ALL heads of its query rows; scores, the mixing,
// the softmax and the accumulators are fp32. Keys live in pages [blocks, G, block_size, D] reached through the block table.
//
//   b200_talking_attn       one query token per CTA (decode tokens, fp32 runs, any sizes): keys are staged in chunks of 32,
//                           a warp owns a head and a lane a key for the scores, the mixing and the online softmax; for the
//                           weighted sum a thread owns a few (head, channel) pairs.
#include "common.cuh"
#include "../include/b200_ops.h"

namespace b200 {

constexpr int kTalkChunk = 32;        // keys per staged chunk: one per lane
constexpr int kTalkThreads = 256;

// U = accumulators per thread (H * D <= U * kTalkThreads)
template <typename T, int U>
__global__ void __launch_bounds__(kTalkThreads)
talking_attn_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ gate, long long ldg, const T* __restrict__ ck,
                    const int* __restrict__ table, int max_blocks, const int* __restrict__ pos, const int* __restrict__ slot,
                    const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ talk,
                    T* __restrict__ out, int H, int G, int D, int bs_log2, float scale, int window, int chunk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int t = blockIdx.x;
  const int i = pos[t], s = slot[t];
  const int lo = window > 0 ? max(0, i - window + 1) : 0;
  const int rep = H / G, GD = G * D, HD = H * D;
  const int BS = 1 << bs_log2;
  const int ldk = GD + (sizeof(T) == 2 ? 2 : 1);          // staged key row, padded to an odd number of 32-bit words
  const int ldr = kTalkChunk + 1;
  float* qs = reinterpret_cast<float*>(smem_raw);         // [H * D]
  float* raw = qs + HD;                                   // [H][ldr]
  float* pw = raw + H * ldr;                              // [H][ldr]
  float* tk = pw + H * ldr;                               // [H * H]
  float* mrow = tk + H * H;                               // [H] running maximum
  float* lrow = mrow + H;                                 // [H] running sum
  float* arow = lrow + H;                                 // [H] rescale of the chunk
  T* ks = reinterpret_cast<T*>(qs + ((HD + 2 * H * ldr + H * H + 3 * H + 3) & ~3));      // [chunk][ldk], 16-byte aligned
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kTalkThreads >> 5;

  const T* qr = q + (long long)t * ldq;
  for (int e = threadIdx.x; e < HD; e += kTalkThreads) qs[e] = to_f32<T>(qr[e]);
  for (int e = threadIdx.x; e < H * H; e += kTalkThreads) tk[e] = talk[e];
  for (int e = threadIdx.x; e < H; e += kTalkThreads) { mrow[e] = -INFINITY; lrow[e] = 0.f; }
  float acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = 0.f;
  const int* trow = table + (long long)s * max_blocks;

  for (int j0 = lo; j0 <= i; j0 += chunk) {               // chunk <= 32 keys: fewer when many wide kv heads fill shared memory
    const int cn = min(chunk, i + 1 - j0);
    __syncthreads();                                      // the previous chunk's keys and weights have been used
    // ---- stage the chunk's key rows (all kv heads of a position side by side)
    for (int e = threadIdx.x; e < cn * GD; e += kTalkThreads) {
      const int jj = e / GD, c = e - jj * GD;
      const int g = c / D, d = c - g * D;
      const int j = j0 + jj;
      const long long blk = trow[j >> bs_log2];
      ks[jj * ldk + c] = ck[((blk * G + g) * BS + (j & (BS - 1))) * D + d];
    }
    __syncthreads();
    // ---- raw scores: warp = head, lane = key
    for (int h = warp; h < H; h += nw) {
      float v = -INFINITY;
      if (lane < cn) {
        const float* qh = qs + h * D;
        const T* kr = ks + lane * ldk + (h / rep) * D;
        float a = 0.f;
        for (int d = 0; d < D; ++d) a = fmaf(qh[d], to_f32<T>(kr[d]), a);
        v = a * scale - r1[h] * log1pf(r2[h] * (float)(i - (j0 + lane)));
      }
      raw[h * ldr + lane] = v;
    }
    __syncthreads();
    // ---- mixing over the heads, then this head's online softmax
    for (int h = warp; h < H; h += nw) {
      float sc = -INFINITY;
      if (lane < cn) {
        sc = 0.f;
        for (int g = 0; g < H; ++g) sc = fmaf(tk[h * H + g], raw[g * ldr + lane], sc);
      }
      const float mo = mrow[h];
      const float mn = fmaxf(mo, warp_max(sc));
      const float p = lane < cn ? expf(sc - mn) : 0.f;
      const float al = expf(mo - mn);                     // 0 at the first chunk (mo = -inf)
      const float ps = warp_sum(p);
      pw[h * ldr + lane] = p;
      if (lane == 0) { mrow[h] = mn; lrow[h] = lrow[h] * al + ps; arow[h] = al; }
    }
    __syncthreads();
    // ---- weighted sum of the keys: a thread owns channels e = tid + u * threads of [H, D]
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int e = threadIdx.x + u * kTalkThreads;
      if (e < HD) {
        const int h = e / D, d = e - h * D;
        const T* kc = ks + (h / rep) * D + d;
        const float* ph = pw + h * ldr;
        float a = acc[u] * arow[h];
        for (int jj = 0; jj < cn; ++jj) a = fmaf(ph[jj], to_f32<T>(kc[jj * ldk]), a);
        acc[u] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int e = threadIdx.x + u * kTalkThreads;
    if (e < HD) {
      float v = acc[u] / lrow[e / D];
      if (gate) v *= 1.f / (1.f + expf(-to_f32<T>(gate[(long long)t * ldg + e])));
      out[(long long)t * HD + e] = from_f32<T>(v);
    }
  }
}

template <typename T>
static int talking_launch(const void* q, long long ldq, const void* gate, long long ldg, const void* ck, const int* table,
                          int max_blocks, const int* pos, const int* slot, const float* r1, const float* r2, const float* talk,
                          void* out, int tokens, int H, int G, int D, int bs_log2, float scale, int window, cudaStream_t st) {
  const int HD = H * D;
  const int ldk = G * D + (sizeof(T) == 2 ? 2 : 1), ldr = kTalkChunk + 1;
  const int nf = HD + 2 * H * ldr + H * H + 3 * H;
  const size_t fixed = ((size_t)((nf + 3) & ~3)) * 4;
  int chunk = kTalkChunk;                                  // as many keys per chunk as fit beside the query and the scores
  while (chunk > 1 && fixed + (size_t)chunk * ldk * sizeof(T) > 200 * 1024) chunk >>= 1;
  const size_t smem = fixed + (size_t)chunk * ldk * sizeof(T);
  if (smem > 200 * 1024 || HD > 32 * kTalkThreads) return B200_ERR_TOO_LARGE;
  const int U = (HD + kTalkThreads - 1) / kTalkThreads;
#define TALK(UU)                                                                                                            \
  do {                                                                                                                      \
    auto kern = talking_attn_kernel<T, UU>;                                                                                 \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    kern<<<tokens, kTalkThreads, smem, st>>>((const T*)q, ldq, (const T*)gate, ldg, (const T*)ck, table, max_blocks, pos, slot, \
                                             r1, r2, talk, (T*)out, H, G, D, bs_log2, scale, window, chunk);                \
  } while (0)
  if (U <= 2) TALK(2); else if (U <= 4) TALK(4); else if (U <= 8) TALK(8); else if (U <= 16) TALK(16); else TALK(32);
#undef TALK
  B200_LAUNCH_CHECK();
  return 0;
}
}  // namespace b200

B200_API int b200_talking_attn(const void* q, long long ldq, const void* gate, long long ldg, const void* ck, const int* table,
                               int max_blocks, const int* pos, const int* slot, const float* r1, const float* r2,
                               const float* talk, void* out, int tokens, int H, int G, int D, int block_size, float scale,
                               int window, int dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || block_size <= 0 || (block_size & (block_size - 1)) || window < 0)
    return B200_ERR_BAD_SHAPE;
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == B200_DT_BF16)
    return talking_launch<__nv_bfloat16>(q, ldq, gate, ldg, ck, table, max_blocks, pos, slot, r1, r2, talk, out, tokens, H, G, D,
                                         bs_log2, scale, window, st);
  if (dtype == B200_DT_FP32)
    return talking_launch<float>(q, ldq, gate, ldg, ck, table, max_blocks, pos, slot, r1, r2, talk, out, tokens, H, G, D, bs_log2,
                                 scale, window, st);
  return B200_ERR_UNSUPPORTED;
}
