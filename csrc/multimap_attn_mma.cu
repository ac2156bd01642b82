// Multi-map attention (see multimap_attn.cu for the definition) for bf16 prompt pieces on the tensor cores.
//
// A CTA owns 64 query rows of one piece (a tile: first row, rows, first position, cache row) and one head; its four warps
// own 16 rows each. The maps are walked one after the other: Q of (head, map) -> fragments, then a flash loop over the 64-key
// blocks the tile can see — the blocks that hold kept first tokens, then the blocks from the window's lower edge of the
// tile's first row up to the diagonal; blocks in between are never fetched — with S = Q K^T and P V on mma.sync.m16n8k16
// (K [64, D] and V [64, Dv] pages gathered through the block table with double-buffered cp.async; P stays in registers as
// the A operand). Scores, running maximum / sum and both accumulators are fp32. After the last map the combination
// a_0 - lambda a_1, the RMS norm over Dv and the post factor are applied in registers and the row is written once.
//
// tcgen05 is not used: tiles are ragged (1 .. 64 rows at any position), D and Dv are independent multiples of 16, and the
// mask has two disjoint key ranges per row; the like kernel of the single-map paged attention makes the same choice.
#include "common.cuh"
#include "mma_sync.cuh"
#include "../include/b200_ops.h"

namespace b200 {

constexpr int kQ = 64, kK = 64;

template <int DK, int DVK>
__global__ void __launch_bounds__(128)
multimap_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ ck,
                         const __nv_bfloat16* __restrict__ cv, const int* __restrict__ tiles, const int* __restrict__ table,
                         int max_blocks, __nv_bfloat16* __restrict__ out, int H, int G, int M, int bs_log2, float scale,
                         int window, int keep_first, int combine, float lambda, float post, float eps) {
  constexpr int D = 16 * DK, Dv = 16 * DVK;
  constexpr int LDK = D + 8, LDV = Dv + 8;
  constexpr int CHK = 2 * DK, CHV = 2 * DVK;            // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [64][LDK]
  __nv_bfloat16* sk = sq + kQ * LDK;                                      // [2][64][LDK]
  __nv_bfloat16* sv = sk + 2 * kK * LDK;                                  // [2][64][LDV]
  const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int g = h / (H / G);
  const int row0 = tiles[tile * 4], nrows = tiles[tile * 4 + 1], pos0 = tiles[tile * 4 + 2], slot = tiles[tile * 4 + 3];
  const int* trow = table + (long long)slot * max_blocks;
  const int kv_len = pos0 + nrows;
  const int nkb = (kv_len + kK - 1) / kK;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bs_mask = (1 << bs_log2) - 1;
  const int lo0 = (window > 0 && pos0 + 1 - window > 0) ? pos0 + 1 - window : 0;       // lower window edge of the first row
  const int keepN = min(max(keep_first, 0), lo0);
  const int nA = (keepN + kK - 1) / kK;                   // blocks [0, nA) hold kept first tokens below the window
  const int bB = max(lo0 / kK, nA);                       // blocks [bB, nkb) reach into the window
  const int nit = nA + (nkb - bB);

  float res[2 * DVK][4];
#pragma unroll
  for (int i = 0; i < 2 * DVK; ++i) res[i][0] = res[i][1] = res[i][2] = res[i][3] = 0.f;
  const int qpos0 = pos0 + warp * 16 + (lane >> 2);       // position of this thread's first row; the second is + 8
  const float LOG2E = 1.4426950408889634f;
  const float sl2 = scale * LOG2E;

  for (int m = 0; m < M; ++m) {
    const int kh = g * M + m;
    auto load_kv = [&](int buf, int kb) {
      for (int c = tid; c < kK * CHK; c += 128) {
        const int r = c / CHK, col = (c % CHK) * 8;
        const int kp = kb * kK + r;
        __nv_bfloat16* dk = sk + (buf * kK + r) * LDK + col;
        if (kp < kv_len) {
          const long long off = ((((long long)trow[kp >> bs_log2] * (G * M) + kh) << bs_log2) + (kp & bs_mask)) * D;
          cp_async16(smem_u32(dk), ck + off + col);
        } else {
          *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
        }
      }
      for (int c = tid; c < kK * CHV; c += 128) {
        const int r = c / CHV, col = (c % CHV) * 8;
        const int kp = kb * kK + r;
        __nv_bfloat16* dv = sv + (buf * kK + r) * LDV + col;
        if (kp < kv_len) {
          const long long off = ((((long long)trow[kp >> bs_log2] * G + g) << bs_log2) + (kp & bs_mask)) * Dv;
          cp_async16(smem_u32(dv), cv + off + col);
        } else {
          *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
        }
      }
    };
    auto block_of = [&](int it) { return it < nA ? it : bB + (it - nA); };

    __syncthreads();                                      // the previous map is done with sq / sk / sv
    for (int c = tid; c < kQ * CHK; c += 128) {
      const int r = c / CHK, col = (c % CHK) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (((long long)(row0 + r) * H + h) * M + m) * D + col);
      *reinterpret_cast<uint4*>(sq + r * LDK + col) = v;
    }
    load_kv(0, block_of(0));
    cp_async_commit();
    __syncthreads();
    uint32_t qa[DK][4];
    {
      const int r = warp * 16 + (lane & 15);
      const int cofs = (lane >> 4) * 8;
#pragma unroll
      for (int k = 0; k < DK; ++k) ldsm_x4(smem_u32(sq + r * LDK + k * 16 + cofs), qa[k][0], qa[k][1], qa[k][2], qa[k][3]);
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[2 * DVK][4];
#pragma unroll
    for (int i = 0; i < 2 * DVK; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int it = 0; it < nit; ++it) {
      const int buf = it & 1;
      const int kb = block_of(it);
      if (it + 1 < nit) load_kv(buf ^ 1, block_of(it + 1));
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* bk = sk + buf * kK * LDK;
      const __nv_bfloat16* bv = sv + buf * kK * LDV;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int k = 0; k + 1 < DK; k += 2) {
        uint32_t b[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
          ldsm_x4(smem_u32(bk + (n * 8 + (lane & 7)) * LDK + k * 16 + (lane >> 3) * 8), b[n][0], b[n][1], b[n][2], b[n][3]);
#pragma unroll
        for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k][0], qa[k][1], qa[k][2], qa[k][3], b[n][0], b[n][1]);
#pragma unroll
        for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k + 1][0], qa[k + 1][1], qa[k + 1][2], qa[k + 1][3], b[n][2], b[n][3]);
      }
      if (DK & 1) {
        constexpr int k = DK - 1;
        uint32_t b[8][2];
#pragma unroll
        for (int n = 0; n < 8; ++n) ldsm_x2(smem_u32(bk + (n * 8 + (lane & 7)) * LDK + k * 16 + ((lane >> 3) & 1) * 8), b[n][0], b[n][1]);
#pragma unroll
        for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k][0], qa[k][1], qa[k][2], qa[k][3], b[n][0], b[n][1]);
      }
      // mask: key j is seen from position i iff j <= i and (no window, or i - j < window, or j < keep_first). Blocks wholly
      // inside every row's range skip the test (uniform over the warp).
      const int k0 = kb * kK;
      const bool diag = k0 + kK - 1 > pos0 + warp * 16;
      const bool edge = window > 0 && k0 < pos0 + warp * 16 + 16 - window && k0 + kK - 1 >= keep_first;
      if (diag || edge) {
        const int kbase = k0 + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int kj = kbase + n * 8 + (j & 1), qi = qpos0 + (j >> 1) * 8;
            const bool seen = kj <= qi && (window <= 0 || qi - kj < window || kj < keep_first);
            if (!seen) s[n][j] = -INFINITY;
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0 * sl2), mn1 = fmaxf(m1, mx1 * sl2);      // scale > 0 (checked by the launcher)
      const float e0 = mn0 == -INFINITY ? 0.f : mn0, e1 = mn1 == -INFINITY ? 0.f : mn1;
      const float r0 = ex2_approx(m0 - e0), r1 = ex2_approx(m1 - e1);
      m0 = mn0; m1 = mn1;
      l0 *= r0; l1 *= r1;
#pragma unroll
      for (int i = 0; i < 2 * DVK; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
      uint32_t pa[4][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p0 = ex2_approx(fmaf(s[n][0], sl2, -e0)), p1 = ex2_approx(fmaf(s[n][1], sl2, -e0));
        const float p2 = ex2_approx(fmaf(s[n][2], sl2, -e1)), p3 = ex2_approx(fmaf(s[n][3], sl2, -e1));
        l0 += p0 + p1;
        l1 += p2 + p3;
        pa[n >> 1][(n & 1) * 2] = pack_bf16x2(p0, p1);
        pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p2, p3);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int n = 0; n < 2 * DVK; n += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(smem_u32(bv + (kk * 16 + (lane & 15)) * LDV + n * 8 + (lane >> 4) * 8), b0, b1, b2, b3);
          mma_bf16_16816(o[n], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
          mma_bf16_16816(o[n + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
        }
      }
      __syncthreads();
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float coef = m == 0 ? 1.f : -lambda;
    const float i0 = (l0 > 0.f ? 1.f / l0 : 0.f) * coef, i1 = (l1 > 0.f ? 1.f / l1 : 0.f) * coef;
#pragma unroll
    for (int n = 0; n < 2 * DVK; ++n) {
      res[n][0] = fmaf(o[n][0], i0, res[n][0]);
      res[n][1] = fmaf(o[n][1], i0, res[n][1]);
      res[n][2] = fmaf(o[n][2], i1, res[n][2]);
      res[n][3] = fmaf(o[n][3], i1, res[n][3]);
    }
  }
  float f0 = 1.f, f1 = 1.f;
  if (combine) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int n = 0; n < 2 * DVK; ++n) {
      s0 += res[n][0] * res[n][0] + res[n][1] * res[n][1];
      s1 += res[n][2] * res[n][2] + res[n][3] * res[n][3];
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    f0 = rsqrtf(s0 / Dv + eps) * post;
    f1 = rsqrtf(s1 / Dv + eps) * post;
  }
  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
#pragma unroll
  for (int n = 0; n < 2 * DVK; ++n) {
    const int d = n * 8 + 2 * (lane & 3);
    if (ra < nrows)
      *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + ra) * H + h) * Dv + d) = pack_bf16x2(res[n][0] * f0, res[n][1] * f0);
    if (rb < nrows)
      *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + rb) * H + h) * Dv + d) = pack_bf16x2(res[n][2] * f1, res[n][3] * f1);
  }
}

template <int DK, int DVK>
static int launch(const void* q, const void* ck, const void* cv, const int* tiles, int n_tiles, const int* table, int max_blocks,
                  void* out, int H, int G, int M, int block_size, float scale, int window, int keep_first, int combine,
                  float lambda, float post, float eps, cudaStream_t st) {
  constexpr int LDK = 16 * DK + 8, LDV = 16 * DVK + 8;
  const size_t smem = ((size_t)(kQ + 2 * kK) * LDK + (size_t)2 * kK * LDV) * sizeof(__nv_bfloat16);
  auto kern = multimap_attn_mma_kernel<DK, DVK>;
  if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  if ((1 << bs_log2) != block_size) return B200_ERR_UNSUPPORTED;
  kern<<<dim3(n_tiles, H), 128, smem, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)ck, (const __nv_bfloat16*)cv, tiles, table,
                                             max_blocks, (__nv_bfloat16*)out, H, G, M, bs_log2, scale, window, keep_first, combine,
                                             lambda, post, eps);
  B200_LAUNCH_CHECK();
  return 0;
}
}  // namespace b200

B200_API int b200_multimap_attn_mma(const void* q, const void* ck, const void* cv, const int* tiles, int n_tiles, const int* table,
                                    int max_blocks, void* out, int H, int G, int M, int D, int Dv, int block_size, float scale,
                                    int window, int keep_first, int combine, float lambda, float post, float eps, int dtype,
                                    void* stream) {
  using namespace b200;
  if (n_tiles <= 0) return 0;
  if (dtype != B200_DT_BF16 || !(scale > 0.f) || M < 1 || M > 2 || (combine && M != 2)) return B200_ERR_UNSUPPORTED;
  if (H <= 0 || G <= 0 || H % G || H > 65535) return B200_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
#define MM(DKV, DVKV)                                                                                                       \
  if (D == 16 * DKV && Dv == 16 * DVKV)                                                                                     \
    return launch<DKV, DVKV>(q, ck, cv, tiles, n_tiles, table, max_blocks, out, H, G, M, block_size, scale, window, keep_first, \
                             combine, lambda, post, eps, st);
#define MMROW(DKV) MM(DKV, 2) MM(DKV, 4) MM(DKV, 6) MM(DKV, 8)
  MMROW(2) MMROW(3) MMROW(4) MMROW(6) MMROW(8)
#undef MMROW
#undef MM
  return B200_ERR_UNSUPPORTED;
}
