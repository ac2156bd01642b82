// Talking-heads attention (see talking_attn.cu for the equations) for bf16 prompt pieces, on mma.sync tensor-core tiles.
//
// The mixing couples all heads of a (query, key) pair, so a CTA owns 16 consecutive query rows of one piece and ALL heads,
// one warp per head. Single tokens (a decode batch: tiles == NULL, positions and cache rows read on the device) run as tiles
// of one row: fifteen of the sixteen rows of every product are idle, which the tensor cores have to spare. Per chunk of 32 keys:
//   A  every warp forms its head's raw scores (Q_h K^T on m16n8k16, fp32 accumulators), applies the scale and the distance
//      penalty and leaves them in shared memory;
//   B  every thread takes a few (row, key) pairs, reads the H raw scores of a pair and writes the H mixed scores in place
//      (fp32 FMAs; pairs outside the window or the causal triangle become -inf);
//   C  every warp runs its head's online softmax on the mixed scores and multiplies P (rounded to bf16, as the operand of the
//      tensor-core product) with the staged key rows of its kv head, which are the values (ldmatrix.trans).
// Key pages are gathered through the block table into shared memory by cp.async, all kv heads of a position side by side,
// one chunk ahead of the one being worked on where two buffers fit. tcgen05 is not
// used: tiles are ragged (2 .. 64 rows at any position), head sizes any multiple of 16, and the scores must pass through
// fp32 CUDA-core work between the two products.
#include "mma_sync.cuh"
#include "../include/b200_ops.h"

namespace b200 {

constexpr int kTmRows = 16;           // query rows per CTA
constexpr int kTmKeys = 32;           // keys per chunk
constexpr int kTmMaxHeads = 16;       // one warp per head

template <int KS>                     // KS = D / 16
__global__ void __launch_bounds__(kTmMaxHeads * 32)
talking_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ gate, long long ldg,
                        const __nv_bfloat16* __restrict__ ck, const int* __restrict__ tiles, const int* __restrict__ pos,
                        const int* __restrict__ slots, const int* __restrict__ table, int max_blocks, const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ talk,
                        __nv_bfloat16* __restrict__ out, int H, int G, int bs_log2, float scale, int window, int nbuf) {
  constexpr int D = KS * 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tile = blockIdx.x, sub = blockIdx.y;
  int row0, nr, p0, slot;
  if (tiles) {
    const int trows = tiles[tile * 4 + 1];
    if (sub * kTmRows >= trows) return;
    row0 = tiles[tile * 4] + sub * kTmRows;
    nr = min(kTmRows, trows - sub * kTmRows);
    p0 = tiles[tile * 4 + 2] + sub * kTmRows;
    slot = tiles[tile * 4 + 3];
  } else {                                                // every token a tile of its own (a decode batch, read on the device)
    row0 = tile; nr = 1; p0 = pos[tile]; slot = slots[tile];
  }
  const int HD = H * D, GD = G * D, rep = H / G, BS = 1 << bs_log2;
  const int ldqs = HD + 8, ldks = GD + 8, ldr = kTmKeys + 1;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][ldqs]
  __nv_bfloat16* Kbuf = Qs + kTmRows * ldqs;                                 // nbuf x [32][ldks]
  float* raw = reinterpret_cast<float*>(Kbuf + nbuf * kTmKeys * ldks);       // [H][16][ldr]
  float* tk = raw + ((H * kTmRows * ldr + 3) & ~3);                          // [16][16], zero outside [H][H], rows read as float4
  const int tid = threadIdx.x, nth = blockDim.x;
  const int h = tid >> 5, lane = tid & 31, qd = lane & 3, rr = lane >> 2;
  const int kvh = h / rep;

  for (int idx = tid; idx < kTmRows * (HD / 8); idx += nth) {
    const int r = idx / (HD / 8), c = idx - r * (HD / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < nr) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + r) * ldq + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ldqs + c * 8) = v;
  }
  for (int e = tid; e < kTmMaxHeads * kTmMaxHeads; e += nth) {
    const int hh = e >> 4, g = e & 15;
    tk[e] = (hh < H && g < H) ? talk[hh * H + g] : 0.f;
  }
  const float r1h = r1[h], r2h = r2[h];
  const int* trow = table + (long long)slot * max_blocks;
  const int lo = window > 0 ? max(0, p0 - window + 1) : 0, hi = p0 + nr - 1;

  float o[2 * KS][4];
#pragma unroll
  for (int nt = 0; nt < 2 * KS; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // key rows of the chunk that starts at j0, all kv heads of a position side by side; rows past the piece's last key are zero
  auto stage = [&](int b, int j0) {
    __nv_bfloat16* Kd = Kbuf + b * kTmKeys * ldks;
    for (int idx = tid; idx < kTmKeys * (GD / 8); idx += nth) {
      const int jj = idx / (GD / 8), c = idx - jj * (GD / 8);
      const int j = j0 + jj;
      if (j <= hi) {
        const int g = (c * 8) / D, d = c * 8 - g * D;
        const long long blk = trow[j >> bs_log2];
        cp_async16(smem_u32(Kd + jj * ldks + c * 8), ck + ((blk * G + g) * BS + (j & (BS - 1))) * D + d);
      } else {
        *reinterpret_cast<uint4*>(Kd + jj * ldks + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  int buf = 0;
  if (nbuf == 2) { stage(0, lo); cp_async_commit(); }
  for (int j0 = lo; j0 <= hi; j0 += kTmKeys) {
    __syncthreads();                                      // the previous chunk's keys and scores have been used (and Qs is there)
    if (nbuf == 2) {                                      // the next chunk travels while this one is worked on
      if (j0 + kTmKeys <= hi) stage(buf ^ 1, j0 + kTmKeys);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      stage(0, j0);
      cp_async_commit();
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* Ks = Kbuf + buf * kTmKeys * ldks;
    // ---- A: raw scores of this warp's head
    {
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const __nv_bfloat16* qa = Qs + h * D + ks * 16 + 2 * qd;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + rr * ldqs);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(qa + (rr + 8) * ldqs);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + rr * ldqs + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(qa + (rr + 8) * ldqs + 8);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const __nv_bfloat16* kb = Ks + (nt * 8 + rr) * ldks + kvh * D + ks * 16 + 2 * qd;
          mma_bf16_16816(s[nt], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = rr + (e >> 1) * 8, c = nt * 8 + 2 * qd + (e & 1);
          const float dist = (float)max(p0 + r - (j0 + c), 0);
          raw[(h * kTmRows + r) * ldr + c] = s[nt][e] * scale - r1h * log1pf(r2h * dist);
        }
    }
    __syncthreads();
    // ---- B: mixing over the heads, pair by pair, in place
    for (int idx = tid; idx < nr * kTmKeys; idx += nth) {  // rows past the piece keep their raw (finite) scores and are never written
      const int r = idx >> 5, jj = idx & 31;
      const int i = p0 + r, j = j0 + jj;
      const bool vis = j <= i && (window == 0 || j > i - window);
      float v[kTmMaxHeads];
#pragma unroll
      for (int g = 0; g < kTmMaxHeads; ++g) v[g] = g < H ? raw[(g * kTmRows + r) * ldr + jj] : 0.f;
#pragma unroll
      for (int hh = 0; hh < kTmMaxHeads; ++hh) {
        if (hh < H) {
          float a = 0.f;
#pragma unroll
          for (int g4 = 0; g4 < kTmMaxHeads / 4; ++g4) {   // the same address in every lane: one broadcast read of four weights
            const float4 w = *reinterpret_cast<const float4*>(tk + hh * kTmMaxHeads + 4 * g4);
            a = fmaf(w.x, v[4 * g4], a); a = fmaf(w.y, v[4 * g4 + 1], a);
            a = fmaf(w.z, v[4 * g4 + 2], a); a = fmaf(w.w, v[4 * g4 + 3], a);
          }
          raw[(hh * kTmRows + r) * ldr + jj] = vis ? a : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- C: this head's online softmax and P V (the values are the staged keys of its kv head)
    {
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = raw[(h * kTmRows + rr + (e >> 1) * 8) * ldr + nt * 8 + 2 * qd + (e & 1)];
      float x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        x0 = fmaxf(x0, fmaxf(s[nt][0], s[nt][1]));
        x1 = fmaxf(x1, fmaxf(s[nt][2], s[nt][3]));
      }
      x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1)); x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
      x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1)); x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
      const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
      const float al0 = n0 == -INFINITY ? 1.f : expf(m0 - n0), al1 = n1 == -INFINITY ? 1.f : expf(m1 - n1);
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = n0 == -INFINITY ? 0.f : expf(s[nt][0] - n0);
        s[nt][1] = n0 == -INFINITY ? 0.f : expf(s[nt][1] - n0);
        s[nt][2] = n1 == -INFINITY ? 0.f : expf(s[nt][2] - n1);
        s[nt][3] = n1 == -INFINITY ? 0.f : expf(s[nt][3] - n1);
        t0 += s[nt][0] + s[nt][1];
        t1 += s[nt][2] + s[nt][3];
      }
      t0 += __shfl_xor_sync(0xffffffffu, t0, 1); t0 += __shfl_xor_sync(0xffffffffu, t0, 2);
      t1 += __shfl_xor_sync(0xffffffffu, t1, 1); t1 += __shfl_xor_sync(0xffffffffu, t1, 2);
      l0 = l0 * al0 + t0; l1 = l1 * al1 + t1;
      m0 = n0; m1 = n1;
#pragma unroll
      for (int nt = 0; nt < 2 * KS; ++nt) { o[nt][0] *= al0; o[nt][1] *= al0; o[nt][2] *= al1; o[nt][3] *= al1; }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        const uint32_t vrow = smem_u32(Ks + (kk * 16 + (lane & 15)) * ldks + kvh * D);
#pragma unroll
        for (int nt = 0; nt < 2 * KS; ++nt) {
          uint32_t b0, b1;
          ldsm_x2_trans(vrow + nt * 16, b0, b1);
          mma_bf16_16816(o[nt], a0, a1, a2, a3, b0, b1);
        }
      }
    }
    if (nbuf == 2) buf ^= 1;
  }
  const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
  for (int nt = 0; nt < 2 * KS; ++nt) {
    const int d = h * D + nt * 8 + 2 * qd;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = rr + half * 8;
      if (r < nr) {
        float v0 = o[nt][2 * half] * (half ? i1 : i0), v1 = o[nt][2 * half + 1] * (half ? i1 : i0);
        if (gate) {
          const __nv_bfloat16* gp = gate + (long long)(row0 + r) * ldg + d;
          v0 *= 1.f / (1.f + expf(-__bfloat162float(gp[0])));
          v1 *= 1.f / (1.f + expf(-__bfloat162float(gp[1])));
        }
        *reinterpret_cast<uint32_t*>(out + (long long)(row0 + r) * HD + d) = pack_bf16x2(v0, v1);
      }
    }
  }
}
}  // namespace b200

B200_API int b200_talking_attn_mma(const void* q, long long ldq, const void* gate, long long ldg, const void* ck, const int* tiles,
                                   int n_tiles, const int* pos, const int* slot, const int* table, int max_blocks, const float* r1, const float* r2,
                                   const float* talk, void* out, int H, int G, int D, int block_size, float scale, int window,
                                   void* stream) {
  using namespace b200;
  if (n_tiles <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || block_size <= 0 || (block_size & (block_size - 1)) || window < 0)
    return B200_ERR_BAD_SHAPE;
  if (H > kTmMaxHeads || D % 16 || D > 128 || D == 80 || D == 112 || ldq % 8 || (reinterpret_cast<uintptr_t>(q) & 15))
    return B200_ERR_UNSUPPORTED;
  const size_t kbytes = (size_t)kTmKeys * (G * D + 8) * 2;
  const size_t fixed = (size_t)kTmRows * (H * D + 8) * 2 + (size_t)((H * kTmRows * (kTmKeys + 1) + 3) & ~3) * 4 +
                       (size_t)kTmMaxHeads * kTmMaxHeads * 4;
  const int nbuf = fixed + 2 * kbytes <= 200 * 1024 ? 2 : 1;       // two key buffers where they fit
  const size_t smem = fixed + nbuf * kbytes;
  if (smem > 200 * 1024) return B200_ERR_UNSUPPORTED;
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  cudaStream_t st = (cudaStream_t)stream;
  if (!tiles && (!pos || !slot)) return B200_ERR_BAD_SHAPE;
  dim3 grid(n_tiles, tiles ? 4 : 1);
  typedef __nv_bfloat16 bf;
#define TMMA(KS)                                                                                                              \
  do {                                                                                                                        \
    auto kern = talking_attn_mma_kernel<KS>;                                                                                  \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    kern<<<grid, H * 32, smem, st>>>((const bf*)q, ldq, (const bf*)gate, ldg, (const bf*)ck, tiles, pos, slot, table, max_blocks, r1, r2, talk, \
                                     (bf*)out, H, G, bs_log2, scale, window, nbuf);                                           \
  } while (0)
  switch (D / 16) {
    case 1: TMMA(1); break;
    case 2: TMMA(2); break;
    case 3: TMMA(3); break;
    case 4: TMMA(4); break;
    case 6: TMMA(6); break;
    default: TMMA(8); break;
  }
#undef TMMA
  B200_LAUNCH_CHECK();
  return 0;
}
