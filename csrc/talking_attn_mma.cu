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

constexpr float kLog2e = 1.4426950408889634f;

template <int N> __device__ __forceinline__ void cp_async_wait_upto(int pending) {
  // wait until at most `pending` (< N) of the committed copy groups are still in flight
  if (pending <= 0) cp_async_wait<0>();
  else if (pending == 1) cp_async_wait<1>();
  else if (pending == 2) cp_async_wait<2>();
  else cp_async_wait<3>();
}

// KS = D / 16. SINGLE: every tile is one token (a decode batch); only row 0 of the 16-row products is live, so the query and
// the scores take one row of shared memory instead of sixteen and the room goes to more key chunks in flight.
template <int KS, bool SINGLE>
__global__ void __launch_bounds__(kTmMaxHeads * 32)
talking_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ gate, long long ldg,
                        const __nv_bfloat16* __restrict__ ck, const int* __restrict__ tiles, const int* __restrict__ pos,
                        const int* __restrict__ slots, const int* __restrict__ table, int max_blocks, const float* __restrict__ r1,
                        const float* __restrict__ r2, const float* __restrict__ talk, __nv_bfloat16* __restrict__ out, int H, int G,
                        int bs_log2, float scale, int window, int nbuf, float* __restrict__ part) {
  constexpr int D = KS * 16;
  constexpr int QR = SINGLE ? 1 : kTmRows;                // rows of the query and score buffers
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tile = blockIdx.x, sub = blockIdx.y;
  int row0, nr, p0, slot;
  if (!SINGLE) {
    const int trows = tiles[tile * 4 + 1];
    if (sub * kTmRows >= trows) return;
    row0 = tiles[tile * 4] + sub * kTmRows;
    nr = min(kTmRows, trows - sub * kTmRows);
    p0 = tiles[tile * 4 + 2] + sub * kTmRows;
    slot = tiles[tile * 4 + 3];
  } else {                                                // positions and cache rows are read on the device (graph replay)
    row0 = tile; nr = 1; p0 = pos[tile]; slot = slots[tile];
  }
  const int HD = H * D, GD = G * D, rep = H / G, BS = 1 << bs_log2;
  const int ldqs = HD + 8, ldks = GD + 8, ldr = kTmKeys + 1;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [QR][ldqs]
  __nv_bfloat16* Kbuf = Qs + QR * ldqs;                                      // nbuf x [32][ldks]
  float* raw = reinterpret_cast<float*>(Kbuf + nbuf * kTmKeys * ldks);       // [H][QR][ldr]
  float* tk = raw + ((H * QR * ldr + 3) & ~3);                               // [16][16] indexed [from][to], zero outside [H][H]
  float* pen = tk + kTmMaxHeads * kTmMaxHeads;                               // [H][48]: this chunk's distance penalties
  const int tid = threadIdx.x, nth = blockDim.x;
  const int h = tid >> 5, lane = tid & 31, qd = lane & 3, rr = lane >> 2;
  const int kvh = h / rep;

  for (int idx = tid; idx < QR * (HD / 8); idx += nth) {
    const int r = idx / (HD / 8), c = idx - r * (HD / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < nr) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + r) * ldq + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ldqs + c * 8) = v;
  }
  for (int e = tid; e < kTmMaxHeads * kTmMaxHeads; e += nth) {
    const int g = e >> 4, hh = e & 15;                      // transposed: the weights of four output heads for one input head
    tk[e] = (hh < H && g < H) ? talk[hh * H + g] : 0.f;     // are one 16-byte read
  }
  const float r1h = r1[h], r2h = r2[h];
  const int* trow = table + (long long)slot * max_blocks;
  const int lo = window > 0 ? max(0, p0 - window + 1) : 0, hi = p0 + nr - 1;
  const int nchunks = (hi - lo) / kTmKeys + 1;
  // a single token's chunks may be shared out over gridDim.y CTAs (`part` given): each walks a run of chunks and leaves its
  // unnormalised sums, running maximum and normaliser per head for the merge kernel
  int k_lo = 0, k_hi = nchunks;
  if (SINGLE && part) {
    const int per = (nchunks + (int)gridDim.y - 1) / (int)gridDim.y;
    k_lo = min(nchunks, sub * per);
    k_hi = min(nchunks, k_lo + per);
  }
  // chunk k (k = 0 is the one nearest to the queries: the running maximum settles early and later chunks seldom rescale)
  auto chunk_j0 = [&](int k) { return lo + (nchunks - 1 - k) * kTmKeys; };

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

  float o[2 * KS][4];
#pragma unroll
  for (int nt = 0; nt < 2 * KS; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int k = k_lo; k < k_lo + nbuf - 1; ++k) {            // the first chunks are on their way before the walk starts
    if (k < k_hi) stage((k - k_lo) % nbuf, chunk_j0(k));
    cp_async_commit();
  }
  for (int k = k_lo; k < k_hi; ++k) {
    const int j0 = chunk_j0(k);
    if (nbuf > 1) {
      // this chunk's copies were issued nbuf - 1 iterations ago: wait for them, then one barrier both publishes them and
      // says that the previous chunk's keys and scores have been used (and that Qs is there); only then is the buffer of
      // the previous chunk refilled, while this chunk is worked on
      cp_async_wait_upto<4>(nbuf - 2);
      __syncthreads();
      if (k + nbuf - 1 < k_hi) stage((k - k_lo + nbuf - 1) % nbuf, chunk_j0(k + nbuf - 1));
      cp_async_commit();
    } else {
      __syncthreads();
      stage(0, j0);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
    }
    const __nv_bfloat16* Ks = Kbuf + ((k - k_lo) % nbuf) * kTmKeys * ldks;
    // the penalty depends on the head and on the distance only: the 47 distances a chunk's (row, key) pairs can have are
    // formed once per head here, not once per pair
    for (int x = lane; x < kTmKeys + kTmRows - 1; x += 32) {
      const int dist = p0 - j0 - (kTmKeys - 1) + x;
      pen[h * 48 + x] = dist > 0 ? r1h * log1pf(r2h * (float)dist) : 0.f;
    }
    __syncwarp();
    // ---- A: raw scores of this warp's head
    {
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const int mi = lane >> 3, l8 = lane & 7;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t a0, a1, a2, a3;
        if (SINGLE) {                                     // only row 0 is there
          const __nv_bfloat16* qa = Qs + h * D + ks * 16 + 2 * qd;
          a0 = rr == 0 ? *reinterpret_cast<const uint32_t*>(qa) : 0u;
          a2 = rr == 0 ? *reinterpret_cast<const uint32_t*>(qa + 8) : 0u;
          a1 = a3 = 0u;
        } else {
          ldsm_x4(smem_u32(Qs + (l8 + (mi & 1) * 8) * ldqs + h * D + ks * 16 + (mi >> 1) * 8), a0, a1, a2, a3);
        }
#pragma unroll
        for (int np = 0; np < 2; ++np) {                  // two key blocks of 8 per ldmatrix
          uint32_t b0, b1, b2, b3;
          ldsm_x4(smem_u32(Ks + ((2 * np + (mi >> 1)) * 8 + l8) * ldks + kvh * D + ks * 16 + (mi & 1) * 8), b0, b1, b2, b3);
          mma_bf16_16816(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = rr + (e >> 1) * 8, c = nt * 8 + 2 * qd + (e & 1);
          if (!SINGLE || r == 0) raw[(h * QR + r) * ldr + c] = s[nt][e] * scale - pen[h * 48 + r - c + (kTmKeys - 1)];
        }
    }
    __syncthreads();
    // ---- B: mixing over the heads, in place. A full tile gives every thread whole pairs (read the H raw scores of a pair,
    // write its H mixed ones); a tile of few rows has fewer pairs than threads, so the heads of a pair are shared out over
    // several threads, which all read before any of them writes. Two output heads per packed fp32 FMA.
    {
      const int npairs = nr * kTmKeys;
      const int ngroups = max(1, nth / npairs);             // threads per pair
      const int hpg = (((H + ngroups - 1) / ngroups) + 3) & ~3;      // heads per thread of a pair, in fours
      auto mix = [&](int r, int jj, const float (&v)[kTmMaxHeads], int h_lo, int h_hi) {
        const int i = p0 + r, j = j0 + jj;
        const bool vis = j <= i && (window == 0 || j > i - window);
#pragma unroll
        for (int h4 = 0; h4 < kTmMaxHeads; h4 += 4) {
          if (h4 >= h_lo && h4 < h_hi) {
            float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
            for (int g = 0; g < kTmMaxHeads; ++g) {        // the same address in every lane: one broadcast read of four weights
              const float4 w = *reinterpret_cast<const float4*>(tk + g * kTmMaxHeads + h4);
              const float2 vg = make_float2(v[g], v[g]);
              a01 = __ffma2_rn(make_float2(w.x, w.y), vg, a01);
              a23 = __ffma2_rn(make_float2(w.z, w.w), vg, a23);
            }
            float* dst = raw + ((h4 * QR + r) * ldr + jj);
            if (h4 < H) dst[0] = vis ? a01.x : -INFINITY;
            if (h4 + 1 < H) dst[QR * ldr] = vis ? a01.y : -INFINITY;
            if (h4 + 2 < H) dst[2 * QR * ldr] = vis ? a23.x : -INFINITY;
            if (h4 + 3 < H) dst[3 * QR * ldr] = vis ? a23.y : -INFINITY;
          }
        }
      };
      if (ngroups > 1) {
        const int pair = tid % npairs, grp = tid / npairs;
        const int r = pair >> 5, jj = pair & 31;
        float v[kTmMaxHeads];
#pragma unroll
        for (int g = 0; g < kTmMaxHeads; ++g) v[g] = g < H ? raw[(g * QR + r) * ldr + jj] : 0.f;
        __syncthreads();
        if (grp < ngroups) mix(r, jj, v, grp * hpg, min(H, (grp + 1) * hpg));
      } else {
        for (int idx = tid; idx < npairs; idx += nth) {     // rows past the piece keep their raw (finite) scores and are never written
          const int r = idx >> 5, jj = idx & 31;
          float v[kTmMaxHeads];
#pragma unroll
          for (int g = 0; g < kTmMaxHeads; ++g) v[g] = g < H ? raw[(g * QR + r) * ldr + jj] : 0.f;
          mix(r, jj, v, 0, H);
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
        for (int e = 0; e < 4; ++e) {
          const int r = rr + (e >> 1) * 8;
          s[nt][e] = (!SINGLE || r == 0) ? raw[(h * QR + r) * ldr + nt * 8 + 2 * qd + (e & 1)] : -INFINITY;
        }
      float x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        x0 = fmaxf(x0, fmaxf(s[nt][0], s[nt][1]));
        x1 = fmaxf(x1, fmaxf(s[nt][2], s[nt][3]));
      }
      x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1)); x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
      x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1)); x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
      const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
      const float al0 = n0 == -INFINITY ? 1.f : ex2_approx((m0 - n0) * kLog2e), al1 = n1 == -INFINITY ? 1.f : ex2_approx((m1 - n1) * kLog2e);
      const float c0 = -n0 * kLog2e, c1 = -n1 * kLog2e;
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = n0 == -INFINITY ? 0.f : ex2_approx(fmaf(s[nt][0], kLog2e, c0));
        s[nt][1] = n0 == -INFINITY ? 0.f : ex2_approx(fmaf(s[nt][1], kLog2e, c0));
        s[nt][2] = n1 == -INFINITY ? 0.f : ex2_approx(fmaf(s[nt][2], kLog2e, c1));
        s[nt][3] = n1 == -INFINITY ? 0.f : ex2_approx(fmaf(s[nt][3], kLog2e, c1));
        t0 += s[nt][0] + s[nt][1];
        t1 += s[nt][2] + s[nt][3];
      }
      t0 += __shfl_xor_sync(0xffffffffu, t0, 1); t0 += __shfl_xor_sync(0xffffffffu, t0, 2);
      t1 += __shfl_xor_sync(0xffffffffu, t1, 1); t1 += __shfl_xor_sync(0xffffffffu, t1, 2);
      l0 = l0 * al0 + t0; l1 = l1 * al1 + t1;
      m0 = n0; m1 = n1;
      if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
        for (int nt = 0; nt < 2 * KS; ++nt) { o[nt][0] *= al0; o[nt][1] *= al0; o[nt][2] *= al1; o[nt][3] *= al1; }
      }
      const int mi = lane >> 3, l8 = lane & 7;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        const uint32_t vrow = smem_u32(Ks + (kk * 16 + (mi & 1) * 8 + l8) * ldks + kvh * D + (mi >> 1) * 8);
#pragma unroll
        for (int np = 0; np < KS; ++np) {                 // two blocks of 8 channels per ldmatrix
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(vrow + np * 32, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * np], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  if (SINGLE && part) {                                     // row 0 lives in the lanes of the first quad row
    if (rr == 0) {
      float* dst = part + (((long long)tile * gridDim.y + sub) * H + h) * (D + 2);
#pragma unroll
      for (int nt = 0; nt < 2 * KS; ++nt) *reinterpret_cast<float2*>(dst + nt * 8 + 2 * qd) = make_float2(o[nt][0], o[nt][1]);
      if (qd == 0) *reinterpret_cast<float2*>(dst + D) = make_float2(m0, l0);
    }
    return;
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

// out[t, h, :] = sum_s w_s o_s / sum_s w_s l_s, w_s = exp(m_s - max_s m_s), over the S partial walks of a token; then the gate.
__global__ void __launch_bounds__(128)
talking_attn_merge_kernel(const float* __restrict__ part, const __nv_bfloat16* __restrict__ gate, long long ldg,
                          __nv_bfloat16* __restrict__ out, int H, int D, int S) {
  const long long t = blockIdx.x;
  const int h = blockIdx.y;
  const float* p = part + ((t * S) * H + h) * (D + 2);
  const long long ss = (long long)H * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, p[s * ss + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int s = 0; s < S; ++s) {
      const float m = p[s * ss + D];
      const float w = m == -INFINITY ? 0.f : expf(m - M);
      num = fmaf(w, p[s * ss + d], num);
      den = fmaf(w, p[s * ss + D + 1], den);
    }
    float v = num / den;
    const long long idx = (long long)h * D + d;
    if (gate) v *= 1.f / (1.f + expf(-__bfloat162float(gate[t * ldg + idx])));
    out[t * (long long)(H * D) + idx] = __float2bfloat16(v);
  }
}
}  // namespace b200

B200_API int b200_talking_attn_mma(const void* q, long long ldq, const void* gate, long long ldg, const void* ck, const int* tiles,
                                   int n_tiles, const int* pos, const int* slot, const int* table, int max_blocks,
                                   const float* r1, const float* r2, const float* talk, void* out, int H, int G, int D,
                                   int block_size, float scale, int window, float* part, int nsplit, void* stream) {
  using namespace b200;
  if (n_tiles <= 0) return 0;
  if (nsplit < 1 || nsplit > 65535 || (nsplit > 1 && (!part || tiles))) return B200_ERR_BAD_SHAPE;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || block_size <= 0 || (block_size & (block_size - 1)) || window < 0)
    return B200_ERR_BAD_SHAPE;
  if (H > kTmMaxHeads || D % 16 || D > 128 || D == 80 || D == 112 || ldq % 8 || (reinterpret_cast<uintptr_t>(q) & 15))
    return B200_ERR_UNSUPPORTED;
  if (!tiles && (!pos || !slot)) return B200_ERR_BAD_SHAPE;
  const bool single = tiles == nullptr;
  const int QR = single ? 1 : kTmRows;
  const size_t kbytes = (size_t)kTmKeys * (G * D + 8) * 2;
  const size_t fixed = (size_t)QR * (H * D + 8) * 2 + (size_t)((H * QR * (kTmKeys + 1) + 3) & ~3) * 4 +
                       (size_t)kTmMaxHeads * kTmMaxHeads * 4 + (size_t)H * 48 * 4;
  // as many key chunks in flight as fit (at most 4): a decode batch streams its keys from HBM and needs the depth; a prompt's
  // neighbouring tiles share their keys through L2 and two buffers are enough to hide the gather
  int nbuf = 1;
  while (nbuf < (single ? 4 : 2) && fixed + (nbuf + 1) * kbytes <= 200 * 1024) ++nbuf;
  const size_t smem = fixed + nbuf * kbytes;
  if (smem > 200 * 1024) return B200_ERR_UNSUPPORTED;
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(n_tiles, single ? nsplit : 4);
  float* pw = nsplit > 1 ? part : nullptr;
  typedef __nv_bfloat16 bf;
#define TMMA_K(KS, SG)                                                                                                        \
  do {                                                                                                                        \
    auto kern = talking_attn_mma_kernel<KS, SG>;                                                                              \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    kern<<<grid, H * 32, smem, st>>>((const bf*)q, ldq, (const bf*)gate, ldg, (const bf*)ck, tiles, pos, slot, table, max_blocks, \
                                     r1, r2, talk, (bf*)out, H, G, bs_log2, scale, window, nbuf, pw);                         \
  } while (0)
#define TMMA(KS)                                                                                                              \
  do {                                                                                                                        \
    if (single) TMMA_K(KS, true); else TMMA_K(KS, false);                                                                     \
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
#undef TMMA_K
  B200_LAUNCH_CHECK();
  if (pw) {
    talking_attn_merge_kernel<<<dim3(n_tiles, H), D >= 128 ? 128 : (D > 32 ? 64 : 32), 0, st>>>(pw, (const bf*)gate, ldg, (bf*)out, H, D, nsplit);
    B200_LAUNCH_CHECK();
  }
  return 0;
}
