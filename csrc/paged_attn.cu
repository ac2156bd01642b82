// Ragged attention over a paged KV cache, with optional attention sinks and an optional sliding window.
//
// A serving step is a flat list of query tokens: token t belongs to the sequence in cache row `slot[t]` and sits at
// position `pos[t]` of it. A prompt piece contributes consecutive positions, a decoding sequence one token, and the two
// kinds share a launch. The cache is [blocks, Hkv, block_size, D] per layer with a block table [rows, max_blocks]
// (logical block j of a row -> physical block). The step first stores the new tokens' K/V, then every query reads keys
// 0 .. pos[t] of its own row, so a piece attends to the pieces before it and to its own earlier tokens with no special case.
//
//   b200_rope_paged_store   rotary embedding on q (in place) and k, k -> cache K; the value rows come either from a v
//                           section of the projection or (v_from_k) are the keys as projected, before rotation.
//                           Pairs are interleaved (2i, 2i+1) or split (i, i + rot/2); only the first `rot` dims turn.
//   b200_paged_attn         per-token attention in fp32 arithmetic over a 16-bit or 32-bit cache, any head size up to 256:
//                           a vector kernel (16-byte row chunks, the query heads of a KV group share the K/V reads) and a
//                           scalar one for head sizes that are not whole chunks. `nsplit` > 1 cuts the keys of every token
//                           into that many ranges (long-context decode); a second kernel merges the partial
//                           (max, sum, acc) triples.
//   b200_paged_attn_mma     bf16 prompt pieces on the tensor cores (mma.sync m16n8k16): 64 query rows of one piece per
//                           CTA, one cache page (or 64 keys of it) per iteration.
//
// A sink is a per-head logit that takes part in the softmax denominator only: the running maximum starts at the sink and
// the running sum at 1, which is exp(sink - max) for that start.
#include "common.cuh"
#include "mma_sync.cuh"
#include "../include/b200_ops.h"

namespace b200 {

// ------------------------------------------------------------------------------------------------------------------
// rotary + cache store
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rope_paged_store_kernel(T* __restrict__ qkv, long long row_stride, const float* __restrict__ cs, const float* __restrict__ sn,
                        const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                        T* __restrict__ ck, T* __restrict__ cv, int H, int G, int D, int rot, int block_size, int interleaved,
                        int v_from_k) {
  const int t = blockIdx.x;
  const int p = pos[t];
  const int s = slot[t];
  T* row = qkv + (long long)t * row_stride;
  const float* c = cs + (long long)p * (rot / 2);
  const float* sgn = sn + (long long)p * (rot / 2);
  const int blk = table[(long long)s * max_blocks + p / block_size];
  const int off = p % block_size;
  const int hr = rot / 2;
  // item i < hr: the rotary pair i; item i >= hr: the pass-through dims rot + 2 (i - hr) and the one after it
  const int items = hr + (D - rot + 1) / 2;
  for (int w = threadIdx.x; w < (H + G) * items; w += blockDim.x) {
    const int h = w / items, i = w % items;
    T* x = row + (long long)h * D;
    int d0, d1;
    bool turn = i < hr;
    if (turn) {
      d0 = interleaved ? 2 * i : i;
      d1 = interleaved ? 2 * i + 1 : i + hr;
    } else {
      d0 = rot + 2 * (i - hr);
      d1 = d0 + 1;
    }
    const bool has1 = d1 < D;
    const float u = to_f32<T>(x[d0]);
    const float v = has1 ? to_f32<T>(x[d1]) : 0.f;
    float ru = u, rv = v;
    if (turn) {
      const float cc = c[i], ss = sgn[i];
      ru = u * cc - v * ss;
      rv = v * cc + u * ss;
      x[d0] = from_f32<T>(ru);
      x[d1] = from_f32<T>(rv);
    }
    if (h >= H) {
      const int g = h - H;
      const long long base = (((long long)blk * G + g) * block_size + off) * D;
      ck[base + d0] = from_f32<T>(ru);
      if (has1) ck[base + d1] = from_f32<T>(rv);
      if (v_from_k && cv) {                             // cv NULL: no value pool (the key rows are read as values)
        cv[base + d0] = from_f32<T>(u);
        if (has1) cv[base + d1] = from_f32<T>(v);
      }
    }
  }
  if (!v_from_k && cv) {
    const T* vsrc = row + (long long)(H + G) * D;
    for (int w = threadIdx.x; w < G * D; w += blockDim.x) {
      const int g = w / D, d = w % D;
      cv[(((long long)blk * G + g) * block_size + off) * D + d] = vsrc[w];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// one warp per (token, query head)
// ------------------------------------------------------------------------------------------------------------------
constexpr int kMaxD = 256;
constexpr int kAccPerLane = kMaxD / 32;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(q[d], to_f32<T>(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int D) {
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

// q: [tokens, q_stride] (head h at h * D); out: [tokens, H * D]; part: [tokens, H, nsplit, D + 2] fp32 when nsplit > 1
template <typename T>
__global__ void __launch_bounds__(256)
paged_attn_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ ck, const T* __restrict__ cv,
                  const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                  const float* __restrict__ sinks, T* __restrict__ out, float* __restrict__ part, int H, int G, int D,
                  int block_size, float scale, int window, int nsplit) {
  extern __shared__ float qs[];                      // [warps, D]
  const int t = blockIdx.x;
  const int g = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int rep = H / G;
  const int p = pos[t];
  const int s = slot[t];
  const int* trow = table + (long long)s * max_blocks;
  int k_lo = 0, k_hi = p + 1;                        // keys [k_lo, k_hi)
  if (window > 0 && p + 1 - window > 0) k_lo = p + 1 - window;
  if (nsplit > 1) {
    const int span = k_hi - k_lo;
    const int chunk = ((span + nsplit - 1) / nsplit + 31) / 32 * 32;
    k_lo = k_lo + split * chunk;
    k_hi = min(k_hi, k_lo + chunk);
  }
  float* myq = qs + warp * D;
  for (int hh = warp; hh < rep; hh += nwarps) {
    const int h = g * rep + hh;
    const T* qr = q + (long long)t * q_stride + (long long)h * D;
    __syncwarp();
    for (int d = lane; d < D; d += 32) myq[d] = to_f32<T>(qr[d]);
    __syncwarp();
    const bool own_sink = sinks != nullptr && nsplit == 1;
    float m = own_sink ? sinks[h] : -INFINITY;
    float l = own_sink ? 1.f : 0.f;
    float acc[kAccPerLane];
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) acc[i] = 0.f;
    for (int k0 = k_lo; k0 < k_hi; k0 += 32) {
      const int kp = k0 + lane;
      const bool valid = kp < k_hi;
      long long rowoff = 0;
      float sc = -INFINITY;
      if (valid) {
        const int blk = trow[kp / block_size];
        rowoff = (((long long)blk * G + g) * block_size + kp % block_size) * D;
        sc = dot_row<T>(myq, ck + rowoff, D) * scale;
      }
      const float m_new = fmaxf(m, warp_max(sc));
      const float pj = valid ? expf(sc - m_new) : 0.f;
      const float resc = (m == -INFINITY) ? 0.f : expf(m - m_new);
      l = l * resc + warp_sum(pj);
      m = m_new;
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) acc[i] *= resc;
      const int nk = min(32, k_hi - k0);
      for (int j = 0; j < nk; ++j) {
        const float w = __shfl_sync(0xffffffffu, pj, j);
        const long long ro = __shfl_sync(0xffffffffu, rowoff, j);
        const T* vr = cv + ro;
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(w, to_f32<T>(vr[d]), acc[i]);
        }
      }
    }
    if (nsplit == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = out + (long long)t * H * D + (long long)h * D;
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = from_f32<T>(acc[i] * inv);
      }
    } else {
      float* pr = part + (((long long)t * H + h) * nsplit + split) * (D + 2);
      if (lane == 0) { pr[0] = m; pr[1] = l; }
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) pr[2 + d] = acc[i];
      }
    }
  }
}

// Vector variant (head size a multiple of one 16-byte chunk, at most 32 chunks): a CTA owns one token, up to HB query heads
// of one KV group and one key range. A lane is (key sub-index, chunk): the CP lanes of a group read one K row and the same V
// row with one 16-byte load each, so a warp instruction covers 32 / CP whole rows; the score is reduced over the group's
// lanes, and every lane keeps its own running (max, sum, acc) for the keys it has seen — nothing crosses groups inside the
// loop. Groups are merged by shuffles at the end, the four warps through shared memory.
template <typename T, int HB>
__global__ void __launch_bounds__(128)
paged_attn_vec_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ ck, const T* __restrict__ cv,
                      const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                      const float* __restrict__ sinks, T* __restrict__ out, float* __restrict__ part, int H, int G, int D,
                      int bs_log2, float scale, int window, int nsplit, int CP, int CPR) {
  constexpr int E = 16 / sizeof(T);                    // elements per chunk
  extern __shared__ float sm[];                        // [4 warps][HB][D + 2]
  const int t = blockIdx.x;
  const int rep = H / G;
  const int passes = (rep + HB - 1) / HB;
  const int g = blockIdx.y / passes;
  const int h0 = g * rep + (blockIdx.y % passes) * HB;
  const int nh = min(HB, g * rep + rep - h0);
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KPI = 32 / CP;                             // keys per warp instruction
  const int kk = lane / CP, c = lane % CP;
  const bool live = c < CPR;
  const int p = pos[t];
  const int* trow = table + (long long)slot[t] * max_blocks;
  int k_lo = 0, k_hi = p + 1;
  if (window > 0 && p + 1 - window > 0) k_lo = p + 1 - window;
  if (nsplit > 1) {
    const int span = k_hi - k_lo;
    const int chunk = ((span + nsplit - 1) / nsplit + 31) / 32 * 32;
    k_lo = k_lo + split * chunk;
    k_hi = min(k_hi, k_lo + chunk);
  }
  float qv[HB][E], acc[HB][E], m[HB], l[HB];
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    m[hh] = -INFINITY;
    l[hh] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      acc[hh][e] = 0.f;
      qv[hh][e] = (live && hh < nh) ? to_f32<T>(q[(long long)t * q_stride + (long long)(h0 + hh) * D + c * E + e]) * scale : 0.f;
    }
  }
  const int bs_mask = (1 << bs_log2) - 1;
  const int stride = 4 * KPI;
  constexpr int U = HB >= 4 ? 2 : 4;                   // keys in flight per lane: their loads are issued before the first is used
                                                       // (four heads per lane leave registers for two)
  for (int kb = k_lo; kb < k_hi; kb += stride * U) {
    uint4 kr[U], vr[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k0 = kb + u * stride + warp * KPI + kk;
      valid[u] = k0 < k_hi;
      kr[u] = vr[u] = make_uint4(0, 0, 0, 0);
      if (valid[u] && live) {
        const long long off = ((((long long)trow[k0 >> bs_log2] * G + g) << bs_log2) + (k0 & bs_mask)) * D + c * E;
        kr[u] = *reinterpret_cast<const uint4*>(ck + off);
        vr[u] = *reinterpret_cast<const uint4*>(cv + off);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kb + u * stride >= k_hi) break;             // uniform over the CTA: no lane has a key in this or a later slot
      float kf[E], vf[E];
      const T* kp = reinterpret_cast<const T*>(&kr[u]);
      const T* vp = reinterpret_cast<const T*>(&vr[u]);
#pragma unroll
      for (int e = 0; e < E; ++e) { kf[e] = to_f32<T>(kp[e]); vf[e] = to_f32<T>(vp[e]); }
#pragma unroll
      for (int hh = 0; hh < HB; ++hh) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) s = fmaf(qv[hh][e], kf[e], s);
        for (int o = CP >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid[u]) {
          const float mn = fmaxf(m[hh], s);
          const float r = expf(m[hh] - mn);           // 0 on the first key (m = -inf)
          const float pj = expf(s - mn);
          m[hh] = mn;
          l[hh] = l[hh] * r + pj;
#pragma unroll
          for (int e = 0; e < E; ++e) acc[hh][e] = fmaf(pj, vf[e], acc[hh][e] * r);
        }
      }
    }
  }
  // merge the key groups of the warp
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    for (int o = CP; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[hh], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[hh], o);
      const float mn = fmaxf(m[hh], m2);
      const float e1 = m[hh] == -INFINITY ? 0.f : expf(m[hh] - mn);
      const float e2 = m2 == -INFINITY ? 0.f : expf(m2 - mn);
      l[hh] = l[hh] * e1 + l2 * e2;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float a2 = __shfl_xor_sync(0xffffffffu, acc[hh][e], o);
        acc[hh][e] = acc[hh][e] * e1 + a2 * e2;
      }
      m[hh] = mn;
    }
    if (kk == 0 && live) {
      float* w = sm + (warp * HB + hh) * (D + 2);
      if (c == 0) { w[0] = m[hh]; w[1] = l[hh]; }
#pragma unroll
      for (int e = 0; e < E; ++e) w[2 + c * E + e] = acc[hh][e];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
    const int hh = i / D, d = i % D;
    const int h = h0 + hh;
    const bool own_sink = sinks != nullptr && nsplit == 1;
    float mt = own_sink ? sinks[h] : -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm[(w * HB + hh) * (D + 2)]);
    float lt = own_sink ? expf(sinks[h] - mt) : 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* ws = sm + (w * HB + hh) * (D + 2);
      if (ws[0] != -INFINITY) {
        const float e = expf(ws[0] - mt);
        lt += ws[1] * e;
        at += ws[2 + d] * e;
      }
    }
    if (nsplit == 1) {
      out[((long long)t * H + h) * D + d] = from_f32<T>(lt > 0.f ? at / lt : 0.f);
    } else {
      float* pr = part + (((long long)t * H + h) * nsplit + split) * (D + 2);
      if (d == 0) { pr[0] = mt; pr[1] = lt; }
      pr[2 + d] = at;
    }
  }
}

template <typename T>
__global__ void paged_attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ sinks, T* __restrict__ out,
                                        int H, int D, int nsplit) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* pr = part + ((long long)t * H + h) * nsplit * (D + 2);
  float m = sinks ? sinks[h] : -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, pr[s * (D + 2)]);
  float l = sinks ? expf(sinks[h] - m) : 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = pr[s * (D + 2)];
    if (ms != -INFINITY) l += pr[s * (D + 2) + 1] * expf(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = pr[s * (D + 2)];
      if (ms != -INFINITY) a += pr[s * (D + 2) + 2 + d] * expf(ms - m);
    }
    out[((long long)t * H + h) * D + d] = from_f32<T>(a * inv);
  }
}


// ------------------------------------------------------------------------------------------------------------------
// prompt pieces on the tensor cores (bf16): 64 query rows x 64 keys per iteration, 4 warps of 16 rows
// ------------------------------------------------------------------------------------------------------------------
constexpr int kTQ = 64, kTK = 64;

// tiles: [n_tiles, 4] = (first row in the batch, rows, position of the first row, cache row)
template <int DK>                                     // head size = 16 * DK
__global__ void __launch_bounds__(128, 3)             // three CTAs per SM: 4 x 17 KB tiles at head size 128, <= 170 registers
paged_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ ck,
                      const __nv_bfloat16* __restrict__ cv, const int* __restrict__ tiles, const int* __restrict__ table,
                      int max_blocks, const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, int H, int G,
                      int bs_log2, float scale) {
  constexpr int D = 16 * DK;
  constexpr int LD = D + 8;                           // padded row (elements): ldmatrix rows land in different banks
  constexpr int CH = D / 8;                           // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [2][64][LD]
  __nv_bfloat16* sv = sk + 2 * kTK * LD;                                      // [2][64][LD]
  __nv_bfloat16* sq = sk + kTK * LD;                                          // Q is staged in K buffer 1 until its fragments are read
  // later tiles of a piece see more keys: taking them first keeps the long CTAs out of the last wave
  const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int g = h / (H / G);
  const int row0 = tiles[tile * 4], nrows = tiles[tile * 4 + 1], pos0 = tiles[tile * 4 + 2], slot = tiles[tile * 4 + 3];
  const int* trow = table + (long long)slot * max_blocks;
  const int kv_len = pos0 + nrows;
  const int nkb = (kv_len + kTK - 1) / kTK;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // two threads per key row, alternating 16-byte chunks (a pair fills whole 32-byte sectors); one page lookup per row
  const int bs_mask = (1 << bs_log2) - 1;
  auto load_kv = [&](int buf, int kb) {
    const int r = tid >> 1, half = tid & 1;
    const int kp = kb * kTK + r;
    __nv_bfloat16* dk = sk + (buf * kTK + r) * LD;
    __nv_bfloat16* dv = sv + (buf * kTK + r) * LD;
    if (kp < kv_len) {
      const long long off = ((((long long)trow[kp >> bs_log2] * G + g) << bs_log2) + (kp & bs_mask)) * D;
#pragma unroll
      for (int i = 0; i < CH / 2; ++i) {
        const int col = (half + 2 * i) * 8;
        cp_async16(smem_u32(dk + col), ck + off + col);
        cp_async16(smem_u32(dv + col), cv + off + col);
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH / 2; ++i) {
        const int col = (half + 2 * i) * 8;
        *reinterpret_cast<uint4*>(dk + col) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv + col) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  for (int c = tid; c < kTQ * CH; c += 128) {
    const int r = c / CH, col = (c % CH) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + r) * q_stride + (long long)h * D + col);
    *reinterpret_cast<uint4*>(sq + r * LD + col) = v;
  }
  load_kv(0, 0);
  cp_async_commit();
  __syncthreads();

  // Q fragments of this warp's 16 rows: DK k-steps of m16k16
  uint32_t qa[DK][4];
  {
    const int r = warp * 16 + (lane & 15);
    const int cofs = (lane >> 4) * 8;
#pragma unroll
    for (int k = 0; k < DK; ++k) ldsm_x4(smem_u32(sq + r * LD + k * 16 + cofs), qa[k][0], qa[k][1], qa[k][2], qa[k][3]);
  }
  __syncthreads();                                      // every warp has its Q fragments: buffer 1 may be refilled with keys

  const float LOG2E = 1.4426950408889634f;
  const float sl2 = scale * LOG2E;
  const float sink2 = sinks ? sinks[h] * LOG2E : -INFINITY;
  float m0 = sink2, m1 = sink2, l0 = 0.f, l1 = 0.f;
  float o[2 * DK][4];
#pragma unroll
  for (int i = 0; i < 2 * DK; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int qpos0 = pos0 + warp * 16 + (lane >> 2);    // position of this thread's first row; the second is + 8

  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) load_kv(buf ^ 1, kb + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* bk = sk + buf * kTK * LD;
    const __nv_bfloat16* bv = sv + buf * kTK * LD;

    // S = Q K^T, k-steps outermost: the eight key tiles of a step are independent accumulators, so consecutive MMAs never
    // wait for each other (tile-outermost would chain the k-steps of one accumulator back to back)
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int k = 0; k + 1 < DK; k += 2) {                // one ldmatrix.x4 feeds two k-steps of a key tile
      uint32_t b[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n)
        ldsm_x4(smem_u32(bk + (n * 8 + (lane & 7)) * LD + k * 16 + (lane >> 3) * 8), b[n][0], b[n][1], b[n][2], b[n][3]);
#pragma unroll
      for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k][0], qa[k][1], qa[k][2], qa[k][3], b[n][0], b[n][1]);
#pragma unroll
      for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k + 1][0], qa[k + 1][1], qa[k + 1][2], qa[k + 1][3], b[n][2], b[n][3]);
    }
    if (DK & 1) {
      constexpr int k = DK - 1;
      uint32_t b[8][2];
#pragma unroll
      for (int n = 0; n < 8; ++n) ldsm_x2(smem_u32(bk + (n * 8 + (lane & 7)) * LD + k * 16 + ((lane >> 3) & 1) * 8), b[n][0], b[n][1]);
#pragma unroll
      for (int n = 0; n < 8; ++n) mma_bf16_16816(s[n], qa[k][0], qa[k][1], qa[k][2], qa[k][3], b[n][0], b[n][1]);
    }
    // causal mask (only blocks that reach past this warp's first query position need one), running max on the raw scores,
    // then p = 2^(s * scale * log2e - max): one FMA and one ex2 per score
    if (kb * kTK + kTK - 1 > pos0 + warp * 16) {
      const int kbase = kb * kTK + 2 * (lane & 3);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (kbase + n * 8 + (j & 1) > qpos0 + (j >> 1) * 8) s[n][j] = -INFINITY;
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
    const float r0 = ex2_approx(m0 - e0), r1 = ex2_approx(m1 - e1);          // 2^(-inf) = 0 when nothing was seen yet
    m0 = mn0; m1 = mn1;
    l0 *= r0; l1 *= r1;
#pragma unroll
    for (int i = 0; i < 2 * DK; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
    uint32_t pa[4][4];                                  // P as A fragments: 4 k-steps of 16 keys
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
      for (int n = 0; n < 2 * DK; n += 2) {             // one ldmatrix.x4.trans feeds two output column tiles
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(smem_u32(bv + (kk * 16 + (lane & 15)) * LD + n * 8 + (lane >> 4) * 8), b0, b1, b2, b3);
        mma_bf16_16816(o[n], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        mma_bf16_16816(o[n + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
      }
    }
    __syncthreads();                                    // everyone is done with `buf` before the next prefetch lands in it
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (sinks) { l0 += ex2_approx(sink2 - m0); l1 += ex2_approx(sink2 - m1); }
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
#pragma unroll
  for (int n = 0; n < 2 * DK; ++n) {
    const int d = n * 8 + 2 * (lane & 3);
    if (ra < nrows)
      *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + ra) * H + h) * D + d) = pack_bf16x2(o[n][0] * i0, o[n][1] * i0);
    if (rb < nrows)
      *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + rb) * H + h) * D + d) = pack_bf16x2(o[n][2] * i1, o[n][3] * i1);
  }
}

template <int DK>
static int launch_mma(const void* q, long long q_stride, const void* ck, const void* cv, const int* tiles, int n_tiles,
                      const int* table, int max_blocks, const float* sinks, void* out, int H, int G, int block_size, float scale,
                      cudaStream_t st) {
  constexpr int LD = 16 * DK + 8;
  const size_t smem = (size_t)(4 * kTK) * LD * sizeof(__nv_bfloat16);
  auto kern = paged_attn_mma_kernel<DK>;
  if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  if ((1 << bs_log2) != block_size) return B200_ERR_UNSUPPORTED;
  kern<<<dim3(n_tiles, H), 128, smem, st>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)ck, (const __nv_bfloat16*)cv,
                                             tiles, table, max_blocks, sinks, (__nv_bfloat16*)out, H, G, bs_log2, scale);
  B200_LAUNCH_CHECK();
  return 0;
}

}  // namespace b200

using namespace b200;

B200_API int b200_rope_paged_store(void* qkv, long long row_stride, const void* cos_t, const void* sin_t, const void* pos,
                                   const void* slot, const void* table, int max_blocks, void* ck, void* cv, int tokens, int H,
                                   int G, int D, int rot, int block_size, int interleaved, int v_from_k, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (H < 0 || G <= 0 || D <= 0 || rot < 0 || rot > D || (rot & 1) || block_size <= 0) return B200_ERR_BAD_SHAPE;
#define ROPE_LAUNCH(T)                                                                                                        \
  rope_paged_store_kernel<T><<<tokens, 128, 0, st>>>((T*)qkv, row_stride, (const float*)cos_t, (const float*)sin_t,           \
                                                     (const int*)pos, (const int*)slot, (const int*)table, max_blocks, (T*)ck, \
                                                     (T*)cv, H, G, D, rot, block_size, interleaved, v_from_k)
  if (dtype == B200_DT_BF16) ROPE_LAUNCH(__nv_bfloat16);
  else if (dtype == B200_DT_FP16) ROPE_LAUNCH(__half);
  else if (dtype == B200_DT_FP32) ROPE_LAUNCH(float);
  else return B200_ERR_UNSUPPORTED;
#undef ROPE_LAUNCH
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_paged_attn(const void* q, long long q_stride, const void* ck, const void* cv, const void* pos, const void* slot,
                             const void* table, int max_blocks, const void* sinks, void* out, void* part, int tokens, int H, int G,
                             int D, int block_size, float scale, int window, int nsplit, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || D > kMaxD || block_size <= 0 || nsplit < 1) return B200_ERR_BAD_SHAPE;
  if (nsplit > 1 && !part) return B200_ERR_BAD_SHAPE;
  const int rep = H / G;
  {
    // vector kernel: rows of whole 16-byte chunks, at most 32 of them, pages of a power-of-two size
    const int E = dtype == B200_DT_FP32 ? 4 : 8;
    const int CPR = D / E;
    int bs_log2 = 0;
    while ((1 << bs_log2) < block_size) ++bs_log2;
    if (D % E == 0 && CPR <= 32 && (1 << bs_log2) == block_size && q_stride % E == 0 && !(reinterpret_cast<uintptr_t>(q) & 15)) {
      int CP = 1;
      while (CP < CPR) CP <<= 1;
      const int HB = rep >= 4 ? 4 : (rep >= 2 ? 2 : 1);
      const int passes = (rep + HB - 1) / HB;
      dim3 vgrid(tokens, G * passes, nsplit);
      const size_t vsmem = (size_t)4 * HB * (D + 2) * sizeof(float);
#define VEC_LAUNCH(T, HBV)                                                                                                     \
  paged_attn_vec_kernel<T, HBV><<<vgrid, 128, vsmem, st>>>((const T*)q, q_stride, (const T*)ck, (const T*)cv, (const int*)pos,  \
                                                           (const int*)slot, (const int*)table, max_blocks, (const float*)sinks, \
                                                           (T*)out, (float*)part, H, G, D, bs_log2, scale, window, nsplit, CP, CPR)
#define VEC_DISPATCH(T)                                                                                                        \
  do {                                                                                                                         \
    if (HB == 4) VEC_LAUNCH(T, 4); else if (HB == 2) VEC_LAUNCH(T, 2); else VEC_LAUNCH(T, 1);                                  \
    if (nsplit > 1)                                                                                                            \
      paged_attn_merge_kernel<T><<<dim3(tokens, H), 64, 0, st>>>((const float*)part, (const float*)sinks, (T*)out, H, D, nsplit); \
  } while (0)
      if (dtype == B200_DT_BF16) VEC_DISPATCH(__nv_bfloat16);
      else if (dtype == B200_DT_FP16) VEC_DISPATCH(__half);
      else if (dtype == B200_DT_FP32) VEC_DISPATCH(float);
      else return B200_ERR_UNSUPPORTED;
#undef VEC_DISPATCH
#undef VEC_LAUNCH
      B200_LAUNCH_CHECK();
      return 0;
    }
  }
  const int warps = rep < 8 ? rep : 8;
  dim3 grid(tokens, G, nsplit), block(32 * warps);
  const size_t smem = (size_t)warps * D * sizeof(float);
#define ATTN_LAUNCH(T)                                                                                                          \
  do {                                                                                                                          \
    paged_attn_kernel<T><<<grid, block, smem, st>>>((const T*)q, q_stride, (const T*)ck, (const T*)cv, (const int*)pos,         \
                                                    (const int*)slot, (const int*)table, max_blocks, (const float*)sinks,       \
                                                    (T*)out, (float*)part, H, G, D, block_size, scale, window, nsplit);         \
    if (nsplit > 1)                                                                                                             \
      paged_attn_merge_kernel<T><<<dim3(tokens, H), 64, 0, st>>>((const float*)part, (const float*)sinks, (T*)out, H, D, nsplit); \
  } while (0)
  if (dtype == B200_DT_BF16) ATTN_LAUNCH(__nv_bfloat16);
  else if (dtype == B200_DT_FP16) ATTN_LAUNCH(__half);
  else if (dtype == B200_DT_FP32) ATTN_LAUNCH(float);
  else return B200_ERR_UNSUPPORTED;
#undef ATTN_LAUNCH
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_paged_attn_mma(const void* q, long long q_stride, const void* ck, const void* cv, const void* tiles, int n_tiles,
                                 const void* table, int max_blocks, const void* sinks, void* out, int H, int G, int D,
                                 int block_size, float scale, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_tiles <= 0) return 0;
  if (dtype != B200_DT_BF16 || D % 16 || D < 16 || D > 128 || !(scale > 0.f)) return B200_ERR_UNSUPPORTED;
  if (H <= 0 || G <= 0 || H % G || block_size <= 0 || (q_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15)) return B200_ERR_BAD_SHAPE;
#define MMA(DK) case DK: return launch_mma<DK>(q, q_stride, ck, cv, (const int*)tiles, n_tiles, (const int*)table, max_blocks, \
                                                (const float*)sinks, out, H, G, block_size, scale, st)
  switch (D / 16) { MMA(1); MMA(2); MMA(3); MMA(4); MMA(5); MMA(6); MMA(7); MMA(8); }
#undef MMA
  return B200_ERR_UNSUPPORTED;
}
