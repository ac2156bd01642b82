// Recurrent mixers of the ragged serving step: short causal convolutions with a carried tail, and linear-attention state
// scans (a decayed outer-product state, and the gated delta rule), all in fp32.
//
// A step is a flat list of tokens; token t sits at position pos[t] of the sequence in state row slot[t]. The tokens of one
// sequence are consecutive and form a run; `runs` int32 [n_runs, 4] = (first row, rows, position of the first row, state
// row), or NULL: every token is a run of its own (a decode batch, read from pos / slot on the device). A run that starts
// at position 0 starts from a zero state whatever its state row held before, so rows are reused without clearing.
//
//   b200_short_conv        y[t, c] = act(sum_j w[c, j] x[t - (taps - 1) + j, c]); inputs before the run come from the tail
//                          kept in `state` [rows, taps - 1, C] (the last taps - 1 inputs; zeros before position 0).
//   b200_silu_rows         x <- silu(x) in place on a column slice of fp32 rows (the activation of projections that enter a
//                          scan without a convolution, done once instead of by every CTA that reads them).
//   b200_short_conv_tail   advances that tail over the step's runs (launched after the convolution has read the old one).
//   b200_delta_gates       q, k -> unit vectors per head (q also times `qscale`); a -> exp(-exp(A_log[h]) softplus(a + bias));
//                          b -> sigmoid(b); in place, fp32.
//   b200_linear_scan       per head, state S [D, Dv] (fp32, in `state` [rows, H, D, Dv]):
//                            mode 0  S <- decay_h S + k v^T ;                                   o = S^T q
//                            mode 1  S <- diag(g) S ; u = beta (v - S^T k) ; S <- S + k u^T ;   o = S^T q
//                            mode 2  S <- a_t S + b_t k v^T  (a, b one number per token and head) ;   o = S^T q
//                          `ones` appends a column of ones to v (the state's last column is then the decayed sum of the
//                          b_t k_t, and o's last column its product with q: the normaliser of an mLSTM read-out).
//   b200_mlstm_gates       capped log gates of an mLSTM with their running maximum m (carried per sequence and head):
//                          i = cap tanh((gi + bi) / cap), f = logsigmoid(cap tanh((gf + bf) / cap)), m' = max(f + m, i);
//                          a = exp(f + m - m'), b = exp(i - m'), e = exp(-m'). m = 0 before position 0.
//   b200_ssm_gates         step sizes of a selective state space: dt = softplus(x + bias), a = exp(-exp(A_log) dt), b = dt.
//   b200_scan_readout      what follows a scan per token: optional division of each head by max(|last column|, e) + den_eps,
//                          optional skip D_h x, optional silu gate BEFORE the norm, RMS norm over equal column groups,
//                          weight (one per column, or shared by the groups), optional sigmoid gate AFTER the norm.
//                          Columns of S are independent, so a thread owns R rows of one column, the lanes that share a
//                          column reduce their partial dot products by shuffles, and a CTA owns a block of columns of one
//                          (run, head): tokens are walked in order, staged through shared memory in chunks.
#include "common.cuh"
#include "../include/b200_ops.h"

namespace b200 {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// V channels per thread (V = 4: rows of x, y, the tail and C are multiples of four floats on 16-byte boundaries)
template <int V, typename TY>
__global__ void short_conv_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                                  const float* __restrict__ bias, const float* __restrict__ state, const int* __restrict__ pos,
                                  const int* __restrict__ slot, TY* __restrict__ y, long long ldy, int tokens, int C, int taps,
                                  int act, int residual) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int CV = C / V;
  if (idx >= (long long)tokens * CV) return;
  const int t = (int)(idx / CV), c = (int)(idx % CV) * V;
  const int p = pos[t], s = slot[t];
  // nb: tokens of the same run right before t (at most taps - 1 matter)
  int nb = 0;
  while (nb < taps - 1 && t - nb - 1 >= 0 && slot[t - nb - 1] == s) ++nb;
  float acc[V], own[V];
#pragma unroll
  for (int e = 0; e < V; ++e) { acc[e] = bias ? bias[c + e] : 0.f; own[e] = 0.f; }
  for (int d = 0; d < taps; ++d) {                       // d tokens back
    if (p - d < 0) break;
    const float* src = d <= nb ? x + (long long)(t - d) * ldx + c : state + ((long long)s * (taps - 1) + (taps - 1 - (d - nb))) * C + c;
    float v[V];
    if (V == 4) *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(src);
    else v[0] = src[0];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      acc[e] = fmaf(w[(long long)(c + e) * taps + (taps - 1 - d)], v[e], acc[e]);
      if (d == 0) own[e] = v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = (act ? silu_f(acc[e]) : acc[e]) + (residual ? own[e] : 0.f);
  TY* dst = y + (long long)t * ldy + c;
  if (V == 4 && sizeof(TY) == 4) *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(acc);
  else {
#pragma unroll
    for (int e = 0; e < V; ++e) dst[e] = from_f32<TY>(acc[e]);
  }
}

constexpr int kMaxTaps = 16;

// x[r, c] <- silu(x[r, c]) over the first `cols` columns of rows of stride ld
template <int V>
__global__ void silu_rows_kernel(float* __restrict__ x, long long ld, long long rows, int cols) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int CV = cols / V;
  if (idx >= rows * CV) return;
  float* px = x + (idx / CV) * ld + (idx % CV) * V;
  float v[V];
  if (V == 4) *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(px);
  else v[0] = px[0];
#pragma unroll
  for (int e = 0; e < V; ++e) v[e] = silu_f(v[e]);
  if (V == 4) *reinterpret_cast<float4*>(px) = *reinterpret_cast<const float4*>(v);
  else px[0] = v[0];
}

__global__ void short_conv_tail_kernel(const float* __restrict__ x, long long ldx, float* __restrict__ state,
                                       const int* __restrict__ runs, const int* __restrict__ pos, const int* __restrict__ slot,
                                       int n_runs, int C, int taps) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_runs * C) return;
  const int r = (int)(idx / C), c = (int)(idx % C);
  int first, n, p0, s;
  if (runs) { first = runs[4 * r]; n = runs[4 * r + 1]; p0 = runs[4 * r + 2]; s = runs[4 * r + 3]; }
  else { first = r; n = 1; p0 = pos[r]; s = slot[r]; }
  const int L = taps - 1;
  float* st = state + (long long)s * L * C + c;
  float nv[kMaxTaps];
  for (int i = 0; i < L; ++i) {
    const int q = p0 + n - L + i;                        // position whose input lands in entry i
    float v = 0.f;
    if (q >= p0) v = x[(long long)(first + (q - p0)) * ldx + c];
    else if (q >= 0) v = st[(long long)(q - p0 + L) * C];
    nv[i] = v;
  }
  for (int i = 0; i < L; ++i) st[(long long)i * C] = nv[i];
}

// one warp per row of q / k / a, one thread per b
__global__ void __launch_bounds__(128)
delta_gates_kernel(float* __restrict__ q, long long ldq, float* __restrict__ k, long long ldk, float* __restrict__ a,
                   long long lda, float* __restrict__ b, long long ldb, const float* __restrict__ dt_bias,
                   const float* __restrict__ A_log, int G, int H, int D, float qscale, float unit_eps) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int r = warp; r < 2 * G + H; r += nw) {
    if (r < 2 * G) {
      float* x = r < G ? q + (long long)t * ldq + (long long)r * D : k + (long long)t * ldk + (long long)(r - G) * D;
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss += x[d] * x[d];
      ss = warp_sum(ss);
      const float sc = rsqrtf(ss + unit_eps) * (r < G ? qscale : 1.f);
      for (int d = lane; d < D; d += 32) x[d] *= sc;
    } else {
      const int h = r - 2 * G;
      float* x = a + (long long)t * lda + (long long)h * D;
      const float rate = expf(A_log[h]);
      for (int d = lane; d < D; d += 32) {
        const float z = x[d] + dt_bias[h * D + d];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        x[d] = expf(-rate * sp);
      }
    }
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float* x = b + (long long)t * ldb + h;
    *x = 1.f / (1.f + expf(-*x));
  }
}

constexpr int kScanChunk = 16;

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16f(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (runs, H, column blocks); block = NW warps; a warp covers 32 / LPC columns, lane = l * (32 / LPC) + jj. The chunk of
// tokens after the one being walked is already on its way into the other shared-memory buffer (cp.async), so the walk
// waits for global memory once per run, not once per chunk. `vec`: rows of q / k / g start on 16-byte boundaries.
template <int R, int MODE, int LPC>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                   const float* __restrict__ v, long long ldv, const float* __restrict__ g, long long ldg,
                   const float* __restrict__ beta, long long ldb, const float* __restrict__ decay, float* __restrict__ state,
                   const int* __restrict__ runs, const int* __restrict__ pos, const int* __restrict__ slot,
                   float* __restrict__ o, int H, int G, int D, int Dv, int act, int vec, int ones) {
  // MODE 2 reads its two per-token numbers through the pointers of mode 1's per-channel decays: g = a [T, H], beta = b [T, H]
  extern __shared__ __align__(16) float sm[];
  const int r_ = blockIdx.x, h = blockIdx.y;
  int first, n, p0, s;
  if (runs) { first = runs[4 * r_]; n = runs[4 * r_ + 1]; p0 = runs[4 * r_ + 2]; s = runs[4 * r_ + 3]; }
  else { first = r_; n = 1; p0 = pos[r_]; s = slot[r_]; }
  const int kvh = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  constexpr int cpw = 32 / LPC;                           // columns per warp
  const int l = lane / cpw, jj = lane % cpw;
  const int ncol = nw * cpw;                              // columns per CTA
  const int col0 = blockIdx.z * ncol;
  const int j = col0 + warp * cpw + jj;
  const bool live = j < Dv;
  const int row0 = l * R;
  constexpr int RP = R + 4;                               // a lane group's rows, padded so that the groups' 16-byte reads
  constexpr int DP = LPC * RP;                            // of one token fall into different banks
  auto at = [](int d) { return (d / R) * RP + d % R; };   // key channel d -> its place in a staged row
  const int ncp = (ncol + 3) & ~3;
  const int vcols = Dv - ones;                            // columns that come from v; column vcols, if any, is all ones
  const int per = kScanChunk * DP * (MODE == 1 ? 3 : 2) + kScanChunk * ncp + 2 * kScanChunk;  // floats per buffer
  auto KS = [&](int b) { return sm + b * per; };                                               // [chunk][DP]
  auto QS = [&](int b) { return sm + b * per + kScanChunk * DP; };
  auto GS = [&](int b) { return sm + b * per + 2 * kScanChunk * DP; };                         // MODE 1 only
  auto VS = [&](int b) { return sm + b * per + (MODE == 1 ? 3 : 2) * kScanChunk * DP; };       // [chunk][ncp]
  auto BS = [&](int b) { return VS(b) + kScanChunk * ncp; };                                   // [chunk]
  auto AS = [&](int b) { return VS(b) + kScanChunk * ncp + kScanChunk; };                      // [chunk], MODE 2 only
  float* os = sm + 2 * per;                               // [chunk][ncol][LPC]: per-lane parts of the read-outs of a chunk
  // padding rows (D <= d < DP) never arrive by copy: k = q = 0 (and a finite g) keep their state at zero
  if (LPC * R > D) {
    const int padw = LPC * R - D;
    for (int i = threadIdx.x; i < 2 * kScanChunk * padw; i += blockDim.x) {
      const int b = i / (kScanChunk * padw), r = i % (kScanChunk * padw);
      const int x = (r / padw) * DP + at(D + r % padw);
      KS(b)[x] = 0.f;
      QS(b)[x] = 0.f;
      if (MODE == 1) GS(b)[x] = 0.f;
    }
  }
  // the state rows of a thread as pairs: the walk runs on packed fp32 FMAs (two IEEE FMAs per instruction, same results)
  float2 S2[R / 2];
  float* sp = state + (((long long)s * H + h) * D) * Dv;
#pragma unroll
  for (int i = 0; i < R / 2; ++i) {
    S2[i].x = (p0 > 0 && live && row0 + 2 * i < D) ? sp[(long long)(row0 + 2 * i) * Dv + j] : 0.f;
    S2[i].y = (p0 > 0 && live && row0 + 2 * i + 1 < D) ? sp[(long long)(row0 + 2 * i + 1) * Dv + j] : 0.f;
  }
  const float dec = MODE == 0 ? decay[h] : 0.f;

  auto stage = [&](int b, int c0) {
    const int cn = min(kScanChunk, n - c0);
    for (int tt = warp; tt < cn; tt += nw) {
      const long long tr = first + c0 + tt;
      const float* kr = k + tr * ldk + (long long)kvh * D;
      const float* qr = q + tr * ldq + (long long)kvh * D;
      const float* gr = MODE == 1 ? g + tr * ldg + (long long)h * D : nullptr;
      if (vec) {
        for (int d = lane * 4; d < D; d += 128) {
          cp_async16f(KS(b) + tt * DP + at(d), kr + d);
          cp_async16f(QS(b) + tt * DP + at(d), qr + d);
          if (MODE == 1) cp_async16f(GS(b) + tt * DP + at(d), gr + d);
        }
      } else {
        for (int d = lane; d < D; d += 32) {
          cp_async4(KS(b) + tt * DP + at(d), kr + d);
          cp_async4(QS(b) + tt * DP + at(d), qr + d);
          if (MODE == 1) cp_async4(GS(b) + tt * DP + at(d), gr + d);
        }
      }
      const float* vr = v + tr * ldv + (long long)h * vcols + col0;
      for (int cc = lane; cc < ncol && col0 + cc < Dv; cc += 32) {
        if (col0 + cc < vcols) cp_async4(VS(b) + tt * ncp + cc, vr + cc);
        else VS(b)[tt * ncp + cc] = 1.f;
      }
      if (MODE >= 1 && lane == 0) cp_async4(BS(b) + tt, beta + tr * ldb + h);
      if (MODE == 2 && lane == 1) cp_async4(AS(b) + tt, g + tr * ldg + h);
    }
  };

  stage(0, 0);
  cp_commit();
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += kScanChunk, buf ^= 1) {
    const int cn = min(kScanChunk, n - c0);
    const bool more = c0 + kScanChunk < n;
    if (more) stage(buf ^ 1, c0 + kScanChunk);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
    if (act) {
      for (int i = threadIdx.x; i < cn * DP; i += blockDim.x) { KS(buf)[i] = silu_f(KS(buf)[i]); QS(buf)[i] = silu_f(QS(buf)[i]); }
      for (int i = threadIdx.x; i < cn * ncp; i += blockDim.x) VS(buf)[i] = silu_f(VS(buf)[i]);
      __syncthreads();
    }
    const float* ks = KS(buf);
    const float* qs = QS(buf);
    const float* gs = GS(buf);
    const float* vs = VS(buf);
    const float* bs = BS(buf);
    const float* as = AS(buf);
    const float* vsp = vs + warp * cpw + jj;
    float* osp = os + (warp * cpw + jj) * LPC + l;
#pragma unroll 4
    for (int tt = 0; tt < cn; ++tt) {
      float2 kr[R / 2], qr[R / 2];
#pragma unroll
      for (int i = 0; i < R / 2; i += 2) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * DP + l * RP + 2 * i);
        const float4 q4 = *reinterpret_cast<const float4*>(qs + tt * DP + l * RP + 2 * i);
        kr[i] = make_float2(k4.x, k4.y); kr[i + 1] = make_float2(k4.z, k4.w);
        qr[i] = make_float2(q4.x, q4.y); qr[i + 1] = make_float2(q4.z, q4.w);
      }
      const float vj = MODE == 2 ? vsp[tt * ncp] * bs[tt] : vsp[tt * ncp];
      float2 oa = make_float2(0.f, 0.f), ob = make_float2(0.f, 0.f);
      if (MODE != 1) {
        const float dt_ = MODE == 2 ? as[tt] : dec;
        const float2 v2 = make_float2(vj, vj), dec2 = make_float2(dt_, dt_);
#pragma unroll
        for (int i = 0; i < R / 2; i += 2) {
          S2[i] = __ffma2_rn(dec2, S2[i], __fmul2_rn(kr[i], v2));
          S2[i + 1] = __ffma2_rn(dec2, S2[i + 1], __fmul2_rn(kr[i + 1], v2));
          oa = __ffma2_rn(S2[i], qr[i], oa);
          ob = __ffma2_rn(S2[i + 1], qr[i + 1], ob);
        }
      } else {
        float2 da = make_float2(0.f, 0.f), db = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < R / 2; i += 2) {
          const float4 g4 = *reinterpret_cast<const float4*>(gs + tt * DP + l * RP + 2 * i);
          S2[i] = __fmul2_rn(S2[i], make_float2(g4.x, g4.y));
          S2[i + 1] = __fmul2_rn(S2[i + 1], make_float2(g4.z, g4.w));
          da = __ffma2_rn(S2[i], kr[i], da);
          db = __ffma2_rn(S2[i + 1], kr[i + 1], db);
        }
        float dot = (da.x + da.y) + (db.x + db.y);
#pragma unroll
        for (int x = cpw; x < 32; x <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
        const float u = bs[tt] * (vj - dot);
        const float2 u2 = make_float2(u, u);
#pragma unroll
        for (int i = 0; i < R / 2; i += 2) {
          S2[i] = __ffma2_rn(kr[i], u2, S2[i]);
          S2[i + 1] = __ffma2_rn(kr[i + 1], u2, S2[i + 1]);
          oa = __ffma2_rn(S2[i], qr[i], oa);
          ob = __ffma2_rn(S2[i + 1], qr[i + 1], ob);
        }
      }
      const float o0 = oa.x + oa.y, o1 = ob.x + ob.y;
      // a token's read-out stays a per-lane part until the chunk is walked: nothing but the state (and, for the delta rule,
      // the reduced S^T k) sits between one token and the next
      osp[tt * ncol * LPC] = o0 + o1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < cn * ncol; i += blockDim.x) {
      const int tt = i / ncol, cc = i - tt * ncol;
      float a = 0.f;
#pragma unroll
      for (int x = 0; x < LPC; ++x) a += os[i * LPC + x];
      if (col0 + cc < Dv) o[((long long)(first + c0 + tt) * H + h) * Dv + col0 + cc] = a;
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < R / 2; ++i) {
      if (row0 + 2 * i < D) sp[(long long)(row0 + 2 * i) * Dv + j] = S2[i].x;
      if (row0 + 2 * i + 1 < D) sp[(long long)(row0 + 2 * i + 1) * Dv + j] = S2[i].y;
    }
  }
}

// One warp per (run, head), a lane per token of a chunk of 32: the gates are formed in parallel and the maximum recurrence
// m_t = max(f_t + m_(t-1), i_t) is a warp scan over max-plus maps; the maximum is carried from chunk to chunk.
__global__ void __launch_bounds__(128)
mlstm_gates_kernel(const float* __restrict__ gi, long long ldi, const float* __restrict__ gf, long long ldf,
                   const float* __restrict__ bi, const float* __restrict__ bf, float cap, float* __restrict__ mstate,
                   const int* __restrict__ runs, const int* __restrict__ pos, const int* __restrict__ slot, int n_runs, int H,
                   float* __restrict__ a, float* __restrict__ b, float* __restrict__ e) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + warp;
  if (w >= (long long)n_runs * H) return;
  const int r = (int)(w / H), h = (int)(w % H);
  int first, n, p0, s;
  if (runs) { first = runs[4 * r]; n = runs[4 * r + 1]; p0 = runs[4 * r + 2]; s = runs[4 * r + 3]; }
  else { first = r; n = 1; p0 = pos[r]; s = slot[r]; }
  float m = p0 > 0 ? mstate[(long long)s * H + h] : 0.f;
  const float bih = bi[h], bfh = bf[h];
  // the next chunk's gate inputs are fetched while this one is walked
  float gin = 0.f, gfn = 0.f;
  if (lane < n) { gin = gi[(long long)(first + lane) * ldi + h]; gfn = gf[(long long)(first + lane) * ldf + h]; }
  for (int c0 = 0; c0 < n; c0 += 32) {
    const int cn = min(32, n - c0);
    const float gic = gin, gfc = gfn;
    if (c0 + 32 + lane < n) {
      gin = gi[(long long)(first + c0 + 32 + lane) * ldi + h];
      gfn = gf[(long long)(first + c0 + 32 + lane) * ldf + h];
    }
    float fv = 0.f, iv = 0.f;
    if (lane < cn) {
      iv = cap * tanhf((gic + bih) / cap);
      const float z = cap * tanhf((gfc + bfh) / cap);
      fv = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));        // log sigmoid(z)
    }
    // token j maps the running maximum x to max(x + f_j, i_j); two such maps compose to one of the same form,
    // (A1, B1) then (A2, B2) = (A1 + A2, max(B1 + A2, B2)), so the 32 tokens of a chunk are a warp scan of five steps
    // instead of 32 dependent ones. Lanes past the chunk hold the identity (0, -inf). How the sums are rounded does not
    // matter downstream: decay and input scale below are formed from the same maxima.
    float A = lane < cn ? fv : 0.f, B = lane < cn ? iv : -INFINITY;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float Ap = __shfl_up_sync(0xffffffffu, A, d), Bp = __shfl_up_sync(0xffffffffu, B, d);
      if (lane >= d) { B = fmaxf(Bp + A, B); A = Ap + A; }
    }
    const float mnew = fmaxf(m + A, B);
    float mprev = __shfl_up_sync(0xffffffffu, mnew, 1);
    if (lane == 0) mprev = m;
    if (lane < cn) {
      const long long t = first + c0 + lane;
      a[t * H + h] = expf(fv + mprev - mnew);
      b[t * H + h] = expf(iv - mnew);
      e[t * H + h] = expf(-mnew);
    }
    m = __shfl_sync(0xffffffffu, mnew, cn - 1);
  }
  if (lane == 0) mstate[(long long)s * H + h] = m;
}

// The same for runs of many tokens: a CTA of eight warps per (run, head) takes 256 tokens per round. Every warp scans its
// chunk of 32 without knowing the incoming maximum (the composite map of a chunk does not depend on it), leaves the
// chunk's composite in shared memory, and then walks the composites of the chunks before it (at most seven steps) to get
// its own incoming maximum.
__global__ void __launch_bounds__(256)
mlstm_gates_run_kernel(const float* __restrict__ gi, long long ldi, const float* __restrict__ gf, long long ldf,
                       const float* __restrict__ bi, const float* __restrict__ bf, float cap, float* __restrict__ mstate,
                       const int* __restrict__ runs, int H, float* __restrict__ a, float* __restrict__ b, float* __restrict__ e) {
  __shared__ float cA[8], cB[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / H, h = blockIdx.x - r * H;
  const int first = runs[4 * r], n = runs[4 * r + 1], p0 = runs[4 * r + 2], s = runs[4 * r + 3];
  float m = p0 > 0 ? mstate[(long long)s * H + h] : 0.f;
  const float bih = bi[h], bfh = bf[h];
  for (int c0 = 0; c0 < n; c0 += 256) {
    const int t0 = c0 + warp * 32;
    const int cn = max(0, min(32, n - t0));
    float fv = 0.f, iv = 0.f;
    if (lane < cn) {
      const long long t = first + t0 + lane;
      iv = cap * tanhf((gi[t * ldi + h] + bih) / cap);
      const float z = cap * tanhf((gf[t * ldf + h] + bfh) / cap);
      fv = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));        // log sigmoid(z)
    }
    float A = lane < cn ? fv : 0.f, B = lane < cn ? iv : -INFINITY;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float Ap = __shfl_up_sync(0xffffffffu, A, d), Bp = __shfl_up_sync(0xffffffffu, B, d);
      if (lane >= d) { B = fmaxf(Bp + A, B); A = Ap + A; }
    }
    if (lane == 31) { cA[warp] = A; cB[warp] = B; }
    __syncthreads();
    float min_ = m, mend = m;
#pragma unroll
    for (int w2 = 0; w2 < 8; ++w2) {
      if (w2 == warp) min_ = mend;
      mend = fmaxf(mend + cA[w2], cB[w2]);
    }
    const float mnew = fmaxf(min_ + A, B);
    float mprev = __shfl_up_sync(0xffffffffu, mnew, 1);
    if (lane == 0) mprev = min_;
    if (lane < cn) {
      const long long t = first + t0 + lane;
      a[t * H + h] = expf(fv + mprev - mnew);
      b[t * H + h] = expf(iv - mnew);
      e[t * H + h] = expf(-mnew);
    }
    m = mend;
    __syncthreads();
  }
  if (threadIdx.x == 0) mstate[(long long)s * H + h] = m;
}

__global__ void ssm_gates_kernel(const float* __restrict__ dt, long long ld, const float* __restrict__ dt_bias,
                                 const float* __restrict__ A_log, float* __restrict__ a, float* __restrict__ b, long long tokens,
                                 int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * H) return;
  const long long t = idx / H;
  const int h = (int)(idx - t * H);
  const float z = dt[t * ld + h] + dt_bias[h];
  const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));  // softplus without a threshold
  a[idx] = expf(-expf(A_log[h]) * sp);
  b[idx] = sp;
}

// One CTA per token; the row [N = H * Dv] lives in shared memory between the passes. o rows have `ocols` columns per head
// (Dv, or Dv + 1 when the scan carried a column of ones).
template <typename TO>
__global__ void __launch_bounds__(256)
scan_readout_kernel(const float* __restrict__ o, int ocols, const float* __restrict__ e, float den_eps, float oscale,
                    const float* __restrict__ skip, const float* __restrict__ x, long long ldx,
                    const float* __restrict__ pre, long long ldpre, const float* __restrict__ post, long long ldpost,
                    const float* __restrict__ w, int w_full, TO* __restrict__ out, int H, int Dv, int groups, float eps) {
  extern __shared__ float row[];                         // [N] + [groups]
  const long long t = blockIdx.x;
  const int N = H * Dv, GS = N / groups;
  float* gsum = row + N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float* orow = o + t * (long long)H * ocols;
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    const int h = c / Dv, d = c - h * Dv;
    float v = orow[h * ocols + d] * oscale;
    if (e) v = v / (fmaxf(fabsf(orow[h * ocols + Dv] * oscale), e[t * H + h]) + den_eps);
    if (skip) v = fmaf(skip[h], x[t * ldx + c], v);
    if (pre) { const float z = pre[t * ldpre + c]; v *= z / (1.f + expf(-z)); }
    row[c] = v;
  }
  __syncthreads();
  for (int g = warp; g < groups; g += nw) {
    float ss = 0.f;
    for (int i = lane; i < GS; i += 32) { const float v = row[g * GS + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if (lane == 0) gsum[g] = 1.f / sqrtf(ss / (float)GS + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float v = row[c] * gsum[c / GS] * w[w_full ? c : c % GS];
    if (post) v *= 1.f / (1.f + expf(-post[t * ldpost + c]));
    out[t * N + c] = from_f32<TO>(v);
  }
}
}  // namespace b200

B200_API int b200_short_conv_ex(const float* x, long long ldx, const float* w, const float* bias, const float* state,
                                const int* pos, const int* slot, void* y, long long ldy, int tokens, int C, int taps, int act,
                                int residual, int y_dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > kMaxTaps) return B200_ERR_BAD_SHAPE;
  if (y_dtype != B200_DT_FP32 && y_dtype != B200_DT_BF16) return B200_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = C % 4 == 0 && ldx % 4 == 0 && ldy % 4 == 0 &&
                   !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(state)) & 15);
  const long long n = (long long)tokens * (vec ? C / 4 : C);
  const unsigned grid = (unsigned)((n + 255) / 256);
#define CONV(VV, TY) short_conv_kernel<VV, TY><<<grid, 256, 0, st>>>(x, ldx, w, bias, state, pos, slot, (TY*)y, ldy, tokens, C, taps, act, residual)
  if (y_dtype == B200_DT_FP32) { if (vec) CONV(4, float); else CONV(1, float); }
  else { if (vec) CONV(4, __nv_bfloat16); else CONV(1, __nv_bfloat16); }
#undef CONV
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_short_conv(const float* x, long long ldx, const float* w, const float* state, const int* pos, const int* slot,
                             float* y, long long ldy, int tokens, int C, int taps, int act, void* stream) {
  return b200_short_conv_ex(x, ldx, w, nullptr, state, pos, slot, y, ldy, tokens, C, taps, act, 0, B200_DT_FP32, stream);
}

B200_API int b200_silu_rows(float* x, long long ld, long long rows, int cols, void* stream) {
  using namespace b200;
  if (rows <= 0 || cols <= 0) return 0;
  const bool vec = cols % 4 == 0 && ld % 4 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15);
  const long long n = rows * (vec ? cols / 4 : cols);
  if (vec) silu_rows_kernel<4><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, ld, rows, cols);
  else silu_rows_kernel<1><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, ld, rows, cols);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_short_conv_tail(const float* x, long long ldx, float* state, const int* runs, const int* pos, const int* slot,
                                  int n_runs, int C, int taps, void* stream) {
  using namespace b200;
  if (n_runs <= 0 || taps <= 1) return 0;
  if (C <= 0 || taps > kMaxTaps) return B200_ERR_BAD_SHAPE;
  const long long n = (long long)n_runs * C;
  short_conv_tail_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, ldx, state, runs, pos, slot, n_runs, C, taps);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_delta_gates(float* q, long long ldq, float* k, long long ldk, float* a, long long lda, float* b, long long ldb,
                              const float* dt_bias, const float* A_log, int tokens, int G, int H, int D, float qscale,
                              float unit_eps, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  delta_gates_kernel<<<tokens, 128, 0, (cudaStream_t)stream>>>(q, ldq, k, ldk, a, lda, b, ldb, dt_bias, A_log, G, H, D, qscale, unit_eps);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_linear_scan(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                              const float* g, long long ldg, const float* beta, long long ldb, const float* decay, float* state,
                              const int* runs, const int* pos, const int* slot, int n_runs, float* o, int H, int G, int D, int Dv,
                              int mode, int act, int ones, void* stream) {
  using namespace b200;
  if (n_runs <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0 || mode < 0 || mode > 2 || H > 65535 || ones < 0 || ones > 1 || Dv - ones < 1)
    return B200_ERR_BAD_SHAPE;
  // rows per thread R in {8, 16, 32}; lanes per column LPC = power of two with LPC * R >= D
  int R = D <= 8 ? 8 : (D <= 256 ? 16 : 32);
  int LPC = 1;
  while (LPC * R < D) LPC *= 2;
  if (LPC > 32) return B200_ERR_TOO_LARGE;
  const int cpw = 32 / LPC;
  int nw = 4;
  while (nw > 1 && (nw - 1) * cpw >= Dv) --nw;            // no warp without columns
  const int ncol = nw * cpw;
  const int zb = (Dv + ncol - 1) / ncol;
  const int DP = LPC * (R + 4);
  const int ncp = (ncol + 3) & ~3;
  const size_t smem = (2 * ((size_t)kScanChunk * DP * (mode == 1 ? 3 : 2) + (size_t)kScanChunk * ncp + 2 * kScanChunk) +
                       (size_t)kScanChunk * ncol * LPC) * 4;
  if (smem > 200 * 1024) return B200_ERR_TOO_LARGE;
  auto al = [](const void* p_, long long ld) { return !(reinterpret_cast<uintptr_t>(p_) & 15) && ld % 4 == 0; };
  const int vec = D % 4 == 0 && al(q, ldq) && al(k, ldk) && (mode != 1 || al(g, ldg));
  dim3 grid(n_runs, H, zb);
  cudaStream_t st = (cudaStream_t)stream;
#define SCAN_K(RR, MM, LL)                                                                                                 \
  do {                                                                                                                     \
    auto kern = linear_scan_kernel<RR, MM, LL>;                                                                            \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
    kern<<<grid, nw * 32, smem, st>>>(q, ldq, k, ldk, v, ldv, g, ldg, beta, ldb, decay, state, runs, pos, slot, o, H, G, D, Dv, act, vec, ones); \
  } while (0)
#define SCAN(RR, LL)                                                                                                       \
  do {                                                                                                                     \
    if (mode == 0) SCAN_K(RR, 0, LL); else if (mode == 1) SCAN_K(RR, 1, LL); else SCAN_K(RR, 2, LL);                       \
  } while (0)
  if (R == 8) SCAN(8, 1);
  else if (R == 16) {
    if (LPC == 1) SCAN(16, 1); else if (LPC == 2) SCAN(16, 2); else if (LPC == 4) SCAN(16, 4); else if (LPC == 8) SCAN(16, 8); else SCAN(16, 16);
  } else {
    if (LPC == 16) SCAN(32, 16); else SCAN(32, 32);
  }
#undef SCAN
#undef SCAN_K
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_mlstm_gates(const float* gi, long long ldi, const float* gf, long long ldf, const float* bi, const float* bf,
                              float cap, float* mstate, const int* runs, const int* pos, const int* slot, int n_runs, int H,
                              float* a, float* b, float* e, void* stream) {
  using namespace b200;
  if (n_runs <= 0) return 0;
  if (H <= 0 || !(cap > 0.f)) return B200_ERR_BAD_SHAPE;
  const long long warps = (long long)n_runs * H;
  if (runs) {                                              // pieces of prompts (and the single tokens beside them)
    if (warps > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
    mlstm_gates_run_kernel<<<(unsigned)warps, 256, 0, (cudaStream_t)stream>>>(gi, ldi, gf, ldf, bi, bf, cap, mstate, runs, H, a, b, e);
    B200_LAUNCH_CHECK();
    return 0;
  }
  mlstm_gates_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>(gi, ldi, gf, ldf, bi, bf, cap, mstate, runs, pos,
                                                                                    slot, n_runs, H, a, b, e);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_ssm_gates(const float* dt, long long ld, const float* dt_bias, const float* A_log, float* a, float* b,
                            long long tokens, int H, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0) return B200_ERR_BAD_SHAPE;
  const long long n = tokens * H;
  ssm_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dt, ld, dt_bias, A_log, a, b, tokens, H);
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_scan_readout(const float* o, int ocols, const float* e, float den_eps, float oscale, const float* skip,
                               const float* x, long long ldx, const float* pre, long long ldpre, const float* post,
                               long long ldpost, const float* w, int w_full, void* out, long long tokens, int H, int Dv,
                               int groups, float eps, int out_dtype, void* stream) {
  using namespace b200;
  if (tokens <= 0) return 0;
  if (H <= 0 || Dv <= 0 || groups <= 0 || (H * Dv) % groups || ocols < Dv || (e && ocols < Dv + 1) || (skip && !x))
    return B200_ERR_BAD_SHAPE;
  const size_t smem = ((size_t)H * Dv + groups) * sizeof(float);
  if (smem > 200 * 1024) return B200_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
#define READOUT(TO)                                                                                                          \
  do {                                                                                                                       \
    auto kern = scan_readout_kernel<TO>;                                                                                     \
    if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    kern<<<(unsigned)tokens, 256, smem, st>>>(o, ocols, e, den_eps, oscale, skip, x, ldx, pre, ldpre, post, ldpost, w, w_full,  \
                                              (TO*)out, H, Dv, groups, eps);                                                 \
  } while (0)
  if (out_dtype == B200_DT_FP32) READOUT(float);
  else if (out_dtype == B200_DT_BF16) READOUT(__nv_bfloat16);
  else return B200_ERR_UNSUPPORTED;
#undef READOUT
  B200_LAUNCH_CHECK();
  return 0;
}
